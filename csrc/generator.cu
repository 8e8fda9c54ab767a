// Memory-bound kernels of the generator models (diffusion transformer, VAE decoder, vocoder):
//   * per-head RMSNorm + rotary embedding in place on strided q/k heads,
//   * row soft-max,
//   * tap gathers that turn 3x3 2-D convolutions (with optional nearest 2x upsampling and SiLU) and
//     dilated causal 1-D convolutions (with optional SnakeBeta) into GEMM operands for the tcgen05 GEMM,
//   * depth-wise causal 1-D convolution, image finalisation (latent range -> uint8 RGB).
// Activations are channels-last ([pixels, C] / [time, C]) so that every access is a 16-byte vector.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum_g(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_g(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void unpack8g(const uint4& w, float (&f)[8]) {
  f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
  f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}
__device__ __forceinline__ uint4 pack8g(const float (&f)[8]) {
  uint4 w;
  w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]);
  w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
  return w;
}
inline unsigned blocks_for(long long n, int per) { return static_cast<unsigned>((n + per - 1) / per); }

// ---------------------------------------------------------------------------------------
// Per-head RMSNorm followed by rotate-half RoPE, in place.  x: [T, heads, d] with token stride ldx;
// w: [d] bf16 or null (no norm); cs: [T, 2, d/2] fp32 or null (no rotation); optional second weight w2 for rows
// whose index within a segment of `seg` rows is >= n_first.  One warp per (token, head);
// lane l owns the pairs (l + 32 j, l + 32 j + d/2).  d is a multiple of 64, d <= 256.
// ---------------------------------------------------------------------------------------
__global__ void head_norm_rope_kernel(__nv_bfloat16* x, long long ldx, long long T, int heads, int d,
                                      const __nv_bfloat16* w, float eps, const float* cs, const __nv_bfloat16* w2,
                                      int seg, int n_first) {
  const long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= T * heads) return;
  const long long t = item / heads;
  // rows come in segments of `seg`; the first `n_first` rows of a segment use w, the others w2 (two token streams)
  if (w2 != nullptr && static_cast<int>(t % seg) >= n_first) w = w2;
  const int h = static_cast<int>(item % heads);
  const int half = d >> 1;
  const int per = half >> 5;  // pairs per lane (1..4)
  __nv_bfloat16* base = x + t * ldx + static_cast<long long>(h) * d;
  float a[4], b[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j < per) {
      a[j] = __bfloat162float(base[lane + 32 * j]);
      b[j] = __bfloat162float(base[lane + 32 * j + half]);
      ss += a[j] * a[j] + b[j] * b[j];
    }
  }
  float rstd = 1.f;
  if (w != nullptr) {
    ss = warp_sum_g(ss);
    rstd = rsqrtf(ss / static_cast<float>(d) + eps);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j < per) {
      const int i = lane + 32 * j;
      float av = a[j], bv = b[j];
      if (w != nullptr) {
        // round to bf16 after the norm, as a separate norm kernel would
        av = __bfloat162float(__float2bfloat16(av * rstd * __bfloat162float(w[i])));
        bv = __bfloat162float(__float2bfloat16(bv * rstd * __bfloat162float(w[i + half])));
      }
      if (cs != nullptr) {
        const float c = cs[t * d + i], s = cs[t * d + half + i];
        const float ra = av * c - bv * s, rb = bv * c + av * s;
        av = ra; bv = rb;
      }
      base[i] = __float2bfloat16(av);
      base[i + half] = __float2bfloat16(bv);
    }
  }
}

// ---------------------------------------------------------------------------------------
// The same operation for d = 128 on the q and the k part of a fused [T, q | k | v] projection in one launch.
// One warp per (token, group of HG heads): the token's rotary row and the four norm weights are loaded once, all
// 2 * HG head rows are fetched before the first is reduced.  Lane l owns the adjacent pair (2l, 2l+1) of the first
// half and its partners (2l+64, 2l+65), so every access is one 4-byte word per lane (128 contiguous bytes per warp).
// ---------------------------------------------------------------------------------------
template <int HG>
__global__ void qk_norm_rope128_kernel(__nv_bfloat16* x, long long ldx, long long T, int heads, long long part_stride,
                                       const __nv_bfloat16* wq, const __nv_bfloat16* wk, const __nv_bfloat16* wq2,
                                       const __nv_bfloat16* wk2, float eps, const float* cs, int seg, int n_first) {
  const long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = heads / HG;
  if (item >= T * groups) return;
  const long long t = item / groups;
  const int g = static_cast<int>(item - t * groups);
  if (wq2 != nullptr && static_cast<int>(t % seg) >= n_first) { wq = wq2; wk = wk2; }
  const float2 c = *reinterpret_cast<const float2*>(cs + t * 128 + 2 * lane);
  const float2 sn = *reinterpret_cast<const float2*>(cs + t * 128 + 64 + 2 * lane);
  __nv_bfloat16* row = x + t * ldx + static_cast<long long>(g) * HG * 128 + 2 * lane;
  __nv_bfloat162 lo[2][HG], hi[2][HG];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int h = 0; h < HG; ++h) {
      const __nv_bfloat16* b = row + p * part_stride + h * 128;
      lo[p][h] = *reinterpret_cast<const __nv_bfloat162*>(b);
      hi[p][h] = *reinterpret_cast<const __nv_bfloat162*>(b + 64);
    }
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const __nv_bfloat16* w = p == 0 ? wq : wk;
    const float2 wl = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + 2 * lane));
    const float2 wh = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + 64 + 2 * lane));
    float ss[HG];
    float2 a[HG], b[HG];
#pragma unroll
    for (int h = 0; h < HG; ++h) {
      a[h] = __bfloat1622float2(lo[p][h]);
      b[h] = __bfloat1622float2(hi[p][h]);
      ss[h] = a[h].x * a[h].x + a[h].y * a[h].y + b[h].x * b[h].x + b[h].y * b[h].y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int h = 0; h < HG; ++h) ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], o);
#pragma unroll
    for (int h = 0; h < HG; ++h) {
      const float rstd = rsqrtf(ss[h] * (1.f / 128.f) + eps);
      // round to bf16 after the norm, as a separate norm kernel would
      const float ax = __bfloat162float(__float2bfloat16(a[h].x * rstd * wl.x));
      const float ay = __bfloat162float(__float2bfloat16(a[h].y * rstd * wl.y));
      const float bx = __bfloat162float(__float2bfloat16(b[h].x * rstd * wh.x));
      const float by = __bfloat162float(__float2bfloat16(b[h].y * rstd * wh.y));
      __nv_bfloat16* d = row + p * part_stride + h * 128;
      *reinterpret_cast<__nv_bfloat162*>(d) = __floats2bfloat162_rn(ax * c.x - bx * sn.x, ay * c.y - by * sn.y);
      *reinterpret_cast<__nv_bfloat162*>(d + 64) = __floats2bfloat162_rn(bx * c.x + ax * sn.x, by * c.y + ay * sn.y);
    }
  }
}

// ---------------------------------------------------------------------------------------
// y[r, :] = softmax(scale * x[r, :]) over `cols` columns, bf16 in / out, one CTA of 256 threads per row.
// ---------------------------------------------------------------------------------------
__global__ void softmax_rows_kernel(const __nv_bfloat16* x, long long ldx, __nv_bfloat16* y, long long ldy,
                                    int cols, float scale) {
  __shared__ float red[8];
  const long long r = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + r * ldx);
  uint4* yr = reinterpret_cast<uint4*>(y + r * ldy);
  const int nvec = cols >> 3;
  float m = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    float f[8];
    unpack8g(xr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, f[j]);
  }
  m = warp_max_g(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    float f[8];
    unpack8g(xr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf((f[j] - m) * scale);
  }
  s = warp_sum_g(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += red[i];
  const float inv = 1.f / s;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    float f[8];
    unpack8g(xr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __expf((f[j] - m) * scale) * inv;
    yr[v] = pack8g(f);
  }
}

// ---------------------------------------------------------------------------------------
// 3x3 tap gather for a channels-last image [B, H, W, C] -> rows [B*Ho*Wo, 9*C], tap-major (ky, kx, c), zero
// padding 1.  up == 2 reads the source through a nearest-neighbour 2x upsampling (Ho = 2H, Wo = 2W); stride 2
// halves the output extent (Ho = (H - 1) / 2 + 1).
// silu != 0 applies SiLU to every gathered value (the activation that precedes the convolution).
// ---------------------------------------------------------------------------------------
__global__ void im2col3x3_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, int B, int H, int W, int C, int up,
                                 int silu, int stride) {
  const int cv = C >> 3;
  const int Hu = H * up, Wu = W * up;                                   // (upsampled) input extent
  const int Ho = (Hu - 1) / stride + 1, Wo = (Wu - 1) / stride + 1;     // output extent
  const long long total = static_cast<long long>(B) * Ho * Wo * 9 * cv;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % cv);
  const int tap = static_cast<int>((idx / cv) % 9);
  const long long pix = idx / (9LL * cv);
  const int xo = static_cast<int>(pix % Wo);
  const int yo = static_cast<int>((pix / Wo) % Ho);
  const int b = static_cast<int>(pix / (static_cast<long long>(Wo) * Ho));
  const int ys = yo * stride + tap / 3 - 1, xs = xo * stride + tap % 3 - 1;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (ys >= 0 && ys < Hu && xs >= 0 && xs < Wu) {
    const long long s = (static_cast<long long>(b) * H + ys / up) * W + xs / up;
    v = *reinterpret_cast<const uint4*>(src + s * C + c * 8);
    if (silu) {
      float f[8];
      unpack8g(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __fdividef(f[j], 1.f + __expf(-f[j]));
      v = pack8g(f);
    }
  }
  *reinterpret_cast<uint4*>(dst + pix * 9 * C + static_cast<long long>(tap) * C + c * 8) = v;
}

// ---------------------------------------------------------------------------------------
// 1-D tap gather for channels-last sequences [B, T, C] -> rows [B*To, taps*C]:
//   dst[b, t, j, :] = act(src[b, t * stride + first + j * dilation, :])   (zero outside [0, T))
// act == 1: SnakeBeta, x + sin^2(x * exp(alpha[c])) / (exp(beta[c]) + 1e-9).
// A causal convolution with kernel k uses first = -(k - 1) * dilation; a stride-s transposed convolution
// with kernel 2s uses taps = 2, first = -1 ... see the Python wrapper.
// ---------------------------------------------------------------------------------------
__global__ void im2col1d_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, int B, int T, int To, int C,
                                int taps, int first, int dilation, int stride, int act, const float* alpha,
                                const float* beta) {
  const int cv = C >> 3;
  const long long total = static_cast<long long>(B) * To * taps * cv;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % cv);
  const int j = static_cast<int>((idx / cv) % taps);
  const long long row = idx / (static_cast<long long>(taps) * cv);
  const int t = static_cast<int>(row % To);
  const int b = static_cast<int>(row / To);
  const int ts = t * stride + first + j * dilation;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (ts >= 0 && ts < T) {
    v = *reinterpret_cast<const uint4*>(src + (static_cast<long long>(b) * T + ts) * C + c * 8);
    if (act == 1) {
      float f[8];
      unpack8g(v, f);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float a = __expf(alpha[c * 8 + q]), bb = __expf(beta[c * 8 + q]);
        const float s = __sinf(f[q] * a);
        f[q] = f[q] + s * s / (bb + 1e-9f);
      }
      v = pack8g(f);
    }
  }
  *reinterpret_cast<uint4*>(dst + row * taps * C + static_cast<long long>(j) * C + c * 8) = v;
}

// Depth-wise causal 1-D convolution, kernel k <= 8: y[b,t,c] = bias[c] + sum_j w[c,j] * x[b, t-(k-1)+j, c].
__global__ void dwconv1d_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, const __nv_bfloat16* w,
                                const __nv_bfloat16* bias, int B, int T, int C, int k) {
  const long long total = static_cast<long long>(B) * T * C;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const int t = static_cast<int>((idx / C) % T);
  const long long b = idx / (static_cast<long long>(C) * T);
  float acc = bias != nullptr ? __bfloat162float(bias[c]) : 0.f;
  for (int j = 0; j < k; ++j) {
    const int ts = t - (k - 1) + j;
    if (ts >= 0) acc += __bfloat162float(w[c * k + j]) * __bfloat162float(x[(b * T + ts) * C + c]);
  }
  y[idx] = __float2bfloat16(acc);
}

// Final image conversion: channels-last [pixels, ldx] bf16 in [-1, 1] (first 3 channels) -> uint8 RGB.
__global__ void to_rgb8_kernel(const __nv_bfloat16* x, long long ldx, unsigned char* y, long long pixels) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= pixels) return;
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    float v = __bfloat162float(x[i * ldx + c]) * 0.5f + 0.5f;
    v = fminf(fmaxf(v, 0.f), 1.f);
    y[i * 3 + c] = static_cast<unsigned char>(__float2int_rn(v * 255.f));
  }
}

}  // namespace

CS_API int cs_head_norm_rope(void* x, long long ldx, long long T, int heads, int d, const void* w, float eps,
                             const void* cs, const void* w2, int seg, int n_first, void* stream) {
  if (T <= 0 || heads <= 0) return 0;
  if ((d & 63) || d > 256 || (w2 != nullptr && (w == nullptr || seg <= 0))) return -1;
  const long long warps = T * heads;
  head_norm_rope_kernel<<<blocks_for(warps, 8), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)x, ldx, T, heads, d, (const __nv_bfloat16*)w, eps, (const float*)cs, (const __nv_bfloat16*)w2, seg,
      n_first);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// q and k parts of x = [T, ...] (q heads at column 0, k heads at column part_stride), d = 128, in one launch.
CS_API int cs_qk_norm_rope128(void* x, long long ldx, long long T, int heads, long long part_stride, const void* wq,
                              const void* wk, const void* wq2, const void* wk2, float eps, const void* cs, int seg,
                              int n_first, void* stream) {
  if (T <= 0 || heads <= 0) return 0;
  if (wq == nullptr || wk == nullptr || cs == nullptr || (ldx & 1) || (part_stride & 1) ||
      ((wq2 == nullptr) != (wk2 == nullptr)) || (wq2 != nullptr && seg <= 0) || (reinterpret_cast<uintptr_t>(x) & 3) ||
      (reinterpret_cast<uintptr_t>(cs) & 7))
    return -1;
  auto s = (cudaStream_t)stream;
#define CS_QK_LAUNCH(HG)                                                                                          \
  qk_norm_rope128_kernel<HG><<<blocks_for(T * (heads / HG), 8), 256, 0, s>>>(                                     \
      (__nv_bfloat16*)x, ldx, T, heads, part_stride, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk,         \
      (const __nv_bfloat16*)wq2, (const __nv_bfloat16*)wk2, eps, (const float*)cs, seg, n_first)
  if (heads % 4 == 0) CS_QK_LAUNCH(4);
  else if (heads % 2 == 0) CS_QK_LAUNCH(2);
  else CS_QK_LAUNCH(1);
#undef CS_QK_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_softmax_rows(const void* x, long long ldx, void* y, long long ldy, int rows, int cols, float scale,
                           void* stream) {
  if (rows <= 0) return 0;
  if ((cols & 7) || (ldx & 7) || (ldy & 7)) return -1;
  softmax_rows_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy,
                                                             cols, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_im2col3x3(const void* src, void* dst, int B, int H, int W, int C, int up, int silu, int stride,
                        void* stream) {
  if (B <= 0 || H <= 0 || W <= 0) return 0;
  if ((C & 7) || (up != 1 && up != 2) || (stride != 1 && stride != 2)) return -1;
  const long long Ho = (H * up - 1) / stride + 1, Wo = (W * up - 1) / stride + 1;
  const long long total = static_cast<long long>(B) * Ho * Wo * 9 * (C >> 3);
  im2col3x3_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, B, H, W, C, up, silu, stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_im2col1d(const void* src, void* dst, int B, int T, int To, int C, int taps, int first, int dilation,
                       int stride, int act, const void* alpha, const void* beta, void* stream) {
  if (B <= 0 || To <= 0) return 0;
  if ((C & 7) || taps <= 0 || stride <= 0 || (act == 1 && (alpha == nullptr || beta == nullptr))) return -1;
  const long long total = static_cast<long long>(B) * To * taps * (C >> 3);
  im2col1d_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, B, T, To, C, taps, first, dilation, stride, act, (const float*)alpha,
      (const float*)beta);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_dwconv1d(const void* x, void* y, const void* w, const void* bias, int B, int T, int C, int k,
                       void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (k <= 0 || k > 8) return -1;
  const long long total = static_cast<long long>(B) * T * C;
  dwconv1d_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, B, T, C, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_to_rgb8(const void* x, long long ldx, void* y, long long pixels, void* stream) {
  if (pixels <= 0) return 0;
  to_rgb8_kernel<<<blocks_for(pixels, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx,
                                                                           (unsigned char*)y, pixels);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// ---------------------------------------------------------------------------------------
// Bilinear lookup in a learned 2-D position table, added in place:
//   x[l, :] += sum_{i<4} wgt[i, l] * table[idx[i, l], :]
// (the four neighbours and weights of every patch are computed on the host).  H is a multiple of 8.
// ---------------------------------------------------------------------------------------
namespace {
__global__ void bilinear_embed_add_kernel(__nv_bfloat16* x, long long ldx, const __nv_bfloat16* table, long long ldt,
                                          const int* idx, const float* wgt, long long L, int H) {
  const int hv = H >> 3;
  const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= L * hv) return;
  const int c = static_cast<int>(g % hv);
  const long long l = g / hv;
  float acc[8];
  unpack8g(*reinterpret_cast<const uint4*>(x + l * ldx + c * 8), acc);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float w = wgt[i * L + l];
    float f[8];
    unpack8g(*reinterpret_cast<const uint4*>(table + static_cast<long long>(idx[i * L + l]) * ldt + c * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
  }
  *reinterpret_cast<uint4*>(x + l * ldx + c * 8) = pack8g(acc);
}
}  // namespace

CS_API int cs_bilinear_embed_add(void* x, long long ldx, const void* table, long long ldt, const void* idx,
                                 const void* wgt, long long L, int H, void* stream) {
  if (L <= 0) return 0;
  if ((H & 7) || (ldx & 7) || (ldt & 7)) return -1;
  bilinear_embed_add_kernel<<<blocks_for(L * (H >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)table, ldt, (const int*)idx, (const float*)wgt, L, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
