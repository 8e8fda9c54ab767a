// Memory-bound kernels: RMSNorm / LayerNorm (with fused residual add and AdaLN modulation),
// rotary embeddings (2-D vision tables, NeoX / M-RoPE with fused paged-KV write), SwiGLU,
// row gather / scatter, embedding lookup, greedy arg-max, flow-match Euler step, PCM16 pack.
// All of them move 16 bytes per thread per access and do their math in fp32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  float r = red[0];
  __syncthreads();
  return r;
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
  f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 w;
  w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]);
  w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
  return w;
}

// ---------------------------------------------------------------------------------------
// Norms.  One CTA of 256 threads per row; the row lives in registers (H <= 256*8*MAXV).
//   mode 0: RMSNorm            y = x * rsqrt(mean(x^2)+eps) * w
//   mode 1: Gemma RMSNorm      y = x * rsqrt(mean(x^2)+eps) * (1 + w)
//   mode 2: LayerNorm          y = (x-mean) * rsqrt(var+eps) * w + b   (w, b may be null)
// Optional: x += residual first (sum is written back to `res_out`), and AdaLN modulation
//   y = y * (1 + scale[row / rpb]) + shift[row / rpb].
// ---------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // up to 8192 columns

struct NormParams {
  const __nv_bfloat16* x; long long ldx;
  const __nv_bfloat16* residual; long long ldres;
  __nv_bfloat16* res_out; long long ldro;
  const __nv_bfloat16* w; const __nv_bfloat16* b;
  const __nv_bfloat16* scale; const __nv_bfloat16* shift; long long ldmod; int rpb;
  __nv_bfloat16* y; long long ldy;
  int rows, H; float eps; int mode;
};

__global__ void __launch_bounds__(NORM_THREADS) norm_kernel(const NormParams p) {
  __shared__ float red[NORM_THREADS / 32];
  pdl_wait();                // launched so that its CTAs may be in place before the kernel ahead of it has ended
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int nvec = p.H >> 3;
  float v[NORM_MAXV][8];
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + (long long)row * p.ldx);
  const uint4* rr = p.residual ? reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldres) : nullptr;
  uint4* ro = p.res_out ? reinterpret_cast<uint4*>(p.res_out + (long long)row * p.ldro) : nullptr;
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      unpack8(xr[c], v[i]);
      if (rr) {
        float r[8];
        unpack8(rr[c], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
      }
      if (ro) {
        uint4 w = pack8(v[i]);
        ro[c] = w;
        unpack8(w, v[i]);  // normalise the value that was stored (bf16-rounded), like the unfused sequence
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
    }
  }
  float mean = 0.f, rstd;
  if (p.mode == 2) {
    mean = block_sum<NORM_THREADS>(s, red) / p.H;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; var += d * d; }
      }
    }
    var = block_sum<NORM_THREADS>(var, red) / p.H;
    rstd = rsqrtf(var + p.eps);
  } else {
    ss = block_sum<NORM_THREADS>(ss, red) / p.H;
    rstd = rsqrtf(ss + p.eps);
  }
  const uint4* w4 = p.w ? reinterpret_cast<const uint4*>(p.w) : nullptr;
  const uint4* b4 = p.b ? reinterpret_cast<const uint4*>(p.b) : nullptr;
  const long long mrow = p.scale ? (long long)(row / p.rpb) * p.ldmod : 0;
  const uint4* sc4 = p.scale ? reinterpret_cast<const uint4*>(p.scale + mrow) : nullptr;
  const uint4* sh4 = p.shift ? reinterpret_cast<const uint4*>(p.shift + mrow) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(p.y + (long long)row * p.ldy);
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float o[8], w[8], b[8];
      if (w4) unpack8(w4[c], w);
      if (b4) unpack8(b4[c], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = (v[i][j] - mean) * rstd;
        if (w4) t *= (p.mode == 1 ? 1.0f + w[j] : w[j]);
        if (b4) t += b[j];
        o[j] = t;
      }
      if (sc4) {
        float sc[8], sh[8];
        unpack8(sc4[c], sc);
        unpack8(sh4[c], sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = o[j] * (1.0f + sc[j]) + sh[j];
      }
      yr[c] = pack8(o);
    }
  }
}

// Same math with one warp per row (no block-wide synchronisation).  The row stays in registers as the packed bf16
// words that were loaded (or stored to `res_out`), so MAXV = 16 (4096 columns) costs 64 registers.
template <int MAXV>
__global__ void __launch_bounds__(256) norm_warp_kernel(const NormParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int nvec = p.H >> 3;
  uint4 raw[MAXV];
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + (long long)row * p.ldx);
  const uint4* rr = p.residual ? reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldres) : nullptr;
  uint4* ro = p.res_out ? reinterpret_cast<uint4*>(p.res_out + (long long)row * p.ldro) : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) raw[i] = xr[c];
  }
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      float v[8];
      unpack8(raw[i], v);
      if (rr) {
        float r[8];
        unpack8(rr[c], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += r[j];
        raw[i] = pack8(v);   // normalise the value that is stored (bf16-rounded), like the unfused sequence
        unpack8(raw[i], v);
      }
      if (ro) ro[c] = raw[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[j]; ss += v[j] * v[j]; }
    }
  }
  float mean = 0.f, rstd;
  if (p.mode == 2) {
    mean = warp_sum(s) / p.H;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float v[8];
        unpack8(raw[i], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[j] - mean; var += d * d; }
      }
    }
    rstd = rsqrtf(warp_sum(var) / p.H + p.eps);
  } else {
    rstd = rsqrtf(warp_sum(ss) / p.H + p.eps);
  }
  const uint4* w4 = p.w ? reinterpret_cast<const uint4*>(p.w) : nullptr;
  const uint4* b4 = p.b ? reinterpret_cast<const uint4*>(p.b) : nullptr;
  const long long mrow = p.scale ? (long long)(row / p.rpb) * p.ldmod : 0;
  const uint4* sc4 = p.scale ? reinterpret_cast<const uint4*>(p.scale + mrow) : nullptr;
  const uint4* sh4 = p.shift ? reinterpret_cast<const uint4*>(p.shift + mrow) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(p.y + (long long)row * p.ldy);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      float v[8], o[8], w[8], b[8];
      unpack8(raw[i], v);
      if (w4) unpack8(__ldg(w4 + c), w);
      if (b4) unpack8(__ldg(b4 + c), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = (v[j] - mean) * rstd;
        if (w4) t *= (p.mode == 1 ? 1.0f + w[j] : w[j]);
        if (b4) t += b[j];
        o[j] = t;
      }
      if (sc4) {
        float sc[8], sh[8];
        unpack8(sc4[c], sc);
        unpack8(sh4[c], sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = o[j] * (1.0f + sc[j]) + sh[j];
      }
      yr[c] = pack8(o);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Rotary embeddings, rotate-half convention: for i < d/2
//   out[i]       = x[i]*cos[i] - x[i+d/2]*sin[i]
//   out[i+d/2]   = x[i+d/2]*cos[i] + x[i]*sin[i]
// `cs` holds per-token tables [T, 2, rot/2] fp32 (cos then sin).  Only the first `rot`
// channels of each head are rotated.  One thread handles 8 pair-columns.
// ---------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* x, long long ldx, int T, int heads, int d, int rot,
                            const float* cs) {
  const int half = rot >> 1;
  const int chunks = half >> 2;  // 4 pairs per thread
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)T * heads * chunks;
  if (idx >= total) return;
  const int c = idx % chunks;
  const int h = (idx / chunks) % heads;
  const long long t = idx / ((long long)chunks * heads);
  __nv_bfloat16* base = x + t * ldx + (long long)h * d + c * 4;
  const float* cosp = cs + t * rot + c * 4;
  const float* sinp = cosp + half;
  uint2 lo = *reinterpret_cast<uint2*>(base);
  uint2 hi = *reinterpret_cast<uint2*>(base + half);
  float a[4] = {bf16lo(lo.x), bf16hi(lo.x), bf16lo(lo.y), bf16hi(lo.y)};
  float b[4] = {bf16lo(hi.x), bf16hi(hi.x), bf16lo(hi.y), bf16hi(hi.y)};
  float oa[4], ob[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float cv = cosp[j], sv = sinp[j];
    oa[j] = a[j] * cv - b[j] * sv;
    ob[j] = b[j] * cv + a[j] * sv;
  }
  *reinterpret_cast<uint2*>(base) = make_uint2(pack_bf16x2(oa[0], oa[1]), pack_bf16x2(oa[2], oa[3]));
  *reinterpret_cast<uint2*>(base + half) = make_uint2(pack_bf16x2(ob[0], ob[1]), pack_bf16x2(ob[2], ob[3]));
}

// cos/sin tables for (M-)RoPE: pos is [3, T] int32 (t/h/w ids; identical rows for text-only),
// section s of the half-dim uses pos row s.  cs out: [T, 2, half] fp32.
__global__ void mrope_table_kernel(const int* pos, int T, int half, float theta, int sec0, int sec1,
                                   float* cs) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * half) return;
  const int i = idx % half;
  const long long t = idx / half;
  const int which = i < sec0 ? 0 : (i < sec0 + sec1 ? 1 : 2);
  const float p = static_cast<float>(pos[(long long)which * T + t]);
  const float inv = powf(theta, -static_cast<float>(2 * i) / static_cast<float>(2 * half));
  float s, c;
  sincosf(p * inv, &s, &c);
  cs[t * 2 * half + i] = c;
  cs[t * 2 * half + half + i] = s;
}

// Rotate q in place, rotate k and write k, v into the paged cache.
// qkv: [T, (Hq + 2*Hkv) * d]; cache: [pages, 2, Hkv, page, d]; slot[t] = page_id*page + offset.
__global__ void rope_kv_write_kernel(__nv_bfloat16* qkv, long long ld, int T, int Hq, int Hkv, int d,
                                     const float* cs, __nv_bfloat16* cache, const int* slot, int page) {
  pdl_wait();
  pdl_launch_dependents();
  const int half = d >> 1;
  const int chunks = half >> 2;
  const int heads = Hq + 2 * Hkv;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)T * heads * chunks;
  if (idx >= total) return;
  const int c = idx % chunks;
  const int h = (idx / chunks) % heads;
  const long long t = idx / ((long long)chunks * heads);
  __nv_bfloat16* base = qkv + t * ld + (long long)h * d + c * 4;
  uint2 lo = *reinterpret_cast<uint2*>(base);
  uint2 hi = *reinterpret_cast<uint2*>(base + half);
  if (h < Hq + Hkv) {
    const float* cosp = cs + t * d + c * 4;
    const float* sinp = cosp + half;
    float a[4] = {bf16lo(lo.x), bf16hi(lo.x), bf16lo(lo.y), bf16hi(lo.y)};
    float b[4] = {bf16lo(hi.x), bf16hi(hi.x), bf16lo(hi.y), bf16hi(hi.y)};
    float oa[4], ob[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float cv = cosp[j], sv = sinp[j];
      oa[j] = a[j] * cv - b[j] * sv;
      ob[j] = b[j] * cv + a[j] * sv;
    }
    lo = make_uint2(pack_bf16x2(oa[0], oa[1]), pack_bf16x2(oa[2], oa[3]));
    hi = make_uint2(pack_bf16x2(ob[0], ob[1]), pack_bf16x2(ob[2], ob[3]));
  }
  if (h < Hq) {
    *reinterpret_cast<uint2*>(base) = lo;
    *reinterpret_cast<uint2*>(base + half) = hi;
  } else {
    const int s = slot[t];
    if (s < 0) return;
    const int kv = h < Hq + Hkv ? 0 : 1;
    const int hh = kv == 0 ? h - Hq : h - Hq - Hkv;
    const long long pg = s / page, off = s % page;
    __nv_bfloat16* dst = cache + (((pg * 2 + kv) * Hkv + hh) * page + off) * d + c * 4;
    *reinterpret_cast<uint2*>(dst) = lo;
    *reinterpret_cast<uint2*>(dst + half) = hi;
  }
}

// ---------------------------------------------------------------------------------------
// y[r, :] = act(g[r, :]) * u[r, :]   (g and u are the two halves of one [rows, 2*I] buffer)
// ---------------------------------------------------------------------------------------
__global__ void act_mul_kernel(const __nv_bfloat16* gu, long long ld, __nv_bfloat16* y, long long ldy,
                               int rows, int I, int act) {
  const int nvec = I >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * nvec) return;
  const int c = idx % nvec;
  const long long r = idx / nvec;
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + c * 8), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + I + c * 8), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float a = g[j];
    if (act == 3) a = a / (1.0f + __expf(-a));
    else if (act == 2) a = 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
    else if (act == 1) a = 0.5f * a * (1.0f + erff(a * 0.70710678118654752f));
    o[j] = a * u[j];
  }
  *reinterpret_cast<uint4*>(y + r * ldy + c * 8) = pack8(o);
}

// ---------------------------------------------------------------------------------------
// Row gather / scatter (16-byte vectors): dst[i, :] = src[idx[i], :] or dst[idx[i], :] = src[i, :]
// Used for embedding lookup, window permutation and placing encoder rows into LLM inputs.
// ---------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const uint4* src, long long src_ld16, uint4* dst, long long dst_ld16,
                                   const int* idx, int n, int vec_per_row, int scatter) {
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (long long)n * vec_per_row) return;
  const int c = g % vec_per_row;
  const long long i = g / vec_per_row;
  const long long j = idx[i];
  if (j < 0) return;
  if (scatter) dst[j * dst_ld16 + c] = src[i * src_ld16 + c];
  else dst[i * dst_ld16 + c] = src[j * src_ld16 + c];
}

// ---------------------------------------------------------------------------------------
// Flat copy whose destination may be another GPU's memory (the sidecar's push of encoder rows into the
// consumer's slab): plain 16-byte loads of local memory and plain stores over NVLink, four vectors in
// flight per thread.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) push_bytes_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                         long long n16, const unsigned char* src_tail,
                                                         unsigned char* dst_tail, int tail) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

__global__ void push_bytes_unaligned_kernel(const unsigned char* src, unsigned char* dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------
// Greedy sampling: arg-max over a [rows, V] logits matrix (bf16 or fp32).  One CTA per row.
// ---------------------------------------------------------------------------------------
// Two-stage so that few rows still fill the GPU: stage 1 scans a slice of the vocabulary per CTA and
// leaves (value, index) candidates, stage 2 (one warp per row) picks the winner.
template <typename T>
__global__ void __launch_bounds__(256) argmax_stage1_kernel(const T* logits, long long ld, int V, int slices,
                                                            float* cand_v, int* cand_i) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const long long row = blockIdx.x;
  const int slice = blockIdx.y;
  const int per = (V + slices - 1) / slices;
  const int lo = slice * per, hi = min(V, lo + per);
  const T* p = logits + row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = static_cast<float>(p[i]);
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    best = l < 8 ? sv[l] : -INFINITY;
    bi = l < 8 ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (l == 0) { cand_v[row * slices + slice] = best; cand_i[row * slices + slice] = bi; }
  }
}

__global__ void argmax_stage2_kernel(const float* cand_v, const int* cand_i, int slices, int rows, int* out) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int l = threadIdx.x & 31;
  if (row >= rows) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int s = l; s < slices; s += 32) {
    const float v = cand_v[(long long)row * slices + s];
    const int i = cand_i[(long long)row * slices + s];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (l == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// ---------------------------------------------------------------------------------------
// Flow-matching Euler step with classifier-free guidance, fp32 latents:
//   v = uncond + cfg * (cond - uncond)   (uncond may be null: v = cond)
//   if norm_rescale: v *= ||cond|| / ||v|| per row (true-CFG norm preservation)
//   x += dt * v
// One CTA per row (token); C channels.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) flow_step_kernel(float* x, const __nv_bfloat16* cond,
                                                        const __nv_bfloat16* uncond, int C, float cfg,
                                                        float dt, int norm_rescale) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  float nc = 0.f, nv = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float c = __bfloat162float(cond[row * C + i]);
    float v = c;
    if (uncond) { float u = __bfloat162float(uncond[row * C + i]); v = u + cfg * (c - u); }
    nc += c * c; nv += v * v;
  }
  float scale = 1.f;
  if (uncond && norm_rescale) {
    nc = block_sum<128>(nc, red);
    nv = block_sum<128>(nv, red);
    scale = sqrtf(nc) / fmaxf(sqrtf(nv), 1e-12f);
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float c = __bfloat162float(cond[row * C + i]);
    float v = c;
    if (uncond) { float u = __bfloat162float(uncond[row * C + i]); v = u + cfg * (c - u); }
    x[row * C + i] += dt * v * scale;
  }
}

// float waveform in [-1,1] -> little-endian PCM16
__global__ void pcm16_kernel(const float* x, short* y, long long n) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = fminf(fmaxf(x[i], -1.0f), 1.0f) * 32767.0f;
  y[i] = static_cast<short>(__float2int_rn(v));
}

// writes `bytes` of zeros-then-pattern; used to evict L2 between timed iterations
__global__ void l2_flush_kernel(uint4* buf, long long n, unsigned v) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) buf[i] = make_uint4(v, v, v, v);
}

// After a decode step: feed the sampled token back as the next input, log it, advance positions,
// key counts and cache slots of every active sequence.  One block, B <= 1024.
__global__ void decode_advance_kernel(const int* sampled, int* input_ids, int* positions, int* kv_len, int* slot,
                                      const int* block_table, int bt_stride, const int* active, int* out_log,
                                      int log_cap, int* step_counter, int B, int page) {
  const int b = threadIdx.x;
  const int step = *step_counter;
  __syncthreads();
  if (b == 0) *step_counter = step + 1;
  if (b >= B) return;
  const int tok = sampled[b];
  input_ids[b] = tok;
  if (step < log_cap) out_log[step * B + b] = tok;
  if (!active[b]) return;
  positions[b] += 1;
  positions[B + b] += 1;
  positions[2 * B + b] += 1;
  const int kv = kv_len[b] + 1;
  kv_len[b] = kv;
  slot[b] = block_table[(long long)b * bt_stride + (kv - 1) / page] * page + (kv - 1) % page;
}

inline int ceil_div_ll(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace

CS_API int cs_norm(const void* x, long long ldx, const void* residual, long long ldres, void* res_out,
                   long long ldro, const void* w, const void* b, const void* scale, const void* shift,
                   long long ldmod, int rpb, void* y, long long ldy, int rows, int H, float eps, int mode,
                   void* stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > NORM_THREADS * 8 * NORM_MAXV || (ldx & 7) || (ldy & 7)) return -1;
  NormParams p{};
  p.x = (const __nv_bfloat16*)x; p.ldx = ldx;
  p.residual = (const __nv_bfloat16*)residual; p.ldres = ldres;
  p.res_out = (__nv_bfloat16*)res_out; p.ldro = ldro;
  p.w = (const __nv_bfloat16*)w; p.b = (const __nv_bfloat16*)b;
  p.scale = (const __nv_bfloat16*)scale; p.shift = (const __nv_bfloat16*)shift;
  p.ldmod = ldmod; p.rpb = rpb > 0 ? rpb : 1;
  p.y = (__nv_bfloat16*)y; p.ldy = ldy;
  p.rows = rows; p.H = H; p.eps = eps; p.mode = mode;
  cudaStream_t st = (cudaStream_t)stream;
  if (H <= 2048 && rows >= 64)
    cs_launch_pdl(norm_warp_kernel<8>, dim3((rows + 7) / 8), dim3(256), 0, st, p);
  else if (H <= 4096 && rows >= 2048 && mode == 2)  // two reductions per row: a warp needs no block-wide barrier for them
    cs_launch_pdl(norm_warp_kernel<16>, dim3((rows + 7) / 8), dim3(256), 0, st, p);
  else
    cs_launch_pdl(norm_kernel, dim3(rows), dim3(NORM_THREADS), 0, st, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_rope(void* x, long long ldx, int T, int heads, int d, int rot, const void* cs, void* stream) {
  if (T <= 0) return 0;
  if ((rot & 7) || rot > d) return -1;
  long long total = (long long)T * heads * (rot >> 3);
  rope_kernel<<<ceil_div_ll(total, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, ldx, T, heads, d,
                                                                        rot, (const float*)cs);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_mrope_table(const void* pos, int T, int half, float theta, int sec0, int sec1, void* cs,
                          void* stream) {
  if (T <= 0) return 0;
  long long total = (long long)T * half;
  mrope_table_kernel<<<ceil_div_ll(total, 256), 256, 0, (cudaStream_t)stream>>>((const int*)pos, T, half, theta,
                                                                               sec0, sec1, (float*)cs);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_rope_kv_write(void* qkv, long long ld, int T, int Hq, int Hkv, int d, const void* cs, void* cache,
                            const void* slot, int page, void* stream) {
  if (T <= 0) return 0;
  if (d & 7) return -1;
  long long total = (long long)T * (Hq + 2 * Hkv) * (d >> 3);
  cs_launch_pdl(rope_kv_write_kernel, dim3((unsigned)ceil_div_ll(total, 256)), dim3(256), 0, (cudaStream_t)stream,
                (__nv_bfloat16*)qkv, ld, T, Hq, Hkv, d, (const float*)cs, (__nv_bfloat16*)cache, (const int*)slot, page);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_act_mul(const void* gu, long long ld, void* y, long long ldy, int rows, int I, int act,
                      void* stream) {
  if (rows <= 0) return 0;
  if ((I & 7) || (ld & 7) || (ldy & 7)) return -1;
  long long total = (long long)rows * (I >> 3);
  act_mul_kernel<<<ceil_div_ll(total, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, ld,
                                                                           (__nv_bfloat16*)y, ldy, rows, I, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// row_bytes, src_ld_bytes and dst_ld_bytes must be multiples of 16.
CS_API int cs_gather_rows(const void* src, long long src_ld_bytes, void* dst, long long dst_ld_bytes,
                          const void* idx, int n, long long row_bytes, int scatter, void* stream) {
  if (n <= 0) return 0;
  if ((row_bytes & 15) || (src_ld_bytes & 15) || (dst_ld_bytes & 15)) return -1;
  const int vpr = static_cast<int>(row_bytes >> 4);
  long long total = (long long)n * vpr;
  gather_rows_kernel<<<ceil_div_ll(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, src_ld_bytes >> 4, (uint4*)dst, dst_ld_bytes >> 4, (const int*)idx, n, vpr, scatter);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// Copies nbytes from src (memory of the launching GPU) to dst (any memory the GPU can address, e.g. a peer's).
CS_API int cs_push_bytes(const void* src, void* dst, long long nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  const auto s = reinterpret_cast<unsigned long long>(src), d = reinterpret_cast<unsigned long long>(dst);
  if ((s & 15) || (d & 15)) {
    long long blocks = ceil_div_ll(nbytes, 256 * 16);
    if (blocks > 148 * 8) blocks = 148 * 8;
    push_bytes_unaligned_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const unsigned char*)src,
                                                                                  (unsigned char*)dst, nbytes);
    return cudaGetLastError() == cudaSuccess ? 0 : -10;
  }
  const long long n16 = nbytes >> 4;
  const int tail = static_cast<int>(nbytes & 15);
  long long blocks = ceil_div_ll(n16 > 0 ? n16 : 1, 256 * 4);
  if (blocks > 148 * 8) blocks = 148 * 8;
  push_bytes_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, (uint4*)dst, n16, (const unsigned char*)src + (n16 << 4), (unsigned char*)dst + (n16 << 4), tail);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// `scratch` must hold rows * 64 floats followed by rows * 64 ints (candidates of stage 1).
CS_API int cs_argmax(const void* logits, long long ld, int rows, int V, int is_fp32, void* out, void* scratch,
                     void* stream) {
  if (rows <= 0) return 0;
  int slices = (148 * 4 + rows - 1) / rows;
  if (slices > 64) slices = 64;
  if (slices < 1) slices = 1;
  float* cv = reinterpret_cast<float*>(scratch);
  int* ci = reinterpret_cast<int*>(cv + static_cast<long long>(rows) * 64);
  dim3 grid(rows, slices);
  if (is_fp32)
    argmax_stage1_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)logits, ld, V, slices, cv, ci);
  else
    argmax_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V,
                                                                                slices, cv, ci);
  argmax_stage2_kernel<<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(cv, ci, slices, rows, (int*)out);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_flow_step(void* x, const void* cond, const void* uncond, int rows, int C, float cfg, float dt,
                        int norm_rescale, void* stream) {
  if (rows <= 0) return 0;
  flow_step_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>((float*)x, (const __nv_bfloat16*)cond,
                                                           (const __nv_bfloat16*)uncond, C, cfg, dt, norm_rescale);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_pcm16(const void* x, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  pcm16_kernel<<<ceil_div_ll(n, 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (short*)y, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_l2_flush(void* buf, long long bytes, unsigned v, void* stream) {
  if (bytes < 16) return 0;
  l2_flush_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((uint4*)buf, bytes >> 4, v);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_decode_advance(const void* sampled, void* input_ids, void* positions, void* kv_len, void* slot,
                             const void* block_table, int bt_stride, const void* active, void* out_log, int log_cap,
                             void* step_counter, int B, int page, void* stream) {
  if (B <= 0) return 0;
  if (B > 1024) return -1;
  decode_advance_kernel<<<1, ((B + 31) / 32) * 32, 0, (cudaStream_t)stream>>>(
      (const int*)sampled, (int*)input_ids, (int*)positions, (int*)kv_len, (int*)slot, (const int*)block_table,
      bt_stride, (const int*)active, (int*)out_log, log_cap, (int*)step_counter, B, page);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
