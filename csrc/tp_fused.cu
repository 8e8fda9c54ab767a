// Row kernels of the tensor-parallel encoder path.  Together with cs_gemm_bf16_tp they replace
// "GEMM -> NCCL reduce-scatter / all-reduce -> add -> RMSNorm -> NCCL all-gather -> GEMM" by three kernels per
// half-block that meet only through counters in peer memory:
//
//   GEMM (epilogue pushes bf16 partial tiles to the owner of the rows)
//     -> tp_reduce_norm_push (this file; per owned row: wait for the partials of all ranks, sum them with bias and
//        residual, store the new residual stream, RMSNorm or LayerNorm, write the normalised row into EVERY rank's copy of
//        the next GEMM's operand and bump that rank's chunk counter)
//     -> GEMM (TMA producer waits per 128-row chunk of its operand)
//
// One warp per row (32 rows per CTA, one flag update per CTA and peer), 16-byte accesses, fp32 math.  Every wait is bounded and records CS_ERR_TIMEOUT_PEER.
#include "common.cuh"

namespace {

constexpr int TP_MAX_WORLD = 8;
constexpr int TP_MAXV = 16;  // 16-byte vectors per lane: H <= 32 * 8 * 16 = 4096

struct ReduceNormPushParams {
  int rows;                    // rows owned by this rank in this call
  int H;
  int world, rank;
  int rows_per_rank;           // ownership stride (multiple of 128)
  // partial sums: recv[slot][row][ldp], slot = source rank; null = no reduction (the input is `residual` itself)
  const __nv_bfloat16* recv; long long ldp;
  const unsigned* recv_flags;  // one counter per 128-row block of this rank's shard
  unsigned recv_target;        // value that means "every rank delivered every tile of the block"
  const __nv_bfloat16* bias;   // [H] or null
  const __nv_bfloat16* residual; long long ldr;  // [rows, ldr] local shard of the residual stream (or null)
  __nv_bfloat16* x_out; long long ldx;            // new residual stream [rows, ldx] (may alias residual; may be null)
  const __nv_bfloat16* norm_w; float eps;          // norm weight [H]; null = push the un-normalised sum
  const __nv_bfloat16* norm_b; int layer_norm;     // LayerNorm (mean removed, optional bias [H]) instead of RMSNorm
  __nv_bfloat16* gather[TP_MAX_WORLD]; long long ldg;  // every rank's copy of the next operand [total rows, ldg]
  unsigned* gather_flags[TP_MAX_WORLD];                // per rank: one counter per `gather_chunk` rows
  int gather_chunk;
  int* err;
};

__device__ __forceinline__ void unpack8t(const uint4& w, float (&f)[8]) {
  f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
  f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}
__device__ __forceinline__ uint4 pack8t(const float (&f)[8]) {
  uint4 w;
  w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]);
  w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
  return w;
}

constexpr int TP_ROWS_PER_CTA = 32;  // 8 warps x 4 rows; divides every flag chunk (multiples of 128 rows)

// NV = 16-byte vectors per lane (H <= 256 * NV).  Per row a warp first issues every load of a source (all NV vectors
// are independent, so they are all in flight together), accumulates in fp32, and only then stores: loads never wait
// behind the stores of the same row (x_out may alias residual), which is what bounded the first version of this kernel.
template <int NV>
__global__ void __launch_bounds__(256) tp_reduce_norm_push_kernel(const ReduceNormPushParams p) {
  __shared__ int wait_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r_first = blockIdx.x * TP_ROWS_PER_CTA;
  const int r_end = min(r_first + TP_ROWS_PER_CTA, p.rows);
  const int nvec = p.H >> 3;
  // ---- wait (once per CTA) until every rank has delivered this 128-row block ----
  if (p.recv != nullptr) {
    if (threadIdx.x == 0) {
      const unsigned* flag = p.recv_flags + (r_first >> 7);
      uint64_t t0 = 0;
      wait_ok = 1;
      for (uint32_t spin = 0;; ++spin) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= p.recv_target) break;
        if ((spin & 0x3f) == 0x3f) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          // on a timeout the rows are still written (with whatever arrived) so that no later wait starves
          if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(p.err, CS_ERR_TIMEOUT_PEER); wait_ok = 0; break; }
        }
      }
    }
    __syncthreads();
  }
  for (int r = r_first + warp; r < r_end; r += 8) {
    // ---- sum partials + bias + residual ----
    float acc[NV][8];
    uint4 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    }
    if (p.recv != nullptr) {
      for (int s = 0; s < p.world; ++s) {
        const __nv_bfloat16* src = p.recv + (static_cast<long long>(s) * p.rows_per_rank + r) * p.ldp;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int v = lane + 32 * i;
          if (v < nvec) raw[i] = __ldcg(reinterpret_cast<const uint4*>(src + v * 8));
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          if (lane + 32 * i < nvec) {
            float f[8];
            unpack8t(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] += f[j];
          }
        }
      }
    }
    if (p.residual != nullptr) {
      const __nv_bfloat16* src = p.residual + static_cast<long long>(r) * p.ldr;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) raw[i] = *reinterpret_cast<const uint4*>(src + v * 8);
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < nvec) {
          float f[8];
          unpack8t(raw[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] += f[j];
        }
      }
    }
    float ss = 0.f, sm = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        if (p.bias != nullptr) {
          float f[8];
          unpack8t(__ldg(reinterpret_cast<const uint4*>(p.bias + v * 8)), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] += f[j];
        }
        // the residual stream is kept in bf16: normalise what is stored
        const uint4 packed = pack8t(acc[i]);
        if (p.x_out != nullptr) *reinterpret_cast<uint4*>(p.x_out + static_cast<long long>(r) * p.ldx + v * 8) = packed;
        unpack8t(packed, acc[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { ss += acc[i][j] * acc[i][j]; sm += acc[i][j]; }
      }
    }
    if (p.gather[0] == nullptr) continue;
    float rstd = 1.f, mean = 0.f;
    if (p.norm_w != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        sm += __shfl_xor_sync(0xffffffffu, sm, o);
      }
      const float inv_h = 1.f / static_cast<float>(p.H);
      if (p.layer_norm) {
        mean = sm * inv_h;
        rstd = rsqrtf(fmaxf(ss * inv_h - mean * mean, 0.f) + p.eps);
      } else {
        rstd = rsqrtf(ss * inv_h + p.eps);
      }
    }
    // ---- normalise and write the row into every rank's operand buffer ----
    const long long g = static_cast<long long>(p.rank) * p.rows_per_rank + r;  // row in the gathered operand
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float y[8];
        if (p.norm_w != nullptr) {
          float w[8];
          unpack8t(__ldg(reinterpret_cast<const uint4*>(p.norm_w + v * 8)), w);
#pragma unroll
          for (int j = 0; j < 8; ++j) y[j] = (acc[i][j] - mean) * rstd * w[j];
          if (p.norm_b != nullptr) {
            float b[8];
            unpack8t(__ldg(reinterpret_cast<const uint4*>(p.norm_b + v * 8)), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] += b[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) y[j] = acc[i][j];
        }
        const uint4 packed = pack8t(y);
        for (int peer = 0; peer < p.world; ++peer)
          *reinterpret_cast<uint4*>(p.gather[peer] + g * p.ldg + v * 8) = packed;
      }
    }
  }
  if (p.gather[0] == nullptr) return;
  // ---- one release per CTA and peer: the CTA's rows all lie in one flag chunk ----
  __syncthreads();
  if (threadIdx.x < p.world && r_end > r_first) {
    const long long g0 = static_cast<long long>(p.rank) * p.rows_per_rank + r_first;
    unsigned* flag = p.gather_flags[threadIdx.x] + g0 / p.gather_chunk;
    const unsigned n = static_cast<unsigned>(r_end - r_first);
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(n) : "memory");
  }
}

}  // namespace

// See the top of this file.  `rows` = rows this rank owns in this call (<= rows_per_rank); `recv` may be null (then
// the kernel only normalises `residual` and pushes it: the entry of the chain).  `gather_ptrs` may be null (then the
// kernel only reduces into `x_out`: the exit of the chain).
CS_API int cs_tp_reduce_norm_push(int rows, int H, int world, int rank, int rows_per_rank, const void* recv, long long ldp,
                                  const void* recv_flags, unsigned recv_target, const void* bias, const void* residual,
                                  long long ldr, void* x_out, long long ldx, const void* norm_w, float eps,
                                  const void* norm_b, int layer_norm, const void* const* gather_ptrs, const void* const* gather_flag_ptrs, long long ldg,
                                  int gather_chunk, void* stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > 32 * 8 * TP_MAXV || world < 1 || world > TP_MAX_WORLD || (ldp & 7) || (ldr & 7) || (ldx & 7) || (ldg & 7))
    return -1;
  ReduceNormPushParams p{};
  p.rows = rows; p.H = H; p.world = world; p.rank = rank; p.rows_per_rank = rows_per_rank;
  p.recv = (const __nv_bfloat16*)recv; p.ldp = ldp;
  p.recv_flags = (const unsigned*)recv_flags; p.recv_target = recv_target;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual; p.ldr = ldr;
  p.x_out = (__nv_bfloat16*)x_out; p.ldx = ldx;
  p.norm_w = (const __nv_bfloat16*)norm_w; p.eps = eps;
  p.norm_b = (const __nv_bfloat16*)norm_b; p.layer_norm = layer_norm;
  p.ldg = ldg; p.gather_chunk = gather_chunk > 0 ? gather_chunk : 128;
  for (int i = 0; i < world; ++i) {
    p.gather[i] = gather_ptrs ? (__nv_bfloat16*)const_cast<void*>(gather_ptrs[i]) : nullptr;
    p.gather_flags[i] = gather_flag_ptrs ? (unsigned*)const_cast<void*>(gather_flag_ptrs[i]) : nullptr;
  }
  p.err = cs_error_word();
  if (p.gather_chunk % TP_ROWS_PER_CTA != 0 || rows_per_rank % TP_ROWS_PER_CTA != 0) return -1;
  const unsigned grid = (rows + TP_ROWS_PER_CTA - 1) / TP_ROWS_PER_CTA;
  if (H <= 256 * 8) tp_reduce_norm_push_kernel<8><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else tp_reduce_norm_push_kernel<16><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}


// ---------------------------------------------------------------------------------------------------------
// Ulysses, the way back: after attention every rank holds ALL tokens for ITS heads, `src` = [world * rows, cols]
// in the order ((b, source rank, row in segment)); token rows return to the rank they came from, landing in
// columns [rank*cols, (rank+1)*cols) of that rank's [rows, world*cols] operand of the output projection.
// The CTA that finishes last publishes the whole transfer with one release per destination (`flags[o][0] += 1`).
// `done` is a local counter that must be zero before the call (the kernel leaves it at zero).
// ---------------------------------------------------------------------------------------------------------
namespace {
struct A2APushParams {
  const __nv_bfloat16* src; long long lds;
  int rows_total, vec_per_row, world, rank, seg;
  __nv_bfloat16* dst[TP_MAX_WORLD]; long long ldd;
  unsigned* flags[TP_MAX_WORLD];
  unsigned* done;
};

__global__ void __launch_bounds__(256) a2a_push_heads_kernel(const A2APushParams p) {
  const long long total = static_cast<long long>(p.rows_total) * p.vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % p.vec_per_row);
    const long long r = i / p.vec_per_row;
    const int in_seg = static_cast<int>(r % p.seg);
    const int owner = static_cast<int>((r / p.seg) % p.world);
    const long long b = r / (static_cast<long long>(p.seg) * p.world);
    const long long drow = b * p.seg + in_seg;
    const uint4 w = *reinterpret_cast<const uint4*>(p.src + r * p.lds + v * 8);
    *reinterpret_cast<uint4*>(p.dst[owner] + drow * p.ldd + static_cast<long long>(p.rank) * p.vec_per_row * 8 + v * 8) = w;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(p.done, 1u);
    if (prev == gridDim.x - 1) {
      *p.done = 0;
      __threadfence();
      for (int o = 0; o < p.world; ++o)
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.flags[o]) : "memory");
    }
  }
}

// One thread waits (bounded) until *flag >= target: orders later kernels of the stream after the peers' pushes.
__global__ void wait_flag_kernel(const unsigned* flag, unsigned target, int* err) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - target) >= 0) return;   // the counters are cumulative and may wrap: compare the difference
    if ((spin & 0x3f) == 0x3f) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(err, CS_ERR_TIMEOUT_PEER); return; }
    }
  }
}
}  // namespace

CS_API int cs_a2a_push_heads(const void* src, long long lds, int rows_total, int cols, int world, int rank, int seg,
                             const void* const* dst_ptrs, long long ldd, const void* const* flag_ptrs, void* done,
                             void* stream) {
  if (rows_total <= 0) return 0;
  if ((cols & 7) || (lds & 7) || (ldd & 7) || world < 1 || world > TP_MAX_WORLD || seg <= 0 || rows_total % (seg * world)) return -1;
  A2APushParams p{};
  p.src = (const __nv_bfloat16*)src; p.lds = lds;
  p.rows_total = rows_total; p.vec_per_row = cols >> 3; p.world = world; p.rank = rank; p.seg = seg;
  p.ldd = ldd;
  for (int i = 0; i < world; ++i) {
    p.dst[i] = (__nv_bfloat16*)const_cast<void*>(dst_ptrs[i]);
    p.flags[i] = (unsigned*)const_cast<void*>(flag_ptrs[i]);
  }
  p.done = (unsigned*)done;
  const long long total = static_cast<long long>(rows_total) * p.vec_per_row;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  a2a_push_heads_kernel<<<static_cast<unsigned>(blocks), 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_wait_flag(const void* flag, unsigned target, void* stream) {
  wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const unsigned*)flag, target, cs_error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
