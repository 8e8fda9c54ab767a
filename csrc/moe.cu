// Mixture-of-experts token movement for expert parallelism over peer memory (and for one GPU, where every "peer" is
// the GPU itself).  A layer is six launches that never return to the host:
//
//   route     softmax + top-k per token (one warp per token); per-expert counts; the last CTA stores this rank's
//             counts into every rank's table and bumps their counters
//   layout    one CTA: waits for all ranks' counts, lays every owner's experts out as row segments padded to the GEMM's
//             row tile, derives (a) where this rank's rows start inside each segment and (b) for the experts of this
//             rank the tile -> expert table that the grouped GEMM reads
//   dispatch  one warp per (token, choice): claims a slot in the expert's segment ON THE OWNER, stores the token row and
//             its return address {rank, token * k + choice} there; the last CTA bumps every rank's counter
//   wait      one thread: all ranks' rows have landed
//   (grouped GEMM gate|up + SwiGLU, grouped GEMM down whose epilogue stores each row at its return address: gemm.cu)
//   combine   waits for all owners, out[t] = sum_j w[t, j] * y[t * k + j] in a fixed order (deterministic); optionally
//             stores the row into every rank's output (tokens were split over ranks that all need the full result)
//
// Counters only grow: their targets are world * (epoch + 1) with the epoch kept on the device and advanced by the last
// CTA of `combine`, so a captured graph of a layer replays correctly.  Every wait is bounded (CS_ERR_TIMEOUT_PEER).
#include "common.cuh"

namespace {

constexpr int MOE_MAX_WORLD = 8;
constexpr int MOE_MAX_E = 256;   // experts in total (8 router values per lane)
constexpr int MOE_MAX_K = 16;

__device__ __forceinline__ bool moe_wait_ge(const unsigned* flag, unsigned target, int* err) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if ((spin & 0x3f) == 0x3f) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(err, CS_ERR_TIMEOUT_PEER); return false; }
    }
  }
}

__device__ __forceinline__ void moe_signal(unsigned* flag) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
}

struct PeerPtrs { void* p[MOE_MAX_WORLD]; };

// ---------------------------------------------------------------------------------------------------------------
// route
// ---------------------------------------------------------------------------------------------------------------
struct RouteParams {
  const float* logits; long long ldl;   // [T, E] fp32
  int T, E, k, norm;
  float* topk_w;                        // [T, k]
  int* topk_e;                          // [T, k]
  int* counts;                          // [E] zero on entry, zero again on exit
  unsigned* done;
  int world, rank;
  PeerPtrs counts_all;                  // per rank: int [world][E]
  PeerPtrs counts_flag;                 // per rank: unsigned
};

__global__ void __launch_bounds__(256) moe_route_kernel(const RouteParams p) {
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int per_lane = (p.E + 31) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < p.T; t += warps) {
    const float* row = p.logits + static_cast<long long>(t) * p.ldl;
    float v[MOE_MAX_E / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MOE_MAX_E / 32; ++i) {
      const int e = lane + 32 * i;
      v[i] = (i < per_lane && e < p.E) ? row[e] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MOE_MAX_E / 32; ++i) sum += __expf(v[i] - mx);   // exp(-inf) = 0 for absent entries
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    float my_w = 0.f, picked = 0.f;   // lane j keeps the j-th choice
    int my_e = 0;
    // the choice is made on the logits themselves (exact comparisons; ties go to the lower expert index)
    for (int j = 0; j < p.k; ++j) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MOE_MAX_E / 32; ++i)
        if (v[i] > best) { best = v[i]; best_e = lane + 32 * i; }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if (best_e >= p.E) best_e = p.E - 1;   // only with NaN / -inf logits: stay inside the tables
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < MOE_MAX_E / 32; ++i)
          if (i == (best_e >> 5)) v[i] = -INFINITY;
      }
      const float pj = __expf(best - mx) * inv;
      if (lane == j) { my_w = pj; my_e = best_e; }
      picked += pj;
    }
    if (lane < p.k) {
      p.topk_w[static_cast<long long>(t) * p.k + lane] = p.norm ? my_w / picked : my_w;
      p.topk_e[static_cast<long long>(t) * p.k + lane] = my_e;
      atomicAdd(&p.counts[my_e], 1);
    }
  }
  // ---- the last CTA publishes this rank's counts to every rank ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    is_last = atomicAdd(p.done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const int c = __ldcg(&p.counts[e]);
    p.counts[e] = 0;
    for (int o = 0; o < p.world; ++o)
      reinterpret_cast<int*>(p.counts_all.p[o])[p.rank * p.E + e] = c;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    *p.done = 0;
    __threadfence();
    for (int o = 0; o < p.world; ++o) moe_signal(reinterpret_cast<unsigned*>(p.counts_flag.p[o]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// layout
// ---------------------------------------------------------------------------------------------------------------
struct LayoutParams {
  const int* counts_all;        // this rank's table [world][E]
  const unsigned* counts_flag;
  const unsigned* epoch;
  int world, rank, E, tile_rows, cap_rows, max_tiles;
  int* base;                    // [E] slot on the owner where this rank's rows of expert e start
  int* cursor;                  // [E] zeroed here
  int* tile_expert;             // [max_tiles] local expert of each row tile of this rank
  int* tile_valid;              // [max_tiles]
  int* num_tiles;               // [1]
  int* overflow;                // [1] set when an owner's segments do not fit into cap_rows
  int* err;
};

__global__ void __launch_bounds__(256) moe_layout_kernel(const LayoutParams p) {
  __shared__ int tot[MOE_MAX_E], before[MOE_MAX_E], start[MOE_MAX_E];
  __shared__ int ok;
  if (threadIdx.x == 0) ok = moe_wait_ge(p.counts_flag, static_cast<unsigned>(p.world) * (*p.epoch + 1u), p.err) ? 1 : 0;
  __syncthreads();
  const int El = p.E / p.world;
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    int t = 0, b = 0;
    if (ok)
      for (int s = 0; s < p.world; ++s) {
        const int c = __ldcg(&p.counts_all[s * p.E + e]);
        if (s < p.rank) b += c;
        t += c;
      }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < p.world) {
    // one thread per owner: running start of its experts' padded segments
    const int o = threadIdx.x;
    int run = 0;
    for (int le = 0; le < El; ++le) {
      const int e = o * El + le;
      start[e] = run;
      run += (tot[e] + p.tile_rows - 1) / p.tile_rows * p.tile_rows;
    }
    if (run > p.cap_rows) { *p.overflow = 1; cs_set_error(p.err, CS_ERR_BAD_ARG); }
    if (o == p.rank) *p.num_tiles = run > p.cap_rows ? 0 : run / p.tile_rows;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    p.base[e] = start[e] + before[e];
    p.cursor[e] = 0;
    if (e / El == p.rank) {
      const int first = start[e] / p.tile_rows;
      const int n = (tot[e] + p.tile_rows - 1) / p.tile_rows;
      for (int i = 0; i < n && first + i < p.max_tiles; ++i) {
        p.tile_expert[first + i] = e - p.rank * El;
        p.tile_valid[first + i] = min(p.tile_rows, tot[e] - i * p.tile_rows);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------------------------------
struct DispatchParams {
  const __nv_bfloat16* x; long long ldx;   // [T, H] tokens of this rank
  int T, k, H, E, world, rank, cap_rows;
  const int* topk_e;
  const int* base;
  int* cursor;
  const int* overflow;
  PeerPtrs x_recv; long long ldr;          // per rank: bf16 [cap_rows, ldr]
  PeerPtrs row_meta;                       // per rank: int2 [cap_rows]
  PeerPtrs flag;                           // per rank: unsigned
  unsigned* done;
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const DispatchParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int El = p.E / p.world;
  const int nvec = p.H >> 3;
  const long long total = static_cast<long long>(p.T) * p.k;
  if (*p.overflow == 0) {
    for (long long a = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; a < total; a += warps) {
      const int e = p.topk_e[a];
      int slot = 0;
      if (lane == 0) slot = p.base[e] + atomicAdd(&p.cursor[e], 1);
      slot = __shfl_sync(0xffffffffu, slot, 0);
      if (slot >= p.cap_rows) continue;   // cannot happen once the layout fitted; keeps a bad table from writing outside
      const int owner = e / El;
      const uint4* src = reinterpret_cast<const uint4*>(p.x + (a / p.k) * p.ldx);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.x_recv.p[owner]) + static_cast<long long>(slot) * p.ldr);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      if (lane == 0) reinterpret_cast<int2*>(p.row_meta.p[owner])[slot] = make_int2(p.rank, static_cast<int>(a));
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
      *p.done = 0;
      __threadfence();
      for (int o = 0; o < p.world; ++o) moe_signal(reinterpret_cast<unsigned*>(p.flag.p[o]));
    }
  }
}

// One thread waits (bounded) until *flag >= world * (epoch + add).
__global__ void moe_wait_kernel(const unsigned* flag, const unsigned* epoch, unsigned world, unsigned add, int* err) {
  moe_wait_ge(flag, world * (*epoch + add), err);
}

// ---------------------------------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------------------------------
struct CombineParams {
  const __nv_bfloat16* y; long long ldy;   // [T * k, H] rows returned by the experts' owners
  const float* topk_w;
  int T, k, H, world;
  const unsigned* flag;                    // owners that have finished
  unsigned* epoch;
  unsigned* done;
  __nv_bfloat16* out; long long ldo;       // [T, H] local result (used when gather_world == 0)
  int gather_world; int row0;              // > 0: store row t at row0 + t of every rank's output, then signal them
  PeerPtrs out_all; PeerPtrs out_flag;
  int* err;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineParams p) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = moe_wait_ge(p.flag, static_cast<unsigned>(p.world) * (*p.epoch + 1u), p.err) ? 1 : 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = p.H >> 3;
  if (ok) {
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < p.T; t += warps) {
      float w[MOE_MAX_K];
#pragma unroll
      for (int j = 0; j < MOE_MAX_K; ++j) w[j] = j < p.k ? p.topk_w[static_cast<long long>(t) * p.k + j] : 0.f;
      for (int v = lane; v < nvec; v += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < MOE_MAX_K; ++j) {
          if (j < p.k) {
            const uint4 q = __ldcg(reinterpret_cast<const uint4*>(p.y + (static_cast<long long>(t) * p.k + j) * p.ldy) + v);
            acc[0] += w[j] * bf16lo(q.x); acc[1] += w[j] * bf16hi(q.x); acc[2] += w[j] * bf16lo(q.y); acc[3] += w[j] * bf16hi(q.y);
            acc[4] += w[j] * bf16lo(q.z); acc[5] += w[j] * bf16hi(q.z); acc[6] += w[j] * bf16lo(q.w); acc[7] += w[j] * bf16hi(q.w);
          }
        }
        uint4 r;
        r.x = pack_bf16x2(acc[0], acc[1]); r.y = pack_bf16x2(acc[2], acc[3]);
        r.z = pack_bf16x2(acc[4], acc[5]); r.w = pack_bf16x2(acc[6], acc[7]);
        if (p.gather_world > 0) {
          for (int o = 0; o < p.gather_world; ++o)
            reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out_all.p[o]) + static_cast<long long>(p.row0 + t) * p.ldo)[v] = r;
        } else {
          reinterpret_cast<uint4*>(p.out + static_cast<long long>(t) * p.ldo)[v] = r;
        }
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
      *p.done = 0;
      *p.epoch = *p.epoch + 1u;
      __threadfence();
      // signalled on every call (also without a gather) so that the counter stays at world * epoch
      for (int o = 0; o < p.world; ++o) moe_signal(reinterpret_cast<unsigned*>(p.out_flag.p[o]));
    }
  }
}

int grid_for_warps(long long warps_needed) {
  long long blocks = (warps_needed + 7) / 8;
  if (blocks < 1) blocks = 1;
  const long long cap = static_cast<long long>(cs_num_sms()) * 8;
  return static_cast<int>(blocks > cap ? cap : blocks);
}

void fill(PeerPtrs& dst, const void* const* src, int world) {
  for (int i = 0; i < MOE_MAX_WORLD; ++i) dst.p[i] = i < world ? const_cast<void*>(src[i]) : nullptr;
}
}  // namespace

CS_API int cs_moe_route(const void* logits, long long ldl, int T, int E, int k, int norm, void* topk_w, void* topk_e, void* counts,
                        void* done, int world, int rank, const void* const* counts_all, const void* const* counts_flag, void* stream) {
  if (T < 0 || E <= 0 || E > MOE_MAX_E || k <= 0 || k > MOE_MAX_K || k > E || world < 1 || world > MOE_MAX_WORLD || E % world) return -1;
  RouteParams p{};
  p.logits = (const float*)logits; p.ldl = ldl; p.T = T; p.E = E; p.k = k; p.norm = norm;
  p.topk_w = (float*)topk_w; p.topk_e = (int*)topk_e; p.counts = (int*)counts; p.done = (unsigned*)done;
  p.world = world; p.rank = rank;
  fill(p.counts_all, counts_all, world);
  fill(p.counts_flag, counts_flag, world);
  moe_route_kernel<<<grid_for_warps(T), 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_moe_layout(const void* counts_all, const void* counts_flag, const void* epoch, int world, int rank, int E, int tile_rows,
                         int cap_rows, int max_tiles, void* base, void* cursor, void* tile_expert, void* tile_valid, void* num_tiles,
                         void* overflow, void* stream) {
  if (E <= 0 || E > MOE_MAX_E || world < 1 || world > MOE_MAX_WORLD || E % world || tile_rows <= 0) return -1;
  LayoutParams p{};
  p.counts_all = (const int*)counts_all; p.counts_flag = (const unsigned*)counts_flag; p.epoch = (const unsigned*)epoch;
  p.world = world; p.rank = rank; p.E = E; p.tile_rows = tile_rows; p.cap_rows = cap_rows; p.max_tiles = max_tiles;
  p.base = (int*)base; p.cursor = (int*)cursor; p.tile_expert = (int*)tile_expert; p.tile_valid = (int*)tile_valid;
  p.num_tiles = (int*)num_tiles; p.overflow = (int*)overflow; p.err = cs_error_word();
  moe_layout_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_moe_dispatch(const void* x, long long ldx, int T, int k, int H, int E, int world, int rank, int cap_rows, const void* topk_e,
                           const void* base, void* cursor, const void* overflow, const void* const* x_recv, long long ldr,
                           const void* const* row_meta, const void* const* flag, void* done, void* stream) {
  if (T < 0 || (H & 7) || (ldx & 7) || (ldr & 7) || world < 1 || world > MOE_MAX_WORLD) return -1;
  DispatchParams p{};
  p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.T = T; p.k = k; p.H = H; p.E = E; p.world = world; p.rank = rank; p.cap_rows = cap_rows;
  p.topk_e = (const int*)topk_e; p.base = (const int*)base; p.cursor = (int*)cursor; p.overflow = (const int*)overflow;
  fill(p.x_recv, x_recv, world); p.ldr = ldr;
  fill(p.row_meta, row_meta, world);
  fill(p.flag, flag, world);
  p.done = (unsigned*)done;
  moe_dispatch_kernel<<<grid_for_warps(static_cast<long long>(T) * k), 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_moe_wait(const void* flag, const void* epoch, int world, int add, void* stream) {
  moe_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const unsigned*)flag, (const unsigned*)epoch, (unsigned)world, (unsigned)add,
                                                     cs_error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_moe_combine(const void* y, long long ldy, const void* topk_w, int T, int k, int H, int world, const void* flag, void* epoch,
                          void* done, void* out, long long ldo, int gather_world, int row0, const void* const* out_all,
                          const void* const* out_flag, void* stream) {
  if (T < 0 || (H & 7) || (ldy & 7) || (ldo & 7) || k <= 0 || k > MOE_MAX_K || gather_world < 0 || gather_world > MOE_MAX_WORLD || world < 1 ||
      world > MOE_MAX_WORLD || out_flag == nullptr)
    return -1;
  CombineParams p{};
  p.y = (const __nv_bfloat16*)y; p.ldy = ldy; p.topk_w = (const float*)topk_w; p.T = T; p.k = k; p.H = H; p.world = world;
  p.flag = (const unsigned*)flag; p.epoch = (unsigned*)epoch; p.done = (unsigned*)done;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.gather_world = gather_world; p.row0 = row0;
  if (gather_world > 0) fill(p.out_all, out_all, gather_world);
  fill(p.out_flag, out_flag, world);
  p.err = cs_error_word();
  moe_combine_kernel<<<grid_for_warps(T), 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
