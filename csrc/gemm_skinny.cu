// Weight-streaming bf16 GEMM for small M (decode):  C[M,N] = epilogue(X[M,K] * W[N,K]^T),  M <= 256.
//
// The operands are swapped relative to gemm.cu: 128 rows of W form the M side of the tcgen05.mma tile
// and the (padded) token rows of X form the N side, so one CTA streams a 128-row slab of W exactly
// once and the tensor core is fed full-width tiles however few tokens there are.  K is split across
// CTAs (split-K) so that every SM streams weights; partial sums go to an fp32 workspace and the last
// CTA to finish a tile reduces them and applies the epilogue (bias, activation, residual, SwiGLU).
//
//   warp 0 (one lane)  TMA producer: ring of stages, each = 2 swizzle atoms (128 K columns) of W and X
//   warp 1 (one lane)  tcgen05.mma issuer, accumulator [128 W rows x M_pad tokens] fp32 in TMEM
//   warps 2..5         epilogue: thread r owns W row r of the tile = output column n0 + r, so for a
//                      fixed token the 32 lanes of a warp write 32 consecutive output columns
//
// Scratch: `ws` holds splits x tiles x M_pad x 128 fp32 partials, `counters` one int per tile (zero before the
// first call; the CTA that leaves a tile last resets its counter, so back-to-back calls on one stream can share
// them).  When the whole grid is resident (tiles x splits <= SMs) the splits of a tile wait for one another and each
// reduces and finishes a share of the tile's 16-token chunks; otherwise the split that arrives last does all of it.
#include "common.cuh"

namespace {

constexpr int BK = 64;
constexpr int KATOMS = 2;          // swizzle atoms per stage
constexpr int W_ATOM = 128 * 128;  // 128 rows x 128 bytes
constexpr int MAX_STAGES = 8;

enum Act : int { ACT_NONE = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_QUICK_GELU = 4, ACT_RELU = 5 };

// The activation is selected once per 16 values (uniform branch), then applied in a straight loop.
__device__ __forceinline__ void act16(float (&f)[16], int act) {
  switch (act) {
    case ACT_GELU_ERF:
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = 0.5f * f[i] * (1.0f + erff(f[i] * 0.70710678118654752f));
      break;
    case ACT_GELU_TANH:
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float u = 0.7978845608028654f * (f[i] + 0.044715f * f[i] * f[i] * f[i]);
        f[i] = 0.5f * f[i] * (2.0f - 2.0f / (__expf(2.0f * u) + 1.0f));
      }
      break;
    case ACT_SILU:
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __fdividef(f[i], 1.0f + __expf(-f[i]));
      break;
    case ACT_QUICK_GELU:
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __fdividef(f[i], 1.0f + __expf(-1.702f * f[i]));
      break;
    case ACT_RELU:
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = fmaxf(f[i], 0.0f);
      break;
    default:
      break;
  }
}

// One-shot all-reduce fused into the epilogue (tensor-parallel row-parallel projections at decode time).
// Every rank pushes its bf16 partial tile into slot [rank] of every peer's receive buffer, bumps the
// peer's per-tile arrival counter, waits until its own counter shows all `world` partials, sums them with
// the residual, and the CTA that finishes last applies RMSNorm to the rows.  Buffers alternate between two
// halves by call parity (a rank can never run two calls ahead of a peer), counters only ever grow, and the
// call number lives in device memory so that a CUDA graph can replay the kernel.
constexpr int AR_MAX_WORLD = 8;
constexpr int AR_STG_PITCH = 128 + 8;  // bf16 elements per staged row (16 bytes of padding against bank conflicts)
struct AllReduceParams {
  int world, rank;
  __nv_bfloat16* recv[AR_MAX_WORLD];  // per peer: [2][world][m_cap][n_cap]
  unsigned* flags[AR_MAX_WORLD];      // per peer: [2][tiles_cap]
  int m_cap, n_cap, tiles_cap;
  float* ssq;                         // local [m_cap] row sums of squares (zero between calls)
  int* done;                          // local int[2]: tiles reduced / tiles normalised (zero between calls)
  unsigned* epoch;                    // local call counter
  const __nv_bfloat16* norm_w;        // RMSNorm weight [N] or null (then no norm output)
  __nv_bfloat16* normed; long long ldn;
  float eps;
};

struct SkinnyParams {
  int M, N, K;          // N = output columns
  int m_pad;            // tokens padded to a multiple of 16
  int splits, stages;
  int swiglu;           // tile = 64 gate rows + 64 up rows, 64 output columns per tile
  int up_row_offset;    // row of W where the "up" half starts
  void* C; long long ldc; int out_fp32;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; long long ldr;
  int act;
  float* ws; int* counters;
  int par_reduce;       // every split CTA of a tile reduces a share of the tile's token chunks (all CTAs resident)
  int w_dynamic;        // W may have been written by the kernel before this one: no weight prefetch ahead of it
  uint32_t idesc;
  uint32_t tmem_cols;
  int* err;
  AllReduceParams ar;
};

__global__ void __launch_bounds__(192, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, is_last;
  __shared__ float xchg[64 * 17];  // SwiGLU: up values of 64 columns x 16 tokens

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int cols_per_tile = p.swiglu ? 64 : 128;
  const int n0 = tile * cols_per_tile;
  const int x_atom = p.m_pad * 128;
  const int stage_bytes = KATOMS * (W_ATOM + x_atom);
  const int total_it = (p.K + BK * KATOMS - 1) / (BK * KATOMS);
  const int it_lo = static_cast<int>((static_cast<long long>(split) * total_it) / p.splits);
  const int it_hi = static_cast<int>((static_cast<long long>(split + 1) * total_it) / p.splits);
  const int n_it = it_hi - it_lo;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    is_last = 0;
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    pdl_launch_dependents();   // the next kernel of the stream may set itself up while this one runs
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, p.tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t tx = static_cast<uint32_t>(stage_bytes);
      auto load_w = [&](int it, int stage) {
        uint8_t* sW = smem + stage * stage_bytes;
        const int k0 = (it_lo + it) * BK * KATOMS;
#pragma unroll
        for (int a = 0; a < KATOMS; ++a) {
          if (p.swiglu) {
            tma_load_2d(sW + a * W_ATOM, &tmW, k0 + a * BK, n0, &full_bar[stage]);
            tma_load_2d(sW + a * W_ATOM + W_ATOM / 2, &tmW, k0 + a * BK, p.up_row_offset + n0, &full_bar[stage]);
          } else {
            tma_load_2d(sW + a * W_ATOM, &tmW, k0 + a * BK, n0, &full_bar[stage]);
          }
        }
      };
      auto load_x = [&](int it, int stage) {
        uint8_t* sX = smem + stage * stage_bytes + KATOMS * W_ATOM;
        const int k0 = (it_lo + it) * BK * KATOMS;
#pragma unroll
        for (int a = 0; a < KATOMS; ++a) tma_load_2d(sX + a * x_atom, &tmX, k0 + a * BK, 0, &full_bar[stage]);
      };
      // The weights do not depend on the kernel before this one: fill the ring with them first, then wait for that
      // kernel (a no-op unless this launch may overlap it) and fetch the activations.
      const int pre = min(n_it, p.stages);
      if (p.w_dynamic) pdl_wait();   // W is an activation here (scores against keys, say), not a stored weight
      for (int it = 0; it < pre; ++it) {
        mbar_arrive_expect_tx(&full_bar[it], tx);
        load_w(it, it);
      }
      pdl_wait();
      for (int it = 0; it < pre; ++it) load_x(it, it);
      int stage = pre == p.stages ? 0 : pre;
      uint32_t phase = pre == p.stages ? 1 : 0;
      for (int it = pre; it < n_it; ++it) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) break;
        mbar_arrive_expect_tx(&full_bar[stage], tx);
        load_w(it, stage);
        load_x(it, stage);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait(&full_bar[stage], phase, abortp, p.err, CS_ERR_TIMEOUT_TMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t w_addr = smem_u32(smem + stage * stage_bytes);
        const uint32_t x_addr = w_addr + KATOMS * W_ATOM;
#pragma unroll
        for (int a = 0; a < KATOMS; ++a) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16_ss(tmem, umma_smem_desc(w_addr + a * W_ATOM + k * 32, 16, 1024),
                        umma_smem_desc(x_addr + a * x_atom + k * 32, 16, 1024), p.idesc,
                        (it | a | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(&acc_full);
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;  // W row of the tile
    const uint32_t t_row = tmem + (static_cast<uint32_t>(q * 32) << 16);
    bool ok = true;
    pdl_wait();   // before the first access to memory that an earlier kernel wrote or still reads
    if (n_it > 0) ok = mbar_wait(&acc_full, 0, abortp, p.err, CS_ERR_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int chunks = p.m_pad / 16;
    const unsigned ar_epoch = p.ar.world > 1 ? *reinterpret_cast<volatile unsigned*>(p.ar.epoch) : 0u;
    const unsigned ar_parity = ar_epoch & 1u;
    const int num_tiles_total = gridDim.x / p.splits;
    // For the fused SwiGLU tile rows 0..63 are gate columns and rows 64..127 the matching up columns.
    const int w_row = p.swiglu ? (r < 64 ? n0 + r : p.up_row_offset + n0 + (r - 64)) : n0 + r;
    const bool row_valid = p.swiglu ? (n0 + (r & 63) < p.N) : (n0 + r < p.N);
    if (p.splits > 1) {
      // 1) publish this split's partial sums
      // layout [split][tile][token][tile row]: the 32 lanes of a warp store (and later load) 128 contiguous bytes
      float* wst = p.ws + (static_cast<long long>(split) * num_tiles_total + tile) * 128 * p.m_pad + r;
      for (int c = 0; c < chunks; ++c) {
        uint32_t v[16];
        if (ok && n_it > 0) { tmem_ld16(t_row + c * 16, v); tmem_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) __stcg(wst + (c * 16 + i) * 128, __uint_as_float(v[i]));
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        if (p.par_reduce) {
          // arrivals count in the low half of the tile's word, departures in the high half; wait (bounded) until
          // every split of this tile has published: all CTAs of the grid are resident (checked by the host)
          atomicAdd(&p.counters[tile], 1);
          uint64_t t0 = 0;
          for (uint32_t spin = 0;; ++spin) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.counters + tile) : "memory");
            if ((v & 0xffff) >= p.splits) break;
            if ((spin & 0xff) == 0xff) {
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(p.err, CS_ERR_TIMEOUT_EPI); ok = false; is_last = -1; break; }
            }
          }
        } else {
          const int prev = atomicAdd(&p.counters[tile], 1);
          if (prev == p.splits - 1) { p.counters[tile] = 0; is_last = 1; }
        }
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const int last_word = *reinterpret_cast<volatile int*>(&is_last);
    const bool reducer = (p.splits == 1) || (p.par_reduce ? last_word == 0 : last_word != 0);
    // token chunks this CTA finishes: all of them, or every splits-th one when the splits share the reduction
    const int c_first = (p.splits > 1 && p.par_reduce) ? split : 0;
    const int c_step = (p.splits > 1 && p.par_reduce) ? p.splits : 1;
    if (reducer) {
      const float bias = (p.bias != nullptr && row_valid) ? __bfloat162float(p.bias[p.swiglu ? (r < 64 ? n0 + r : p.N + n0 + r - 64) : n0 + r]) : 0.f;
      (void)w_row;
      for (int c = c_first; c < chunks; c += c_step) {
        float f[16];
        if (p.splits == 1) {
          uint32_t v[16];
          if (ok && n_it > 0) { tmem_ld16(t_row + c * 16, v); tmem_wait_ld(); }
          else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = 0.f;
          // four splits' worth of loads are in flight before the first sum (one L2 round trip per group)
          const long long split_stride = static_cast<long long>(num_tiles_total) * 128 * p.m_pad;
          const float* src0 = p.ws + static_cast<long long>(tile) * 128 * p.m_pad + (c * 16) * 128 + r;
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float t[4][16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float* src = src0 + min(s0 + j, p.splits - 1) * split_stride;
#pragma unroll
              for (int i = 0; i < 16; ++i) t[j][i] = __ldcg(src + i * 128);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (s0 + j < p.splits) {
#pragma unroll
                for (int i = 0; i < 16; ++i) f[i] += t[j][i];
              }
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] += bias;
        if (p.swiglu) {
          // hand the up values (rows 64..127) to the threads that hold the matching gate columns
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (r >= 64) {
#pragma unroll
            for (int i = 0; i < 16; ++i) xchg[(r - 64) * 17 + i] = f[i];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (r < 64) {
            act16(f, p.act);
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] *= xchg[r * 17 + i];
          }
        } else {
          act16(f, p.act);
        }
        const bool writer = row_valid && (!p.swiglu || r < 64);
        if (p.ar.world > 1) {
          // stage this rank's partial (bias already applied on rank 0 only by the caller) row-major in shared memory
          // (the operand ring is free: every MMA of this CTA has completed); it leaves as 16-byte row pieces below
          if (writer) {
            const int mmax = min(16, p.M - c * 16);
            __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(smem) + static_cast<long long>(c * 16) * AR_STG_PITCH + r;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (i < mmax) st[i * AR_STG_PITCH] = __float2bfloat16(f[i]);
          }
          continue;
        }
        if (writer) {
          const int n = n0 + r;
          const int mmax = min(16, p.M - c * 16);
          if (p.residual != nullptr) {
            const __nv_bfloat16* rp = p.residual + static_cast<long long>(c * 16) * p.ldr + n;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (i < mmax) f[i] += __bfloat162float(rp[static_cast<long long>(i) * p.ldr]);
          }
          if (p.out_fp32) {
            float* op = reinterpret_cast<float*>(p.C) + static_cast<long long>(c * 16) * p.ldc + n;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (i < mmax) op[static_cast<long long>(i) * p.ldc] = f[i];
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(c * 16) * p.ldc + n;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (i < mmax) op[static_cast<long long>(i) * p.ldc] = __float2bfloat16(f[i]);
          }
        }
      }
      if (p.splits > 1 && p.par_reduce) {
        // departures count in the high half of the tile's word; the last one re-arms it for the next call
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&p.counters[tile], 0x10000);
          if ((prev >> 16) == p.splits - 1) p.counters[tile] = 0;
        }
      }
      if (p.ar.world > 1) {
        // Work item u = (row, 8-column group) of the M x 128 tile: 16 consecutive lanes cover one row, so every
        // global access below is a 16-byte piece of a 256-byte row segment.
        const int units = p.M * 16;
        const unsigned slot_base = ar_parity * static_cast<unsigned>(p.ar.world);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // ---- push this rank's partial tile into slot [rank] of every peer ----
        for (int base = 0; base < units; base += 128) {
          const int u = base + r, row = u >> 4, col = n0 + (u & 15) * 8;
          if (u < units && col < p.N) {
            const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(smem) +
                                                            static_cast<long long>(row) * AR_STG_PITCH + (u & 15) * 8);
            const long long off = (static_cast<long long>(slot_base + p.ar.rank) * p.ar.m_cap + row) * p.ar.n_cap + col;
            for (int peer = 0; peer < p.ar.world; ++peer) *reinterpret_cast<uint4*>(p.ar.recv[peer] + off) = v;
          }
        }
        // ---- signal: all stores of this CTA are visible system-wide before the counters move ----
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r < p.ar.world) {
          unsigned* flag = p.ar.flags[r] + static_cast<long long>(ar_parity) * p.ar.tiles_cap + tile;
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
        }
        // ---- wait for the partials of all ranks for this tile ----
        const unsigned target = (ar_epoch / 2 + 1) * static_cast<unsigned>(p.ar.world);
        const unsigned* mine = p.ar.flags[p.ar.rank] + static_cast<long long>(ar_parity) * p.ar.tiles_cap + tile;
        if (r == 0) {
          uint64_t t0 = 0;
          for (uint32_t spin = 0;; ++spin) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v >= target) break;
            if ((spin & 0xff) == 0xff) {
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(p.err, CS_ERR_TIMEOUT_PEER); break; }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // ---- reduce: sum the world partials (+ residual), keep the new residual, gather row norms ----
        for (int base = 0; base < units; base += 128) {
          const int u = base + r, row = u >> 4, col = n0 + (u & 15) * 8;
          const bool live = u < units && col < p.N;
          float sq = 0.f;
          if (live) {
            float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int src = 0; src < p.ar.world; ++src) {
              const uint4 q4 = __ldcg(reinterpret_cast<const uint4*>(
                  p.ar.recv[p.ar.rank] + (static_cast<long long>(slot_base + src) * p.ar.m_cap + row) * p.ar.n_cap + col));
              h[0] += bf16lo(q4.x); h[1] += bf16hi(q4.x); h[2] += bf16lo(q4.y); h[3] += bf16hi(q4.y);
              h[4] += bf16lo(q4.z); h[5] += bf16hi(q4.z); h[6] += bf16lo(q4.w); h[7] += bf16hi(q4.w);
            }
            if (p.residual != nullptr) {
              const uint4 q4 = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(row) * p.ldr + col);
              h[0] += bf16lo(q4.x); h[1] += bf16hi(q4.x); h[2] += bf16lo(q4.y); h[3] += bf16hi(q4.y);
              h[4] += bf16lo(q4.z); h[5] += bf16hi(q4.z); h[6] += bf16lo(q4.w); h[7] += bf16hi(q4.w);
            }
            uint4 o;
            o.x = pack_bf16x2(h[0], h[1]); o.y = pack_bf16x2(h[2], h[3]); o.z = pack_bf16x2(h[4], h[5]); o.w = pack_bf16x2(h[6], h[7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col) = o;
            // the norm sees the stored (rounded) values
            const float g0 = bf16lo(o.x), g1 = bf16hi(o.x), g2 = bf16lo(o.y), g3 = bf16hi(o.y);
            const float g4 = bf16lo(o.z), g5 = bf16hi(o.z), g6 = bf16lo(o.w), g7 = bf16hi(o.w);
            sq = g0 * g0 + g1 * g1 + g2 * g2 + g3 * g3 + g4 * g4 + g5 * g5 + g6 * g6 + g7 * g7;
          }
          if (p.ar.norm_w != nullptr) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);  // the 16 lanes of a row
            if ((lane & 15) == 0 && u < units) atomicAdd(&p.ar.ssq[row], sq);
          }
        }
        // ---- once every tile of this rank is reduced, each tile CTA normalises its own 128 columns ----
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r == 0) {
          atomicAdd(&p.ar.done[0], 1);
          if (p.ar.norm_w != nullptr) {
            // all tile CTAs of the grid are resident (checked by the host), so this wait cannot starve
            uint64_t t0 = 0;
            for (uint32_t spin = 0;; ++spin) {
              if (*reinterpret_cast<volatile int*>(&p.ar.done[0]) >= num_tiles_total) break;
              if ((spin & 0xff) == 0xff) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > CS_WAIT_LIMIT_NS) { cs_set_error(p.err, CS_ERR_TIMEOUT_EPI); break; }
              }
            }
            __threadfence();
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (p.ar.norm_w != nullptr) {
          const float inv_n = 1.0f / static_cast<float>(p.N);
          for (int base = 0; base < units; base += 128) {
            const int u = base + r, row = u >> 4, col = n0 + (u & 15) * 8;
            if (u < units && col < p.N) {
              const uint4 hq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.C) +
                                                               static_cast<long long>(row) * p.ldc + col);
              const uint4 wq = *reinterpret_cast<const uint4*>(p.ar.norm_w + col);
              const float s = rsqrtf(__ldcg(&p.ar.ssq[row]) * inv_n + p.ar.eps);
              uint4 o;
              o.x = pack_bf16x2(bf16lo(hq.x) * s * bf16lo(wq.x), bf16hi(hq.x) * s * bf16hi(wq.x));
              o.y = pack_bf16x2(bf16lo(hq.y) * s * bf16lo(wq.y), bf16hi(hq.y) * s * bf16hi(wq.y));
              o.z = pack_bf16x2(bf16lo(hq.z) * s * bf16lo(wq.z), bf16hi(hq.z) * s * bf16hi(wq.z));
              o.w = pack_bf16x2(bf16lo(hq.w) * s * bf16lo(wq.w), bf16hi(hq.w) * s * bf16hi(wq.w));
              *reinterpret_cast<uint4*>(p.ar.normed + static_cast<long long>(row) * p.ar.ldn + col) = o;
            }
          }
        }
        // ---- the CTA that leaves last re-arms the scratch for the next call ----
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r == 0) {
          const int prev = atomicAdd(&p.ar.done[1], 1);
          is_last = (prev == num_tiles_total - 1) ? 2 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*reinterpret_cast<volatile int*>(&is_last) == 2) {
          for (int m = r; m < p.ar.m_cap; m += 128) p.ar.ssq[m] = 0.f;
          if (r == 0) { p.ar.done[0] = 0; p.ar.done[1] = 0; *p.ar.epoch = ar_epoch + 1; }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, p.tmem_cols); }
}

}  // namespace

// Workspace sizes for cs_gemm_skinny: bytes of fp32 partials and number of int counters.
CS_API long long cs_gemm_skinny_ws_bytes(int M, int N, int splits, int swiglu) {
  const long long m_pad = (M + 15) & ~15;
  const long long tiles = (N + (swiglu ? 64 : 128) - 1) / (swiglu ? 64 : 128);
  return splits > 1 ? static_cast<long long>(splits) * tiles * 128 * m_pad * 4 : 0;
}

// Picks the split count used when `splits` is passed as 0.
CS_API int cs_gemm_skinny_auto_splits(int N, int K, int swiglu) {
  const int tiles = (N + (swiglu ? 64 : 128) - 1) / (swiglu ? 64 : 128);
  const int sms = cs_num_sms();
  const int total_it = (K + BK * KATOMS - 1) / (BK * KATOMS);
  int splits = 1;
  if (tiles < sms) {
    splits = sms / tiles;
    if (splits > total_it) splits = total_it;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  return splits;
}

// C[M,N] = act(X W^T + bias) + residual   (swiglu == 0),  W: [N,K]
// C[M,N] = act(X Wg^T + bg) * (X Wu^T + bu), W = [Wg; Wu] ([2N,K])   (swiglu == 1)
// M <= 256.  `ws` / `counters` as described at the top of this file (`counters` needs one int per tile).
// `out_fp32`: bit 0 = fp32 output; bit 1 = W is not a stored weight but may have been written by the kernel that
// precedes this call on the stream (the kernel then fetches nothing before that kernel has completed).
CS_API int cs_gemm_skinny(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc,
                          const void* bias, const void* residual, long long ldr, int M, int N, int K, int act,
                          int swiglu, int out_fp32, int splits, void* ws, long long ws_bytes, void* counters,
                          int num_counters, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 256 || K <= 0 || (ldx & 7) || (ldw & 7)) return -1;
  SkinnyParams p{};
  p.M = M; p.N = N; p.K = K;
  p.m_pad = (M + 15) & ~15;
  p.swiglu = swiglu;
  p.up_row_offset = N;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32 & 1;
  p.w_dynamic = (out_fp32 >> 1) & 1;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = act;
  p.err = cs_error_word();
  const int cols_per_tile = swiglu ? 64 : 128;
  const int tiles = (N + cols_per_tile - 1) / cols_per_tile;
  if (splits <= 0) splits = cs_gemm_skinny_auto_splits(N, K, swiglu);
  const int total_it = (K + BK * KATOMS - 1) / (BK * KATOMS);
  if (splits > total_it) splits = total_it;
  if (splits > 1) {
    if (ws == nullptr || counters == nullptr || tiles > num_counters ||
        cs_gemm_skinny_ws_bytes(M, N, splits, swiglu) > ws_bytes)
      return -5;
  }
  p.splits = splits;
  p.par_reduce = (splits > 1 && tiles * splits <= cs_num_sms()) ? 1 : 0;
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = reinterpret_cast<int*>(counters);
  const int stage_bytes = KATOMS * (W_ATOM + p.m_pad * 128);
  int stages = MAX_STAGES;
  const int max_smem = 220 * 1024;
  while (stages > 2 && stages * stage_bytes + 1024 > max_smem) --stages;
  p.stages = stages;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(p.m_pad)) cols <<= 1;
  p.tmem_cols = cols;
  p.idesc = umma_idesc_bf16(128, p.m_pad, 0, 0);

  CUtensorMap tmW, tmX;
  const int w_rows = swiglu ? 2 * N : N;
  if (cs_encode_tmap_2d(&tmW, W, K, w_rows, ldw * 2, BK, swiglu ? 64 : 128, 2, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmX, X, K, M, ldx * 2, BK, p.m_pad, 2, 1) != 0) return -3;
  const int smem = stages * stage_bytes + 1024;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    attr_done[dev] = true;
  }
  // may start (set-up, weight prefetch) while the previous kernel of the stream is still running
  if (cs_launch_pdl(gemm_skinny_kernel, dim3(tiles * splits), dim3(192), smem, stream, tmW, tmX, p) != cudaSuccess) return -10;
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// Fused row-parallel projection + one-shot all-reduce + residual + RMSNorm over NVLink peer memory:
//   h      = sum_over_ranks(X_r W_r^T (+ bias on rank 0)) + residual       -> `H`      [M,N] bf16
//   normed = RMSNorm(h) * norm_w                                           -> `normed` [M,N] bf16 (if norm_w)
// `recv_ptrs[p]` / `flag_ptrs[p]` are rank p's symmetric receive buffer ([2][world][m_cap][n_cap] bf16) and
// arrival counters ([2][tiles_cap] u32, zero at start, never reset); `ssq` ([m_cap] f32), `done` (int[2]) and
// `epoch` (u32) are local scratch, zero before the first call.  Every rank must call with the same shapes,
// in the same order, on streams that do not run two of these calls concurrently.  M <= 256, N % 8 == 0.
CS_API int cs_gemm_skinny_allreduce(const void* X, long long ldx, const void* W, long long ldw, void* H, long long ldh,
                                    const void* bias, const void* residual, long long ldr, const void* norm_w,
                                    void* normed, long long ldn, float eps, int M, int N, int K, int splits,
                                    void* ws, long long ws_bytes, void* counters, int num_counters, int world,
                                    int rank, const void* const* recv_ptrs, const void* const* flag_ptrs, int m_cap,
                                    int n_cap, int tiles_cap, void* ssq, void* done, void* epoch, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 256 || K <= 0 || (ldx & 7) || (ldw & 7) || (N & 7) || world < 1 || world > AR_MAX_WORLD) return -1;
  // the reduction works on 16-byte row pieces of H, the residual, the norm weight and the normalised output
  if ((ldh & 7) || (residual != nullptr && (ldr & 7)) || (normed != nullptr && (ldn & 7)) || (n_cap & 7) ||
      ((reinterpret_cast<uintptr_t>(H) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(normed) |
        reinterpret_cast<uintptr_t>(norm_w)) & 15))
    return -1;
  SkinnyParams p{};
  p.M = M; p.N = N; p.K = K;
  p.m_pad = (M + 15) & ~15;
  if (p.m_pad > m_cap || N > n_cap) return -6;
  p.swiglu = 0;
  p.up_row_offset = N;
  p.C = H; p.ldc = ldh; p.out_fp32 = 0;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = ACT_NONE;
  p.err = cs_error_word();
  const int tiles = (N + 127) / 128;
  if (tiles > tiles_cap) return -6;
  if (splits <= 0) splits = cs_gemm_skinny_auto_splits(N, K, 0);
  const int total_it = (K + BK * KATOMS - 1) / (BK * KATOMS);
  if (splits > total_it) splits = total_it;
  if (splits > 1 && (ws == nullptr || counters == nullptr || tiles > num_counters ||
                     cs_gemm_skinny_ws_bytes(M, N, splits, 0) > ws_bytes))
    return -5;
  // every CTA of every rank must be resident at once (tile CTAs wait for their peers' tile CTAs)
  while (splits > 1 && tiles * splits > cs_num_sms()) --splits;
  if (tiles * splits > cs_num_sms()) return -6;
  p.splits = splits;
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = reinterpret_cast<int*>(counters);
  p.ar.world = world; p.ar.rank = rank;
  for (int i = 0; i < world; ++i) {
    p.ar.recv[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(recv_ptrs[i]));
    p.ar.flags[i] = reinterpret_cast<unsigned*>(const_cast<void*>(flag_ptrs[i]));
  }
  p.ar.m_cap = m_cap; p.ar.n_cap = n_cap; p.ar.tiles_cap = tiles_cap;
  p.ar.ssq = reinterpret_cast<float*>(ssq);
  p.ar.done = reinterpret_cast<int*>(done);
  p.ar.epoch = reinterpret_cast<unsigned*>(epoch);
  p.ar.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.ar.normed = reinterpret_cast<__nv_bfloat16*>(normed);
  p.ar.ldn = ldn;
  p.ar.eps = eps;
  if (world == 1) return -7;  // use cs_gemm_skinny + cs_norm on a single GPU
  const int stage_bytes = KATOMS * (W_ATOM + p.m_pad * 128);
  int stages = MAX_STAGES;
  const int max_smem = 220 * 1024;
  while (stages > 2 && stages * stage_bytes + 1024 > max_smem) --stages;
  p.stages = stages;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(p.m_pad)) cols <<= 1;
  p.tmem_cols = cols;
  p.idesc = umma_idesc_bf16(128, p.m_pad, 0, 0);
  CUtensorMap tmW, tmX;
  if (cs_encode_tmap_2d(&tmW, W, K, N, ldw * 2, BK, 128, 2, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmX, X, K, M, ldx * 2, BK, p.m_pad, 2, 1) != 0) return -3;
  const int smem = stages * stage_bytes + 1024;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    attr_done[dev] = true;
  }
  gemm_skinny_kernel<<<tiles * splits, 192, smem, stream>>>(tmW, tmX, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free entry point (contract and audience: cornserve_noalloc.h).  The split-K scratch and the
// word that records a bounded wait running out are one static device array of this library; nothing below
// allocates host or device memory.
// ---------------------------------------------------------------------------------------------------------
#include <mutex>
#include <stdio.h>

#include "cornserve_noalloc.h"

// [partial sums | arrival counters | error word].  In host code this name is only the handle given to
// cudaGetSymbolAddress; it is never handed to a kernel as if it were a device pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CS_NOALLOC_SCRATCH_BYTES + 256];

namespace {
constexpr int kNoallocMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_dev[kNoallocMaxDevices] = {nullptr};  // device address of the array, per device
thread_local char g_noalloc_msg[320] = "ok";

int noalloc_fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), fmt, a, b);
  return code;
}

// Device address of the scratch array on the current device.  The first call on a device looks the address
// up (cudaGetSymbolAddress with that device current) and raises the kernel's shared-memory limit.
unsigned char* noalloc_scratch_of_current_device(int* code) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) {
    *code = noalloc_fail(CS_NOALLOC_SETUP_FAILED, "cs_gemm_skinny_noalloc: no usable current device (%lld)", dev);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_dev[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      *code = noalloc_fail(CS_NOALLOC_SETUP_FAILED,
                           "cs_gemm_skinny_noalloc: cudaGetSymbolAddress failed with CUDA error %lld on device %lld",
                           static_cast<long long>(e), dev);
      return nullptr;
    }
    const cudaError_t a = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (a != cudaSuccess) {
      *code = noalloc_fail(CS_NOALLOC_SETUP_FAILED, "cs_gemm_skinny_noalloc: cudaFuncSetAttribute failed with CUDA error %lld",
                           static_cast<long long>(a));
      return nullptr;
    }
    g_noalloc_dev[dev] = ptr;
  }
  return g_noalloc_dev[dev];
}

int noalloc_effective_splits(int N, int K, int swiglu, int splits) {
  if (splits <= 0) splits = cs_gemm_skinny_auto_splits(N, K, swiglu);
  const int total_it = (K + BK * KATOMS - 1) / (BK * KATOMS);
  return splits > total_it ? total_it : splits;
}
}  // namespace

CS_API long long cs_gemm_skinny_noalloc_need_bytes(int M, int N, int K, int swiglu, int splits) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return cs_gemm_skinny_ws_bytes(M, N, noalloc_effective_splits(N, K, swiglu, splits), swiglu);
}

CS_API const char* cs_noalloc_last_message(void) { return g_noalloc_msg; }

// Copies the error word of the current device back (synchronises with the device; no allocation): 0, or the
// CsError code of a bounded wait that ran out inside a cs_gemm_skinny_noalloc kernel since the last call here.
CS_API int cs_gemm_skinny_noalloc_kernel_error(void) {
  int code = 0;
  unsigned char* base = noalloc_scratch_of_current_device(&code);
  if (base == nullptr) return code;
  int word = 0;
  if (cudaMemcpy(&word, base + CS_NOALLOC_SCRATCH_BYTES, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return CS_NOALLOC_SETUP_FAILED;
  if (word != 0) cudaMemset(base + CS_NOALLOC_SCRATCH_BYTES, 0, sizeof(int));
  return word;
}

CS_API int cs_gemm_skinny_noalloc(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc,
                                  const void* bias, const void* residual, long long ldr, int M, int N, int K, int act,
                                  int swiglu, int out_fp32, int splits, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 256 || K <= 0 || (ldx & 7) || (ldw & 7))
    return noalloc_fail(-1, "cs_gemm_skinny_noalloc: needs 1 <= M <= 256, K > 0 and row strides that are multiples of 8 elements");
  splits = noalloc_effective_splits(N, K, swiglu, splits);
  const int cols_per_tile = swiglu ? 64 : 128;
  const int tiles = (N + cols_per_tile - 1) / cols_per_tile;
  const long long need = cs_gemm_skinny_ws_bytes(M, N, splits, swiglu);
  if (need > CS_NOALLOC_PARTIAL_BYTES)
    return noalloc_fail(CS_NOALLOC_TOO_LARGE,
                        "cs_gemm_skinny_noalloc: this problem needs %lld bytes of partial sums but the built-in scratch holds "
                        "%lld; pass a smaller `splits` (1 needs none) or call cs_gemm_skinny with your own workspace",
                        need, CS_NOALLOC_PARTIAL_BYTES);
  if (splits > 1 && tiles > CS_NOALLOC_MAX_TILES)
    return noalloc_fail(CS_NOALLOC_TOO_LARGE, "cs_gemm_skinny_noalloc: %lld output tiles exceed the %lld built-in arrival counters",
                        tiles, CS_NOALLOC_MAX_TILES);
  int code = 0;
  unsigned char* base = noalloc_scratch_of_current_device(&code);
  if (base == nullptr) return code;
  int* counters = reinterpret_cast<int*>(base + CS_NOALLOC_PARTIAL_BYTES);
  if (splits > 1) {
    // the counters must start at zero; a call that ended in an error may have left some raised
    if (cudaMemsetAsync(counters, 0, static_cast<size_t>(tiles) * sizeof(int), stream) != cudaSuccess)
      return noalloc_fail(CS_NOALLOC_SETUP_FAILED, "cs_gemm_skinny_noalloc: clearing the arrival counters failed");
  }
  SkinnyParams p{};
  p.M = M; p.N = N; p.K = K;
  p.m_pad = (M + 15) & ~15;
  p.swiglu = swiglu;
  p.up_row_offset = N;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = act;
  p.err = reinterpret_cast<int*>(base + CS_NOALLOC_SCRATCH_BYTES);
  p.splits = splits;
  p.par_reduce = (splits > 1 && tiles * splits <= cs_num_sms()) ? 1 : 0;
  p.ws = reinterpret_cast<float*>(base);
  p.counters = counters;
  const int stage_bytes = KATOMS * (W_ATOM + p.m_pad * 128);
  int stages = MAX_STAGES;
  while (stages > 2 && stages * stage_bytes + 1024 > 220 * 1024) --stages;
  p.stages = stages;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(p.m_pad)) cols <<= 1;
  p.tmem_cols = cols;
  p.idesc = umma_idesc_bf16(128, p.m_pad, 0, 0);
  CUtensorMap tmW, tmX;
  if (cs_encode_tmap_2d(&tmW, W, K, swiglu ? 2 * N : N, ldw * 2, BK, swiglu ? 64 : 128, 2, 1) != 0)
    return noalloc_fail(-2, "cs_gemm_skinny_noalloc: W cannot be described to the TMA unit (16-byte aligned base and row stride needed)");
  if (cs_encode_tmap_2d(&tmX, X, K, M, ldx * 2, BK, p.m_pad, 2, 1) != 0)
    return noalloc_fail(-3, "cs_gemm_skinny_noalloc: X cannot be described to the TMA unit (16-byte aligned base and row stride needed)");
  gemm_skinny_kernel<<<tiles * splits, 192, stages * stage_bytes + 1024, stream>>>(tmW, tmX, p);
  if (cudaGetLastError() != cudaSuccess) return noalloc_fail(-10, "cs_gemm_skinny_noalloc: the kernel launch failed");
  snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ok");
  return 0;
}
