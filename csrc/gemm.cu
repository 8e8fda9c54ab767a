// bf16 GEMM for sm_100a:  C[M,N] = epilogue(A[M,K] * W[N,K]^T)
//
// Persistent, warp-specialised kernel.  One CTA per SM walks a list of 128 x BN output tiles:
//   warp 0 (one lane)  : TMA producer, fills a ring of (A,B) K-blocks of 64 columns
//   warp 1 (one lane)  : issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//                        accumulators, releases ring slots with tcgen05.commit
//   warps 2..5         : epilogue; each warp owns 32 TMEM lanes (= 32 output rows), reads the
//                        accumulator with tcgen05.ld and applies bias / activation / gate /
//                        residual / SwiGLU before storing bf16 (or fp32)
// While the epilogue drains accumulator i, the MMA warp already fills accumulator i^1.
//
// Operands are K-major (A row-major [M,K]; W is the nn.Linear layout [N,K]), staged by TMA with
// the 128-byte swizzle; edges in M, N and K are handled by TMA zero fill plus masked stores.
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int MAX_STAGES = 16;
constexpr int GROUP_M = 16;

enum Act : int { ACT_NONE = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_QUICK_GELU = 4, ACT_RELU = 5 };

struct GemmParams {
  int M, N, K;            // N = number of output columns
  void* C;                // bf16 or fp32 [M, ldc]
  long long ldc;
  const __nv_bfloat16* bias;      // [N] (or [2N] for SwiGLU), may be null
  const __nv_bfloat16* residual;  // [M, ldr], may be null
  long long ldr;
  const __nv_bfloat16* gate;      // [M / gate_rpb, ldg] multiplicative gate applied before the residual
  long long ldg;
  int gate_rpb;
  int act;
  int out_fp32;
  int stages;
  int a_rows;             // rows of the A box actually fetched (<= 128)
  int a_bytes;            // shared-memory bytes reserved per stage for the A tile (multiple of 1024)
  int up_row_offset;      // SwiGLU: row of W where the "up" half starts
  uint32_t idesc;
  int* err;
  // ---- tensor-parallel coupling (COMM variant of the kernel only) ----
  // A-side: A is a buffer that peers fill row by row (an all-gather in flight).  a_flags[c] counts the rows of
  // chunk c that have landed (each "pushed row" is 1/a_rpr of a GEMM row); a tile waits for the chunks it reads.
  const unsigned* a_flags;   // null = A is ready
  int a_chunk;               // pushed rows per flag (128 * a_rpr)
  int a_total;               // pushed rows in total (M * a_rpr)
  unsigned a_epoch;          // flag value per pushed row of this call
  int m_rot;                 // tile-row rotation so that every rank starts with the rows it owns
  // C-side: partial sums go to the rank that owns the output rows (a reduce-scatter in flight) instead of C.
  __nv_bfloat16* push_dst[8];  // per owner: [world][rows_per_rank][push_ld]
  unsigned* push_flags[8];     // per owner: one arrival counter per 128-row block of its shard
  int push_world, push_rank, rows_per_rank;
  long long push_ld;
  // push_mode 2 (all-to-all of heads, Ulysses): a tile of output columns goes to the rank that owns those heads.
  // Columns are [part][D] (q | k | v); within a part, rank o owns columns [o*own, (o+1)*own).  Rows are this rank's
  // tokens: row r lands at ((r0+r)/seg)*seg*world + rank*seg + (r0+r)%seg of the owner's [world*rows, parts*own] buffer.
  int push_mode;             // 1 = by row owner (reduce-scatter), 2 = by column owner, 3 = by per-row table
  int a2a_part_cols, a2a_own_cols, a2a_seg, a2a_row0;
  int a2a_run, a2a_stride;   // input row m sits at row a2a_row0 + (m / run) * stride + m % run of this rank's token order
  // ---- grouped GEMM (mixture of experts; COMM variant only) ----
  // A holds the rows of every local expert, each expert's segment padded to a multiple of grp_tile_rows.  Row tile t
  // covers rows [t * grp_tile_rows, ...) and multiplies with rows [e * grp_w_rows, ...) of W, e = grp_tile_expert[t].
  // The tables are written on the device by the layout kernel of the same stream (no host round trip).
  const int* grp_tile_expert;  // null = not grouped
  const int* grp_tile_valid;   // rows of tile t that hold tokens (the rest is padding)
  const int* grp_num_tiles;    // device word: row tiles in use
  int grp_tile_rows, grp_w_rows;
  // push_mode 3 (expert outputs return to the token owners): A row r goes to row grp_row_meta[r].y of rank
  // grp_row_meta[r].x; the last CTA to finish bumps every rank's arrival counter once (grp_done counts CTAs).
  const int2* grp_row_meta;
  unsigned* grp_done;
};

constexpr uint64_t kFlagSpinCheck = 0x3f;

// f[j] += bias[j] for the first n (<= 32) columns; bias + 0 is 16-byte aligned when col0 is.
__device__ __forceinline__ void add_bias32(float (&f)[32], const __nv_bfloat16* b, int n) {
  if (n == 32 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) {
    const uint4* b4 = reinterpret_cast<const uint4*>(b);
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
      const uint4 w = __ldg(b4 + j4);
      f[j4 * 8 + 0] += bf16lo(w.x); f[j4 * 8 + 1] += bf16hi(w.x);
      f[j4 * 8 + 2] += bf16lo(w.y); f[j4 * 8 + 3] += bf16hi(w.y);
      f[j4 * 8 + 4] += bf16lo(w.z); f[j4 * 8 + 5] += bf16hi(w.z);
      f[j4 * 8 + 6] += bf16lo(w.w); f[j4 * 8 + 7] += bf16hi(w.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < n) f[j] += __bfloat162float(b[j]);
  }
}

// The activation is chosen once per 32 columns (uniform branch), then applied in a straight loop.
__device__ __forceinline__ void apply_act32(float (&f)[32], int act) {
  switch (act) {
    case ACT_GELU_ERF:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = 0.5f * f[j] * (1.0f + erff(f[j] * 0.70710678118654752f));
      break;
    case ACT_GELU_TANH:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float u = 0.7978845608028654f * (f[j] + 0.044715f * f[j] * f[j] * f[j]);
        // tanh(u) = 1 - 2 / (exp(2u) + 1)
        f[j] = 0.5f * f[j] * (2.0f - __fdividef(2.0f, __expf(2.0f * u) + 1.0f));
      }
      break;
    case ACT_SILU:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __fdividef(f[j], 1.0f + __expf(-f[j]));
      break;
    case ACT_QUICK_GELU:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __fdividef(f[j], 1.0f + __expf(-1.702f * f[j]));
      break;
    case ACT_RELU:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = fmaxf(f[j], 0.0f);
      break;
    default:
      break;
  }
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  int per_band = GROUP_M * tiles_n;
  int band = t / per_band;
  int r = t - band * per_band;
  int m_first = band * GROUP_M;
  int gm = min(GROUP_M, tiles_m - m_first);
  tm = m_first + (r % gm);
  tn = r / gm;
}

// Bounded wait until *flag >= target (flag written by other GPUs with release semantics).
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned target, volatile int* abort_flag, int* err) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if ((spin & kFlagSpinCheck) == kFlagSpinCheck) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > CS_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        cs_set_error(err, CS_ERR_TIMEOUT_PEER);
        return false;
      }
    }
  }
}

template <int BN, bool SWIGLU, bool COMM = false>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;
  constexpr int B_BYTES = BN * BK * 2;
  const int A_BYTES = p.a_bytes;
  const int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[MAX_STAGES];
  __shared__ uint64_t empty_bar[MAX_STAGES];
  __shared__ uint64_t acc_full[2];
  __shared__ uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int push_cnt[4];  // COMM push: epilogue warps that have sent their rows of the current / next tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int stages = p.stages;
  const bool grouped = COMM && p.grp_tile_expert != nullptr;
  const int tile_rows = grouped ? p.grp_tile_rows : BM;
  const int tiles_m = grouped ? *p.grp_num_tiles : (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN_OUT - 1) / BN_OUT;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    push_cnt[0] = push_cnt[1] = push_cnt[2] = push_cnt[3] = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  // COMM push: each epilogue warp stages its 32 x BN_OUT bf16 sub-tile here so that rows leave as contiguous
  // 16-byte-per-lane stores (scattered 16-byte stores are slow over NVLink).  Row pitch padded against conflicts.
  constexpr int STG_PITCH = BN_OUT * 2 + 16;
  uint8_t* stg_base = smem + stages * STAGE_BYTES + (BM * BK * 2 - A_BYTES);

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = static_cast<uint32_t>(p.a_rows * BK * 2 + B_BYTES);
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        if (COMM) tm = (tm + p.m_rot) % tiles_m;
        const int m0 = tm * tile_rows;
        const int n0 = tn * BN_OUT + (grouped ? p.grp_tile_expert[tm] * p.grp_w_rows : 0);  // row of W
        if (COMM && p.a_flags != nullptr) {
          // the rows of this tile are chunk tm of the gathered operand: wait until all of them have landed
          const int rows = min(p.a_chunk, p.a_total - tm * p.a_chunk);
          if (!wait_flag_ge(p.a_flags + tm, p.a_epoch * static_cast<unsigned>(rows), abortp, p.err)) { ok = false; break; }
          // the rows were written by ordinary stores (of other GPUs); the TMA unit reads through the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], tx_bytes);
          tma_load_2d(sA, &tmA, kb * BK, m0, &full_bar[stage]);
          if (SWIGLU) {
            tma_load_2d(sB, &tmB, kb * BK, n0, &full_bar[stage]);
            tma_load_2d(sB + B_BYTES / 2, &tmB, kb * BK, p.up_row_offset + n0, &full_bar[stage]);
          } else {
            tma_load_2d(sB, &tmB, kb * BK, n0, &full_bar[stage]);
          }
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------ MMA issuer --------------------------------
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_EPI)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abortp, p.err, CS_ERR_TIMEOUT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // -------------------------------- epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    int acc = 0;
    uint32_t acc_phase = 0;
    int n_push = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      if (COMM) tm = (tm + p.m_rot) % tiles_m;
      const int row = tm * tile_rows + q * 32 + lane;
      const int n0 = tn * BN_OUT;
      const int tile_valid = grouped ? p.grp_tile_valid[tm] : BM;
      if (!mbar_wait(&acc_full[acc], acc_phase, abortp, p.err, CS_ERR_TIMEOUT_MMA)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool row_ok = grouped ? (q * 32 + lane < tile_valid) : (row < p.M);
      const __nv_bfloat16* gate_row =
          (p.gate != nullptr && row_ok) ? p.gate + static_cast<long long>(row / p.gate_rpb) * p.ldg : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN_OUT / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        const bool full = (col0 + 32 <= p.N);
        uint32_t v[32];
        float f[32];
        tmem_ld32(t_row + c * 32, v);
        if (SWIGLU) {
          uint32_t u[32];
          tmem_ld32(t_row + BN_OUT + c * 32, u);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias != nullptr) {
            add_bias32(f, p.bias + col0, full ? 32 : p.N - col0);
            float fu[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) fu[j] = __uint_as_float(u[j]);
            add_bias32(fu, p.bias + p.N + col0, full ? 32 : p.N - col0);
#pragma unroll
            for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(fu[j]);
          }
          apply_act32(f, p.act);
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] *= __uint_as_float(u[j]);
        } else {
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias != nullptr) add_bias32(f, p.bias + col0, full ? 32 : p.N - col0);
          apply_act32(f, p.act);
        }
        if (row_ok) {
          if (gate_row != nullptr) {
            const __nv_bfloat16* gr = gate_row + col0;
            if (full && ((reinterpret_cast<uintptr_t>(gr) & 15) == 0)) {
              const uint4* g4 = reinterpret_cast<const uint4*>(gr);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const uint4 w = g4[j4];
                f[j4 * 8 + 0] *= bf16lo(w.x); f[j4 * 8 + 1] *= bf16hi(w.x);
                f[j4 * 8 + 2] *= bf16lo(w.y); f[j4 * 8 + 3] *= bf16hi(w.y);
                f[j4 * 8 + 4] *= bf16lo(w.z); f[j4 * 8 + 5] *= bf16hi(w.z);
                f[j4 * 8 + 6] *= bf16lo(w.w); f[j4 * 8 + 7] *= bf16hi(w.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) f[j] *= __bfloat162float(gr[j]);
            }
          }
          if (p.residual != nullptr) {
            const __nv_bfloat16* rr = p.residual + static_cast<long long>(row) * p.ldr + col0;
            if (full && ((reinterpret_cast<uintptr_t>(rr) & 15) == 0)) {
              const uint4* r4 = reinterpret_cast<const uint4*>(rr);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                uint4 w = r4[j4];
                f[j4 * 8 + 0] += bf16lo(w.x); f[j4 * 8 + 1] += bf16hi(w.x);
                f[j4 * 8 + 2] += bf16lo(w.y); f[j4 * 8 + 3] += bf16hi(w.y);
                f[j4 * 8 + 4] += bf16lo(w.z); f[j4 * 8 + 5] += bf16hi(w.z);
                f[j4 * 8 + 6] += bf16lo(w.w); f[j4 * 8 + 7] += bf16hi(w.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) f[j] += __bfloat162float(rr[j]);
            }
          }
          if (p.out_fp32) {
            float* out = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
              float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4)
                o4[j4] = make_float4(f[j4 * 4], f[j4 * 4 + 1], f[j4 * 4 + 2], f[j4 * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) out[j] = f[j];
            }
          } else if (COMM && p.push_world > 0) {
            // stage this lane's 32 columns; the warp sends whole rows once the tile is complete (below)
            uint4* sp = reinterpret_cast<uint4*>(stg_base + (q * 32 + lane) * STG_PITCH + c * 64);
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              uint4 w;
              w.x = pack_bf16x2(f[j4 * 8 + 0], f[j4 * 8 + 1]);
              w.y = pack_bf16x2(f[j4 * 8 + 2], f[j4 * 8 + 3]);
              w.z = pack_bf16x2(f[j4 * 8 + 4], f[j4 * 8 + 5]);
              w.w = pack_bf16x2(f[j4 * 8 + 6], f[j4 * 8 + 7]);
              sp[j4] = w;
            }
          } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
              uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                uint4 w;
                w.x = pack_bf16x2(f[j4 * 8 + 0], f[j4 * 8 + 1]);
                w.y = pack_bf16x2(f[j4 * 8 + 2], f[j4 * 8 + 3]);
                w.z = pack_bf16x2(f[j4 * 8 + 4], f[j4 * 8 + 5]);
                w.w = pack_bf16x2(f[j4 * 8 + 6], f[j4 * 8 + 7]);
                o4[j4] = w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) out[j] = __float2bfloat16(f[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
      if (COMM && p.push_world > 0) {
        // partial sums of this rank go to slot [rank] of the receive buffer of the rank that owns the rows:
        // lanes_per_row lanes cover one row with consecutive 16-byte pieces
        __syncwarp();
        constexpr int LPR = BN_OUT / 8;               // lanes per row (32 for 256 columns, 16 for 128)
        constexpr int RPI = 32 / LPR;                 // rows per store instruction
        const int cc = lane % LPR;
        const bool col_ok = n0 + cc * 8 < p.N;
        int owner = 0;
        if (p.push_mode == 3) {
#pragma unroll 4
          for (int r0 = 0; r0 < 32; r0 += RPI) {
            const int rr = q * 32 + r0 + lane / LPR;    // row within the tile
            if (col_ok && rr < tile_valid) {
              const int2 meta = __ldcg(&p.grp_row_meta[tm * tile_rows + rr]);  // written by peers: not through L1
              const uint4 w = *reinterpret_cast<const uint4*>(stg_base + rr * STG_PITCH + cc * 16);
              *reinterpret_cast<uint4*>(p.push_dst[meta.x] + static_cast<long long>(meta.y) * p.push_ld + n0 + cc * 8) = w;
            }
          }
        } else if (p.push_mode == 2) {
          const int part = n0 / p.a2a_part_cols, within = n0 - part * p.a2a_part_cols;
          owner = within / p.a2a_own_cols;
          const int dcol = part * p.a2a_own_cols + (within - owner * p.a2a_own_cols) + cc * 8;
#pragma unroll 4
          for (int r0 = 0; r0 < 32; r0 += RPI) {
            const int rr = q * 32 + r0 + lane / LPR;    // row within the tile
            if (col_ok && tm * BM + rr < p.M) {
              const int mrow = tm * BM + rr;             // row in this rank's token order: runs of a2a_run rows
              const int lr = p.a2a_row0 + (mrow / p.a2a_run) * p.a2a_stride + mrow % p.a2a_run;
              const long long drow = static_cast<long long>(lr / p.a2a_seg) * p.a2a_seg * p.push_world +
                                     static_cast<long long>(p.push_rank) * p.a2a_seg + lr % p.a2a_seg;
              const uint4 w = *reinterpret_cast<const uint4*>(stg_base + rr * STG_PITCH + cc * 16);
              *reinterpret_cast<uint4*>(p.push_dst[owner] + drow * p.push_ld + dcol) = w;
            }
          }
        } else {
          owner = (tm * BM) / p.rows_per_rank;
          const long long slot_row0 = static_cast<long long>(p.push_rank) * p.rows_per_rank + (tm * BM - owner * p.rows_per_rank);
#pragma unroll 4
          for (int r0 = 0; r0 < 32; r0 += RPI) {
            const int rr = q * 32 + r0 + lane / LPR;    // row within the tile
            if (col_ok && tm * BM + rr < p.M) {
              const uint4 w = *reinterpret_cast<const uint4*>(stg_base + rr * STG_PITCH + cc * 16);
              *reinterpret_cast<uint4*>(p.push_dst[owner] + (slot_row0 + rr) * p.push_ld + n0 + cc * 8) = w;
            }
          }
        }
        // The last of the four epilogue warps to finish the tile tells the owner of the rows (one system-scope
        // release per tile: such releases are expensive).  The warps meet through a shared-memory counter, not a
        // barrier, so a warp that gave up on a wait cannot strand the others; the owner's wait is bounded too.
        __syncwarp();
        if (lane == 0 && p.push_mode != 3) {
          __threadfence_block();
          const int par = n_push & 3;  // a warp cannot get four tiles ahead of another (two accumulators)
          const int prev = atomicAdd(&push_cnt[par], 1);
          if (prev == 3) {
            push_cnt[par] = 0;
            __threadfence_block();
            const int blk = p.push_mode == 2 ? 0 : (tm * BM - owner * p.rows_per_rank) / BM;
            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.push_flags[owner] + blk) : "memory");
          }
        }
        ++n_push;
      }
    }
  }

  if (COMM && p.push_mode == 3) __threadfence();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (COMM && p.push_mode == 3 && threadIdx.x == 0) {
    // every row of this CTA has left; the last CTA of the grid tells all ranks that this rank's experts are done
    __threadfence();
    const unsigned prev = atomicAdd(p.grp_done, 1u);
    if (prev == gridDim.x - 1) {
      *p.grp_done = 0;
      __threadfence();
      for (int o = 0; o < p.push_world; ++o)
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.push_flags[o]) : "memory");
    }
  }
}

template <int BN, bool SWIGLU, bool COMM = false>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, cudaStream_t stream) {
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;
  const int stage_bytes = p.a_bytes + BN * BK * 2;
  int stages = p.stages;
  const int max_smem = 220 * 1024;
  if (stages <= 0) stages = MAX_STAGES;
  // The MMA always reads 128 rows of A; when fewer rows are fetched the read runs past the A slot,
  // so keep a tail pad that makes the last stage's read stay inside the allocation.
  const int tail_pad = BM * BK * 2 - p.a_bytes;
  const int staging = COMM ? BM * (BN_OUT * 2 + 16) : 0;  // epilogue staging of the push variant
  while (stages > 2 && stages * stage_bytes + 1024 + tail_pad + staging > max_smem) --stages;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  p.stages = stages;
  const int smem = stages * stage_bytes + 1024 + tail_pad + staging;
  static bool attr_done[64] = {false};
  auto kern = gemm_bf16_kernel<BN, SWIGLU, COMM>;
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    attr_done[dev] = true;
  }
  const int rows_per_tile = (COMM && p.grp_tile_expert != nullptr) ? p.grp_tile_rows : BM;
  const int tiles = ((p.M + rows_per_tile - 1) / rows_per_tile) * ((p.N + BN_OUT - 1) / BN_OUT);
  int grid = tiles < cs_num_sms() ? tiles : cs_num_sms();
  if (grid < 1) return 0;
  p.idesc = umma_idesc_bf16(128, BN, 0, 0);
  kern<<<grid, 192, smem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

}  // namespace

// C[M,N] = act(A[M,K] W[N,K]^T + bias) * gate + residual         (swiglu == 0)
// C[M,N] = act(A Wg^T + bg) * (A Wu^T + bu), W = [Wg; Wu] ([2N,K]) (swiglu == 1)
// All matrices bf16 row-major with the given leading dimensions (elements); lda/ldw must be
// multiples of 8.  `bn` picks the tile width (0 = choose from the problem size).
CS_API int cs_gemm_bf16(const void* A, long long lda, const void* W, long long ldw, void* C,
                        long long ldc, const void* bias, const void* residual, long long ldr,
                        const void* gate, long long ldg, int gate_rpb, int M, int N, int K, int act,
                        int swiglu, int out_fp32, int bn, int stages, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda & 7) || (ldw & 7)) return -1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.gate = reinterpret_cast<const __nv_bfloat16*>(gate);
  p.ldg = ldg;
  p.gate_rpb = gate_rpb > 0 ? gate_rpb : 1;
  p.act = act;
  p.out_fp32 = out_fp32;
  p.stages = stages;
  p.up_row_offset = N;
  p.err = cs_error_word();
  p.a_rows = M >= BM ? BM : ((M + 7) & ~7);
  p.a_bytes = p.a_rows * BK * 2;

  const int sms = cs_num_sms();
  const int tiles_m = (M + BM - 1) / BM;
  if (bn == 0) {
    if (swiglu) {
      bn = (tiles_m * ((N + 127) / 128) >= sms) ? 256 : 128;
    } else {
      // Wide tiles re-read the activation rows less often (a column tile reads all K of its 128 rows): measured at
      // 256..512 rows, a 128- or 256-wide tile on 96 of the 148 SMs beats narrower tiles on all of them by
      // 1.3-1.8x.  So narrow only until about five eighths of the SMs have a tile, and not below 64 columns.
      bn = 256;
      const int want = (5 * sms) / 8;
      while (bn > 64 && tiles_m * ((N + bn - 1) / bn) < want) bn >>= 1;
      if (N <= 32) bn = 32;
      if (M > 2048 && bn < 128) bn = 128;
    }
  }
  const int w_rows = swiglu ? 2 * N : N;
  CUtensorMap tmA, tmB;
  if (cs_encode_tmap_2d(&tmA, A, K, M, lda * 2, BK, p.a_rows, 2, 1) != 0) return -2;
  const int b_box = swiglu ? bn / 2 : bn;
  if (cs_encode_tmap_2d(&tmB, W, K, w_rows, ldw * 2, BK, b_box, 2, 1) != 0) return -3;

  if (swiglu) {
    switch (bn) {
      case 256: return launch<256, true>(tmA, tmB, p, stream);
      case 128: return launch<128, true>(tmA, tmB, p, stream);
      case 64: return launch<64, true>(tmA, tmB, p, stream);
      default: return -4;
    }
  }
  switch (bn) {
    case 256: return launch<256, false>(tmA, tmB, p, stream);
    case 128: return launch<128, false>(tmA, tmB, p, stream);
    case 64: return launch<64, false>(tmA, tmB, p, stream);
    case 32: return launch<32, false>(tmA, tmB, p, stream);
    default: return -4;
  }
}

// Tensor-parallel coupled GEMM (one kernel per rank, the ranks meet only through flags in peer memory):
//   * `a_flags` != null: A is the local copy of an operand that peers are still pushing row by row (the
//     all-gather half of a column-parallel layer).  Tile row i waits until a_flags[i] >= a_epoch * (pushed rows in
//     chunk i); a pushed row is 1/a_rpr of a GEMM row (a_rpr = 4 when [S, H] rows are read as [S/4, 4H]).
//   * `push_world` > 0: the result is a partial sum of a row-parallel layer.  Tile rows go, as bf16, into slot
//     [push_rank] of the receive buffer of the rank that owns them (rank o owns rows [o*rows_per_rank, ...),
//     rows_per_rank a multiple of 128) and that rank's arrival counter of the 128-row block is bumped once per tile;
//     C is unused.
// `m_rot` rotates the tile rows so that a rank starts with rows that are already local.  Epilogue options as in
// cs_gemm_bf16 (bias and residual are normally left to the reduction kernel when pushing).
CS_API int cs_gemm_bf16_tp(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                           const void* bias, int M, int N, int K, int act, int swiglu, int bn, const void* a_flags,
                           int a_rpr, unsigned a_epoch, int m_rot, int push_world, int push_rank,
                           const void* const* push_dst, const void* const* push_flags, int rows_per_rank,
                           long long push_ld, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda & 7) || (ldw & 7) || push_world > 8 || M < BM) return -1;
  if (push_world > 0 && (rows_per_rank % BM != 0 || swiglu || (push_ld & 7))) return -1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.gate_rpb = 1;
  p.act = act;
  p.up_row_offset = N;
  p.err = cs_error_word();
  p.a_rows = BM;
  p.a_bytes = BM * BK * 2;
  p.a_flags = reinterpret_cast<const unsigned*>(a_flags);
  p.a_chunk = BM * (a_rpr > 0 ? a_rpr : 1);
  p.a_total = M * (a_rpr > 0 ? a_rpr : 1);
  p.a_epoch = a_epoch;
  const int tiles_m = (M + BM - 1) / BM;
  p.m_rot = ((m_rot % tiles_m) + tiles_m) % tiles_m;
  p.push_world = push_world; p.push_rank = push_rank; p.rows_per_rank = rows_per_rank > 0 ? rows_per_rank : BM;
  p.push_ld = push_ld;
  p.push_mode = 1;
  for (int i = 0; i < push_world; ++i) {
    p.push_dst[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(push_dst[i]));
    p.push_flags[i] = reinterpret_cast<unsigned*>(const_cast<void*>(push_flags[i]));
  }
  if (bn == 0) bn = swiglu ? 256 : ((tiles_m * ((N + 255) / 256) >= cs_num_sms()) ? 256 : 128);
  CUtensorMap tmA, tmB;
  if (cs_encode_tmap_2d(&tmA, A, K, M, lda * 2, BK, BM, 2, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmB, W, K, swiglu ? 2 * N : N, ldw * 2, BK, swiglu ? bn / 2 : bn, 2, 1) != 0) return -3;
  if (swiglu) {
    switch (bn) {
      case 256: return launch<256, true, true>(tmA, tmB, p, stream);
      case 128: return launch<128, true, true>(tmA, tmB, p, stream);
      default: return -4;
    }
  }
  switch (bn) {
    case 256: return launch<256, false, true>(tmA, tmB, p, stream);
    case 128: return launch<128, false, true>(tmA, tmB, p, stream);
    default: return -4;
  }
}

// Column-parallel projection whose output leaves as an all-to-all (Ulysses sequence parallelism): this rank holds
// `M` token rows and all `parts * part_cols` output columns (q | k | v over all heads); the column tile of heads
// [o*own_cols, (o+1)*own_cols) of every part goes, from the epilogue, to rank o's buffer [world * rows, parts*own_cols]
// at row ((row0+r)/seg)*seg*world + rank*seg + (row0+r)%seg.  One arrival per tile on `flag_ptrs[o][0]`.
// Tiles are 128 columns wide: own_cols and part_cols must be multiples of 128.  M >= 128.
CS_API int cs_gemm_bf16_a2a(const void* A, long long lda, const void* W, long long ldw, const void* bias, int M, int N, int K,
                            int world, int rank, const void* const* dst_ptrs, const void* const* flag_ptrs, long long dst_ld,
                            int part_cols, int own_cols, int seg, int row0, int run, int run_stride, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda & 7) || (ldw & 7) || world < 1 || world > 8 || run <= 0 || (own_cols % 128) || (part_cols % 128) ||
      (N % part_cols) || seg <= 0 || (dst_ld & 7))
    return -1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.gate_rpb = 1;
  p.up_row_offset = N;
  p.err = cs_error_word();
  p.a_rows = M >= BM ? BM : ((M + 7) & ~7);
  p.a_bytes = p.a_rows * BK * 2;
  p.a_chunk = BM; p.a_total = M;
  p.push_world = world; p.push_rank = rank; p.rows_per_rank = BM; p.push_ld = dst_ld;
  p.push_mode = 2;
  p.a2a_part_cols = part_cols; p.a2a_own_cols = own_cols; p.a2a_seg = seg; p.a2a_row0 = row0;
  p.a2a_run = run; p.a2a_stride = run_stride;
  for (int i = 0; i < world; ++i) {
    p.push_dst[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dst_ptrs[i]));
    p.push_flags[i] = reinterpret_cast<unsigned*>(const_cast<void*>(flag_ptrs[i]));
  }
  CUtensorMap tmA, tmB;
  if (cs_encode_tmap_2d(&tmA, A, K, M, lda * 2, BK, p.a_rows, 2, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmB, W, K, N, ldw * 2, BK, 128, 2, 1) != 0) return -3;
  return launch<128, false, true>(tmA, tmB, p, stream);
}

// Grouped GEMM over the rows of this rank's experts (see GemmParams::grp_*): C = A W_e^T per row tile, with the SwiGLU
// epilogue (W_e = [gate; up], 2N rows) or, with push_world > 0, with every valid output row stored at
// (rank, row) = row_meta[A row] of dst_ptrs and one arrival on every rank's flag when the whole launch is done.
// M_cap bounds the rows of A (the grid is sized from it; the tiles actually in use are read on the device).
CS_API int cs_gemm_bf16_grouped(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int M_cap,
                                int N, int K, int swiglu, int experts, int tile_rows, const void* tile_expert,
                                const void* tile_valid, const void* num_tiles, int push_world, const void* const* dst_ptrs,
                                const void* const* flag_ptrs, long long push_ld, const void* row_meta, void* done,
                                void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M_cap <= 0 || N <= 0 || experts <= 0) return 0;
  if (K <= 0 || (lda & 7) || (ldw & 7) || push_world < 0 || push_world > 8 || tile_rows < 8 || tile_rows > BM || (tile_rows & 7) ||
      tile_expert == nullptr || tile_valid == nullptr || num_tiles == nullptr || (push_world > 0 && (swiglu || (push_ld & 7))))
    return -1;
  GemmParams p{};
  p.M = M_cap; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.gate_rpb = 1;
  p.act = swiglu ? ACT_SILU : ACT_NONE;
  p.up_row_offset = N;
  p.err = cs_error_word();
  p.a_rows = tile_rows;
  p.a_bytes = tile_rows * BK * 2;
  p.a_chunk = BM; p.a_total = M_cap;
  p.grp_tile_expert = reinterpret_cast<const int*>(tile_expert);
  p.grp_tile_valid = reinterpret_cast<const int*>(tile_valid);
  p.grp_num_tiles = reinterpret_cast<const int*>(num_tiles);
  p.grp_tile_rows = tile_rows;
  p.grp_w_rows = swiglu ? 2 * N : N;
  if (push_world > 0) {
    p.push_world = push_world; p.push_mode = 3; p.push_ld = push_ld; p.rows_per_rank = BM;
    p.grp_row_meta = reinterpret_cast<const int2*>(row_meta);
    p.grp_done = reinterpret_cast<unsigned*>(done);
    for (int i = 0; i < push_world; ++i) {
      p.push_dst[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dst_ptrs[i]));
      p.push_flags[i] = reinterpret_cast<unsigned*>(const_cast<void*>(flag_ptrs[i]));
    }
  }
  CUtensorMap tmA, tmB;
  if (cs_encode_tmap_2d(&tmA, A, K, M_cap, lda * 2, BK, tile_rows, 2, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmB, W, K, static_cast<long long>(experts) * p.grp_w_rows, ldw * 2, BK, 128, 2, 1) != 0) return -3;
  if (swiglu) return launch<256, true, true>(tmA, tmB, p, stream);
  return launch<128, false, true>(tmA, tmB, p, stream);
}
