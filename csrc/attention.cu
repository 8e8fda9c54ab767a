// Variable-length attention for sm_100a (tcgen05 + TMEM + TMA), one kernel for:
//   * packed var-len self attention without mask (vision towers, windows and full images, DiT)
//   * causal prefill over a paged KV cache (LLM), with grouped-query heads
//   * decode over a paged KV cache: the G query heads that share a KV head are packed into the
//     rows of one tile, so K/V pages are read once per KV head
//
// One CTA = one tile of up to 128 query rows of one sequence and one (group of) head(s).
//   warps 0-7 : softmax; two threads per query row (= TMEM lane), one per half of the 128 keys
//   warp 8    : TMA producer (Q once per item, then a 2-deep ring of K and V tiles of 128 keys)
//   warp 9    : issues tcgen05.mma:  S_j = Q K_j^T  (two S buffers in TMEM, so S_{j+1} is computed
//               while the softmax of S_j runs)  and  O += P_j V_j  (P_j staged in shared memory
//               as a swizzled K-major bf16 tile, V consumed as an MN-major operand)
// Online softmax in base 2; O lives in TMEM and is rescaled in place when the row max moves.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int KV_TILE = 128;
constexpr int KV_STAGES = 2;
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows x 64 bf16

struct AttnParams {
  __nv_bfloat16* O; long long ldo;
  const int* cu_q;        // [B+1] packed query offsets (tokens)
  const int* cu_k;        // [B+1] packed key offsets (contiguous mode)
  const int* kv_len;      // [B] key length (paged mode)
  const int* block_table; // [B, bt_stride] page ids (paged mode)
  int bt_stride;
  int Hq, Hkv, d, G;      // G = query heads packed per tile (1, or Hq/Hkv)
  int causal, paged;
  int window;             // > 0 (with causal): query i only sees the last `window` keys up to its own position
  // packed segments (several short sequences, e.g. attention windows, share one 128-row tile): query token t only
  // sees keys [seg_lo[t], seg_hi[t]) (indices in the packed token numbering); null = not used
  const int* seg_lo; const int* seg_hi;
  int max_q_tiles, head_blks, total_items;
  int kv_splits;          // > 1: every item covers 1/kv_splits of the key tiles and writes fp32 partials
  float* ws_o;            // [Tq*Hq, kv_splits, d] unnormalised partial outputs
  float* ws_ml;           // [Tq*Hq, kv_splits, 2] running max (base-2 scaled) and normaliser
  float scale_log2;
  uint32_t idesc_s, idesc_pv;
  int* err;
};

// Geometry of one work item = one tile of query rows of one sequence and one (group of) head(s).
struct Item {
  int seq, head_blk, q_beg, t0, n_tok, k_beg, k_len, k_end, shift, n_kv, hk, hq0, split, j0;
  bool valid;
};

// 2^x on the special-function unit (ex2.approx: 2 ulp, flushes denormals; -inf -> 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ Item decode_item(const AttnParams& p, int w) {
  Item it;
  it.split = w % p.kv_splits;
  w /= p.kv_splits;
  const int tile = w % p.max_q_tiles;
  const int rest = w / p.max_q_tiles;
  it.head_blk = rest % p.head_blks;
  it.seq = rest / p.head_blks;
  const int tok_per_tile = 128 / p.G;
  it.q_beg = p.cu_q[it.seq];
  const int q_len = p.cu_q[it.seq + 1] - it.q_beg;
  it.t0 = tile * tok_per_tile;
  it.valid = it.t0 < q_len;
  it.k_beg = p.paged ? 0 : p.cu_k[it.seq];
  it.k_len = p.paged ? p.kv_len[it.seq] : (p.cu_k[it.seq + 1] - it.k_beg);
  it.hk = p.G > 1 ? it.head_blk : it.head_blk / (p.Hq / p.Hkv);
  it.hq0 = p.G > 1 ? it.head_blk * p.G : it.head_blk;
  it.n_tok = min(tok_per_tile, q_len - it.t0);
  it.shift = it.k_len - q_len;  // causal: query token i sees keys j <= i + shift
  int k_end = it.k_len;
  if (p.causal) k_end = min(it.k_len, it.t0 + it.n_tok + it.shift);
  it.k_end = k_end;
  const int n_all = (it.valid && k_end > 0) ? (k_end + KV_TILE - 1) / KV_TILE : 0;
  // this item's share of the key tiles: [j0, j0 + n_kv)
  it.j0 = static_cast<int>((static_cast<long long>(it.split) * n_all) / p.kv_splits);
  it.n_kv = static_cast<int>((static_cast<long long>(it.split + 1) * n_all) / p.kv_splits) - it.j0;
  return it;
}

// Persistent: every CTA walks work items blockIdx.x, blockIdx.x + gridDim.x, ...; barriers and TMEM
// are set up once and all pipeline phases are derived from running counters, so the producer already
// fetches Q/K of the next item while the softmax / PV of the current one are still in flight.
template <bool kWindow>
__global__ void __launch_bounds__(320, 1)
attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
            const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  const int tok_per_tile = 128 / p.G;
  const int n_atoms = (p.d + 63) / 64;
  const int d16 = (p.d + 15) / 16;  // 16-column groups in O, and K-steps of Q K^T

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                // n_atoms * 16 KB
  uint8_t* sP = sQ + 2 * ATOM_BYTES;                 // 2 atoms (128 keys)
  uint8_t* sK = sP + 2 * ATOM_BYTES;                 // KV_STAGES * 2 atoms
  uint8_t* sV = sK + KV_STAGES * 2 * ATOM_BYTES;
  __shared__ uint64_t q_full, q_empty, k_full[KV_STAGES], v_full[KV_STAGES], k_empty[KV_STAGES], v_empty[KV_STAGES];
  __shared__ uint64_t s_full[2], p_full, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xmax[2][2][128];  // softmax: the two column halves of a row exchange their maxima here
  __shared__ float xl[2][128];       // ... and their normalisers once per item

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&p_full, 256);
    mbar_init(&o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 9) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 256;
  volatile int* abortp = &abort_flag;

  if (warp == 8) {
    if (lane == 0) {
      // ------------------------------- TMA producer -------------------------------
      uint32_t n_item = 0, n_tile = 0;  // running counts: items with work, KV tiles
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_items && ok; w += gridDim.x) {
        const Item it = decode_item(p, w);
        if (it.n_kv == 0) continue;
        if (!mbar_wait(&q_empty, (n_item & 1) ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) break;
        mbar_arrive_expect_tx(&q_full, static_cast<uint32_t>(n_atoms * p.G * tok_per_tile * 128));
        for (int a = 0; a < n_atoms; ++a)
          tma_load_3d(sQ + a * ATOM_BYTES, &tmQ, a * 64, it.hq0, it.q_beg + it.t0, &q_full);
        ++n_item;
        for (int jj = 0; jj < it.n_kv; ++jj, ++n_tile) {
          const int j = it.j0 + jj;
          const int stage = n_tile % KV_STAGES;
          const uint32_t phase = (n_tile / KV_STAGES) & 1;
          if (!mbar_wait(&k_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[stage], static_cast<uint32_t>(n_atoms * ATOM_BYTES));
          int page = 0;
          if (p.paged) page = p.block_table[(long long)it.seq * p.bt_stride + j];
          for (int a = 0; a < n_atoms; ++a) {
            uint8_t* dst = sK + (stage * 2 + a) * ATOM_BYTES;
            if (p.paged) tma_load_3d(dst, &tmK, a * 64, 0, (page * 2 + 0) * p.Hkv + it.hk, &k_full[stage]);
            else tma_load_3d(dst, &tmK, a * 64, it.hk, it.k_beg + j * KV_TILE, &k_full[stage]);
          }
          if (!mbar_wait(&v_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[stage], static_cast<uint32_t>(n_atoms * ATOM_BYTES));
          for (int a = 0; a < n_atoms; ++a) {
            uint8_t* dst = sV + (stage * 2 + a) * ATOM_BYTES;
            if (p.paged) tma_load_3d(dst, &tmV, a * 64, 0, (page * 2 + 1) * p.Hkv + it.hk, &v_full[stage]);
            else tma_load_3d(dst, &tmV, a * 64, it.hk, it.k_beg + j * KV_TILE, &v_full[stage]);
          }
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // -------------------------------- MMA issuer --------------------------------
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      uint32_t n_item = 0, n_s = 0, n_pv = 0;  // running counts: items, S tiles issued, PV tiles issued
      bool ok = true;
      auto issue_s = [&](bool last_of_item) -> bool {
        const int stage = n_s % KV_STAGES;
        const uint32_t ph = (n_s / KV_STAGES) & 1;
        if (!mbar_wait(&k_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + stage * 2 * ATOM_BYTES);
        for (int kk = 0; kk < d16; ++kk) {
          const uint32_t off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
          umma_f16_ss(tS0 + (n_s & 1) * 128, umma_smem_desc(q_addr + off, 16, 1024),
                      umma_smem_desc(k_addr + off, 16, 1024), p.idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);
        if (last_of_item) umma_commit(&q_empty);
        umma_commit(&s_full[n_s & 1]);
        ++n_s;
        return true;
      };
      for (int w = blockIdx.x; w < p.total_items && ok; w += gridDim.x) {
        const Item it = decode_item(p, w);
        if (it.n_kv == 0) continue;
        if (!mbar_wait(&q_full, n_item & 1, abortp, p.err, CS_ERR_TIMEOUT_TMA)) break;
        ++n_item;
        if (!issue_s(it.n_kv == 1)) break;
        for (int j = 0; j < it.n_kv; ++j) {
          if (j + 1 < it.n_kv) { if (!issue_s(j + 2 == it.n_kv)) { ok = false; break; } }
          const int stage = n_pv % KV_STAGES;
          const uint32_t ph = (n_pv / KV_STAGES) & 1;
          if (!mbar_wait(&p_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_EPI)) { ok = false; break; }
          if (!mbar_wait(&v_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sV + stage * 2 * ATOM_BYTES);
          for (int kk = 0; kk < KV_TILE / 16; ++kk) {
            const uint32_t a_off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
            // V: rows = keys (K index), 64 head-dim columns per atom (N index) -> MN-major operand:
            // 16 keys = two 8-row groups 1024 B apart; the next 64 columns are one atom further.
            umma_f16_ss(tO, umma_smem_desc(p_addr + a_off, 16, 1024),
                        umma_smem_desc(v_addr + kk * 2048, ATOM_BYTES, 1024), p.idesc_pv,
                        (j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&v_empty[stage]);
          umma_commit(&o_full);
          ++n_pv;
        }
      }
    }
  } else {
    // ---------------------------------- softmax -----------------------------------
    // 8 warps: warp w works on TMEM lanes (w % 4) * 32 .. + 31 (= query rows) and on the column half
    // w / 4 of every S tile (64 keys) and of O (d/2 channels); the two threads of a row exchange their
    // partial row maxima through shared memory once per key tile and their normalisers once per item.
    const int hf = warp >> 2;                       // column half
    const int r = (warp & 3) * 32 + lane;           // tile row == TMEM lane
    const int tl = r / p.G, g = r - tl * p.G;       // token in tile, head within group
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint8_t* p_row = sP + hf * ATOM_BYTES + r * 128;  // this thread's 64 keys are exactly one swizzle atom row
    const int oc_lo = hf * ((d16 + 1) / 2), oc_hi = hf ? d16 : (d16 + 1) / 2;  // O column groups of this half
    uint32_t n_s = 0, n_pv = 0;  // running counts of S tiles consumed / PV tiles awaited
    bool ok = true;
    // A failed wait never leaves the loops early: all 256 softmax threads must keep meeting at the named
    // barriers below (after a failure every later wait returns at once because the abort flag is set).
    for (int w = blockIdx.x; w < p.total_items; w += gridDim.x) {
      const Item it = decode_item(p, w);
      if (!it.valid) continue;
      const bool row_ok = tl < it.n_tok;
      const int qi = it.t0 + tl;
      int lim = p.causal ? min(it.k_len, qi + it.shift + 1) : it.k_len;  // keys [lo, lim) are visible
      int lo = (kWindow && p.window > 0) ? max(0, qi + it.shift + 1 - p.window) : 0;
      if (kWindow && p.seg_lo != nullptr && row_ok) {
        lo = p.seg_lo[it.q_beg + qi] - it.k_beg;
        lim = min(lim, p.seg_hi[it.q_beg + qi] - it.k_beg);
      }
      float m = -INFINITY, l = 0.f;
      // A warp whose 32 tile rows all lie beyond the item's tokens (decode: 7 of 128 rows are real) only keeps
      // the barriers company: it neither reads S nor writes P (rows of the MMA are independent, and the rows
      // it would have produced are never stored).
      const bool warp_active = ((warp & 3) * 32) / p.G < it.n_tok;
      for (int j = 0; j < it.n_kv; ++j) {
        if (!mbar_wait(&s_full[n_s & 1], (n_s >> 1) & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) ok = false;
        tc_fence_after();
        const uint32_t tS = tS0 + (n_s & 1) * 128 + lane_off + hf * 64;
        ++n_s;
        if (!warp_active) {
          asm volatile("bar.sync 2, 256;" ::: "memory");
          if (j > 0) ++n_pv;
          tc_fence_before();
          mbar_arrive(&p_full);
          continue;
        }
        const int kbase = (it.j0 + j) * KV_TILE + hf * 64;
        // 32-key chunks of this half that hold any visible key of the tile (uniform over the CTA)
        const int n_ch = max(0, min(2, (it.k_end - kbase + 31) / 32));
        // the scores of this half are read from TMEM once and stay in registers for both passes
        uint32_t sv[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c)
          if (c < n_ch) tmem_ld32(tS + c * 32, sv[c]);
        if (n_ch > 0) tmem_wait_ld();
        // pass 1: row max over this half
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c < n_ch) {
            const int nvalid = lim - (kbase + c * 32);
            const int nlow = lo - (kbase + c * 32);
            if (kWindow && nlow > 0) {  // sliding window: keys below the window count as -inf
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nlow) sv[c][i] = 0xff800000u;
            }
            if (nvalid >= 32) {  // every key of the chunk is visible to this row: no per-element tests
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(sv[c][i]));
                mx1 = fmaxf(mx1, __uint_as_float(sv[c][i + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(sv[c][i + 2]));
                mx3 = fmaxf(mx3, __uint_as_float(sv[c][i + 3]));
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                if (i < nvalid) mx0 = fmaxf(mx0, __uint_as_float(sv[c][i]));
                if (i + 1 < nvalid) mx1 = fmaxf(mx1, __uint_as_float(sv[c][i + 1]));
                if (i + 2 < nvalid) mx2 = fmaxf(mx2, __uint_as_float(sv[c][i + 2]));
                if (i + 3 < nvalid) mx3 = fmaxf(mx3, __uint_as_float(sv[c][i + 3]));
              }
            }
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        xmax[j & 1][hf][r] = mx;  // double-buffered by tile parity: the next write to this slot is two barriers away
        asm volatile("bar.sync 2, 256;" ::: "memory");
        const float mx_row = fmaxf(mx, xmax[j & 1][hf ^ 1][r]);
        // The reference point of the exponents only moves when the row maximum has grown by more than 2^8 since it was
        // set: probabilities then stay below 256 (exact enough in bf16, harmless in the fp32 normaliser), and most key
        // tiles need no rescaling of O at all.  Both threads of a row see the same maxima, so they decide alike.
        const float m_cand = fmaxf(m, mx_row * p.scale_log2);
        const float m_new = (m_cand - m > 8.f) ? m_cand : m;   // m = -inf: the difference is +inf (or NaN when both are)
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2(m - m_use);  // m = -inf -> 0
        // pass 2: probabilities of this half, packed to bf16
        uint32_t pk[32];
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c < n_ch) {
            const int nvalid = lim - (kbase + c * 32);
            // (keys masked by the window hold -inf and come out as 0; the normaliser sums the unrounded values)
            if (nvalid >= 32) {
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float e0 = fast_exp2(__uint_as_float(sv[c][i]) * p.scale_log2 - m_use);
                const float e1 = fast_exp2(__uint_as_float(sv[c][i + 1]) * p.scale_log2 - m_use);
                sum0 += e0;
                sum1 += e1;
                pk[c * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float e0 = (i < nvalid) ? fast_exp2(__uint_as_float(sv[c][i]) * p.scale_log2 - m_use) : 0.f;
                const float e1 = (i + 1 < nvalid) ? fast_exp2(__uint_as_float(sv[c][i + 1]) * p.scale_log2 - m_use) : 0.f;
                sum0 += e0;
                sum1 += e1;
                pk[c * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[c * 16 + i] = 0u;
          }
        }
        l = l * alpha + (sum0 + sum1);  // partial normaliser of this half; both halves share m
        m = m_new;
        tc_fence_before();
        if (j > 0) {
          // PV of the previous tile must be finished: P buffer free, O up to date
          if (!mbar_wait(&o_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) ok = false;
          ++n_pv;
          tc_fence_after();
        }
        // P -> shared memory, K-major with the 128-byte swizzle (16-byte chunk index XOR row%8)
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 wv = make_uint4(pk[cc * 4], pk[cc * 4 + 1], pk[cc * 4 + 2], pk[cc * 4 + 3]);
          *reinterpret_cast<uint4*>(p_row + ((cc ^ (r & 7)) << 4)) = wv;
        }
        // tcgen05.ld/st are warp-collective: decide by vote whether this warp rescales its part of O
        const bool need = __any_sync(0xffffffffu, j > 0 && alpha != 1.0f);
        if (need) {
          for (int c = oc_lo; c < oc_hi; ++c) {
            uint32_t o[16];
            tmem_ld16(tO + lane_off + c * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(
                    tO + lane_off + c * 16),
                "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
                "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15])
                : "memory");
          }
          tmem_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full);
      }
      // ---------------------------------- write O ------------------------------------
      if (ok && it.n_kv > 0) {
        ok = mbar_wait(&o_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA);
        ++n_pv;
      }
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      // total normaliser of the row = sum of the two halves
      xl[hf][r] = l;
      asm volatile("bar.sync 2, 256;" ::: "memory");
      l += xl[hf ^ 1][r];
      asm volatile("bar.sync 2, 256;" ::: "memory");  // xl and xmax are reused by the next item
      if (p.kv_splits > 1) {
        // split-KV: leave the unnormalised partial and its (max, normaliser) for the combine kernel
        const long long prow = ((long long)(it.q_beg + qi) * p.Hq + (it.hq0 + g)) * p.kv_splits + it.split;
        float* po = p.ws_o + prow * p.d;
        if (row_ok && hf == 0) {
          p.ws_ml[prow * 2] = m;
          p.ws_ml[prow * 2 + 1] = l;
        }
        for (int c = oc_lo; c < oc_hi; ++c) {
          uint32_t o[16];
          if (ok && it.n_kv > 0) {
            tmem_ld16(tO + lane_off + c * 16, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = 0;
          }
          if (row_ok) {
            const int col = c * 16;
            for (int i = 0; i < 16 && col + i < p.d; i += 4)
              *reinterpret_cast<float4*>(po + col + i) = make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]),
                                                                     __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
          }
        }
        tc_fence_before();
        continue;
      }
      __nv_bfloat16* orow = p.O + (long long)(it.q_beg + qi) * p.ldo + (long long)(it.hq0 + g) * p.d;
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      for (int c = oc_lo; c < oc_hi; ++c) {
        uint32_t o[16];
        if (ok && it.n_kv > 0) {
          tmem_ld16(tO + lane_off + c * 16, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0;
        }
        if (row_ok) {
          const int col = c * 16;
          if (col + 16 <= p.d) {
            uint4 w0, w1;
            w0.x = pack_bf16x2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
            w0.y = pack_bf16x2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
            w0.z = pack_bf16x2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
            w0.w = pack_bf16x2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
            w1.x = pack_bf16x2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
            w1.y = pack_bf16x2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
            w1.z = pack_bf16x2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
            w1.w = pack_bf16x2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
            uint4* dst = reinterpret_cast<uint4*>(orow + col);
            dst[0] = w0; dst[1] = w1;
          } else {
            for (int i = 0; i < 16 && col + i < p.d; ++i)
              orow[col + i] = __float2bfloat16(__uint_as_float(o[i]) * inv);
          }
        }
      }
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Merge the split-KV partials of one (token, head) row: one warp per row.
__global__ void attn_combine_kernel(const float* ws_o, const float* ws_ml, __nv_bfloat16* O, long long ldo,
                                    int rows, int Hq, int d, int splits) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mmax = -INFINITY;
  for (int s = 0; s < splits; ++s) mmax = fmaxf(mmax, ws_ml[((long long)row * splits + s) * 2]);
  float lsum = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const long long pr = (long long)row * splits + s;
    const float ms = ws_ml[pr * 2], ls = ws_ml[pr * 2 + 1];
    if (ls <= 0.f) continue;
    const float sc = exp2f(ms - mmax);
    lsum += ls * sc;
    if (lane * 4 < d) {
      const float4 v = *reinterpret_cast<const float4*>(ws_o + pr * d + lane * 4);
      acc[0] += v.x * sc; acc[1] += v.y * sc; acc[2] += v.z * sc; acc[3] += v.w * sc;
    }
  }
  if (lane * 4 < d) {
    const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
    const int t = row / Hq, h = row % Hq;
    __nv_bfloat16* o = O + (long long)t * ldo + (long long)h * d + lane * 4;
    *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
  }
}

}  // namespace

int cs_encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// q: [Tq, Hq, d] view with token stride ldq (elements).  Contiguous mode: k, v: [Tk, Hkv, d] views with
// token strides ldk / ldv and packed offsets cu_k.  Paged mode (block_table != null): `k` is the cache
// [pages, 2, Hkv, 128, d] (v ignored), kv_len gives the key count per sequence.
// pack_gqa != 0 packs the Hq/Hkv query heads of one KV head into the rows of a tile (use for decode).
// window > 0 (causal only) restricts every query to the last `window` keys up to and including its own position.
// kv_splits > 1 divides the key tiles of every item over that many CTAs (flash-decoding); `ws` must then hold
// Tq*Hq*kv_splits*(d+2) floats of scratch.  Calls sharing `ws` must be ordered on one stream.
CS_API int cs_attention(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                        void* o, long long ldo, const void* cu_q, const void* cu_k, const void* kv_len,
                        const void* block_table, int bt_stride, int num_pages, int B, int Tq, int Tk,
                        int max_q_len, int Hq, int Hkv, int d, float scale, int causal, int pack_gqa,
                        int kv_splits, void* ws, long long ws_bytes, int window, const void* seg_lo, const void* seg_hi,
                        void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0 || Tq <= 0) return 0;
  if (d > 128 || (d & 7) || Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int paged = block_table != nullptr;
  const int G = pack_gqa ? Hq / Hkv : 1;
  if (G > 128) return -1;
  const int tok_per_tile = 128 / G;
  AttnParams p{};
  p.O = (__nv_bfloat16*)o; p.ldo = ldo;
  p.cu_q = (const int*)cu_q; p.cu_k = (const int*)cu_k; p.kv_len = (const int*)kv_len;
  p.block_table = (const int*)block_table; p.bt_stride = bt_stride;
  p.Hq = Hq; p.Hkv = Hkv; p.d = d; p.G = G; p.causal = causal; p.paged = paged;
  p.window = (window > 0 && causal) ? window : 0;
  p.seg_lo = reinterpret_cast<const int*>(seg_lo);
  p.seg_hi = reinterpret_cast<const int*>(seg_hi);
  if ((p.seg_lo == nullptr) != (p.seg_hi == nullptr) || (p.seg_lo != nullptr && (paged || pack_gqa))) return -1;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int dpad = (d + 15) & ~15;
  p.idesc_s = umma_idesc_bf16(128, 128, 0, 0);
  p.idesc_pv = umma_idesc_bf16(128, dpad, 0, 1);
  p.err = cs_error_word();

  CUtensorMap tmQ, tmK, tmV;
  if (cs_encode_tmap_3d(&tmQ, q, d, Hq, Tq, (uint64_t)d * 2, (uint64_t)ldq * 2, 64, G, tok_per_tile)) return -2;
  if (paged) {
    const uint64_t rows = (uint64_t)num_pages * 2 * Hkv;
    if (cs_encode_tmap_3d(&tmK, k, d, 128, rows, (uint64_t)d * 2, (uint64_t)128 * d * 2, 64, 128, 1)) return -3;
    tmV = tmK;
  } else {
    if (cs_encode_tmap_3d(&tmK, k, d, Hkv, Tk, (uint64_t)d * 2, (uint64_t)ldk * 2, 64, 1, 128)) return -3;
    if (cs_encode_tmap_3d(&tmV, v, d, Hkv, Tk, (uint64_t)d * 2, (uint64_t)ldv * 2, 64, 1, 128)) return -4;
  }
  const int smem = (2 + 2 + 2 * KV_STAGES * 2) * ATOM_BYTES + 1024;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev] = true;
  }
  p.max_q_tiles = (max_q_len + tok_per_tile - 1) / tok_per_tile;
  p.head_blks = pack_gqa ? Hkv : Hq;
  if (kv_splits < 1) kv_splits = 1;
  if (kv_splits > 1) {
    // scratch: partial outputs then (max, normaliser) pairs
    const long long rows = static_cast<long long>(Tq) * Hq * kv_splits;
    const long long need = rows * d * 4 + rows * 8;
    if (ws == nullptr || need > ws_bytes || (d & 3)) return -5;
    p.ws_o = reinterpret_cast<float*>(ws);
    p.ws_ml = p.ws_o + rows * d;
  }
  p.kv_splits = kv_splits;
  const long long total = static_cast<long long>(p.max_q_tiles) * p.head_blks * B * kv_splits;
  if (total <= 0 || total > 0x7fffffffLL) return -1;
  p.total_items = static_cast<int>(total);
  const int grid = p.total_items < cs_num_sms() ? p.total_items : cs_num_sms();
  if (p.window > 0 || p.seg_lo != nullptr) attn_kernel<true><<<grid, 320, smem, stream>>>(tmQ, tmK, tmV, p);
  else attn_kernel<false><<<grid, 320, smem, stream>>>(tmQ, tmK, tmV, p);
  if (kv_splits > 1) {
    const int rows = Tq * Hq;
    attn_combine_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(p.ws_o, p.ws_ml, p.O, ldo, rows, Hq, d, kv_splits);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
