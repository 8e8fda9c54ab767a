// Decode attention over a paged KV cache for sm_100a: one new query token per sequence, grouped-query heads.
//
// The general kernel (attention.cu) puts queries on the 128-row side of the tcgen05 tile; at decode time only
// the G query heads that share a KV head are real rows, so it spends a full 128 x 128 x d MMA pair and a
// 128-row softmax per 128 keys.  Here the operands are swapped: the 128 KEYS of a cache page are the M side and
// the G <= 16 query heads the N side,
//
//     S^T [128 keys x 16]  = K_page [128 x d] . Q^T [d x 16]
//     O^T [d = 128 x 16]  += V_page^T [128 x 128 keys] . P [128 keys x 16]
//
// which cuts tensor time and softmax work per page by 8x and leaves shared memory for a three-page K/V ring.
//   warps 0-3 : softmax; thread t owns key t of the page (= TMEM lane t of S^T) and output channel t of O^T
//   warp 4    : TMA producer (Q once per item, then K and V pages through a ring)
//   warp 5    : tcgen05.mma issuer
// The soft-max runs over TMEM lanes: per query head the page maximum is a warp reduction plus a 4-entry exchange
// through shared memory; normalisers stay per thread until the end of the item.  Requires head_dim == 128.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int PAGE = 128;
constexpr int NQ = 16;                 // query heads per tile (padded)
constexpr int RING = 3;                // K/V pages in flight
constexpr int KV_ATOM = 128 * 128;     // 128 keys x 64 bf16
constexpr int QP_ATOM = NQ * 128;      // 16 rows x 64 bf16

struct DecParams {
  __nv_bfloat16* O; long long ldo;     // [B, Hq, d] with token stride ldo
  const int* kv_len;                   // [B]
  const int* block_table; int bt_stride;
  int B, Hq, Hkv, G;
  int kv_splits, total_items;
  float* ws_o;                         // [B*Hq, kv_splits, 128] unnormalised partial outputs
  float* ws_ml;                        // [B*Hq, kv_splits, 2]  (running max in base-2 units, normaliser)
  float scale_log2;
  uint32_t idesc_s, idesc_pv;
  int* err;
};

struct DItem { int seq, hk, split, k_len, j0, n_kv; };

__device__ __forceinline__ DItem dec_item(const DecParams& p, int w) {
  DItem it;
  it.split = w % p.kv_splits;
  w /= p.kv_splits;
  it.hk = w % p.Hkv;
  it.seq = w / p.Hkv;
  it.k_len = p.kv_len[it.seq];
  const int n_all = (it.k_len + PAGE - 1) / PAGE;
  it.j0 = static_cast<int>((static_cast<long long>(it.split) * n_all) / p.kv_splits);
  it.n_kv = static_cast<int>((static_cast<long long>(it.split + 1) * n_all) / p.kv_splits) - it.j0;
  return it;
}

// order-preserving float -> int so that the integer warp reduction gives the float maximum
__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 8) tmem_ld8(taddr, r); else tmem_ld16(taddr, r);
}
template <int N>
__device__ __forceinline__ void tmem_stn(uint32_t taddr, const uint32_t (&r)[N]) {
  if constexpr (N == 8) tmem_st8(taddr, r); else tmem_st16(taddr, r);
}

// NG = query heads the softmax looks at (8 or 16): the MMAs always produce 16 columns, columns >= NG belong to
// other KV heads' queries (or to zero fill) and are never read.
template <int NG>
__global__ void __launch_bounds__(192, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, const DecParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // 2 atoms of 16 rows
  uint8_t* sP = sQ + 2 * QP_ATOM;           // 2 atoms of 16 rows (64 keys each)
  uint8_t* sK = sP + 2 * QP_ATOM;           // RING pages, 2 atoms each
  uint8_t* sV = sK + RING * 2 * KV_ATOM;
  __shared__ uint64_t q_full, q_empty, k_full[RING], v_full[RING], k_empty[RING], v_empty[RING];
  __shared__ uint64_t s_full[2], p_full, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float wmax[2][4][NQ];   // per-warp page maxima, double-buffered by page parity
  __shared__ __align__(16) float wsum[4][NQ];      // per-warp normalisers at the end of an item

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&p_full, 128);
    mbar_init(&o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmKV);
  }
  if (warp == 5) { tmem_alloc(&tmem_slot, 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // barriers and TMEM were set up while the kernel ahead in the stream may still have been running; its results
  // (queries, the cache rows of this step) are read from here on
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 64;  // S^T buffers at columns 0 and 32, O^T at column 64
  volatile int* abortp = &abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------- TMA producer -------------------------------
      uint32_t n_item = 0, n_page = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_items && ok; w += gridDim.x) {
        const DItem it = dec_item(p, w);
        if (it.n_kv == 0) continue;
        if (!mbar_wait(&q_empty, (n_item & 1) ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) break;
        mbar_arrive_expect_tx(&q_full, 2 * QP_ATOM);
        tma_load_3d(sQ, &tmQ, 0, it.hk * p.G, it.seq, &q_full);
        tma_load_3d(sQ + QP_ATOM, &tmQ, 64, it.hk * p.G, it.seq, &q_full);
        ++n_item;
        int page_next = p.block_table[(long long)it.seq * p.bt_stride + it.j0];
        for (int jj = 0; jj < it.n_kv; ++jj, ++n_page) {
          const int page = page_next;
          if (jj + 1 < it.n_kv) page_next = p.block_table[(long long)it.seq * p.bt_stride + it.j0 + jj + 1];  // prefetch
          const int stage = n_page % RING;
          const uint32_t phase = (n_page / RING) & 1;
          if (!mbar_wait(&k_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[stage], 2 * KV_ATOM);
          tma_load_3d(sK + (stage * 2) * KV_ATOM, &tmKV, 0, 0, (page * 2 + 0) * p.Hkv + it.hk, &k_full[stage]);
          tma_load_3d(sK + (stage * 2 + 1) * KV_ATOM, &tmKV, 64, 0, (page * 2 + 0) * p.Hkv + it.hk, &k_full[stage]);
          if (!mbar_wait(&v_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[stage], 2 * KV_ATOM);
          tma_load_3d(sV + (stage * 2) * KV_ATOM, &tmKV, 0, 0, (page * 2 + 1) * p.Hkv + it.hk, &v_full[stage]);
          tma_load_3d(sV + (stage * 2 + 1) * KV_ATOM, &tmKV, 64, 0, (page * 2 + 1) * p.Hkv + it.hk, &v_full[stage]);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // -------------------------------- MMA issuer --------------------------------
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      uint32_t n_item = 0, n_s = 0, n_pv = 0;
      bool ok = true;
      auto issue_s = [&](bool last_of_item) -> bool {
        const int stage = n_s % RING;
        const uint32_t ph = (n_s / RING) & 1;
        if (!mbar_wait(&k_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + stage * 2 * KV_ATOM);
        for (int kk = 0; kk < 8; ++kk) {  // 8 x 16 channels
          umma_f16_ss(tS0 + (n_s & 1) * 32, umma_smem_desc(k_addr + (kk >> 2) * KV_ATOM + (kk & 3) * 32, 16, 1024),
                      umma_smem_desc(q_addr + (kk >> 2) * QP_ATOM + (kk & 3) * 32, 16, 1024), p.idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);
        if (last_of_item) umma_commit(&q_empty);
        umma_commit(&s_full[n_s & 1]);
        ++n_s;
        return true;
      };
      for (int w = blockIdx.x; w < p.total_items && ok; w += gridDim.x) {
        const DItem it = dec_item(p, w);
        if (it.n_kv == 0) continue;
        if (!mbar_wait(&q_full, n_item & 1, abortp, p.err, CS_ERR_TIMEOUT_TMA)) break;
        ++n_item;
        if (!issue_s(it.n_kv == 1)) break;
        for (int j = 0; j < it.n_kv; ++j) {
          if (j + 1 < it.n_kv) { if (!issue_s(j + 2 == it.n_kv)) { ok = false; break; } }
          const int stage = n_pv % RING;
          const uint32_t ph = (n_pv / RING) & 1;
          if (!mbar_wait(&p_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_EPI)) { ok = false; break; }
          if (!mbar_wait(&v_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sV + stage * 2 * KV_ATOM);
          for (int kk = 0; kk < 8; ++kk) {  // 8 x 16 keys
            // A = V^T: channels are the M index and contiguous in memory (MN-major): 16 keys = two 8-row groups
            // 1024 B apart, the second 64 channels one atom further.  B = P: [16 heads x 128 keys], K-major.
            umma_f16_ss(tO, umma_smem_desc(v_addr + kk * 2048, KV_ATOM, 1024),
                        umma_smem_desc(p_addr + (kk >> 2) * QP_ATOM + (kk & 3) * 32, 16, 1024), p.idesc_pv,
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
    const int t = threadIdx.x;                                  // key within the page / output channel
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t n_s = 0, n_pv = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total_items; w += gridDim.x) {
      const DItem it = dec_item(p, w);
      float m_run[NG], l_thr[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) { m_run[g] = -INFINITY; l_thr[g] = 0.f; }
      for (int j = 0; j < it.n_kv; ++j) {
        if (!mbar_wait(&s_full[n_s & 1], (n_s >> 1) & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) ok = false;
        tc_fence_after();
        uint32_t v[NG];
        tmem_ldn<NG>(tS0 + (n_s & 1) * 32 + lane_off, v);
        tmem_wait_ld();
        ++n_s;
        const bool valid = (it.j0 + j) * PAGE + t < it.k_len;
        float s[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) s[g] = valid ? __uint_as_float(v[g]) * p.scale_log2 : -INFINITY;
        // page maximum per head: integer warp reduction, then the four warps exchange through shared memory
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const int mx = __reduce_max_sync(0xffffffffu, f2ord(s[g]));
          if (lane == g) wmax[j & 1][warp][g] = ord2f(mx);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        float alpha[NG];
        bool rescale = false;
        uint32_t pk[NG / 2];
#pragma unroll
        for (int g4 = 0; g4 < NG / 4; ++g4) {
          float4 a = *reinterpret_cast<const float4*>(&wmax[j & 1][0][g4 * 4]);
#pragma unroll
          for (int ww = 1; ww < 4; ++ww) {
            const float4 b = *reinterpret_cast<const float4*>(&wmax[j & 1][ww][g4 * 4]);
            a.x = fmaxf(a.x, b.x); a.y = fmaxf(a.y, b.y); a.z = fmaxf(a.z, b.z); a.w = fmaxf(a.w, b.w);
          }
          const float mt[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int g = g4 * 4 + i;
            const float m_new = fmaxf(m_run[g], mt[i]);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[g] = exp2f(m_run[g] - m_use);   // m_run = -inf -> 0
            rescale |= (alpha[g] != 1.0f);
            const float e = exp2f(s[g] - m_use);   // s = -inf -> 0
            const __nv_bfloat16 eb = __float2bfloat16(e);
            // accumulate the rounded value so that the normaliser matches what the MMA sums
            l_thr[g] = l_thr[g] * alpha[g] + __bfloat162float(eb);
            m_run[g] = m_new;
            const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(eb));
            if (i & 1) pk[g >> 1] |= bits << 16; else pk[g >> 1] = bits;
          }
        }
        tc_fence_before();
        if (j > 0) {
          // PV of the previous page must be finished: P buffer free, O^T up to date
          if (!mbar_wait(&o_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) ok = false;
          ++n_pv;
          tc_fence_after();
        }
        // P[g][key] -> shared memory, K-major rows of 64 keys with the 128-byte swizzle
        {
          uint8_t* atom = sP + (t >> 6) * QP_ATOM;
          const int kc = t & 63;
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            const uint32_t bits = (g & 1) ? (pk[g >> 1] >> 16) : (pk[g >> 1] & 0xffffu);
            uint8_t* dst = atom + (g >> 3) * 1024 + (g & 7) * 128 + (((kc >> 3) ^ (g & 7)) << 4) + (kc & 7) * 2;
            *reinterpret_cast<unsigned short*>(dst) = static_cast<unsigned short>(bits);
          }
        }
        // alpha is the same in every thread (the maxima are global), so the decision is uniform
        if (j > 0 && rescale) {
          uint32_t o[NG];
          tmem_ldn<NG>(tO + lane_off, o);
          tmem_wait_ld();
#pragma unroll
          for (int g = 0; g < NG; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
          tmem_stn<NG>(tO + lane_off, o);
          tmem_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full);
      }
      // ---------------------------------- write O ------------------------------------
      if (it.n_kv > 0) {
        if (!mbar_wait(&o_full, n_pv & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) ok = false;
        ++n_pv;
      }
      tc_fence_after();
      // normalisers: sum the per-thread parts over the 128 threads
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float sg = l_thr[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, o);
        if (lane == g) wsum[warp][g] = sg;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      uint32_t o[NG];
      if (ok && it.n_kv > 0) {
        tmem_ldn<NG>(tO + lane_off, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int g = 0; g < NG; ++g) o[g] = 0;
      }
      const long long row0 = (long long)it.seq * p.Hq + (long long)it.hk * p.G;  // first (token, head) row of the item
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        if (g < p.G) {
          const float l = wsum[0][g] + wsum[1][g] + wsum[2][g] + wsum[3][g];
          if (p.kv_splits > 1) {
            const long long prow = (row0 + g) * p.kv_splits + it.split;
            p.ws_o[prow * 128 + t] = __uint_as_float(o[g]);
            if (t == 0) { p.ws_ml[prow * 2] = m_run[g]; p.ws_ml[prow * 2 + 1] = l; }
          } else {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            p.O[(long long)it.seq * p.ldo + ((long long)it.hk * p.G + g) * 128 + t] = __float2bfloat16(__uint_as_float(o[g]) * inv);
          }
        }
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");  // wsum / wmax are reused by the next item
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem, 128); }
}

// Merge the split-KV partials of one (token, head) row: one warp per row, d = 128.
__global__ void attn_decode_combine_kernel(const float* ws_o, const float* ws_ml, __nv_bfloat16* O, long long ldo,
                                           int rows, int Hq, int splits) {
  pdl_wait();
  pdl_launch_dependents();
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
    const float4 v = *reinterpret_cast<const float4*>(ws_o + pr * 128 + lane * 4);
    acc[0] += v.x * sc; acc[1] += v.y * sc; acc[2] += v.z * sc; acc[3] += v.w * sc;
  }
  const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
  const int tok = row / Hq, h = row % Hq;
  __nv_bfloat16* o = O + (long long)tok * ldo + (long long)h * 128 + lane * 4;
  *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
}

}  // namespace

int cs_encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// Decode attention: q [B, Hq, 128] (token stride ldq), one query token per sequence; cache [pages, 2, Hkv, 128, 128];
// kv_len[b] keys are visible to sequence b (including the token just appended).  Hq / Hkv <= 16.
// kv_splits > 1 spreads the pages of a sequence over that many work items; `ws` must then hold
// B*Hq*kv_splits*130 floats.  Calls sharing `ws` must be ordered on one stream.
CS_API int cs_attention_decode(const void* q, long long ldq, const void* cache, void* o, long long ldo, const void* kv_len,
                               const void* block_table, int bt_stride, int num_pages, int B, int Hq, int Hkv, float scale,
                               int kv_splits, void* ws, long long ws_bytes, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > NQ) return -1;
  DecParams p{};
  p.O = (__nv_bfloat16*)o; p.ldo = ldo;
  p.kv_len = (const int*)kv_len;
  p.block_table = (const int*)block_table; p.bt_stride = bt_stride;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.idesc_s = umma_idesc_bf16(128, NQ, 0, 0);
  p.idesc_pv = umma_idesc_bf16(128, NQ, 1, 0);
  p.err = cs_error_word();
  if (kv_splits < 1) kv_splits = 1;
  if (kv_splits > 1) {
    const long long rows = static_cast<long long>(B) * Hq * kv_splits;
    if (ws == nullptr || rows * 130 * 4 > ws_bytes) return -5;
    p.ws_o = reinterpret_cast<float*>(ws);
    p.ws_ml = p.ws_o + rows * 128;
  }
  p.kv_splits = kv_splits;
  const long long total = static_cast<long long>(B) * Hkv * kv_splits;
  if (total > 0x7fffffffLL) return -1;
  p.total_items = static_cast<int>(total);
  CUtensorMap tmQ, tmKV;
  if (cs_encode_tmap_3d(&tmQ, q, 128, Hq, B, 256, (uint64_t)ldq * 2, 64, NQ, 1)) return -2;
  if (cs_encode_tmap_3d(&tmKV, cache, 128, 128, (uint64_t)num_pages * 2 * Hkv, 256, (uint64_t)128 * 256, 64, 128, 1)) return -3;
  const int smem = 4 * QP_ATOM + 2 * RING * 2 * KV_ATOM + 1024;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(attn_decode_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(attn_decode_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev] = true;
  }
  const int grid = p.total_items < cs_num_sms() ? p.total_items : cs_num_sms();
  if (p.G <= 8) cs_launch_pdl(attn_decode_kernel<8>, dim3(grid), dim3(192), smem, stream, tmQ, tmKV, p);
  else cs_launch_pdl(attn_decode_kernel<16>, dim3(grid), dim3(192), smem, stream, tmQ, tmKV, p);
  if (kv_splits > 1) {
    const int rows = B * Hq;
    cs_launch_pdl(attn_decode_combine_kernel, dim3((rows + 7) / 8), dim3(256), 0, stream, p.ws_o, p.ws_ml, p.O, ldo, rows, Hq,
                  kv_splits);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
