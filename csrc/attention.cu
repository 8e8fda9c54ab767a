// Variable-length attention for sm_100a (tcgen05 + TMEM + TMA), one kernel for:
//   * packed var-len self attention without mask (vision towers, windows and full images, DiT)
//   * causal prefill over a paged KV cache (LLM), with grouped-query heads
//   * decode over a paged KV cache: the G query heads that share a KV head are packed into the
//     rows of one tile, so K/V pages are read once per KV head
//
// One CTA = one tile of up to 128 query rows of one sequence and one (group of) head(s).
//   warps 0-3 : softmax; thread r owns query row r = TMEM lane r (no shuffles needed)
//   warp 4    : TMA producer (Q once, then a 2-deep ring of K and V tiles of 128 keys)
//   warp 5    : issues tcgen05.mma:  S_j = Q K_j^T  (two S buffers in TMEM, so S_{j+1} is computed
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
  float scale_log2;
  uint32_t idesc_s, idesc_pv;
  int* err;
};

__global__ void __launch_bounds__(192, 1)
attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
            const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  const int seq = blockIdx.z;
  const int head_blk = blockIdx.y;  // kv-head index when G > 1, else query head
  const int q_beg = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_beg;
  const int tok_per_tile = 128 / p.G;
  const int t0 = blockIdx.x * tok_per_tile;  // first query token (within the sequence) of this tile
  if (t0 >= q_len) return;
  const int k_beg = p.paged ? 0 : p.cu_k[seq];
  const int k_len = p.paged ? p.kv_len[seq] : (p.cu_k[seq + 1] - k_beg);
  const int hk = p.G > 1 ? head_blk : head_blk / (p.Hq / p.Hkv);
  const int hq0 = p.G > 1 ? head_blk * p.G : head_blk;
  const int n_tok = min(tok_per_tile, q_len - t0);
  // causal: query token i sees keys j <= i + (k_len - q_len)
  const int shift = k_len - q_len;
  int k_end = k_len;
  if (p.causal) k_end = min(k_len, t0 + n_tok + shift);
  const int n_kv = k_end > 0 ? (k_end + KV_TILE - 1) / KV_TILE : 0;

  const int n_atoms = (p.d + 63) / 64;
  const int d16 = (p.d + 15) / 16;  // 16-column groups in O, and K-steps of Q K^T

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                // n_atoms * 16 KB
  uint8_t* sP = sQ + 2 * ATOM_BYTES;                 // 2 atoms (128 keys)
  uint8_t* sK = sP + 2 * ATOM_BYTES;                 // KV_STAGES * n_atoms * 16 KB (sized for 2 atoms)
  uint8_t* sV = sK + KV_STAGES * 2 * ATOM_BYTES;
  __shared__ uint64_t q_full, k_full[KV_STAGES], v_full[KV_STAGES], k_empty[KV_STAGES], v_empty[KV_STAGES];
  __shared__ uint64_t s_full[2], p_full, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&p_full, 128);
    mbar_init(&o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 5) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 256;
  volatile int* abortp = &abort_flag;

  if (warp == 4) {
    if (lane == 0 && n_kv > 0) {
      // ------------------------------- TMA producer -------------------------------
      mbar_arrive_expect_tx(&q_full, static_cast<uint32_t>(n_atoms * p.G * tok_per_tile * 128));
      for (int a = 0; a < n_atoms; ++a)
        tma_load_3d(sQ + a * ATOM_BYTES, &tmQ, a * 64, hq0, q_beg + t0, &q_full);
      int stage = 0; uint32_t phase = 0;
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait(&k_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) break;
        mbar_arrive_expect_tx(&k_full[stage], static_cast<uint32_t>(n_atoms * ATOM_BYTES));
        int page = 0;
        if (p.paged) page = p.block_table[(long long)seq * p.bt_stride + j];
        for (int a = 0; a < n_atoms; ++a) {
          uint8_t* dst = sK + (stage * 2 + a) * ATOM_BYTES;
          if (p.paged) tma_load_3d(dst, &tmK, a * 64, 0, (page * 2 + 0) * p.Hkv + hk, &k_full[stage]);
          else tma_load_3d(dst, &tmK, a * 64, hk, k_beg + j * KV_TILE, &k_full[stage]);
        }
        if (!mbar_wait(&v_empty[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) break;
        mbar_arrive_expect_tx(&v_full[stage], static_cast<uint32_t>(n_atoms * ATOM_BYTES));
        for (int a = 0; a < n_atoms; ++a) {
          uint8_t* dst = sV + (stage * 2 + a) * ATOM_BYTES;
          if (p.paged) tma_load_3d(dst, &tmV, a * 64, 0, (page * 2 + 1) * p.Hkv + hk, &v_full[stage]);
          else tma_load_3d(dst, &tmV, a * 64, hk, k_beg + j * KV_TILE, &v_full[stage]);
        }
        if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && n_kv > 0) {
      // -------------------------------- MMA issuer --------------------------------
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(&q_full, 0, abortp, p.err, CS_ERR_TIMEOUT_TMA);
      auto issue_s = [&](int j) -> bool {
        const int stage = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&k_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + stage * 2 * ATOM_BYTES);
        for (int kk = 0; kk < d16; ++kk) {
          const uint32_t off = (kk >> 2) * ATOM_BYTES + (kk & 3) * 32;
          umma_f16_ss(tS0 + (j & 1) * 128, umma_smem_desc(q_addr + off, 16, 1024),
                      umma_smem_desc(k_addr + off, 16, 1024), p.idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { if (!issue_s(j + 1)) break; }
        const int stage = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&p_full, j & 1, abortp, p.err, CS_ERR_TIMEOUT_EPI)) break;
        if (!mbar_wait(&v_full[stage], ph, abortp, p.err, CS_ERR_TIMEOUT_TMA)) break;
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
      }
    }
  } else {
    // ---------------------------------- softmax -----------------------------------
    const int r = threadIdx.x;                 // tile row == TMEM lane
    const int tl = r / p.G, g = r - tl * p.G;  // token in tile, head within group
    const bool row_ok = tl < n_tok;
    const int qi = t0 + tl;
    const int lim = p.causal ? min(k_len, qi + shift + 1) : k_len;  // keys [0, lim) are visible
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    uint8_t* p_row = sP + r * 128;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = tS0 + (j & 1) * 128 + lane_off;
      const int kbase = j * KV_TILE;
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tS + c * 32, v);
        tmem_wait_ld();
        const int nvalid = lim - (kbase + c * 32);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < nvalid) mx = fmaxf(mx, __uint_as_float(v[i]));
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m - m_use);  // m = -inf -> 0
      // pass 2: probabilities, packed to bf16
      uint32_t pk[64];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tS + c * 32, v);
        tmem_wait_ld();
        const int nvalid = lim - (kbase + c * 32);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = (i < nvalid) ? exp2f(__uint_as_float(v[i]) * p.scale_log2 - m_use) : 0.f;
          float e1 = (i + 1 < nvalid) ? exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - m_use) : 0.f;
          const uint32_t w = pack_bf16x2(e0, e1);
          // accumulate the rounded values so that the normaliser matches what the MMA sums
          sum += bf16lo(w) + bf16hi(w);
          pk[c * 16 + (i >> 1)] = w;
        }
      }
      l = l * alpha + sum;
      m = m_new;
      tc_fence_before();
      if (j > 0) {
        if (!mbar_wait(&o_full, (j - 1) & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
      }
      // P -> shared memory, K-major with the 128-byte swizzle (16-byte chunk index XOR row%8)
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const int atom = ch >> 3, cc = ch & 7;
        uint4 w = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(p_row + atom * ATOM_BYTES + ((cc ^ (r & 7)) << 4)) = w;
      }
      // tcgen05.ld/st are warp-collective: decide by vote whether this warp rescales O
      const bool need = __any_sync(0xffffffffu, j > 0 && alpha != 1.0f);
      if (need) {
        for (int c = 0; c < d16; ++c) {
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
    if (ok && n_kv > 0) ok = mbar_wait(&o_full, (n_kv - 1) & 1, abortp, p.err, CS_ERR_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    __nv_bfloat16* orow = p.O + (long long)(q_beg + qi) * p.ldo + (long long)(hq0 + g) * p.d;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int c = 0; c < d16; ++c) {
      uint32_t o[16];
      if (ok && n_kv > 0) {
        tmem_ld16(tO + lane_off + c * 16, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0;
      }
      if (row_ok && g < p.G) {
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace

int cs_encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// q: [Tq, Hq, d] view with token stride ldq (elements).  Contiguous mode: k, v: [Tk, Hkv, d] views with
// token strides ldk / ldv and packed offsets cu_k.  Paged mode (block_table != null): `k` is the cache
// [pages, 2, Hkv, 128, d] (v ignored), kv_len gives the key count per sequence.
// pack_gqa != 0 packs the Hq/Hkv query heads of one KV head into the rows of a tile (use for decode).
CS_API int cs_attention(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                        void* o, long long ldo, const void* cu_q, const void* cu_k, const void* kv_len,
                        const void* block_table, int bt_stride, int num_pages, int B, int Tq, int Tk,
                        int max_q_len, int Hq, int Hkv, int d, float scale, int causal, int pack_gqa,
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
    cudaFuncSetAttribute(attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev] = true;
  }
  dim3 grid((max_q_len + tok_per_tile - 1) / tok_per_tile, pack_gqa ? Hkv : Hq, B);
  attn_kernel<<<grid, 192, smem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
