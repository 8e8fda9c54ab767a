// fp8 (e4m3) GEMM with block scales for sm_100a:   C[M,N] = sum_kb  sa[kb][m] * sw[n/128][kb] * (Aq[m, kb] . Wq[n, kb])
//
//   Aq [M, K] e4m3, one fp32 scale per row and 128-wide K block (sa, stored [K/128][M] so that rows coalesce)
//   Wq [N, K] e4m3, one fp32 scale per 128 x 128 block            (sw, stored [ceil(N/128)][K/128])
//
// The tensor core accumulates in fp32 inside one 128-wide K block only (tcgen05.mma kind::f8f6f4, four K=32
// instructions per block) into one of two TMEM buffers; the epilogue warps read that partial product, multiply it
// by the block's scale pair and add it to the running sum they keep in registers (one output row per thread, 128
// columns), while the tensor core already works on the next K block in the other buffer.  So the scaling costs no
// extra pass over memory and the sum over K blocks is exact fp32.
//
//   warp 0 (one lane): TMA producer, ring of (A, W) K blocks: 128 rows x 128 bytes each, 128-byte swizzle
//   warp 1 (one lane): MMA issuer
//   warps 2..9       : scale-and-accumulate, then bias / bf16 store; warp w works on TMEM lanes (w % 4) * 32 .. + 31
//                      (32 output rows) and on the column half (w - 2) / 4 of the tile, so that two warps share the
//                      reads and multiply-adds of every row quarter
//
// Also here: the row-wise quantiser that produces Aq and sa from bf16 activations.
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_STAGE_BYTES = (F8_BM + F8_BN) * F8_BK;  // 32 KiB
constexpr int F8_MAX_STAGES = 6;

struct Fp8Params {
  int M, N, K;
  __nv_bfloat16* C; long long ldc;
  const float* sa; long long ld_sa;   // [K/128][ld_sa >= M]
  const float* sw; int kb_total;      // [tiles_n][kb_total]
  const __nv_bfloat16* bias;
  int stages;
  uint32_t idesc;
  int* err;
};

// kind::f8f6f4, A and B e4m3 (format 0), fp32 accumulate, both operands K-major
__host__ __device__ inline uint32_t umma_idesc_e4m3(uint32_t m, uint32_t n) {
  uint32_t d = 0;
  d |= 1u << 4;                   // D format fp32
  d |= ((n >> 3) & 0x3f) << 17;
  d |= ((m >> 4) & 0x1f) << 24;
  return d;
}

__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(320, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[F8_MAX_STAGES], empty_bar[F8_MAX_STAGES];
  __shared__ uint64_t part_full[2], part_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + F8_BM - 1) / F8_BM, tiles_n = (p.N + F8_BN - 1) / F8_BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = p.K / F8_BK;
  const int stages = p.stages;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&part_full[b], 1); mbar_init(&part_empty[b], 8); }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 2 * F8_BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tm = t % tiles_m, tn = t / tiles_m;   // neighbouring CTAs share the W tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp, p.err, CS_ERR_TIMEOUT_SLOT)) { ok = false; break; }
          uint8_t* sA = smem + stage * F8_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], F8_STAGE_BYTES);
          tma_load_2d(sA, &tmA, kb * F8_BK, tm * F8_BM, &full_bar[stage]);
          tma_load_2d(sA + F8_BM * F8_BK, &tmB, kb * F8_BK, tn * F8_BN, &full_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      uint32_t g = 0;   // K blocks issued so far: buffer g & 1, use number g >> 1
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const uint32_t buf = g & 1u;
          if (!mbar_wait(&part_empty[buf], ((g >> 1) & 1u) ^ 1u, abortp, p.err, CS_ERR_TIMEOUT_EPI)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abortp, p.err, CS_ERR_TIMEOUT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * F8_STAGE_BYTES);
          const uint32_t b_addr = a_addr + F8_BM * F8_BK;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)   // K = 32 elements (32 bytes) per instruction
            umma_f8_ss(tmem + buf * F8_BN, umma_smem_desc(a_addr + k * 32, 16, 1024), umma_smem_desc(b_addr + k * 32, 16, 1024),
                       p.idesc, k != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[buf]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;            // which 64 columns of the tile
    constexpr int HC = F8_BN / 2;
    uint32_t g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int tm = t % tiles_m, tn = t / tiles_m;
      const int row = tm * F8_BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      float acc[HC];
#pragma unroll
      for (int j = 0; j < HC; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++g) {
        const uint32_t buf = g & 1u;
        const float s = (row_ok ? __ldg(p.sa + static_cast<long long>(kb) * p.ld_sa + row) : 0.f) *
                        __ldg(p.sw + static_cast<long long>(tn) * p.kb_total + kb);
        if (!mbar_wait(&part_full[buf], (g >> 1) & 1u, abortp, p.err, CS_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_row = tmem + buf * F8_BN + half * HC + (static_cast<uint32_t>(q * 32) << 16);
        uint32_t v0[32], v1[32];
        tmem_ld32(t_row, v0);
        tmem_ld32(t_row + 32, v1);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[buf]);   // the values are in registers: the buffer may be overwritten
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(s, __uint_as_float(v0[j]), acc[j]);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(s, __uint_as_float(v1[j]), acc[32 + j]);
      }
      if (!ok) break;
      if (row_ok) {
        const int n0 = tn * F8_BN + half * HC;
        __nv_bfloat16* out = p.C + static_cast<long long>(row) * p.ldc + n0;
        const bool vec = (n0 + HC <= p.N) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll
        for (int j8 = 0; j8 < HC / 8; ++j8) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = n0 + j8 * 8 + j;
            f[j] = acc[j8 * 8 + j] + ((p.bias != nullptr && col < p.N) ? __bfloat162float(p.bias[col]) : 0.f);
          }
          if (vec) {
            uint4 w;
            w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]); w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
            reinterpret_cast<uint4*>(out)[j8] = w;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n0 + j8 * 8 + j < p.N) out[j8 * 8 + j] = __float2bfloat16(f[j]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 2 * F8_BN); }
}

// One warp per (row, 128-wide K block): amax -> scale = amax / 448, values / scale -> e4m3 (saturating).
__global__ void __launch_bounds__(256) quant_fp8_rows_kernel(const __nv_bfloat16* x, long long ldx, int M, int K, uint8_t* q, long long ldq,
                                                             float* scales, long long ld_s) {
  const int lane = threadIdx.x & 31;
  const int kbs = K / 128;
  const long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (item >= static_cast<long long>(M) * kbs) return;
  const int row = static_cast<int>(item / kbs), kb = static_cast<int>(item % kbs);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<long long>(row) * ldx + kb * 128 + lane * 4);
  float v[4] = {bf16lo(raw.x), bf16hi(raw.x), bf16lo(raw.y), bf16hi(raw.y)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
    packed |= static_cast<uint32_t>(b) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * ldq + kb * 128 + lane * 4) = packed;
  if (lane == 0) scales[static_cast<long long>(kb) * ld_s + row] = scale;
}
}  // namespace

// Aq: [M, K] e4m3 (lda bytes per row), Wq: [N, K] e4m3 (ldw), sa: [K/128][ld_sa] fp32, sw: [ceil(N/128)][K/128] fp32,
// C: [M, ldc] bf16, bias: [N] bf16 or null.  K % 128 == 0.
CS_API int cs_gemm_fp8_blockscaled(const void* Aq, long long lda, const void* Wq, long long ldw, const void* sa, long long ld_sa,
                                   const void* sw, void* C, long long ldc, const void* bias, int M, int N, int K, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % F8_BK) || (lda & 15) || (ldw & 15) || ld_sa < M) return -1;
  Fp8Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.sa = reinterpret_cast<const float*>(sa); p.ld_sa = ld_sa;
  p.sw = reinterpret_cast<const float*>(sw); p.kb_total = K / F8_BK;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.stages = F8_MAX_STAGES;
  p.idesc = umma_idesc_e4m3(F8_BM, F8_BN);
  p.err = cs_error_word();
  CUtensorMap tmA, tmB;
  if (cs_encode_tmap_2d(&tmA, Aq, K, M, lda, F8_BK, F8_BM, 1, 1) != 0) return -2;
  if (cs_encode_tmap_2d(&tmB, Wq, K, N, ldw, F8_BK, F8_BN, 1, 1) != 0) return -3;
  const int smem = F8_MAX_STAGES * F8_STAGE_BYTES + 1024;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_done[dev]) {
    cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev] = true;
  }
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < cs_num_sms() ? tiles : cs_num_sms();
  gemm_fp8_kernel<<<grid, 320, smem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// x: [M, K] bf16 -> q: [M, K] e4m3 and scales [K/128][ld_s >= M] (one per row and 128-wide K block).  K % 128 == 0.
CS_API int cs_quant_fp8_rows(const void* x, long long ldx, int M, int K, void* q, long long ldq, void* scales, long long ld_s,
                             void* stream) {
  if (M <= 0) return 0;
  if (K <= 0 || (K % 128) || (ldx & 3) || (ldq & 3) || ld_s < M) return -1;
  const long long warps = static_cast<long long>(M) * (K / 128);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  quant_fp8_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, M, K,
                                                                 reinterpret_cast<uint8_t*>(q), ldq, reinterpret_cast<float*>(scales), ld_s);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
