// Token sampling on the device: temperature, top-k and top-p (nucleus) over fp32 logits, one CTA per row.
//
// No sort: the cut-off is found by a radix select over the order-preserving 32-bit key of each logit, eight bits per
// pass.  One routine serves both limits: every element carries an integer weight (1 for top-k, its probability in
// 2^-36 fixed point for top-p) and the select returns the largest key T whose upper set {key >= T} weighs at least
// the target.  Ties at T are kept.  With both limits, top-p applies to the distribution renormalised over the top-k
// set.  The token is then drawn by inverting the cumulative weight of the kept set in index order.  All sums are
// integers, so a row's result depends only on (logits, parameters, seed, draw index), never on the order in which
// threads arrive.  Rows with temperature <= 0 take the arg-max (lowest index on ties).
#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr float kFixedOne = 68719476736.0f;  // 2^36
constexpr int kSplitBits = 18;              // a weight enters the histograms as two 18-bit halves (32-bit counters)

__device__ __forceinline__ unsigned order_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// probability of a logit in 2^-36 fixed point, relative to the row maximum (which maps to 2^36)
__device__ __forceinline__ unsigned long long fixed_prob(float logit, float mx, float inv_t_log2) {
  return static_cast<unsigned long long>(exp2f((logit - mx) * inv_t_log2) * kFixedOne);
}

struct SelectScratch {
  unsigned long long hist[256];
  unsigned long long warp_sums[SAMPLE_THREADS / 32];
  unsigned long long total;
  unsigned prefix;
  unsigned long long remaining;
};

__device__ unsigned long long block_sum_u64(unsigned long long v, SelectScratch& sc) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sc.warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += sc.warp_sums[w];
    sc.total = t;
  }
  __syncthreads();
  return sc.total;
}

// Largest key T such that the weight of {i : key_i >= T, key_i >= floor_key} is >= target (target >= 1; if the whole
// set weighs less, the smallest key of the set is returned through the same walk).  kByMass: weight = fixed_prob,
// else weight = 1.
// The 256-bucket histogram of a pass is kept once per lane (`lanes_lo/hi[bucket * 32 + lane]`, 32-bit counters): the
// lanes of a warp never meet on an address or a bank however skewed the digits are, and a column receives at most
// V / 32 < 2^13 additions of an 18-bit half, which fits.
template <bool kByMass>
__device__ unsigned radix_select(const float* row, int V, float mx, float inv_t_log2, unsigned floor_key,
                                 unsigned long long target, SelectScratch& sc, unsigned* lanes_lo, unsigned* lanes_hi) {
  unsigned prefix = 0;
  unsigned long long remaining = target;
  const int lane = threadIdx.x & 31;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256 * 32; b += SAMPLE_THREADS) {
      lanes_lo[b] = 0;
      if (kByMass) lanes_hi[b] = 0;
    }
    __syncthreads();
    const unsigned hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
      const float x = row[i];
      const unsigned k = order_key(x);
      if (k >= floor_key && (k & hi_mask) == prefix) {
        const int slot = static_cast<int>((k >> shift) & 255u) * 32 + lane;
        if (kByMass) {
          const unsigned long long w = fixed_prob(x, mx, inv_t_log2);
          if (w) {
            atomicAdd(&lanes_lo[slot], static_cast<unsigned>(w & ((1u << kSplitBits) - 1u)));
            atomicAdd(&lanes_hi[slot], static_cast<unsigned>(w >> kSplitBits));
          }
        } else {
          atomicAdd(&lanes_lo[slot], 1u);
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      const int b = threadIdx.x;
      unsigned long long lo = 0, hi = 0;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) {
        const int l = (j + b) & 31;  // skewed: the threads of a warp read 32 different banks
        lo += lanes_lo[b * 32 + l];
        if (kByMass) hi += lanes_hi[b * 32 + l];
      }
      sc.hist[b] = (hi << kSplitBits) + lo;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long acc = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + sc.hist[b] >= remaining) break;
        acc += sc.hist[b];
      }
      sc.prefix = prefix | (static_cast<unsigned>(b) << shift);
      sc.remaining = remaining - acc;
    }
    __syncthreads();
    prefix = sc.prefix;
    remaining = sc.remaining;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* logits, long long ld, int V, const float* temperature, const float* top_p,
                   const int* top_k, const long long* seed, int* draws, int* out) {
  extern __shared__ unsigned lane_hist[];  // [2][256 * 32]
  unsigned* lanes_lo = lane_hist;
  unsigned* lanes_hi = lane_hist + 256 * 32;
  __shared__ SelectScratch sc;
  __shared__ float red_v[SAMPLE_THREADS / 32];
  __shared__ int red_i[SAMPLE_THREADS / 32];
  __shared__ unsigned long long scan[SAMPLE_THREADS / 32];
  __shared__ int winner;
  const int r = blockIdx.x;
  const float* row = logits + static_cast<long long>(r) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // ---- row maximum and its lowest index --------------------------------------------------------------
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = red_v[lane];
    bi = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { red_v[0] = best; red_i[0] = bi; }
  }
  __syncthreads();
  const float mx = red_v[0];
  const int arg = red_i[0];
  const float temp = temperature[r];
  const int draw = draws[r];
  __syncthreads();
  if (threadIdx.x == 0) draws[r] = draw + 1;
  if (!(temp > 0.f) || !(mx > -INFINITY)) {
    if (threadIdx.x == 0) out[r] = arg;
    return;
  }
  const float inv_t_log2 = 1.4426950408889634f / temp;

  // ---- cut-off key -------------------------------------------------------------------------------------
  unsigned thr = 0;
  const int k = top_k[r];
  if (k > 0 && k < V) thr = radix_select<false>(row, V, mx, inv_t_log2, 0u, static_cast<unsigned long long>(k), sc, lanes_lo, lanes_hi);
  const float pp = top_p[r];
  if (pp > 0.f && pp < 1.f) {
    unsigned long long mass = 0;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
      const float x = row[i];
      if (order_key(x) >= thr) mass += fixed_prob(x, mx, inv_t_log2);
    }
    mass = block_sum_u64(mass, sc);
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(mass) * static_cast<double>(pp));
    if (target < 1) target = 1;
    const unsigned tp = radix_select<true>(row, V, mx, inv_t_log2, thr, target, sc, lanes_lo, lanes_hi);
    thr = max(thr, tp);
  }

  // ---- draw: invert the cumulative weight of the kept set, in index order ---------------------------------
  const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(V, static_cast<int>(threadIdx.x) * per), hi = min(V, lo + per);
  unsigned long long mine = 0;
  for (int i = lo; i < hi; ++i) {
    const float x = row[i];
    if (order_key(x) >= thr) mine += fixed_prob(x, mx, inv_t_log2);
  }
  // inclusive scan over the block (warp scan, then the warp totals)
  unsigned long long incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) scan[warp] = incl;
  if (threadIdx.x == 0) winner = arg;  // fallback: the maximum is always in the kept set
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    scan[lane] = w;  // inclusive totals of warps 0..lane
  }
  __syncthreads();
  const unsigned long long total = scan[SAMPLE_THREADS / 32 - 1];
  const unsigned long long base = (warp ? scan[warp - 1] : 0ull) + incl - mine;  // weight before this thread's slice
  const unsigned long long rnd = mix64(mix64(static_cast<unsigned long long>(seed[r])) ^
                                       (0x9E3779B97F4A7C15ull * (static_cast<unsigned long long>(draw) + 1ull)));
  const unsigned long long target = __umul64hi(rnd, total);  // uniform in [0, total)
  if (total > 0 && mine > 0 && target >= base && target < base + mine) {
    unsigned long long acc = base;
    int pick = lo;
    for (int i = lo; i < hi; ++i) {
      const float x = row[i];
      if (order_key(x) >= thr) {
        const unsigned long long w = fixed_prob(x, mx, inv_t_log2);
        if (w && target < acc + w) { pick = i; break; }
        acc += w;
      }
    }
    winner = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = winner;
}

}  // namespace

// logits fp32 [rows, ld]; temperature / top_p f32 [rows]; top_k i32 [rows] (<= 0: off); seed i64 [rows]; draws i32 [rows]
// (index of this draw in the row's stream, advanced by one here); out i32 [rows].
CS_API int cs_sample_rows(const void* logits, long long ld, int rows, int V, const void* temperature, const void* top_p,
                          const void* top_k, const void* seed, void* draws, void* out, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0 || logits == nullptr || temperature == nullptr || top_p == nullptr || top_k == nullptr || seed == nullptr ||
      draws == nullptr || out == nullptr)
    return -1;
  constexpr int kSmem = 2 * 256 * 32 * static_cast<int>(sizeof(unsigned));
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -10;
    attr_set[dev] = true;
  }
  if (static_cast<long long>(V) >= (1ll << 18)) return -1;  // a lane's column would no longer fit 32 bits
  sample_rows_kernel<<<rows, SAMPLE_THREADS, kSmem, (cudaStream_t)stream>>>(
      (const float*)logits, ld, V, (const float*)temperature, (const float*)top_p, (const int*)top_k,
      (const long long*)seed, (int*)draws, (int*)out);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// ---------------------------------------------------------------------------------------
// OpenAI-style repetition control: logits[r][t] -= frequency[r] * count[r][t] + presence[r] * (count[r][t] > 0),
// where count[r][t] is how often row r has generated token t so far.  Applied before the sampling kernel; the
// counts are advanced by cs_count_tokens after it, both inside the decode graph.
// ---------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) apply_penalties_kernel(float* logits, long long ld, const int* counts, long long ldc,
                                                              const float* freq, const float* pres, int V) {
  const int r = blockIdx.y;
  const float f = freq[r], p = pres[r];
  if (f == 0.f && p == 0.f) return;
  float* row = logits + r * ld;
  const int* crow = counts + r * ldc;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < V; t += gridDim.x * blockDim.x) {
    const int c = crow[t];
    if (c > 0) row[t] -= f * static_cast<float>(c) + p;
  }
}

__global__ void count_tokens_kernel(int* counts, long long ldc, const int* tokens, const int* active, int rows, int V) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  if (active != nullptr && active[r] == 0) return;
  const int t = tokens[r];
  if (t >= 0 && t < V) counts[r * ldc + t] += 1;
}
}  // namespace

CS_API int cs_apply_penalties(void* logits, long long ld, const void* counts, long long ldc, const void* freq,
                              const void* pres, int rows, int V, void* stream) {
  if (rows <= 0 || V <= 0) return 0;
  if (logits == nullptr || counts == nullptr || freq == nullptr || pres == nullptr) return -1;
  int bx = (V + 256 * 8 - 1) / (256 * 8);
  if (bx < 1) bx = 1;
  apply_penalties_kernel<<<dim3(bx, rows), 256, 0, (cudaStream_t)stream>>>((float*)logits, ld, (const int*)counts, ldc,
                                                                           (const float*)freq, (const float*)pres, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

CS_API int cs_count_tokens(void* counts, long long ldc, const void* tokens, const void* active, int rows, int V,
                           void* stream) {
  if (rows <= 0) return 0;
  if (counts == nullptr || tokens == nullptr) return -1;
  count_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>((int*)counts, ldc, (const int*)tokens,
                                                                          (const int*)active, rows, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}
