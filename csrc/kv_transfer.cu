// KV-cache page transfer for prefill/decode disaggregation: the decode executor pulls the pages that a prefill executor
// filled straight out of that executor's cache, which is mapped into this process (CUDA IPC; over NVLink when the two
// executors sit on different GPUs).  One launch moves every layer of every page of a request:
//
//   dst[layer][dst_pages[i]][:] = src[layer][src_pages[i]][:]      (page = K and V of all local heads, contiguous)
//
// Each CTA copies one (page, layer) pair with 16-byte loads and stores, several in flight per thread so that the
// read latency of the peer link is covered.  The page lists live on the device (no host round trip per page).
#include "common.cuh"

namespace {

struct KvCopyParams {
  uint8_t* dst; const uint8_t* src;
  long long dst_layer_stride, src_layer_stride;  // bytes
  long long page_bytes;                          // multiple of 16
  int layers, n, dst_num_pages, src_num_pages;
  const int* src_pages; const int* dst_pages;
  int* err;
};

__global__ void __launch_bounds__(256) kv_copy_pages_kernel(const KvCopyParams p) {
  const int i = blockIdx.x, layer = blockIdx.y;
  const int sp = p.src_pages[i], dp = p.dst_pages[i];
  if (sp < 0 || sp >= p.src_num_pages || dp < 0 || dp >= p.dst_num_pages) {   // a bad list must not touch memory
    if (threadIdx.x == 0) cs_set_error(p.err, CS_ERR_BAD_ARG);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(p.src + layer * p.src_layer_stride + sp * p.page_bytes);
  uint4* d = reinterpret_cast<uint4*>(p.dst + layer * p.dst_layer_stride + dp * p.page_bytes);
  const long long nvec = p.page_bytes >> 4;
  long long v = threadIdx.x;
  for (; v + 3 * 256 < nvec; v += 4 * 256) {
    const uint4 a = __ldcs(s + v), b = __ldcs(s + v + 256), c = __ldcs(s + v + 512), e = __ldcs(s + v + 768);
    d[v] = a; d[v + 256] = b; d[v + 512] = c; d[v + 768] = e;
  }
  for (; v < nvec; v += 256) d[v] = __ldcs(s + v);
}
}  // namespace

CS_API int cs_kv_copy_pages(void* dst, const void* src, long long dst_layer_stride, long long src_layer_stride, long long page_bytes,
                            int layers, int n, int dst_num_pages, int src_num_pages, const void* src_pages, const void* dst_pages,
                            void* stream) {
  if (n <= 0 || layers <= 0) return 0;
  if ((page_bytes & 15) || (dst_layer_stride & 15) || (src_layer_stride & 15) || layers > 65535 ||
      (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15))
    return -1;
  KvCopyParams p{};
  p.dst = (uint8_t*)dst; p.src = (const uint8_t*)src;
  p.dst_layer_stride = dst_layer_stride; p.src_layer_stride = src_layer_stride; p.page_bytes = page_bytes;
  p.layers = layers; p.n = n; p.dst_num_pages = dst_num_pages; p.src_num_pages = src_num_pages;
  p.src_pages = (const int*)src_pages; p.dst_pages = (const int*)dst_pages;
  p.err = cs_error_word();
  kv_copy_pages_kernel<<<dim3(n, layers), 256, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -10;
}

// Lets kernels of the current device read memory of `peer_device` (needed once per pair before the first pull).
// Returns 0 when access is (already) enabled, 1 when the two devices cannot reach each other.
CS_API int cs_enable_peer_access(int peer_device) {
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) return -1;
  if (cur == peer_device) return 0;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, cur, peer_device) != cudaSuccess || !can) { cudaGetLastError(); return 1; }
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  cudaGetLastError();
  return -1;
}
