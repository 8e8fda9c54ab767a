// Allocation-free entry point of the small-M weight-streaming GEMM.
//
// This entry point has no counterpart in the reference project (which has no native code at all); it exists
// for users of this library whose process must not allocate GPU memory at the time of the call.  Examples: an
// LLM executor that handed every free byte of the device to its KV cache when it started, so a later
// cudaMalloc would simply fail; a serving loop in which an allocation would stall every stream of the device;
// a plug-in running under a host framework that owns the allocator and forbids calls around it.
//
// cs_gemm_skinny (gemm_skinny.cu) needs two scratch areas from its caller when it splits K over several
// thread blocks: fp32 partial sums and per-tile arrival counters.  Here both live in one array that is part of
// the library image itself, `static __device__ __align__(256)`, CS_NOALLOC_SCRATCH_BYTES (+ one status word) long.  Every GPU
// that loads the library carries that array until the process exits, whether or not this function is used.
//
//   C[M,N] = act(X[M,K] W[N,K]^T + bias) + residual              (swiglu == 0)
//   C[M,N] = act(X Wg^T + bg) * (X Wu^T + bu),  W = [Wg; Wu]     (swiglu == 1)
//
// Arguments are those of cs_gemm_skinny without the scratch pointers; the caller still owns every input and
// output buffer.  Returns 0 on success.  CS_NOALLOC_TOO_LARGE means the partial sums of this problem
// (splits * N * round_up(M,16) * 4 bytes, twice that with swiglu) or its tile count do not fit the built-in
// array: lower `splits` (1 needs no scratch at all) or use cs_gemm_skinny with your own buffers.
// cs_noalloc_last_message() describes the most recent failure of the calling thread in words.
//
// Things to know:
//  * The first call on each device looks up the device address of the array (cudaGetSymbolAddress with that
//    device current) and sets a kernel attribute.  Make that first call during start-up, before any stream
//    capture begins on that device.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
//  * All calls on one device share the same array, and it keeps what the previous call left in it.  The
//    arrival counters are cleared on the caller's stream at the start of every call (a memset node, not an
//    allocation); the partial sums are always written before they are read.  Two calls that can overlap on
//    the GPU (different streams without ordering between them, or two host threads) race on the array and
//    give wrong results: order them on one stream or with events.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define CS_NOALLOC_PARTIAL_BYTES (8ll << 20) /* fp32 partial sums */
#define CS_NOALLOC_MAX_TILES 1024            /* one int arrival counter per 128-column tile */
#define CS_NOALLOC_SCRATCH_BYTES (CS_NOALLOC_PARTIAL_BYTES + CS_NOALLOC_MAX_TILES * 4)

#define CS_NOALLOC_TOO_LARGE (-20)
#define CS_NOALLOC_SETUP_FAILED (-21)

int cs_gemm_skinny_noalloc(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc,
                           const void* bias, const void* residual, long long ldr, int M, int N, int K, int act,
                           int swiglu, int out_fp32, int splits, void* stream);

/* Bytes of fp32 partial sums the call would need (0 when it would not split K). */
long long cs_gemm_skinny_noalloc_need_bytes(int M, int N, int K, int swiglu, int splits);

const char* cs_noalloc_last_message(void);

/* Reads back (and clears) the word in which a kernel of this entry point records a bounded wait that ran out:
   0 = none.  Synchronises with the current device; allocates nothing. */
int cs_gemm_skinny_noalloc_kernel_error(void);

#ifdef __cplusplus
}
#endif
