// ksana_gemm_smallm_noalloc: the skinny (decode-sized) GEMM for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine. It exists for hosts that embed the
// kernel library where device allocation is off limits at call time: code running inside a region
// that forbids cudaMalloc (a latency-critical serving loop that pre-reserved all device memory, a
// plugin called from another framework's stream callback or capture-adjacent section, a process
// whose memory pool is owned and fully handed out by someone else). Such callers can pass inputs
// and outputs they already own, but cannot provide or grow a scratch buffer.
//
// What it does: D[M,N] = X[M,K] * W[N,K]^T (+bias)(+residual), exactly like ksana_gemm_smallm, but
// the split-K scratch (fp32 partial tiles) and the tile arrival counters live in a file-scope
// device array of fixed size that is part of the library image. Every GPU that loads the library
// carries that array (kKsanaNoAllocScratchBytes + counters) until the process exits.
//
// Contract:
//   * Allocates nothing: no cudaMalloc / cudaFree / allocating library call, on any path.
//   * Limits: M <= 128; the scratch the chosen split needs must fit kKsanaNoAllocScratchBytes and
//     the output may have at most kKsanaNoAllocMaxTiles 128-column tiles (N <= 128 * that). Larger
//     problems are rejected with KSANA_NOALLOC_TOO_LARGE and a message from
//     ksana_noalloc_last_error(); nothing is launched.
//   * First call on a device: resolves the device address of the built-in scratch with
//     cudaGetSymbolAddress while that device is current (checked), once per device; host threads
//     that make their first call together are serialised on that step. Make this first call
//     outside of any stream capture.
//   * kind must be 0 or 1; anything else is rejected with KSANA_NOALLOC_BAD_ARGUMENT before any launch.
//   * All calls on one device share the one scratch array, which keeps whatever the previous call
//     left in it. The counters that must start at zero are cleared on the caller's stream before
//     each launch. Two calls that overlap on the GPU (different streams without ordering) race on
//     the scratch and produce wrong results: order the calls.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kKsanaNoAllocScratchBytes = 8 << 20, kKsanaNoAllocMaxTiles = 1024 };
enum { KSANA_NOALLOC_OK = 0, KSANA_NOALLOC_TOO_LARGE = -30, KSANA_NOALLOC_SETUP_FAILED = -31,
       KSANA_NOALLOC_BAD_ARGUMENT = -32 };

// kind 0: X and W are bf16. kind 1: X and W are e4m3 with a_scale [K/128][a_scale_ld] and
// w_scale [ceil(N/128)][K/128] (fp32). D is bf16 with row stride ldd. bias / residual may be null.
int ksana_gemm_smallm_noalloc(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld, const void* W,
                              int ldw, const float* w_scale, void* D, int ldd, const void* bias, const void* residual,
                              int ldr, int M, int N, int K, int* err_flag, cudaStream_t stream);

// Text of the last rejection / set-up failure on the calling thread ("" if none).
const char* ksana_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
