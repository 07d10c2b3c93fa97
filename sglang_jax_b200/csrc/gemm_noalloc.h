// Allocation-free bf16 GEMM entry point of libsglb200.  It has no counterpart in the reference
// project (sgl-project/sglang-jax), whose dense projections are XLA `dot_general` calls.
//
// Who needs it: hosts that must not allocate device memory once serving has started.  Typical
// cases are an engine that has committed (almost) all of HBM to its weight arena and KV pool at
// start-up — a later cudaMalloc there can fail outright or stall the whole device while the
// driver reclaims memory — and plugin-style embedders whose host runtime owns every device
// allocation and forbids the plugin to make its own.  The regular entry point
// (`sglb_gemm_bf16`) leaves scratch to its caller; its Python wrapper obtains that scratch from
// torch's allocator.  This one carries its scratch inside the library instead.
//
//   out[M, N] = x[M, K] . w[N, K]^T (+ bias[N])       bf16, row-major, fp32 accumulation
//
// Limits: M <= 256 (the decode-shaped "weights on the MMA M dimension" variant only); N and K
// multiples of 8; x, w, out 16-byte aligned.  Split-K partial tiles are kept in an 8 MiB
// file-scope device array (plus an 8 KiB header with the status word and tile counters), i.e.
// ceil(N/128) * splits * 128 * BN * 4 bytes must fit in 8 MiB, where BN is M rounded up to
// 16/32/64/128/256.  `splits = 0` lets the library choose a split count that fits; an explicit
// `splits` that does not fit is rejected (negative return, text in
// sglb_gemm_bf16_noalloc_last_error()).  Every GPU that loads the library holds the array
// (sglb_gemm_bf16_noalloc_scratch_bytes()) until the process exits.
//
// Behaviour to know about:
//   * The first call on a device looks up the device address of the scratch array
//     (cudaGetSymbolAddress, with that device current) and caches it.  Make that first call
//     before any stream capture.
//   * All calls share the one array, which keeps the contents of the previous call: the header
//     (status + counters) is cleared with cudaMemsetAsync on `stream` at the start of each call,
//     which also erases a status word of the previous call that nobody has read yet: read the
//     status between calls if a failure must not go unnoticed.
//     Calls that overlap on the GPU (different streams, no ordering between them) race on it;
//     serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called; the caller provides
//     x, w, bias (may be null) and out.
//   * Waits inside the kernel are bounded; sglb_gemm_bf16_noalloc_status() copies the status word
//     (0 = ok) to the host with a blocking cudaMemcpy.  That copy waits for work of the legacy
//     default stream only: a caller that launched on another stream (in particular one created
//     with cudaStreamNonBlocking) must synchronise that stream itself before asking for the
//     status, or it can read 0 while the GEMM is still running.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int sglb_gemm_bf16_noalloc(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                           int splits, cudaStream_t stream);
size_t sglb_gemm_bf16_noalloc_scratch_bytes(void);
const char* sglb_gemm_bf16_noalloc_last_error(void);
int sglb_gemm_bf16_noalloc_status(int* out4);

#ifdef __cplusplus
}
#endif
