// Allocation-free entry point of libfsb200.
//
// This entry point has no counterpart in the reference library. It exists for callers that may
// not allocate device memory at the moment they need the kernel: code that runs inside another
// runtime's execution callback (an inference-server plugin, a custom-call hook of a compiler
// runtime, a real-time control loop) where the host application has handed out all device memory
// up front and treats a cudaMalloc on the hot path as an error, because it may synchronise the
// device, fragment a budget that was sized exactly, or simply fail.
//
// fsb_rmsnorm_bwd_noalloc computes the same result as fsb_rmsnorm_bwd, but the per-block partial
// sums of the weight gradient, for which fsb_rmsnorm_bwd needs a caller-allocated scratch buffer of
// ceil(T/32) * D floats, live in a fixed 8 MiB array inside the library image (every GPU that loads
// the library carries that array until the process exits). The caller still provides every input
// and output; the function calls no cudaMalloc, cudaFree or allocating library routine.
//
//  * Limit: ceil(T/32) * D <= 2 097 152 floats (for example T = 16 384 rows at D = 4096) and
//    D <= 8192, D % 8 == 0. Larger problems are rejected with FSB_ERR_TOO_LARGE (64) and a message
//    on stderr; nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current). Make that first call before starting any stream capture.
//  * All calls on a device share the one array, and it keeps what the previous call left there.
//    The kernel overwrites every entry it later reads, so nothing has to be cleared between calls,
//    but two calls that overlap on the GPU (different streams, no ordering between them) race on
//    it: serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// dy, x, dx: bf16 [T, D]; w: bf16 [D]; rstd: fp32 [T]; dres: optional bf16 [T, D] added to dx
// (may be null); dw_out: [D], fp32 when dw_fp32 != 0 else bf16; dw_accumulate != 0 adds to dw_out.
// Returns 0 on success; 1 for a bad argument (shape outside the limits above, a null required pointer, or
// a pointer that is not aligned as the kernels read it: 16 bytes for dy / x / w / dx / dres, element size
// for rstd and dw_out); 3 for a failed launch or address lookup; 64 when the problem exceeds the built-in
// scratch array (checked before the pointers, so a size can be probed with null pointers).
int fsb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                            const void* dres, void* dx, void* dw_out, int dw_fp32, int dw_accumulate,
                            long long T, int D, cudaStream_t stream);

// Capacity of the built-in scratch array, in floats.
long long fsb_rmsnorm_bwd_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
