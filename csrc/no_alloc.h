// Entry points of libtyr_kernels.so that never allocate.
//
// This header has no counterpart in the reference: there every native op goes through libtorch,
// which allocates outputs and temporaries from its caching allocator.
//
// Who needs this: code that must not (or cannot) obtain device memory while it runs.  Examples are
// a serving process whose memory pool already owns the whole device, so a cudaMalloc would fail or
// evict; a control loop that cannot tolerate the device-wide synchronisation a cudaMalloc/cudaFree
// implies; and a plugin that lives inside a host application with a fixed memory contract.  Such
// callers still own their inputs and outputs and pass them in; only the *temporary* memory the
// operation needs comes from the library.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest temporary footprint the allocation-free entry accepts, in bytes: enough for one
// 1280 x 5120 (or 5120 x 1280) bf16 matrix, or any batch whose requirement
// tyr_newton_schulz_scratch_bytes(batch, R, C) does not exceed it.
#define TYR_NS_STATIC_SCRATCH_BYTES 19660800LL

// Newton-Schulz orthogonalisation chain (the same math and the same GEMM launches as
// tyr_newton_schulz_bf16) whose temporaries live in a fixed array inside the library image
// instead of caller-provided or freshly allocated memory.
//
//   x        in/out, bf16 [batch, R, C], already Frobenius-normalised, 16-byte aligned
//   returns  0 on success, -1 bad shape, -2 bad alignment, -8 if the shape needs more than
//            TYR_NS_STATIC_SCRATCH_BYTES, 9000+e if resolving the array's device address failed
//            with CUDA error e, other positive values as tyr_gemm_bf16.
//
// * The array occupies TYR_NS_STATIC_SCRATCH_BYTES on every GPU that uses the library's code, until the
//   process exits.  With CUDA's lazy module loading the driver reserves it when the module is first
//   used on a device, which is at the latest this entry's first call there: a process whose pool wants
//   the whole device should make one warm-up call at start-up, before the pool takes the rest.
// * The first call on each device looks up the array's address on that device (the calling
//   thread's current device), raises the kernels' shared-memory limit there, and remembers both.
//   Make that first call outside any stream capture.
// * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
// * Every call uses the same array.  Nothing in it has to start at zero (each launch overwrites what
//   it later reads), and it keeps whatever the previous call left.  Two calls that overlap on the
//   GPU - different streams, or different host threads without ordering - race on it; serialise them.
int tyr_newton_schulz_bf16_static(void* x, int batch, int R, int C, int iters, float a, float b,
                                  float c, int* err, void* stream);

#ifdef __cplusplus
}
#endif
