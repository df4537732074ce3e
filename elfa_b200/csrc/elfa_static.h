// Entry point of libelfa_b200.so that never allocates memory.
//
// This function has no counterpart in the reference project: it exists for hosts that embed the
// library but are not allowed to allocate device memory themselves - for example a plug-in running
// inside another runtime that owns the whole memory pool and forbids cudaMalloc, or a caller that
// is already inside a section where allocation is prohibited. Such callers cannot provide the
// scratch buffer that elfa_sumsq() asks for, so this variant keeps its scratch in a fixed array
// that is part of the library image.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest input the static scratch supports: 1024 partial sums of at most 2^24 elements each.
#define ELFA_SUMSQ_STATIC_MAX_ELEMS (1024LL << 24)

// out[0] = sum of x[i]^2 over n elements (x is fp32 when grad_type == 0, bf16 when 1).
// `x` and `out` are device pointers supplied by the caller; nothing is allocated or freed.
//
// * Scratch: a 4 KiB array of the library, resident on every GPU that loads the library until the
//   process exits. All calls share it; it keeps the last call's partial sums. Each call overwrites
//   every slot it later reads, so nothing has to be cleared, but two calls that overlap on the GPU
//   (different streams, or different threads) race on it: serialise them.
// * The first call on each device looks up the device address of that array (with that device
//   current). Make this first call before starting any stream capture.
// * n must be in [1, ELFA_SUMSQ_STATIC_MAX_ELEMS]; larger inputs are rejected with ELFA_ERR_ARG and
//   a message in elfa_last_error().
int elfa_sumsq_static(const void* x, int grad_type, long long n, float* out, void* stream);

#ifdef __cplusplus
}
#endif
