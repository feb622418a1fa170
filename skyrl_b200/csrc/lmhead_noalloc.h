// Allocation-free variant of the fused LM-head log-probability entry point.
//
// This entry point has no counterpart in the reference; it exists for callers of this library that are
// not allowed to allocate device memory at the point where they need token log-probabilities: code
// running inside a memory-frozen region (for example a serving loop whose allocator has been handed
// over to another component, or a host that forbids cudaMalloc after start-up because every byte of
// HBM is budgeted), and foreign-language callers that only have raw pointers for inputs and outputs.
//
// The regular path (sb_lmhead_partials + sb_lmhead_combine) needs a scratch buffer of per-(row, split)
// softmax records that its caller allocates.  Here that scratch is a fixed array inside the library's
// device image, so the call needs nothing beyond the caller's own input and output buffers.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Upper bound on rows * vocabulary-splits that fit the built-in scratch (16 bytes per record, 4 MiB in
// total; every GPU that loads the library reserves it until the process exits).
#define SB_LMHEAD_NOALLOC_MAX_RECORDS 262144

// logprob[t] = log softmax(hidden[t] @ W^T * inv_temp)[targets[t]], entropy[t], lse[t] (any output may be null).
//   hidden [T, K] bf16 (row stride ldh), W [V, K] bf16 (row stride ldw), targets [T] int32, all on the current device.
// Returns 0 on success, SB_ERR_TOO_LARGE (4) when T * splits(T, V) exceeds SB_LMHEAD_NOALLOC_MAX_RECORDS,
// SB_ERR_ARG (1) for unsupported strides, SB_ERR_CUDA (2) / SB_ERR_TMAP (3) when a CUDA call fails.
//
// * The first call on each device resolves the scratch array's device address and sets the kernel's
//   shared-memory attribute; make that first call outside of any stream capture.  That one-time set-up is
//   guarded by a per-device mutex, so first calls may come from several host threads at once.
// * All calls on a device share the one scratch array.  Two calls whose kernels overlap on the GPU (different
//   streams, or different host threads) race on it; serialise them on one stream.
// * Nothing in the scratch has to start at zero: each call overwrites every record it later reads, so stale
//   contents from the previous call are never observed.
// * No cudaMalloc / cudaFree / host allocation happens inside the call.
int sb_lmhead_logprob_noalloc(const void* hidden, const void* W, const int* targets, int T, int V, int K,
                              long long ldh, long long ldw, float inv_temp, float* logprob, float* entropy,
                              float* lse, void* stream);

#ifdef __cplusplus
}
#endif
