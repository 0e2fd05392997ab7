// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference plugin.  It exists for host code
// that runs where device allocation is off the table: inside a region that a CUDA
// allocator owns exclusively (a serving process whose memory pool has already claimed the
// whole device), in a plugin or callback that is forbidden to call cudaMalloc / cudaFree
// because either would synchronise the device, or in a runtime embedded through the C ABI
// that has no allocator of its own to hand a workspace from.
//
// b200_paged_decode (attention.cu) needs a caller-provided workspace for its split-KV
// partial results.  b200_paged_decode_noalloc is the same kernel with that workspace in a
// fixed array inside the library image, so the caller passes inputs and outputs only.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in workspace.  A call needs B * Hq * num_splits * HD floats of
// partial outputs and B * Hq * num_splits floats of log-sum-exp values; anything larger is
// rejected with B200_NOALLOC_TOO_LARGE before any kernel is launched.
#define B200_NOALLOC_MAX_OUT_FLOATS (2 * 1024 * 1024) /* 8 MiB */
#define B200_NOALLOC_MAX_LSE_FLOATS (32 * 1024)       /* 128 KiB */
#define B200_NOALLOC_TOO_LARGE (-12)
#define B200_NOALLOC_SETUP_FAILED (-13)

// Same arguments and semantics as b200_paged_decode without tmp_out / tmp_lse.
//
// * Calls no cudaMalloc / cudaFree and no allocating library routine.  Every GPU that loads
//   the library holds the ~8.1 MiB workspace until the process exits.
// * The first call on each device resolves the device address of the workspace (one
//   cudaGetSymbolAddress, with that device current).  Make that first call outside any
//   stream capture.
// * All calls on a device share the one workspace, and it keeps whatever the previous call
//   left in it.  Nothing in it has to start at zero (every slot that is read was written by
//   the same call), but two calls that overlap on the GPU (different streams) race on it:
//   serialise them.
// Returns 0, a CUDA error code, or one of the negative codes above;
// b200_noalloc_last_error() describes the last failure of the calling thread.
int b200_paged_decode_noalloc(const void* q, long long ldq, void* out, long long ldo,
                              const void* k_cache, const void* v_cache, long long slot_stride,
                              long long head_stride, long long num_slots,
                              const int* block_tables, int max_blocks, int block_size,
                              const int* seq_lens, int num_splits, int B, int Hq, int Hkv, int HD,
                              float scale, int dtype, void* stream);

const char* b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
