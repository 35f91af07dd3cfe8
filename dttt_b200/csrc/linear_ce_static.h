// Forward of linear + cross-entropy for callers that must not allocate.
//
// This entry point has no counterpart in the reference (tianhux2/dttt has no native code at all); it exists for
// callers that run where device allocation is off the table: inside a region where the caching allocator must not
// be touched (a replayed step whose memory plan is frozen, an allocator-free C host, a signal-safe diagnostics path).
// dttt_linear_ce_fwd needs a scratch buffer of per-tile (max, sum-exp) pairs and leaves its allocation to the
// caller; this variant keeps that scratch in a fixed array in the library's own device image instead, so a call
// performs no cudaMalloc / cudaFree and calls no allocating library routine.
//
//   lse[r] = logsumexp_v(h_r . E_v)      nll[r] = lse[r] - h_r . E_{targets[r]}
//
//   h [rows, K] bf16 (row stride ldh elements), E [classes, K] bf16 (row stride ldE), targets [rows] int32,
//   tgt_logit / lse / nll [rows] f32 device buffers owned by the caller (nll may be null).  A row whose target is
//   outside [0, classes) leaves its tgt_logit entry as it was, exactly as dttt_linear_ce_fwd does.
//
// Limit: ceil(rows / 128) * 128 * ceil(classes / 256) <= DTTT_LINEAR_CE_STATIC_MAX_ELEMS (2 Mi pairs, 16 MiB; e.g.
// 4096 rows x 131072 classes).  Larger problems are refused with DTTT_LINEAR_CE_STATIC_TOO_LARGE and nothing is
// launched; dttt_linear_ce_static_strerror() gives the message.
//
// Set-up: the first call on a device (with that device current) resolves the array's device address, sets the
// kernel's shared-memory attribute for that device and loads the kernels; make that first call before any stream
// capture begins.  The state is kept per device, so one process may call this on several devices in turn.
// Sharing: every call on a device uses the same array.  Nothing in it has to start at zero (each entry that is read
// was written earlier by the same call), but two calls in flight at once -- on different streams, or from different
// threads without ordering between their streams -- race on it and give wrong results.  Calls on one stream are safe.
#pragma once
#include <cuda_runtime.h>

#define DTTT_LINEAR_CE_STATIC_MAX_ELEMS (2ll * 1024 * 1024)
#define DTTT_LINEAR_CE_STATIC_TOO_LARGE (-10)
#define DTTT_LINEAR_CE_STATIC_SETUP_FAILED (-11)

#ifdef __cplusplus
extern "C" {
#endif

int dttt_linear_ce_fwd_static(const void* h, const void* E, const int* targets, int rows, int classes, int K, long long ldh,
                              long long ldE, float* tgt_logit, float* lse, float* nll, int* status, cudaStream_t stream);

const char* dttt_linear_ce_static_strerror(int code);

#ifdef __cplusplus
}
#endif
