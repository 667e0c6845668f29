// Allocation-free top-k entry point.  It has no counterpart in the reference, which runs torch.topk on
// freshly allocated tensors (engine/model_runner.py:1034-1081).
//
// Who needs it: callers that hold raw device pointers and must not allocate while they run: code on a
// latency-critical serving thread where a cudaMalloc would serialise the device, a host written in another
// language that links this library without PyTorch's caching allocator, or a process whose memory budget is
// fixed at start-up.  Such a caller passes the logits and the two output buffers; the intermediate
// per-chunk candidates, which ti_topk() takes from caller-provided workspace, live here in a file-scope
// device array instead.
//
// Limits: rows <= TI_TOPK_STATIC_MAX_ROWS, k <= 64, vocab <= 524288, single rank (no candidate exchange).
// The scratch array is TI_TOPK_STATIC_SCRATCH_BYTES per GPU and stays resident from the moment the library
// is loaded on that GPU until the process exits.
//
// Sharing: every call on a GPU uses the same scratch.  Nothing in it has to start at zero (each call
// overwrites every entry it later reads), but two calls that overlap on the GPU (different streams, or a
// second thread) corrupt each other: serialise them.
//
// Device ownership: the scratch is per GPU.  The CURRENT device of the calling thread must own `logits`, both
// outputs and the stream; a device pointer of another GPU is rejected with code -6.
//
// First call on a device: it resolves the device address of the scratch array (one cudaGetSymbolAddress,
// no allocation; guarded so that two threads may make it at the same time).  Make that first call outside any
// stream capture.
#pragma once

#define TI_TOPK_STATIC_MAX_ROWS 16
#define TI_TOPK_STATIC_MAX_ENTRIES (TI_TOPK_STATIC_MAX_ROWS * 8192)
#define TI_TOPK_STATIC_SCRATCH_BYTES (TI_TOPK_STATIC_MAX_ENTRIES * 8)

#ifdef __cplusplus
extern "C" {
#endif

// out_val[rows, k] (descending) and out_idx[rows, k] (token id + vocab_start; ties go to the smaller id) of
// logits[rows, ld] (fp32, first `vocab` columns).  All pointers are device pointers owned by the caller.
// Returns 0, a negative code explained by ti_topk_static_error(), or a positive cudaError_t.
int ti_topk_static(const float* logits, int rows, int vocab, int ld, int k, int vocab_start, float* out_val,
                   int* out_idx, void* stream);

const char* ti_topk_static_error(int code);

#ifdef __cplusplus
}
#endif
