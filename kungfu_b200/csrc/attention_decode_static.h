// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (nickheyer/kungfu); it exists for hosts of this library
// that cannot call cudaMalloc: code that runs while a CUDA graph is being captured around it, plug-ins that
// are handed a fixed arena by an embedding runtime, and real-time loops where an allocation (and the implicit
// device synchronisation it may cause) is not allowed.  The ordinary entry point, kf_attention_decode, needs two
// scratch buffers from its caller (the partial results of the key splits and one arrival counter per group of
// heads); here they are two arrays that are part of the library image:
//
//     KF_DECODE_STATIC_MAX_PARTIAL_FLOATS floats (8 MiB) and KF_DECODE_STATIC_MAX_COUNTERS ints (16 KiB).
//
// Every GPU that loads the library holds these arrays until the process exits.  A call that cuts the keys into
// several splits and whose rows * heads * splits * (head_dim + 4) or rows * kv_heads * head_groups exceeds them is
// refused with KF_ERR_SIZE (2) and touches nothing; a call planned with one split (many rows, or few keys) needs
// neither array and is taken at any size.  The function calls no cudaMalloc, cudaFree or other allocating routine.
//
// Set-up: the first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress, once per
// device, with that device current).  Make that first call outside any stream capture.
// Sharing: all calls use the same arrays, which keep the previous call's contents; the counters are cleared by a
// memset on `stream` at the start of every call that uses them.  Two calls that overlap on the GPU (different streams without
// an ordering between them) race on the arrays; keep calls on one stream or order them with events.
//
// Arguments are those of kf_attention_decode for rows 0..n_rows-1 (one query row per request):
// q, out [n_rows, nh*d] bfloat16; pages [n_pages, 2, nkv, page_size, d] bfloat16; positions, row_req [n_rows];
// table [n_requests, table_stride]; max_keys: the longest key range any row reads (it only steers how many
// splits are used).  Returns 0 when the work was queued on `stream`.
#pragma once
#include <cuda_runtime.h>

#define KF_DECODE_STATIC_MAX_PARTIAL_FLOATS (2 * 1024 * 1024)
#define KF_DECODE_STATIC_MAX_COUNTERS 4096

#ifdef __cplusplus
extern "C" {
#endif
// The size rule alone, without a launch: 0 if a call with `splits` key splits and `ht` heads per block fits the
// built-in arrays, 2 (with a message for kf_last_cuda_error) if not.  kf_attention_decode_static applies it to the
// split count its planner chooses for the device.
__attribute__((visibility("default")))
int kf_attention_decode_static_fits(int n_rows, int nh, int nkv, int d, int ht, int splits);

__attribute__((visibility("default")))
int kf_attention_decode_static(const void* q, void* out, const void* pages, int n_rows, const int* positions,
                               const int* row_req, const int* table, int table_stride, int page_size, int nh,
                               int nkv, int d, float scale, float softcap, int window, int max_keys,
                               cudaStream_t stream);
#ifdef __cplusplus
}
#endif
