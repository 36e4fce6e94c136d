// Entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (KoduruChandrasekhar/TokenMill): there every
// buffer comes from PyTorch's allocator. It exists for hosts that embed this library next to another
// owner of the GPU's memory: a process whose memory pool was sized up front and handed out completely
// (a serving runtime that reserves the whole device for weights and cache, a plugin running inside
// someone else's allocator), or a latency-critical loop that cannot afford cudaMalloc / cudaFree, which
// synchronise the whole device. Such callers can still pass their own inputs and outputs, but they have
// nowhere to get the scratch that split-key decode attention needs for its partial results.
//
// tm_decode_attention_bf16_noalloc is the decode attention of tm_decode_attention_bf16 (its last block per
// request and kv head merges the key splits), with the partial results and the arrival counters kept in fixed
// arrays that are part of the library image itself (TM_NOALLOC_SCRATCH_FLOATS floats, 8 MiB, and 4,096
// counters; every GPU that loads the library holds them until the process exits). It calls no cudaMalloc,
// cudaFree or allocating library routine.
//
// Rules for the caller:
//  * Sizes: T * nh * max_splits * (D + 2) floats must fit the array (T = tokens in the step, nh = query
//    heads, D = head size), and requests x kv heads the 4,096 counters; larger steps are refused with
//    TM_ERR_NOALLOC_TOO_LARGE (90004) before anything is launched. Batch 64, 14 heads of 64, contexts up to
//    4096 (16 splits of 256 keys) need 0.95 M floats.
//  * What the host cannot see (the requests' lengths are device arrays): max_splits * split_keys must exceed
//    the longest context of the step, and no request may bring more than 16 / (nh / nkv) tokens. A launch
//    that meets a request beyond either limit leaves that request's output incomplete and raises an error
//    word inside the library, which tm_decode_attention_bf16_noalloc_status reads (32); the counters still
//    end at zero.
//  * First call on a device: it looks up the array's device address once (cudaGetSymbolAddress, with that
//    device current) and remembers it. Make that first call outside any stream capture.
//  * The arrays are shared by every call. The floats keep the last call's contents and need not start at
//    zero (each call writes every partial it later reads); the counters are zero in the image and every call
//    leaves them zero. A call that returned a CUDA error (a failed launch, a fault in an earlier kernel of the
//    stream) leaves them undefined: call tm_decode_attention_bf16_noalloc_reset before the next one. Two calls that overlap on the GPU (different streams, or one call racing a graph
//    replay that contains another) would write the same floats and counters: keep calls to this entry point
//    ordered on one stream.
#pragma once

#include <cuda_runtime.h>

#define TM_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TM_ERR_NOALLOC_TOO_LARGE 90004

#ifdef __cplusplus
extern "C" {
#endif

// q, out [T, nh, D] bfloat16; kcache, vcache [pages, page_size, nkv, D] bfloat16; block_table [n_seqs,
// bt_stride] int; cu_q [n_seqs + 1]; kv_before [n_seqs]; seq_of_token [T] (unused, kept for callers). Each request brings at most
// 16 / (nh / nkv) tokens; D is 64 or 128; split_keys a multiple of 64. Returns 0, a TM_ERR_* code, or a
// cudaError_t.
int tm_decode_attention_bf16_noalloc(const void* q, const void* kcache, const void* vcache,
                                     const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                                     const int* seq_of_token, int n_seqs, int n_tokens, void* out, int nh, int nkv,
                                     int D, int page_size, float scale, int window, int split_keys, int max_splits,
                                     cudaStream_t stream);

// Zeroes the arrival counters and the error word on `stream` (no allocation). Use after a failed launch.
int tm_decode_attention_bf16_noalloc_reset(cudaStream_t stream);

// Copies the current device's error word to *code (host memory) and waits for `stream`: 0, or 32 after a launch
// that met a request beyond the size rules above.
int tm_decode_attention_bf16_noalloc_status(int* code, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
