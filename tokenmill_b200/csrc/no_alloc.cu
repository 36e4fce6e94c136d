// Decode attention for callers that cannot allocate: see no_alloc.h for who they are and the rules.
#include "no_alloc.h"

#include "common.cuh"

// The partial results of split-key attention live here instead of in caller- or allocator-provided
// memory, and so do the arrival counters by which the last block of a (request, kv head) knows to merge
// them (zero in the image, left zero by every launch). In host code these names are only stand-ins for the
// device arrays: their device addresses have to be asked for (cudaGetSymbolAddress) and are what the kernel
// receives.
static __device__ __align__(256) float tm_noalloc_scratch[TM_NOALLOC_SCRATCH_FLOATS];
constexpr int kNoallocCounters = 4096;
static __device__ int tm_noalloc_done[kNoallocCounters];
static __device__ int tm_noalloc_error;       // raised (32) by a launch whose requests broke the rules on sizes

extern "C" int tm_decode_attention_bf16(const void* q, const void* kcache, const void* vcache,
                                        const int* block_table, int bt_stride, const int* cu_q,
                                        const int* kv_before, int n_seqs, float* part_acc, float* part_ml,
                                        void* out, int* done, int nh, int nkv, int D, int page_size, float scale,
                                        int window, int split_keys, int max_splits, int* error,
                                        cudaStream_t stream);

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch[kMaxDevices] = {};   // device address of tm_noalloc_scratch, per device, once looked up
int* g_done[kMaxDevices] = {};        // and of tm_noalloc_done
int* g_error[kMaxDevices] = {};       // and of tm_noalloc_error

// The arrays' addresses on the current device. The first call per device does the look-up.
int scratch_for_current_device(float** ptr, int** done, int** error) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return TM_ERR_UNSUPPORTED_SHAPE;
  if (!g_scratch[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, tm_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    int* d = nullptr;
    e = cudaGetSymbolAddress((void**)&d, tm_noalloc_done);
    if (e != cudaSuccess) return (int)e;
    int* w = nullptr;
    e = cudaGetSymbolAddress((void**)&w, tm_noalloc_error);
    if (e != cudaSuccess) return (int)e;
    g_error[dev] = w;
    g_done[dev] = d;
    g_scratch[dev] = p;
  }
  *ptr = g_scratch[dev];
  *done = g_done[dev];
  *error = g_error[dev];
  return 0;
}

}  // namespace

extern "C" int tm_decode_attention_bf16_noalloc(const void* q, const void* kcache, const void* vcache,
                                                const int* block_table, int bt_stride, const int* cu_q,
                                                const int* kv_before, const int* seq_of_token, int n_seqs,
                                                int n_tokens, void* out, int nh, int nkv, int D, int page_size,
                                                float scale, int window, int split_keys, int max_splits,
                                                cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || D <= 0 || max_splits <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  (void)seq_of_token;                         // (kept in the signature; the merge no longer needs it)
  const long long rows = (long long)n_tokens * nh * max_splits;
  if (rows * (D + 2) > (long long)TM_NOALLOC_SCRATCH_FLOATS || (long long)n_seqs * nkv > kNoallocCounters)
    return TM_ERR_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  int* done = nullptr;
  int* error = nullptr;
  const int status = scratch_for_current_device(&scratch, &done, &error);
  if (status != 0) return status;
  float* part_acc = scratch;                  // [rows, D]
  float* part_ml = scratch + rows * D;        // [rows, 2]
  return tm_decode_attention_bf16(q, kcache, vcache, block_table, bt_stride, cu_q, kv_before, n_seqs, part_acc,
                                  part_ml, out, done, nh, nkv, D, page_size, scale, window, split_keys, max_splits,
                                  error, stream);
}

// Puts the arrival counters and the error word back to zero, on `stream` (cudaMemsetAsync at the arrays' own
// addresses: nothing is allocated). For after a launch that failed or was cut short.
extern "C" int tm_decode_attention_bf16_noalloc_reset(cudaStream_t stream) {
  float* scratch = nullptr;
  int* done = nullptr;
  int* error = nullptr;
  const int status = scratch_for_current_device(&scratch, &done, &error);
  if (status != 0) return status;
  cudaError_t e = cudaMemsetAsync(done, 0, sizeof(int) * kNoallocCounters, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(error, 0, sizeof(int), stream);
  return (int)e;
}

// Reads the error word of the current device into *code (0: every launch so far kept the rules; 32: some
// request had more rows than a tile holds, or keys beyond max_splits * split_keys). Waits for `stream`.
extern "C" int tm_decode_attention_bf16_noalloc_status(int* code, cudaStream_t stream) {
  float* scratch = nullptr;
  int* done = nullptr;
  int* error = nullptr;
  const int status = scratch_for_current_device(&scratch, &done, &error);
  if (status != 0) return status;
  cudaError_t e = cudaMemcpyAsync(code, error, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return (int)e;
}
