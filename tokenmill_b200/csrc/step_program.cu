// A step program: the launches of one forward pass as a flat list that the host walks in ONE native call.
//
// The reference drives its model from Python, one library call per operation
// (src/infer/model/qwen2.py:13-52, src/infer/engine/model_runner.py:80-97). Doing the same with this library's
// kernels costs 8 to 10 microseconds of interpreter time per launch; a prompt step of a 24-layer model has
// about 200 launches, so every prompt step took at least 3 ms however few tokens it had, and a 2,048-token step
// was bound by the host as much as by the GPU. Here the parts of a model write their launches ONCE into a list
// of fixed-size records; a value in a record is either fixed for the model's lifetime (a weight, a workspace
// buffer, a size from the configuration) or the index of a per-step parameter (the number of tokens, a pointer
// into the step's input buffer, whether this step's attention takes the decode kernel). Each step then fills the
// small parameter table and calls tm_program_run.
//
// Matrix products go to the same library the reference's F.linear reaches (cuBLAS, GemmEx with float32
// accumulation). The library is not linked: its entry points are looked up in the copy that the process has
// already loaded (PyTorch's), so the build needs nothing beyond the CUDA toolkit's headers.
#include <cublas_v2.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstring>

#include "common.cuh"

extern "C" {
int tm_add_rmsnorm(int dtype, float* resid, const void* branch, const float* partials, int n_partials,
                   long long partial_stride, const int* ids, const void* table, const int* rows, const float* weight,
                   float eps, void* out, int n_rows, int H, cudaStream_t stream);
int tm_qkv_rope_write(int in_dtype, int dtype, const void* qkv, const float* bias, const int* positions,
                      const float* cos_t, const float* sin_t, const int* slot_map, void* q_out, void* kcache,
                      void* vcache, int T, int nh, int nkv, int D, int n_pos, int* error, cudaStream_t stream);
int tm_swiglu(int dtype, const void* gu, void* out, int T, int I, cudaStream_t stream);
int tm_tc_linear(const void* x, int ldx, const void* w, void* out, int ldo, int T, int N, int K, int* error,
                 cudaStream_t stream);
int tm_tc_qkv_rope_write(const void* x, int ldx, const void* w, const float* bias, const int* positions,
                         const float* cos_t, const float* sin_t, const int* slot_map, void* q_out, void* kcache,
                         void* vcache, int T, int K, int nh, int nkv, int D, int n_pos, int* error, cudaStream_t stream);
int tm_prefill_attention_tc_bf16(const void* q, const void* kcache, const void* vcache, const int* block_table,
                                 int bt_stride, const int* unit_rec, int n_units, int chunk_keys, float* part_acc,
                                 float* part_ml, int* tile_done, int* counters, void* out, int nh, int nkv, int D,
                                 int page_size, float scale, int window, int* error, cudaStream_t stream);
int tm_prefill_attention_bf16(const void* q, const void* kcache, const void* vcache, const int* block_table,
                              int bt_stride, const int* unit_rec, int n_units, int chunk_keys, float* part_acc,
                              float* part_ml, int* tile_done, int* counters, void* out, int nh, int nkv, int D,
                              int page_size, float scale, int window, cudaStream_t stream);
int tm_decode_attention_bf16(const void* q, const void* kcache, const void* vcache, const int* block_table,
                             int bt_stride, const int* cu_q, const int* kv_before, int n_seqs, float* part_acc,
                             float* part_ml, void* out, int* done, int nh, int nkv, int D, int page_size, float scale,
                             int window, int split_keys, int max_splits, int* error, cudaStream_t stream);
int tm_decode_attention_units_bf16(const void* q, const void* kcache, const void* vcache, long long n_pages,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                                   const int* units, const int* n_work, int max_work, int grid_blocks, float* part_acc,
                                   float* part_ml, void* out, int* done, int nh, int nkv, int D, int page_size,
                                   float scale, int window, int max_parts, int* error, cudaStream_t stream);
}

#define TM_ERR_PROGRAM 90010          // a malformed record (unknown kind, parameter index out of range)
#define TM_ERR_NO_CUBLAS 90011        // the matrix library could not be found in the process

namespace tmk {

enum ProgramOpKind : int32_t {
  kOpAddRmsNorm = 1,
  kOpGemmBf16 = 2,
  kOpQkvRopeWrite = 3,
  kOpPrefillAttentionTc = 4,
  kOpPrefillAttention = 5,
  kOpDecodeAttention = 6,
  kOpSwiglu = 7,
  kOpTcQkvRopeWrite = 8,
  kOpTcLinear = 9,
  kOpDecodeAttentionUnits = 10,
};
constexpr int kOpKinds = 16;

constexpr int kProgramArgs = 24;

// One launch. arg[i] is the value itself, or, where bit i of param_mask is set, the index of the step
// parameter that holds it. Pointers and integers are stored as they are, floats as their bit pattern in the
// low 32 bits. cond >= 0: the launch is skipped in steps whose parameter `cond` is zero.
struct ProgramOp {
  int32_t kind;
  int32_t cond;
  uint32_t param_mask;
  int32_t n_args;
  int64_t arg[kProgramArgs];
};

using GemmExFn = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                    const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                    cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);

struct Cublas {
  cublasHandle_t handle = nullptr;
  GemmExFn gemm_ex = nullptr;
  decltype(&cublasSetStream_v2) set_stream = nullptr;
  cudaStream_t stream = nullptr;
  bool stream_set = false;
};

static Cublas g_cublas;

static void* cublas_symbol(void* lib, const char* name) { return lib ? dlsym(lib, name) : nullptr; }

// Finds the matrix library in the process (it is there once PyTorch is: libcublas.so.12), creates a handle and
// gives it `workspace` (the library then has room for its faster split and stream-k kernels, as under PyTorch).
static int cublas_setup(void* workspace, size_t workspace_bytes) {
  if (g_cublas.handle) return 0;
  void* lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
  if (!lib) lib = dlopen("libcublas.so.12", RTLD_NOW);
  if (!lib) lib = dlopen("libcublas.so", RTLD_NOW);
  auto create = reinterpret_cast<decltype(&cublasCreate_v2)>(cublas_symbol(lib, "cublasCreate_v2"));
  auto set_ws = reinterpret_cast<decltype(&cublasSetWorkspace_v2)>(cublas_symbol(lib, "cublasSetWorkspace_v2"));
  g_cublas.gemm_ex = reinterpret_cast<GemmExFn>(cublas_symbol(lib, "cublasGemmEx"));
  g_cublas.set_stream = reinterpret_cast<decltype(&cublasSetStream_v2)>(cublas_symbol(lib, "cublasSetStream_v2"));
  if (!create || !set_ws || !g_cublas.gemm_ex || !g_cublas.set_stream) return TM_ERR_NO_CUBLAS;
  cublasHandle_t h = nullptr;
  if (create(&h) != CUBLAS_STATUS_SUCCESS) return TM_ERR_NO_CUBLAS;
  if (workspace && workspace_bytes && set_ws(h, workspace, workspace_bytes) != CUBLAS_STATUS_SUCCESS) return TM_ERR_NO_CUBLAS;
  g_cublas.handle = h;
  return 0;
}

// x [T, K] . w [N, K]^T -> out [T, N], all row-major; bfloat16 in, float32 accumulation, bfloat16 or float32 out.
// In the library's column-major terms: out^T [N, T] = w^T-as-stored [K, N]^T . x-as-stored [K, T].
static int gemm_bf16(const void* x, const void* w, void* out, int T, int N, int K, int out_f32, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!g_cublas.handle) return TM_ERR_NO_CUBLAS;
  if (!g_cublas.stream_set || g_cublas.stream != stream) {
    if (g_cublas.set_stream(g_cublas.handle, stream) != CUBLAS_STATUS_SUCCESS) return TM_ERR_NO_CUBLAS;
    g_cublas.stream = stream;
    g_cublas.stream_set = true;
  }
  const float alpha = 1.0f, beta = 0.0f;
  const cublasStatus_t st =
      g_cublas.gemm_ex(g_cublas.handle, CUBLAS_OP_T, CUBLAS_OP_N, N, T, K, &alpha, w, CUDA_R_16BF, K, x, CUDA_R_16BF, K,
                       &beta, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 91000 + (int)st;
}

static inline float as_float(int64_t v) {
  const uint32_t bits = (uint32_t)v;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
template <typename T> static inline T* as_ptr(int64_t v) { return reinterpret_cast<T*>(static_cast<uintptr_t>(v)); }

static long long g_kind_launches[kOpKinds] = {};   // launches issued per kind since the library was loaded

static int run_op(const ProgramOp& op, const int64_t* a, cudaStream_t s) {
  if (op.kind > 0 && op.kind < kOpKinds) ++g_kind_launches[op.kind];
  switch (op.kind) {
    case kOpAddRmsNorm:   // dtype, resid, branch, ids, table, rows, weight, eps, out, n_rows, H
      if (op.n_args != 11) return TM_ERR_PROGRAM;
      return tm_add_rmsnorm((int)a[0], as_ptr<float>(a[1]), as_ptr<const void>(a[2]), nullptr, 0, 0, as_ptr<const int>(a[3]),
                            as_ptr<const void>(a[4]), as_ptr<const int>(a[5]), as_ptr<const float>(a[6]), as_float(a[7]),
                            as_ptr<void>(a[8]), (int)a[9], (int)a[10], s);
    case kOpGemmBf16:     // x, w, out, T, N, K, out_f32
      if (op.n_args != 7) return TM_ERR_PROGRAM;
      return gemm_bf16(as_ptr<const void>(a[0]), as_ptr<const void>(a[1]), as_ptr<void>(a[2]), (int)a[3], (int)a[4], (int)a[5],
                       (int)a[6], s);
    case kOpQkvRopeWrite:  // in_dtype, dtype, qkv, bias, positions, cos, sin, slot_map, q_out, kcache, vcache, T, nh, nkv, D,
                           // n_pos, error
      if (op.n_args != 17) return TM_ERR_PROGRAM;
      return tm_qkv_rope_write((int)a[0], (int)a[1], as_ptr<const void>(a[2]), as_ptr<const float>(a[3]), as_ptr<const int>(a[4]),
                               as_ptr<const float>(a[5]), as_ptr<const float>(a[6]), as_ptr<const int>(a[7]), as_ptr<void>(a[8]),
                               as_ptr<void>(a[9]), as_ptr<void>(a[10]), (int)a[11], (int)a[12], (int)a[13], (int)a[14],
                               (int)a[15], as_ptr<int>(a[16]), s);
    case kOpPrefillAttentionTc:  // q, k, v, table, bt_stride, units, n_units, chunk, acc, ml, tile_done, counters, out,
                                 // nh, nkv, D, page, scale, window, error
      if (op.n_args != 20) return TM_ERR_PROGRAM;
      return tm_prefill_attention_tc_bf16(as_ptr<const void>(a[0]), as_ptr<const void>(a[1]), as_ptr<const void>(a[2]),
                                          as_ptr<const int>(a[3]), (int)a[4], as_ptr<const int>(a[5]), (int)a[6], (int)a[7],
                                          as_ptr<float>(a[8]), as_ptr<float>(a[9]), as_ptr<int>(a[10]), as_ptr<int>(a[11]),
                                          as_ptr<void>(a[12]), (int)a[13], (int)a[14], (int)a[15], (int)a[16], as_float(a[17]),
                                          (int)a[18], as_ptr<int>(a[19]), s);
    case kOpPrefillAttention:    // the same without the error word
      if (op.n_args != 19) return TM_ERR_PROGRAM;
      return tm_prefill_attention_bf16(as_ptr<const void>(a[0]), as_ptr<const void>(a[1]), as_ptr<const void>(a[2]),
                                       as_ptr<const int>(a[3]), (int)a[4], as_ptr<const int>(a[5]), (int)a[6], (int)a[7],
                                       as_ptr<float>(a[8]), as_ptr<float>(a[9]), as_ptr<int>(a[10]), as_ptr<int>(a[11]),
                                       as_ptr<void>(a[12]), (int)a[13], (int)a[14], (int)a[15], (int)a[16], as_float(a[17]),
                                       (int)a[18], s);
    case kOpDecodeAttention:     // q, k, v, table, bt_stride, cu_q, kv_before, n_seqs, acc, ml, out, done, nh, nkv, D, page,
                                 // scale, window, split_keys, max_splits, error
      if (op.n_args != 21) return TM_ERR_PROGRAM;
      return tm_decode_attention_bf16(as_ptr<const void>(a[0]), as_ptr<const void>(a[1]), as_ptr<const void>(a[2]),
                                      as_ptr<const int>(a[3]), (int)a[4], as_ptr<const int>(a[5]), as_ptr<const int>(a[6]),
                                      (int)a[7], as_ptr<float>(a[8]), as_ptr<float>(a[9]), as_ptr<void>(a[10]), as_ptr<int>(a[11]),
                                      (int)a[12], (int)a[13], (int)a[14], (int)a[15], as_float(a[16]), (int)a[17], (int)a[18],
                                      (int)a[19], as_ptr<int>(a[20]), s);
    case kOpDecodeAttentionUnits:  // q, k, v, n_pages, table, bt_stride, cu_q, kv_before, units, n_work, max_work, grid, acc, ml,
                                   // out, done, nh, nkv, D, page, scale, window, max_parts, error
      if (op.n_args != 24) return TM_ERR_PROGRAM;
      return tm_decode_attention_units_bf16(
          as_ptr<const void>(a[0]), as_ptr<const void>(a[1]), as_ptr<const void>(a[2]), (long long)a[3],
          as_ptr<const int>(a[4]), (int)a[5], as_ptr<const int>(a[6]), as_ptr<const int>(a[7]), as_ptr<const int>(a[8]),
          as_ptr<const int>(a[9]), (int)a[10], (int)a[11], as_ptr<float>(a[12]), as_ptr<float>(a[13]), as_ptr<void>(a[14]),
          as_ptr<int>(a[15]), (int)a[16], (int)a[17], (int)a[18], (int)a[19], as_float(a[20]), (int)a[21], (int)a[22],
          as_ptr<int>(a[23]), s);
    case kOpSwiglu:       // dtype, gu, out, T, I
      if (op.n_args != 5) return TM_ERR_PROGRAM;
      return tm_swiglu((int)a[0], as_ptr<const void>(a[1]), as_ptr<void>(a[2]), (int)a[3], (int)a[4], s);
    case kOpTcQkvRopeWrite:  // x, ldx, w, bias, positions, cos, sin, slot_map, q_out, kcache, vcache, T, K, nh, nkv, D, n_pos, error
      if (op.n_args != 18) return TM_ERR_PROGRAM;
      return tm_tc_qkv_rope_write(as_ptr<const void>(a[0]), (int)a[1], as_ptr<const void>(a[2]), as_ptr<const float>(a[3]),
                                  as_ptr<const int>(a[4]), as_ptr<const float>(a[5]), as_ptr<const float>(a[6]),
                                  as_ptr<const int>(a[7]), as_ptr<void>(a[8]), as_ptr<void>(a[9]), as_ptr<void>(a[10]),
                                  (int)a[11], (int)a[12], (int)a[13], (int)a[14], (int)a[15], (int)a[16], as_ptr<int>(a[17]), s);
    case kOpTcLinear:     // x, ldx, w, out, ldo, T, N, K, error
      if (op.n_args != 9) return TM_ERR_PROGRAM;
      return tm_tc_linear(as_ptr<const void>(a[0]), (int)a[1], as_ptr<const void>(a[2]), as_ptr<void>(a[3]), (int)a[4],
                          (int)a[5], (int)a[6], (int)a[7], as_ptr<int>(a[8]), s);
    default:
      return TM_ERR_PROGRAM;
  }
}

}  // namespace tmk

extern "C" int tm_program_op_size() { return (int)sizeof(tmk::ProgramOp); }

// Once per process, before the first tm_program_run with a matrix product: `workspace` (device memory that stays
// alive, 32 MiB is what PyTorch gives the library) may be null.
extern "C" int tm_program_setup(void* workspace, long long workspace_bytes) {
  return tmk::cublas_setup(workspace, (size_t)workspace_bytes);
}

// How many launches of each kind (index = kind, 16 values) programs have issued in this process: lets a caller
// check which kernels a step took.
extern "C" int tm_program_kind_launches(long long* out) {
  for (int i = 0; i < tmk::kOpKinds; ++i) out[i] = tmk::g_kind_launches[i];
  return 0;
}

// Walks the list. Returns 0, or the first failing launch's code with its index in report[0] (launches before
// it have been issued); report[1] receives the number of launches issued. Nothing here waits for the GPU.
extern "C" int tm_program_run(const void* ops, int n_ops, const long long* params, int n_params, int* report,
                              cudaStream_t stream) {
  int issued = 0;
  const tmk::ProgramOp* list = static_cast<const tmk::ProgramOp*>(ops);
  int64_t a[tmk::kProgramArgs];
  for (int i = 0; i < n_ops; ++i) {
    const tmk::ProgramOp& op = list[i];
    int rc = 0;
    if (op.n_args < 0 || op.n_args > tmk::kProgramArgs || op.cond >= n_params) {
      rc = TM_ERR_PROGRAM;
    } else if (op.cond < 0 || params[op.cond] != 0) {
      for (int j = 0; j < op.n_args && !rc; ++j) {
        if (op.param_mask >> j & 1u) {
          if (op.arg[j] < 0 || op.arg[j] >= n_params) rc = TM_ERR_PROGRAM;
          else a[j] = params[op.arg[j]];
        } else {
          a[j] = op.arg[j];
        }
      }
      if (!rc) {
        rc = tmk::run_op(op, a, stream);
        ++issued;
      }
    }
    if (rc) {
      if (report) {
        report[0] = i;
        report[1] = issued;
      }
      return rc;
    }
  }
  if (report) report[1] = issued;
  return 0;
}
