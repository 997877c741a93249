// Library matrix product for steps of many tokens, called without the tensor library in between:
//   out[M, N] = x[M, K] . w[N, K]^T, bfloat16 in, float32 accumulate, bfloat16 or float32 out,
// through cuBLASLt with the algorithm chosen once per (N, K, output type, size class of M) and
// kept.  A serving step has a new token count nearly every time; asked shape by shape, the
// library searches its heuristics again for each (about 40 us of host time per product, 4 ms per
// step of a 26-layer model), which is more than such a step's kernels take to launch.
//
// The library is the one the process already holds (it is opened by name, not linked).
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <map>
#include <mutex>
#include <tuple>

namespace {

struct LtApi {
  decltype(&cublasLtCreate) create;
  decltype(&cublasLtMatmulDescCreate) desc_create;
  decltype(&cublasLtMatmulDescSetAttribute) desc_set;
  decltype(&cublasLtMatrixLayoutCreate) layout_create;
  decltype(&cublasLtMatrixLayoutDestroy) layout_destroy;
  decltype(&cublasLtMatmulPreferenceCreate) pref_create;
  decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set;
  decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy;
  decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic;
  decltype(&cublasLtMatmul) matmul;
  cublasLtHandle_t handle = nullptr;
  cublasLtMatmulDesc_t op = nullptr;  // transa = T, transb = N, float32 compute and scale
  bool ok = false;
};

LtApi* lt_api() {
  static LtApi api;
  static bool tried = false;
  if (tried) return api.ok ? &api : nullptr;
  tried = true;
  void* lib = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_NOLOAD);
  if (!lib) lib = dlopen("libcublasLt.so.12", RTLD_NOW);
  if (!lib) lib = dlopen("/usr/local/cuda/lib64/libcublasLt.so.12", RTLD_NOW);
  if (!lib) lib = dlopen("libcublasLt.so", RTLD_NOW);
  if (!lib) return nullptr;
#define SB_SYM(field, name)                                    \
  api.field = (decltype(api.field))dlsym(lib, #name);          \
  if (!api.field) return nullptr;
  SB_SYM(create, cublasLtCreate)
  SB_SYM(desc_create, cublasLtMatmulDescCreate)
  SB_SYM(desc_set, cublasLtMatmulDescSetAttribute)
  SB_SYM(layout_create, cublasLtMatrixLayoutCreate)
  SB_SYM(layout_destroy, cublasLtMatrixLayoutDestroy)
  SB_SYM(pref_create, cublasLtMatmulPreferenceCreate)
  SB_SYM(pref_set, cublasLtMatmulPreferenceSetAttribute)
  SB_SYM(pref_destroy, cublasLtMatmulPreferenceDestroy)
  SB_SYM(heuristic, cublasLtMatmulAlgoGetHeuristic)
  SB_SYM(matmul, cublasLtMatmul)
#undef SB_SYM
  if (api.create(&api.handle) != CUBLAS_STATUS_SUCCESS) return nullptr;
  if (api.desc_create(&api.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return nullptr;
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  if (api.desc_set(api.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)) != CUBLAS_STATUS_SUCCESS) return nullptr;
  if (api.desc_set(api.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)) != CUBLAS_STATUS_SUCCESS) return nullptr;
  api.ok = true;
  return &api;
}

// Row-major out[M, N] = x . w^T is, column-major, out^T[N, M] = op_T(w as [K, N]) . (x as [K, M]):
// M is only the number of columns of two operands, so an algorithm found for one M serves others.
struct Layouts {
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
};

bool make_layouts(LtApi* api, int M, int N, int K, bool out_f32, Layouts& l) {
  return api->layout_create(&l.a, CUDA_R_16BF, K, N, K) == CUBLAS_STATUS_SUCCESS &&
         api->layout_create(&l.b, CUDA_R_16BF, K, M, K) == CUBLAS_STATUS_SUCCESS &&
         api->layout_create(&l.c, out_f32 ? CUDA_R_32F : CUDA_R_16BF, N, M, N) == CUBLAS_STATUS_SUCCESS;
}

void drop_layouts(LtApi* api, Layouts& l) {
  if (l.a) api->layout_destroy(l.a);
  if (l.b) api->layout_destroy(l.b);
  if (l.c) api->layout_destroy(l.c);
}

// Size classes of M: up to 64, then powers of two.  The class's largest M stands for it.
int size_class(int M) {
  int c = 64;
  while (c < M && c < (1 << 30)) c <<= 1;
  return c;
}

struct Chosen {
  cublasLtMatmulAlgo_t algo;
  size_t workspace;
};

std::mutex g_mutex;
std::map<std::tuple<int, int, int, int, long long>, Chosen> g_chosen;

bool choose(LtApi* api, int M, int N, int K, bool out_f32, size_t workspace_bytes, Chosen& out) {
  Layouts l;
  bool found = false;
  if (make_layouts(api, M, N, K, out_f32, l)) {
    cublasLtMatmulPreference_t pref = nullptr;
    if (api->pref_create(&pref) == CUBLAS_STATUS_SUCCESS) {
      api->pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes, sizeof(workspace_bytes));
      cublasLtMatmulHeuristicResult_t result;
      int count = 0;
      if (api->heuristic(api->handle, api->op, l.a, l.b, l.c, l.c, pref, 1, &result, &count) ==
              CUBLAS_STATUS_SUCCESS && count > 0) {
        out.algo = result.algo;
        out.workspace = result.workspaceSize;
        found = true;
      }
      api->pref_destroy(pref);
    }
  }
  drop_layouts(api, l);
  return found;
}

}  // namespace

// Returns 0, -9 when the library or an algorithm is not to be had (the caller then goes through
// the tensor library), or a positive cuBLAS status.
extern "C" int sb_gemm_library_bf16(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                    void* workspace, long long workspace_bytes, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K <= 0 || K % 8 != 0 || (N % 8 != 0 && !out_f32) || N % 4 != 0) return -9;  // 16-byte rows for every operand
  std::lock_guard<std::mutex> lock(g_mutex);
  LtApi* api = lt_api();
  if (!api) return -9;
  const int cls = size_class(M);
  const auto key = std::make_tuple(cls, N, K, out_f32, workspace_bytes);
  auto it = g_chosen.find(key);
  if (it == g_chosen.end()) {
    Chosen c;
    if (!choose(api, cls, N, K, out_f32 != 0, (size_t)workspace_bytes, c)) return -9;
    it = g_chosen.emplace(key, c).first;
  }
  Layouts l;
  int rc = -9;
  if (make_layouts(api, M, N, K, out_f32 != 0, l)) {
    const float alpha = 1.0f, beta = 0.0f;
    cublasStatus_t st = api->matmul(api->handle, api->op, &alpha, w, l.a, x, l.b, &beta, out, l.c, out, l.c,
                                    &it->second.algo, workspace, it->second.workspace, stream);
    if (st == CUBLAS_STATUS_NOT_SUPPORTED) {
      // The class's algorithm does not take this M: ask for this very shape (not kept).
      Chosen c;
      if (choose(api, M, N, K, out_f32 != 0, (size_t)workspace_bytes, c))
        st = api->matmul(api->handle, api->op, &alpha, w, l.a, x, l.b, &beta, out, l.c, out, l.c, &c.algo,
                         workspace, c.workspace, stream);
    }
    rc = st == CUBLAS_STATUS_SUCCESS ? 0 : (st == CUBLAS_STATUS_NOT_SUPPORTED ? -9 : (int)st);
  }
  drop_layouts(api, l);
  return rc;
}
