// The vendor library's product for bfloat16 operands, called from this library's own host code.
//
// out[M, N] = x[M, K] * W[N, K]^T, float32 accumulation, bfloat16 or float32 out: the products of
// more than 32 rows that no hand-written kernel of this package is the default for (QKV, O, down and
// the head in prompt-sized steps). The reference's engine calls the same vendor library for every
// projection (pegainfer-kernels/csrc/shared/linear.cu:312-362, cublasGemmEx with CUBLAS_COMPUTE_32F).
//
// cuBLASLt is looked up at run time (dlopen / dlsym): the copy that the process has loaded already
// (torch's) if there is one, else the path given to oi_library_gemm_init. Nothing is linked at build
// time, so the package builds and loads on a machine without the library; a product that needs it
// then fails with a message, and the dispatcher (host_step.cu) uses the hand-written tcgen05 kernel instead.
// A plan (operation and layout descriptors, the algorithm the library's heuristic ranks first) is made
// once per shape and kept, so a call costs one cublasLtMatmul. Partial sums of a split K are never
// rounded to the output type: reduction schemes that do so are excluded from the search.
#include <cublasLt.h>
#include <dlfcn.h>

#include <mutex>
#include <unordered_map>

#include "oi_api.h"

namespace {

struct Api {
  void* handle = nullptr;
  cublasStatus_t (*create)(cublasLtHandle_t*) = nullptr;
  cublasStatus_t (*desc_create)(cublasLtMatmulDesc_t*, cublasComputeType_t, cudaDataType_t) = nullptr;
  cublasStatus_t (*desc_set)(cublasLtMatmulDesc_t, cublasLtMatmulDescAttributes_t, const void*, size_t) = nullptr;
  cublasStatus_t (*layout_create)(cublasLtMatrixLayout_t*, cudaDataType, uint64_t, uint64_t, int64_t) = nullptr;
  cublasStatus_t (*pref_create)(cublasLtMatmulPreference_t*) = nullptr;
  cublasStatus_t (*pref_set)(cublasLtMatmulPreference_t, cublasLtMatmulPreferenceAttributes_t, const void*, size_t) = nullptr;
  cublasStatus_t (*pref_destroy)(cublasLtMatmulPreference_t) = nullptr;
  cublasStatus_t (*heuristic)(cublasLtHandle_t, cublasLtMatmulDesc_t, cublasLtMatrixLayout_t, cublasLtMatrixLayout_t,
                              cublasLtMatrixLayout_t, cublasLtMatrixLayout_t, cublasLtMatmulPreference_t, int,
                              cublasLtMatmulHeuristicResult_t*, int*) = nullptr;
  cublasStatus_t (*matmul)(cublasLtHandle_t, cublasLtMatmulDesc_t, const void*, const void*, cublasLtMatrixLayout_t,
                           const void*, cublasLtMatrixLayout_t, const void*, const void*, cublasLtMatrixLayout_t, void*,
                           cublasLtMatrixLayout_t, const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t) = nullptr;
};

struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
  size_t workspace = 0;
};

struct Key {
  int M, N, K, out_dtype;
  long long ldx, ldw, ldc;
  int align;   // bytes to which x, W and out are all aligned (16 ... 256): an algorithm is chosen for what it may assume
  bool operator==(const Key& o) const {
    return M == o.M && N == o.N && K == o.K && out_dtype == o.out_dtype && ldx == o.ldx && ldw == o.ldw && ldc == o.ldc &&
           align == o.align;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = 1469598103934665603ull;
    for (long long v : {(long long)k.M, (long long)k.N, (long long)k.K, (long long)k.out_dtype, k.ldx, k.ldw, k.ldc, (long long)k.align})
      h = (h ^ (size_t)v) * 1099511628211ull;
    return h;
  }
};

Api g_api;
cublasLtHandle_t g_lt = nullptr;
void* g_workspace = nullptr;
size_t g_workspace_bytes = 0;
std::mutex g_mutex;
std::unordered_map<Key, Plan, KeyHash> g_plans;

template <typename F>
bool sym(void* handle, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(handle, name));
  return *out != nullptr;
}

}  // namespace

// Whether oi_library_gemm can be called.
OI_API int oi_library_gemm_ready() { return g_lt != nullptr ? 1 : 0; }

// Find cuBLASLt and create a handle. `path`: where to load the library from if the process has not loaded
// one (may be null: the dynamic linker's search path is tried). `workspace`: device memory the library may
// use as scratch, owned by the caller and kept alive as long as products are computed; all products share
// it, so they must be issued on one stream at a time.
OI_API int oi_library_gemm_init(const char* path, void* workspace, long long workspace_bytes) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_workspace = workspace;
  g_workspace_bytes = workspace_bytes > 0 ? (size_t)workspace_bytes : 0;
  if (g_lt) return OI_OK;
  void* h = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_NOLOAD);
  if (!h && path && *path) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) h = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_LOCAL);
  if (!h) h = dlopen("libcublasLt.so", RTLD_NOW | RTLD_LOCAL);
  OI_REQUIRE(h != nullptr, "library_gemm: cuBLASLt could not be loaded (%s)", dlerror());
  Api a;
  a.handle = h;
  const bool ok = sym(h, "cublasLtCreate", &a.create) && sym(h, "cublasLtMatmulDescCreate", &a.desc_create) &&
                  sym(h, "cublasLtMatmulDescSetAttribute", &a.desc_set) &&
                  sym(h, "cublasLtMatrixLayoutCreate", &a.layout_create) &&
                  sym(h, "cublasLtMatmulPreferenceCreate", &a.pref_create) &&
                  sym(h, "cublasLtMatmulPreferenceSetAttribute", &a.pref_set) &&
                  sym(h, "cublasLtMatmulPreferenceDestroy", &a.pref_destroy) &&
                  sym(h, "cublasLtMatmulAlgoGetHeuristic", &a.heuristic) && sym(h, "cublasLtMatmul", &a.matmul);
  OI_REQUIRE(ok, "library_gemm: the loaded cuBLASLt lacks an entry point this package calls");
  cublasLtHandle_t lt = nullptr;
  const cublasStatus_t st = a.create(&lt);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: cublasLtCreate failed (%d)", (int)st);
  g_api = a;
  g_lt = lt;
  return OI_OK;
}

static int make_plan(const Key& k, Plan* plan) {
  const Api& a = g_api;
  Plan p;
  cublasStatus_t st = a.desc_create(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: operation descriptor (%d)", (int)st);
  // Row-major out[M, N] = x[M, K] W[N, K]^T is, column-major, out^T[N, M] = (W as K x N)^T (x as K x M).
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  a.desc_set(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
  a.desc_set(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
  const cudaDataType_t out_type = k.out_dtype == OI_BF16 ? CUDA_R_16BF : CUDA_R_32F;
  st = a.layout_create(&p.a, CUDA_R_16BF, (uint64_t)k.K, (uint64_t)k.N, (int64_t)k.ldw);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: layout of W (%d)", (int)st);
  st = a.layout_create(&p.b, CUDA_R_16BF, (uint64_t)k.K, (uint64_t)k.M, (int64_t)k.ldx);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: layout of x (%d)", (int)st);
  st = a.layout_create(&p.c, out_type, (uint64_t)k.N, (uint64_t)k.M, (int64_t)k.ldc);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: layout of out (%d)", (int)st);
  cublasLtMatmulPreference_t pref = nullptr;
  st = a.pref_create(&pref);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: preference (%d)", (int)st);
  const uint64_t ws = g_workspace_bytes;
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof(ws));
  const uint32_t align = (uint32_t)k.align;
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_MIN_ALIGNMENT_A_BYTES, &align, sizeof(align));
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_MIN_ALIGNMENT_B_BYTES, &align, sizeof(align));
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_MIN_ALIGNMENT_C_BYTES, &align, sizeof(align));
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_MIN_ALIGNMENT_D_BYTES, &align, sizeof(align));
  // partial sums of a split K stay in the compute type (float32), never in the output type
  const uint32_t schemes = CUBLASLT_REDUCTION_SCHEME_NONE | CUBLASLT_REDUCTION_SCHEME_INPLACE | CUBLASLT_REDUCTION_SCHEME_COMPUTE_TYPE;
  a.pref_set(pref, CUBLASLT_MATMUL_PREF_REDUCTION_SCHEME_MASK, &schemes, sizeof(schemes));
  cublasLtMatmulHeuristicResult_t result;
  int found = 0;
  st = a.heuristic(g_lt, p.op, p.a, p.b, p.c, p.c, pref, 1, &result, &found);
  a.pref_destroy(pref);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS && found > 0, "library_gemm: no algorithm for M=%d N=%d K=%d (%d)", k.M, k.N, k.K,
             (int)st);
  p.algo = result.algo;
  p.workspace = result.workspaceSize;
  *plan = p;
  return OI_OK;
}

// x: [M, K] bfloat16 (row stride ldx), W: [N, K] bfloat16 (row stride ldw), out: [M, N] bfloat16 or float32
// (row stride ldc).
OI_API int oi_library_gemm(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
                           long long ldw, int M, int N, int K, void* stream) {
  OI_REQUIRE(g_lt != nullptr, "library_gemm: not initialised (oi_library_gemm_init)");
  OI_REQUIRE(M >= 1 && N >= 1 && K >= 1 && ldx >= K && ldw >= K && ldc >= N, "library_gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  OI_REQUIRE(out_dtype == OI_BF16 || out_dtype == OI_F32, "library_gemm: unknown output dtype code %d", out_dtype);
  int align = 256;
  for (const void* ptr : {x, W, (const void*)out})
    while (align > 1 && ((uintptr_t)ptr & (uintptr_t)(align - 1))) align >>= 1;
  OI_REQUIRE(align >= 2, "library_gemm: operands must be aligned to their element size");
  const Key key{M, N, K, out_dtype, ldx, ldw, ldc, align};
  Plan plan;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_plans.find(key);
    if (it == g_plans.end()) {
      if (g_plans.size() > 4096) g_plans.clear();   // descriptors of shapes long gone; a few hundred bytes each
      Plan fresh;
      const int rc = make_plan(key, &fresh);
      if (rc != OI_OK) return rc;
      it = g_plans.emplace(key, fresh).first;
    }
    plan = it->second;
  }
  const float one = 1.f, zero = 0.f;
  const cublasStatus_t st = g_api.matmul(g_lt, plan.op, &one, W, plan.a, x, plan.b, &zero, out, plan.c, out, plan.c,
                                         &plan.algo, g_workspace, plan.workspace <= g_workspace_bytes ? g_workspace_bytes : 0,
                                         (cudaStream_t)stream);
  OI_REQUIRE(st == CUBLAS_STATUS_SUCCESS, "library_gemm: cublasLtMatmul failed (%d) for M=%d N=%d K=%d", (int)st, M, N, K);
  return OI_OK;
}
