// The vendor library's matrix product (cuBLASLt) with a MEASURED choice of algorithm.
//
// out[M, N] = x[M, K] . W[N, K]^T, bfloat16 in, 32-bit accumulate, bfloat16 or float32 out.  The library's own
// choice for a shape is the first entry of its heuristic list; for the few-row products of a decode step, which
// only stream W once, the entries further down are sometimes faster.  On the first call for a shape outside a
// stream capture the candidates are timed (L2 flushed before each run) and the fastest is kept for the life of
// the process; during a capture an untimed shape takes the list's first entry.
//
// The library is reached through dlopen of its soname, which resolves to the copy the process has already loaded
// (PyTorch's); nothing is linked at build time.
#include <cublasLt.h>
#include <dlfcn.h>

#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "common.cuh"

// reads `n` 16-byte words and writes nothing (the condition never holds for a zero-filled buffer)
__global__ void lt_flush_read_kernel(const uint4* __restrict__ src, long long n, uint4* sink) {
  unsigned acc = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    acc |= v.x | v.y | v.z | v.w;
  }
  if (acc == 0xFFFFFFFFu) sink[0] = make_uint4(acc, 0, 0, 0);
}

namespace {

struct LtApi {
  void* lib = nullptr;
  decltype(&cublasLtCreate) create = nullptr;
  decltype(&cublasLtMatmulDescCreate) desc_create = nullptr;
  decltype(&cublasLtMatmulDescSetAttribute) desc_set = nullptr;
  decltype(&cublasLtMatrixLayoutCreate) layout_create = nullptr;
  decltype(&cublasLtMatmulPreferenceCreate) pref_create = nullptr;
  decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set = nullptr;
  decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy = nullptr;
  decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic = nullptr;
  decltype(&cublasLtMatmul) matmul = nullptr;
  cublasLtHandle_t handle = nullptr;
  bool ok = false;
};

LtApi& lt_api() {
  static LtApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  api.lib = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_LOCAL);
  if (api.lib == nullptr) api.lib = dlopen("libcublasLt.so", RTLD_NOW | RTLD_LOCAL);
  if (api.lib == nullptr) return api;
#define LT_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.lib, name))
  LT_SYM(create, "cublasLtCreate");
  LT_SYM(desc_create, "cublasLtMatmulDescCreate");
  LT_SYM(desc_set, "cublasLtMatmulDescSetAttribute");
  LT_SYM(layout_create, "cublasLtMatrixLayoutCreate");
  LT_SYM(pref_create, "cublasLtMatmulPreferenceCreate");
  LT_SYM(pref_set, "cublasLtMatmulPreferenceSetAttribute");
  LT_SYM(pref_destroy, "cublasLtMatmulPreferenceDestroy");
  LT_SYM(heuristic, "cublasLtMatmulAlgoGetHeuristic");
  LT_SYM(matmul, "cublasLtMatmul");
#undef LT_SYM
  if (!api.create || !api.desc_create || !api.desc_set || !api.layout_create || !api.pref_create || !api.pref_set ||
      !api.pref_destroy || !api.heuristic || !api.matmul)
    return api;
  if (api.create(&api.handle) != CUBLAS_STATUS_SUCCESS) return api;
  api.ok = true;
  return api;
}

struct LtPlan {
  cublasLtMatmulDesc_t desc = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  std::vector<cublasLtMatmulHeuristicResult_t> cands;
  int chosen = 0;
  bool tuned = false;
  float best_us = 0.f, first_us = 0.f;
};

typedef std::tuple<int, int, int, int, long long> LtKey;  // M, N, K, out_f32, workspace bytes
std::map<LtKey, LtPlan> g_plans;
std::mutex g_lt_mutex;
int g_lt_last_chosen = -1, g_lt_last_cands = 0;
float g_lt_last_best_us = 0.f, g_lt_last_first_us = 0.f;

bool lt_make_plan(LtApi& api, LtPlan& plan, int M, int N, int K, int out_f32, long long ws_bytes) {
  // Row-major out[M, N] = x[M, K] W[N, K]^T is, read column-major, out^T[N, M] = W^T(K x N)^T . x^T(K x M).
  if (api.desc_create(&plan.desc, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return false;
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  if (api.desc_set(plan.desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)) != CUBLAS_STATUS_SUCCESS ||
      api.desc_set(plan.desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)) != CUBLAS_STATUS_SUCCESS)
    return false;
  if (api.layout_create(&plan.a, CUDA_R_16BF, K, N, K) != CUBLAS_STATUS_SUCCESS ||
      api.layout_create(&plan.b, CUDA_R_16BF, K, M, K) != CUBLAS_STATUS_SUCCESS ||
      api.layout_create(&plan.c, out_f32 ? CUDA_R_32F : CUDA_R_16BF, N, M, N) != CUBLAS_STATUS_SUCCESS)
    return false;
  cublasLtMatmulPreference_t pref = nullptr;
  if (api.pref_create(&pref) != CUBLAS_STATUS_SUCCESS) return false;
  const size_t ws = (size_t)ws_bytes;
  api.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof(ws));
  plan.cands.resize(24);
  int found = 0;
  const cublasStatus_t st = api.heuristic(api.handle, plan.desc, plan.a, plan.b, plan.c, plan.c, pref, (int)plan.cands.size(),
                                          plan.cands.data(), &found);
  api.pref_destroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found <= 0) return false;
  plan.cands.resize(found);
  return true;
}

cublasStatus_t lt_run(LtApi& api, const LtPlan& plan, int which, const void* x, const void* w, void* out, void* ws,
                      long long ws_bytes, cudaStream_t st) {
  const float alpha = 1.f, beta = 0.f;
  const cublasLtMatmulHeuristicResult_t& h = plan.cands[which];
  return api.matmul(api.handle, plan.desc, &alpha, w, plan.a, x, plan.b, &beta, out, plan.c, out, plan.c, &h.algo, ws,
                    h.workspaceSize <= (size_t)ws_bytes ? h.workspaceSize : 0, st);
}

}  // namespace

// 1 when the library could be opened and a handle made.
extern "C" int ullm_lt_available(void) { return lt_api().ok ? 1 : 0; }

// What the last timed choice was: index in the heuristic list, candidates, microseconds of the chosen one and
// of the list's first entry.
extern "C" void ullm_lt_last_choice(int* chosen, int* cands, float* best_us, float* first_us) {
  *chosen = g_lt_last_chosen;
  *cands = g_lt_last_cands;
  *best_us = g_lt_last_best_us;
  *first_us = g_lt_last_first_us;
}

// `tune`: time the candidates at the first call for a shape (never during a stream capture).  `flush`: a buffer
// larger than L2 that is cleared before every timed run, so that W comes from memory as it does in a decode step.
extern "C" int ullm_lt_linear(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, void* workspace,
                              long long ws_bytes, int tune, void* flush, long long flush_bytes, void* stream) {
  LtApi& api = lt_api();
  if (!api.ok) return ULLM_ERR_UNSUPPORTED;
  if (M <= 0 || N <= 0 || K <= 0) return ULLM_ERR_BAD_SIZE;
  if (K % 8 || (!out_f32 && N % 8) || (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15)) return ULLM_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  std::lock_guard<std::mutex> lock(g_lt_mutex);
  const LtKey key(M, N, K, out_f32, ws_bytes);
  auto it = g_plans.find(key);
  if (it == g_plans.end()) {
    LtPlan plan;
    if (!lt_make_plan(api, plan, M, N, K, out_f32, ws_bytes)) return ULLM_ERR_UNSUPPORTED;
    it = g_plans.emplace(key, plan).first;
  }
  LtPlan& plan = it->second;
  if (tune && !plan.tuned && plan.cands.size() > 1) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
      cudaEvent_t e0, e1;
      if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
        // Rounds over all candidates (so that a drift of the clocks touches them alike), the fastest run of each.
        // Before every run the flush buffer is READ: L2 then holds clean lines of something else, as it does
        // when the product runs inside a step (a memset would leave dirty lines to be written back meanwhile).
        const int n = (int)plan.cands.size();
        std::vector<float> t_min(n, 1e30f);
        std::vector<char> failed(n, 0);
        // Few rows (the product streams W once: memory-bound): one launch per timing, W cold.  Many rows (bound by
        // the tensor cores, W re-read from L2 by the kernel itself): three launches back to back per timing and no
        // flush, so that the clocks are those of sustained work.
        const bool cold = M < 512 && flush != nullptr;
        const int reps = cold ? 1 : 3;
        const int rounds = cold ? 12 : 6;  // cold runs are short and noisier: more of them
        for (int r = 0; r < rounds; ++r) {
          for (int i = 0; i < n; ++i) {
            if (failed[i]) continue;
            if (cold) lt_flush_read_kernel<<<1024, 256, 0, st>>>((const uint4*)flush, flush_bytes / 16, (uint4*)flush);
            cudaEventRecord(e0, st);
            bool bad = false;
            for (int k = 0; k < reps && !bad; ++k)
              bad = lt_run(api, plan, i, x, w, out, workspace, ws_bytes, st) != CUBLAS_STATUS_SUCCESS;
            cudaEventRecord(e1, st);
            if (cudaEventSynchronize(e1) != cudaSuccess) bad = true;
            float ms = 0.f;
            if (!bad && r > 0 && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && ms / reps < t_min[i]) t_min[i] = ms / reps;
            if (bad) failed[i] = 1;
          }
        }
        float best = 1e30f, first = t_min[0];
        int best_i = 0;
        for (int i = 0; i < n; ++i)
          if (!failed[i] && t_min[i] < best) best = t_min[i], best_i = i;
        if (failed[0]) first = best;
        // the list's first entry stays unless another one is faster by more than 3 %
        if (best_i != 0 && !failed[0] && best > first * 0.97f) best_i = 0, best = first;
        plan.chosen = best_i;
        plan.best_us = best * 1000.f;
        plan.first_us = first * 1000.f;
        plan.tuned = true;
        g_lt_last_chosen = best_i;
        g_lt_last_cands = (int)plan.cands.size();
        g_lt_last_best_us = plan.best_us;
        g_lt_last_first_us = plan.first_us;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
      }
    }
  }
  if (lt_run(api, plan, plan.chosen, x, w, out, workspace, ws_bytes, st) != CUBLAS_STATUS_SUCCESS) return ULLM_ERR_LAUNCH;
  return ULLM_OK;
}
