// Dense bfloat16 products of steps with many rows, through cuBLASLt with the algorithm chosen by
// measurement. y[M, N] = x[M, K] W[N, K]^T, row-major, float32 accumulation: the product that the
// reference gives to torch (F.linear in engine/model.py of willzeng274/kernel-rush-kawk), which takes
// the first algorithm of the library's heuristic. The heuristic's first choice is not always its best
// one: on a B200, 2,048 rows of the Qwen3-4B gate/up projection take 140 us with it and 131 us with
// another of the eight algorithms it proposes. So, the first time a shape class is seen outside a
// stream capture, every proposed algorithm is timed on the caller's own buffers and the fastest is
// kept for the class; under capture, and for classes not yet timed, the heuristic's first choice runs.
//
// One workspace per device: products of one device are meant to run on one stream at a time, as the
// engine's do. The first call on a device allocates it, so that call must not come under stream capture.
//
// A shape class is (rows rounded up to a multiple of 256, or the exact row count up to 256; N; K;
// the leading dimensions). A plan (descriptors, the heuristic's proposals) is kept per exact shape.
#include "common.cuh"

#include <cublasLt.h>

#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace {

constexpr size_t WORKSPACE_BYTES = 64u << 20;
constexpr int PROPOSALS = 8;

using Shape = std::tuple<int, int, int, int, int, int>;  // M, N, K, ldx, ldw, ldy

struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t w = nullptr, x = nullptr, y = nullptr;
  std::vector<cublasLtMatmulHeuristicResult_t> proposals;
};

struct State {
  std::mutex mu;
  cublasLtHandle_t handle = nullptr;
  void* workspace = nullptr;
  std::map<Shape, Plan> plans;
  std::map<Shape, cublasLtMatmulAlgo_t> chosen;  // by shape class
  std::map<Shape, int> chosen_index;             // for reports: the proposal's index at the time it was chosen
};

// one state per device: a handle and its workspace belong to the device that was current when they were made
State* state() {
  static std::mutex mu;
  static std::map<int, State*> by_device;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  State*& s = by_device[device];
  if (!s) s = new State();  // lives as long as the process
  return s;
}

int row_class(int M) { return M <= 256 ? M : (M + 255) / 256 * 256; }

// In column-major terms: y^T [N x M] = op_T(W as K x N, ld = ldw) * (x as K x M, ld = ldx)
int make_plan(State& s, Plan& p, int M, int N, int K, int ldx, int ldw, int ldy) {
  if (cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return -21;
  const cublasOperation_t t = CUBLAS_OP_T, n = CUBLAS_OP_N;
  cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &t, sizeof t);
  cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &n, sizeof n);
  if (cublasLtMatrixLayoutCreate(&p.w, CUDA_R_16BF, K, N, ldw) != CUBLAS_STATUS_SUCCESS) return -22;
  if (cublasLtMatrixLayoutCreate(&p.x, CUDA_R_16BF, K, M, ldx) != CUBLAS_STATUS_SUCCESS) return -22;
  if (cublasLtMatrixLayoutCreate(&p.y, CUDA_R_16BF, N, M, ldy) != CUBLAS_STATUS_SUCCESS) return -22;
  cublasLtMatmulPreference_t pref;
  if (cublasLtMatmulPreferenceCreate(&pref) != CUBLAS_STATUS_SUCCESS) return -23;
  const size_t ws = WORKSPACE_BYTES;
  cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof ws);
  p.proposals.resize(PROPOSALS);
  int found = 0;
  const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(s.handle, p.op, p.w, p.x, p.y, p.y, pref, PROPOSALS, p.proposals.data(), &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found == 0) return -24;
  p.proposals.resize(found);
  return 0;
}

int run(State& s, const Plan& p, const cublasLtMatmulAlgo_t& algo, const void* x, const void* w, void* y, cudaStream_t stream) {
  const float one = 1.f, zero = 0.f;
  const cublasStatus_t st = cublasLtMatmul(s.handle, p.op, &one, w, p.w, x, p.x, &zero, y, p.y, y, p.y, &algo, s.workspace, WORKSPACE_BYTES, stream);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : -25;
}

}  // namespace

// tune != 0: time the proposals if this shape class has none chosen yet and the stream is not capturing.
// Returns 0, or a negative code; *picked (may be null) receives the index of the proposal that ran, -1 if
// the algorithm came from another shape of the class.
KRK_API int krk_lt_gemm_bf16(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int ldw, int ldy, int tune,
                             int* picked, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  State* sp = state();
  if (!sp) return -20;
  State& s = *sp;
  std::lock_guard<std::mutex> lock(s.mu);
  if (!s.handle) {
    cublasLtHandle_t handle = nullptr;
    if (cublasLtCreate(&handle) != CUBLAS_STATUS_SUCCESS) return -20;
    if (cudaMalloc(&s.workspace, WORKSPACE_BYTES) != cudaSuccess) {
      cublasLtDestroy(handle);
      s.workspace = nullptr;
      return -20;
    }
    s.handle = handle;
  }
  const Shape shape{M, N, K, ldx, ldw, ldy};
  auto it = s.plans.find(shape);
  if (it == s.plans.end()) {
    Plan p;
    const int rc = make_plan(s, p, M, N, K, ldx, ldw, ldy);
    if (rc) {
      if (p.op) cublasLtMatmulDescDestroy(p.op);
      if (p.w) cublasLtMatrixLayoutDestroy(p.w);
      if (p.x) cublasLtMatrixLayoutDestroy(p.x);
      if (p.y) cublasLtMatrixLayoutDestroy(p.y);
      return rc;
    }
    it = s.plans.emplace(shape, std::move(p)).first;
  }
  const Plan& plan = it->second;
  const Shape cls{row_class(M), N, K, ldx, ldw, ldy};
  auto chosen = s.chosen.find(cls);
  if (chosen != s.chosen.end()) {
    // an algorithm timed on another row count of the class: use it if the library accepts it for this one
    cublasLtMatmulHeuristicResult_t check;
    if (cublasLtMatmulAlgoCheck(s.handle, plan.op, plan.w, plan.x, plan.y, plan.y, &chosen->second, &check) == CUBLAS_STATUS_SUCCESS &&
        check.workspaceSize <= WORKSPACE_BYTES) {
      if (picked) *picked = row_class(M) == M ? s.chosen_index[cls] : -1;
      return run(s, plan, chosen->second, x, w, y, stream);
    }
    if (picked) *picked = 0;
    return run(s, plan, plan.proposals[0].algo, x, w, y, stream);
  }
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(stream, &capturing);
  if (!tune || capturing != cudaStreamCaptureStatusNone || plan.proposals.size() == 1) {
    if (picked) *picked = 0;
    return run(s, plan, plan.proposals[0].algo, x, w, y, stream);
  }
  // time every proposal: one warm-up run and the fastest of three timed ones, on the caller's stream and buffers
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -26;
  int best = 0;
  float best_ms = 1e30f;
  for (int a = 0; a < (int)plan.proposals.size(); ++a) {
    if (plan.proposals[a].state != CUBLAS_STATUS_SUCCESS || plan.proposals[a].workspaceSize > WORKSPACE_BYTES) continue;
    if (run(s, plan, plan.proposals[a].algo, x, w, y, stream)) continue;
    float fastest = 1e30f;
    bool ok = true;
    for (int rep = 0; rep < 3 && ok; ++rep) {
      cudaEventRecord(e0, stream);
      ok = run(s, plan, plan.proposals[a].algo, x, w, y, stream) == 0;
      cudaEventRecord(e1, stream);
      if (cudaEventSynchronize(e1) != cudaSuccess) { cudaEventDestroy(e0); cudaEventDestroy(e1); return -27; }
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      fastest = ms < fastest ? ms : fastest;
    }
    if (ok && fastest < best_ms) { best_ms = fastest; best = a; }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  s.chosen[cls] = plan.proposals[best].algo;
  s.chosen_index[cls] = best;
  if (picked) *picked = best;
  return run(s, plan, plan.proposals[best].algo, x, w, y, stream);
}

// How many shape classes have a measured choice, and how many of them kept the heuristic's first proposal.
KRK_API int krk_lt_gemm_report(int* classes, int* kept_first) {
  State* sp = state();
  if (!sp) return -20;
  State& s = *sp;
  std::lock_guard<std::mutex> lock(s.mu);
  *classes = (int)s.chosen.size();
  int first = 0;
  for (const auto& kv : s.chosen_index) first += kv.second == 0;
  *kept_first = first;
  return 0;
}
