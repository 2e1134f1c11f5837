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
// A shape class is (the row count up to 256 rows, its next multiple of 256 up to 2,048, its next power of
// two beyond; N; K; the leading dimensions): a serving process meets a bounded number of classes, and a
// class is measured on 4,096 rows at most. A plan (descriptors, the heuristic's proposals) is kept per
// exact shape.
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

struct Choice {
  cublasLtMatmulAlgo_t algo;
  int index;  // among the proposals for `rows` rows
  int rows;   // the row count it was measured on
};

struct State {
  std::mutex mu;
  cublasLtHandle_t handle = nullptr;
  void* workspace = nullptr;
  std::map<Shape, Plan> plans;
  std::map<Shape, Choice> chosen;  // by shape class
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

constexpr int MEASURED_ROWS = 4096;
constexpr size_t MAX_PLANS = 4096;

// exact up to 256 rows (decode batch sizes), multiples of 256 up to 2,048, powers of two beyond
int row_class(int M) {
  if (M <= 256) return M;
  if (M <= 2048) return (M + 255) / 256 * 256;
  int c = 4096;
  while (c < M && c < (1 << 30)) c *= 2;
  return c;
}

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

// the plan of an exact shape, made at its first use
int plan_for(State& s, int M, int N, int K, int ldx, int ldw, int ldy, const Plan** out) {
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
  *out = &it->second;
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
// the algorithm was measured on another row count.
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
  if (s.plans.size() > MAX_PLANS) {  // a process that has met this many row counts starts its list over
    for (auto& kv : s.plans) {
      cublasLtMatmulDescDestroy(kv.second.op);
      cublasLtMatrixLayoutDestroy(kv.second.w);
      cublasLtMatrixLayoutDestroy(kv.second.x);
      cublasLtMatrixLayoutDestroy(kv.second.y);
    }
    s.plans.clear();
  }
  const Plan* plan = nullptr;
  int rc = plan_for(s, M, N, K, ldx, ldw, ldy, &plan);
  if (rc) return rc;
  const Shape cls{row_class(M), N, K, ldx, ldw, ldy};
  auto chosen = s.chosen.find(cls);
  if (chosen == s.chosen.end()) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &capturing);
    if (!tune || capturing != cudaStreamCaptureStatusNone) {
      if (picked) *picked = 0;
      return run(s, *plan, plan->proposals[0].algo, x, w, y, stream);
    }
    // Time every proposal on the caller's stream and buffers: one warm-up run and the faster of two timed ones.
    // Long steps are measured on their first MEASURED_ROWS rows, so that a new class costs a bounded time
    // (the runs write into y, which the real product then overwrites).
    const int rows = M < MEASURED_ROWS ? M : MEASURED_ROWS;
    const Plan* trial = plan;
    if (rows != M && (rc = plan_for(s, rows, N, K, ldx, ldw, ldy, &trial))) return rc;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -26;
    int best = 0;
    float best_ms = 1e30f;
    for (int a = 0; a < (int)trial->proposals.size(); ++a) {
      if (trial->proposals[a].state != CUBLAS_STATUS_SUCCESS || trial->proposals[a].workspaceSize > WORKSPACE_BYTES) continue;
      if (run(s, *trial, trial->proposals[a].algo, x, w, y, stream)) continue;
      float fastest = 1e30f;
      bool ok = true;
      for (int rep = 0; rep < 2 && ok; ++rep) {
        cudaEventRecord(e0, stream);
        ok = run(s, *trial, trial->proposals[a].algo, x, w, y, stream) == 0;
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
    chosen = s.chosen.emplace(cls, Choice{trial->proposals[best].algo, best, rows}).first;
  }
  // an algorithm measured on another row count runs if the library accepts it for this one
  const Choice& c = chosen->second;
  if (c.rows == M) {
    if (picked) *picked = c.index;
    return run(s, *plan, c.algo, x, w, y, stream);
  }
  cublasLtMatmulHeuristicResult_t check;
  if (cublasLtMatmulAlgoCheck(s.handle, plan->op, plan->w, plan->x, plan->y, plan->y, &c.algo, &check) == CUBLAS_STATUS_SUCCESS &&
      check.workspaceSize <= WORKSPACE_BYTES) {
    if (picked) *picked = -1;
    return run(s, *plan, c.algo, x, w, y, stream);
  }
  if (picked) *picked = 0;
  return run(s, *plan, plan->proposals[0].algo, x, w, y, stream);
}

// How many shape classes have a measured choice, and how many of them kept the heuristic's first proposal.
KRK_API int krk_lt_gemm_report(int* classes, int* kept_first) {
  State* sp = state();
  if (!sp) return -20;
  State& s = *sp;
  std::lock_guard<std::mutex> lock(s.mu);
  *classes = (int)s.chosen.size();
  int first = 0;
  for (const auto& kv : s.chosen) first += kv.second.index == 0;
  *kept_first = first;
  return 0;
}
