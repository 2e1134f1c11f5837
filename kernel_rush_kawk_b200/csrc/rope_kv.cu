// Per-head q/k RMSNorm + rotate-half RoPE + cache write, one launch.
//
// Input rows are the QKV projection, [rows, (HQ + 2*HKV) * D], heads in the order
// q heads, k heads, v heads (engine/model.py:112-115 of willzeng274/kernel-rush-kawk).
// For every q and k head: r = rsqrt(mean(x^2) + eps); n = round(x*r);
// y = round(w*n); then with the head's halves y1, y2 and the row's cos/sin:
//   out1 = round(round(y1*cos) + round(-y2*sin)), out2 = round(round(y2*cos) + round(y1*sin))
// (engine/kernels/rope.py:19-30). q heads are rewritten in place; k heads go to the
// cache page of the row's position, v heads are copied there raw (rope.py:139-144).
// HKV may be 0: a run that reads another run's cache has queries only.
// One warp per (row, head); the head size is a run-time argument (even, <= 512).
#include "common.cuh"

namespace {

template <typename T>
__global__ void qk_norm_rope_write_kernel(T* __restrict__ qkv, const void* __restrict__ q_gain,
                                          const void* __restrict__ k_gain, int gain_f32, const T* __restrict__ cos_t,
                                          const T* __restrict__ sin_t, const int* __restrict__ row_seq,
                                          const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                                          const int* __restrict__ table, int width, T* __restrict__ k_cache,
                                          T* __restrict__ v_cache, int rows, int HQ, int HKV, int D, float eps,
                                          int n_pos, int* error) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int heads = HQ + 2 * HKV;
  if (item >= (long long)rows * heads) return;
  const int row = (int)(item / heads);
  const int head = (int)(item % heads);
  const int pos = row_pos[row];
  const int half = D / 2;
  T* src = qkv + (size_t)row * heads * D + (size_t)head * D;

  T* dst = src;
  if (head >= HQ) {
    const int kh = (head - HQ) % HKV;
    const int slot = seq_slot[row_seq[row]];
    const int page = page_of(table, width, slot, pos);
    T* cache = head < HQ + HKV ? k_cache : v_cache;
    dst = cache + (((size_t)page * HKV + kh) * KRK_PAGE + (pos % KRK_PAGE)) * D;
  }
  if (head >= HQ + HKV) {  // a value head: raw copy
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  const void* gain = head < HQ ? q_gain : k_gain;
  if (pos < 0 || pos >= n_pos) {
    if (lane == 0 && error) atomicExch(error, 2);
    return;
  }
  // each lane owns the pairs (i, i + half), i = lane, lane + 32, ...
  float sq = 0.f;
  for (int i = lane; i < half; i += 32) {
    const float a = to_float<T>(src[i]), b = to_float<T>(src[i + half]);
    sq += a * a + b * b;
  }
  sq = warp_sum(sq);
  const float r = gain ? rsqrtf(sq / (float)D + eps) : 1.f;
  for (int i = lane; i < half; i += 32) {
    float y1 = to_float<T>(src[i]), y2 = to_float<T>(src[i + half]);
    if (gain) {
      y1 = round_to<T>(load_gain<T>(gain, i, gain_f32) * round_to<T>(y1 * r));
      y2 = round_to<T>(load_gain<T>(gain, i + half, gain_f32) * round_to<T>(y2 * r));
    }
    if (cos_t) {
      const float c = to_float<T>(cos_t[(size_t)pos * half + i]);
      const float s = to_float<T>(sin_t[(size_t)pos * half + i]);
      const float o1 = round_to<T>(y1 * c) + round_to<T>(-y2 * s);
      const float o2 = round_to<T>(y2 * c) + round_to<T>(y1 * s);
      y1 = o1;
      y2 = o2;
    }
    dst[i] = from_float<T>(y1);
    dst[i + half] = from_float<T>(y2);
  }
}

}  // namespace

// gains may be null (no q/k norm); cos/sin may be null (no rotation); the cache
// pointers are unused when HKV == 0.
KRK_API int krk_qk_norm_rope_write(void* qkv, const void* q_gain, const void* k_gain, int gain_f32, const void* cos_t,
                                   const void* sin_t, const int* row_seq, const int* row_pos, const int* seq_slot,
                                   const int* table, int width, void* k_cache, void* v_cache, int rows, int HQ, int HKV,
                                   int D, float eps, int n_pos, int* error, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (D % 2 || D > 4096) return -2;
  const long long items = (long long)rows * (HQ + 2 * HKV);
  const int warps = 8;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(qk_norm_rope_write_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
        (float*)qkv, q_gain, k_gain, gain_f32, (const float*)cos_t, (const float*)sin_t, row_seq, row_pos, seq_slot,
        table, width, (float*)k_cache, (float*)v_cache, rows, HQ, HKV, D, eps, n_pos, error);
  return (int)launch_pdl(qk_norm_rope_write_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
        (bf16*)qkv, q_gain, k_gain, gain_f32, (const bf16*)cos_t, (const bf16*)sin_t, row_seq, row_pos, seq_slot, table,
        width, (bf16*)k_cache, (bf16*)v_cache, rows, HQ, HKV, D, eps, n_pos, error);
}
