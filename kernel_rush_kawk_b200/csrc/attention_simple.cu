// Causal grouped-query attention over the paged cache, one warp per (row, head),
// one key after the other. This is the kernel of the true 32-bit path; it is
// slow and its result for a row depends on nothing but that row's own keys, in
// their order, so it is the same however the tokens were cut into steps or
// batched.
//
// s = (q . k) * scale; a query at position p sees keys max(0, p - window + 1)..p
// (window 0: all keys 0..p); running max and sum in float32; the probability is
// rounded to the element type before it multiplies v; the sum divides once at
// the end; q head h reads kv head h / (HQ / HKV) (engine/kernels/attention.py:
// 9-11,70-73,104-122 of willzeng274/kernel-rush-kawk). The keys and values of
// this step's own rows are already in the cache when this runs.
//
// Compiled once per head size: -DKRK_HEAD_DIM=<D>.
#include "common.cuh"

#ifndef KRK_HEAD_DIM
#error "compile with -DKRK_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = KRK_HEAD_DIM;
constexpr int PER_LANE = (D + 31) / 32;

template <typename T>
__global__ void attention_simple_kernel(T* __restrict__ out, const T* __restrict__ q, int q_row_stride, int HQ, int HKV,
                                        const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                        const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                                        const T* __restrict__ k_cache, const T* __restrict__ v_cache, int rows,
                                        float scale, int window) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * HQ) return;
  const int row = (int)(item / HQ), head = (int)(item % HQ);
  const int kh = head / (HQ / HKV);
  const int pos = row_pos[row];
  const int slot = seq_slot[row_seq[row]];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;

  float qv[PER_LANE], acc[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < D ? to_float<T>(q[(size_t)row * q_row_stride + (size_t)head * D + d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  int page = -1, page_index = -1;
  for (int key = first; key <= pos; ++key) {
    if (key / KRK_PAGE != page_index) {
      page_index = key / KRK_PAGE;
      page = page_of(table, width, slot, key);
    }
    const size_t base = (((size_t)page * HKV + kh) * KRK_PAGE + (key % KRK_PAGE)) * D;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < D) dot += qv[i] * to_float<T>(k_cache[base + d]);
    }
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float alpha = expf(m - m_new);  // exp(-inf) = 0 on the first key
    const float p = expf(s - m_new);
    l = l * alpha + p;
    const float pr = round_to<T>(p);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] = acc[i] * alpha + pr * to_float<T>(v_cache[base + d]);
    }
    m = m_new;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out[(size_t)row * HQ * D + (size_t)head * D + d] = from_float<T>(acc[i] / l);
  }
}

}  // namespace

KRK_API int krk_attention_simple(void* out, const void* q, int q_row_stride, int HQ, int HKV, const int* row_seq,
                                 const int* row_pos, const int* seq_slot, const int* table, int width,
                                 const void* k_cache, const void* v_cache, int rows, float scale, int window, int dtype,
                                 cudaStream_t stream) {
  if (rows == 0) return 0;
  const long long items = (long long)rows * HQ;
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    attention_simple_kernel<float><<<(unsigned)blocks, warps * 32, 0, stream>>>(
        (float*)out, (const float*)q, q_row_stride, HQ, HKV, row_seq, row_pos, seq_slot, table, width,
        (const float*)k_cache, (const float*)v_cache, rows, scale, window);
  else
    attention_simple_kernel<bf16><<<(unsigned)blocks, warps * 32, 0, stream>>>(
        (bf16*)out, (const bf16*)q, q_row_stride, HQ, HKV, row_seq, row_pos, seq_slot, table, width,
        (const bf16*)k_cache, (const bf16*)v_cache, rows, scale, window);
  KRK_CHECK_LAUNCH();
  return 0;
}

KRK_API int krk_attention_head_dim(void) { return D; }
