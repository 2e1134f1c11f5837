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

// bfloat16 and a head size of 16, 32, 64, 128 or 256: D/8 lanes share a head, 16 bytes each,
// so a warp handles 32 / (D/8) heads with vector loads and stores. The partner of element i
// (i < D/2) is element i + D/2, which sits D/16 lanes further; a shuffle brings it over.
__global__ void qk_norm_rope_write_vec_kernel(bf16* __restrict__ qkv, const void* __restrict__ q_gain,
                                              const void* __restrict__ k_gain, int gain_f32,
                                              const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
                                              const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                              const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                                              bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int rows, int HQ,
                                              int HKV, int D, float eps, int n_pos, int* error) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lph = D / 8;  // lanes per head
  const int lane = threadIdx.x & 31;
  const int sub = lane % lph;  // this lane's 8 elements are [8 * sub, 8 * sub + 8)
  const int heads = HQ + 2 * HKV;
  const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32 / lph) + lane / lph;
  const bool live = item < (long long)rows * heads;
  const int row = live ? (int)(item / heads) : 0;
  const int head = live ? (int)(item % heads) : 0;
  const int raw_pos = row_pos[row];
  const bool bad = raw_pos < 0 || raw_pos >= n_pos;  // flagged below; nothing is stored for such a row
  const int pos = bad ? 0 : raw_pos;
  const int half = D / 2;
  bf16* src = qkv + (size_t)row * heads * D + (size_t)head * D + 8 * sub;
  bf16* dst = src;
  if (head >= HQ) {
    const int kh = (head - HQ) % HKV;
    const int page = page_of(table, width, seq_slot[row_seq[row]], pos);
    bf16* cache = head < HQ + HKV ? k_cache : v_cache;
    dst = cache + (((size_t)page * HKV + kh) * KRK_PAGE + (pos % KRK_PAGE)) * D + 8 * sub;
  }
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (live) raw = *reinterpret_cast<const uint4*>(src);
  const bool is_v = head >= HQ + HKV;
  const void* gain = head < HQ ? q_gain : k_gain;
  if (bad && live && error) atomicExch(error, 2);
  float y[8];
  const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    y[2 * j] = __low2float(rp[j]);
    y[2 * j + 1] = __high2float(rp[j]);
    sq += y[2 * j] * y[2 * j] + y[2 * j + 1] * y[2 * j + 1];
  }
  for (int o = lph >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);  // over the head's lanes
  if (gain && !is_v) {
    const float r = rsqrtf(sq / (float)D + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = round_to<bf16>(load_gain<bf16>(gain, 8 * sub + j, gain_f32) * round_to<bf16>(y[j] * r));
  }
  float other[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) other[j] = __shfl_xor_sync(0xffffffffu, y[j], lph >> 1);
  if (cos_t && !is_v) {
    const bool first = 8 * sub < half;
    const int i0 = first ? 8 * sub : 8 * sub - half;  // index into the half tables
    const uint4 cv = *reinterpret_cast<const uint4*>(cos_t + (size_t)pos * half + i0);
    const uint4 sv = *reinterpret_cast<const uint4*>(sin_t + (size_t)pos * half + i0);
    const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&cv);
    const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = (j & 1) ? __high2float(cp[j >> 1]) : __low2float(cp[j >> 1]);
      const float s = (j & 1) ? __high2float(sp[j >> 1]) : __low2float(sp[j >> 1]);
      // first half: y1*c - y2*s with y2 = other; second half: y2*c + y1*s with y1 = other
      y[j] = first ? round_to<bf16>(y[j] * c) + round_to<bf16>(-other[j] * s)
                   : round_to<bf16>(y[j] * c) + round_to<bf16>(other[j] * s);
    }
  }
  if (live && !bad) {
    uint4 ov;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
    *reinterpret_cast<uint4*>(dst) = is_v ? raw : ov;
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
  if (dtype == KRK_DTYPE_BF16 && (D == 16 || D == 32 || D == 64 || D == 128 || D == 256)) {
    const int per_warp = 32 / (D / 8);
    const long long n_warps = (items + per_warp - 1) / per_warp;
    const long long n_blocks = (n_warps + 7) / 8;
    if (n_blocks > 0x7fffffffLL) return -3;
    return (int)launch_pdl(qk_norm_rope_write_vec_kernel, dim3((unsigned)n_blocks), dim3(256), 0, stream, (bf16*)qkv,
                           q_gain, k_gain, gain_f32, (const bf16*)cos_t, (const bf16*)sin_t, row_seq, row_pos, seq_slot,
                           table, width, (bf16*)k_cache, (bf16*)v_cache, rows, HQ, HKV, D, eps, n_pos, error);
  }
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
