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
// A rotation of part of the head (rot < D, the tables then [positions, rot/2]) pairs element i
// with element i + rot/2 for i < rot/2 and leaves elements rot..D-1 as the norm made them; the
// norm is over the whole head. The general kernel serves it; the 16-byte-lane kernels rotate the whole head.
#include "common.cuh"

namespace {

template <typename T>
__global__ void qk_norm_rope_write_kernel(T* __restrict__ qkv, const void* __restrict__ q_gain,
                                          const void* __restrict__ k_gain, int gain_f32, const T* __restrict__ cos_t,
                                          const T* __restrict__ sin_t, const int* __restrict__ row_seq,
                                          const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                                          const int* __restrict__ table, int width, T* __restrict__ k_cache,
                                          T* __restrict__ v_cache, int rows, int HQ, int HKV, int D, int rot, float eps,
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
  if (rot < D) {  // part of the head is rotated: pairs (i, i + rot/2) below rot, the rest only normalised
    const int rh = rot / 2;
    float sq = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float a = to_float<T>(src[i]);
      sq += a * a;
    }
    sq = warp_sum(sq);
    const float r = gain ? rsqrtf(sq / (float)D + eps) : 1.f;
    auto normed = [&](int i) {
      const float y = to_float<T>(src[i]);
      return gain ? round_to<T>(load_gain<T>(gain, i, gain_f32) * round_to<T>(y * r)) : y;
    };
    for (int i = lane; i < rh; i += 32) {  // both elements of a pair are read before either is written (q in place)
      float y1 = normed(i), y2 = normed(i + rh);
      if (cos_t) {
        const float c = to_float<T>(cos_t[(size_t)pos * rh + i]);
        const float s = to_float<T>(sin_t[(size_t)pos * rh + i]);
        const float o1 = round_to<T>(y1 * c) + round_to<T>(-y2 * s);
        const float o2 = round_to<T>(y2 * c) + round_to<T>(y1 * s);
        y1 = o1;
        y2 = o2;
      }
      dst[i] = from_float<T>(y1);
      dst[i + rh] = from_float<T>(y2);
    }
    for (int i = rot + lane; i < D; i += 32) dst[i] = from_float<T>(normed(i));
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
//
// The arithmetic is packed: x * r is a 32-bit product rounded to bfloat16 (r is a float), and every later
// step multiplies or adds two bfloat16 values and rounds, which mul.rn.bf16x2 and add.rn.bf16x2 do in one
// instruction with the same result (the 32-bit product of two bfloat16 values is exact, and the 32-bit sum
// of two is exact whenever it could matter to the second rounding). The _rn forms are never fused.
struct RopeLane {
  __nv_bfloat162 c[4];  // this lane's 8 cosines
  __nv_bfloat162 s[4];  // its sines, negated in the first half of the head: out1 = y1*c - y2*s, out2 = y2*c + y1*s
};

__device__ __forceinline__ RopeLane rope_lane(const bf16* cos_t, const bf16* sin_t, int pos, int D, int sub) {
  const int half = D / 2;
  const bool first = 8 * sub < half;
  const int i0 = first ? 8 * sub : 8 * sub - half;  // index into the half tables
  const uint4 cv = *reinterpret_cast<const uint4*>(cos_t + (size_t)pos * half + i0);
  const uint4 sv = *reinterpret_cast<const uint4*>(sin_t + (size_t)pos * half + i0);
  RopeLane t;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    t.c[j] = reinterpret_cast<const __nv_bfloat162*>(&cv)[j];
    const __nv_bfloat162 sj = reinterpret_cast<const __nv_bfloat162*>(&sv)[j];
    t.s[j] = first ? __hneg2(sj) : sj;
  }
  return t;
}

// One lane's 8 elements of one head through the norm (gain != null) and the rotation (rope). Every lane of
// the warp must call it: the head's lanes exchange their sums and their partner elements by shuffle.
__device__ __forceinline__ uint4 norm_rope_piece(uint4 raw, int lph, int D, float eps, const void* gain, int gain_f32,
                                                 int sub, bool rope, const RopeLane& t) {
  __nv_bfloat162 h[4];
  float y[8];
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    h[j] = reinterpret_cast<const __nv_bfloat162*>(&raw)[j];
    y[2 * j] = __low2float(h[j]);
    y[2 * j + 1] = __high2float(h[j]);
    sq += y[2 * j] * y[2 * j] + y[2 * j + 1] * y[2 * j + 1];
  }
  for (int o = lph >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);  // over the head's lanes
  if (gain) {
    const float r = rsqrtf(sq / (float)D + eps);
    if (gain_f32) {
      const float* g = reinterpret_cast<const float*>(gain) + 8 * sub;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 n = __bfloat1622float2(__floats2bfloat162_rn(y[2 * j] * r, y[2 * j + 1] * r));
        h[j] = __floats2bfloat162_rn(g[2 * j] * n.x, g[2 * j + 1] * n.y);
      }
    } else {
      const uint4 gv = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(gain) + 8 * sub);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        h[j] = __hmul2_rn(reinterpret_cast<const __nv_bfloat162*>(&gv)[j], __floats2bfloat162_rn(y[2 * j] * r, y[2 * j + 1] * r));
    }
  }
  uint4 out;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t mine = *reinterpret_cast<const uint32_t*>(&h[j]);
    const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, lph >> 1);
    const __nv_bfloat162 other = *reinterpret_cast<const __nv_bfloat162*>(&theirs);
    if (rope) h[j] = __hadd2_rn(__hmul2_rn(h[j], t.c[j]), __hmul2_rn(other, t.s[j]));
    reinterpret_cast<__nv_bfloat162*>(&out)[j] = h[j];
  }
  return out;
}

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
  if (bad && live && error) atomicExch(error, 2);
  RopeLane t;
  if (cos_t) t = rope_lane(cos_t, sin_t, pos, D, sub);
  const uint4 done = norm_rope_piece(raw, lph, D, eps, is_v ? nullptr : (head < HQ ? q_gain : k_gain), gain_f32, sub,
                                     cos_t && !is_v, t);
  if (live && !bad) *reinterpret_cast<uint4*>(dst) = done;
}

// The same lanes-per-head layout for steps with many rows: one block per row. What depends on the row only
// (position, cache page, this lane's cosines and sines) is fetched once, and the block's lane groups walk
// the row's heads, two at a time with their loads issued together. 2,048 rows of 48 heads of size 128 take
// 23 us with a cold L2 where the flat kernel takes 26 us (and took 34 us with unpacked arithmetic).
__global__ void __launch_bounds__(256)
qk_norm_rope_write_row_kernel(bf16* __restrict__ qkv, const void* __restrict__ q_gain, const void* __restrict__ k_gain,
                              int gain_f32, const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
                              const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                              const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                              bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int HQ, int HKV, int D, float eps,
                              int n_pos, int* error) {
  grid_launch_dependents();
  grid_dependency_wait();
  constexpr int U = 2;
  const int lph = D / 8;
  const int sub = threadIdx.x % lph;
  const int group = threadIdx.x / lph, groups = blockDim.x / lph;
  const int heads = HQ + 2 * HKV;
  const int row = blockIdx.x;
  bf16* src_row = qkv + (size_t)row * heads * D + 8 * sub;
  const int raw_pos = row_pos[row];
  const bool bad = raw_pos < 0 || raw_pos >= n_pos;  // flagged below; nothing is stored for such a row
  const int pos = bad ? 0 : raw_pos;
  if (bad && threadIdx.x == 0 && error) atomicExch(error, 2);
  size_t cache_row = 0;
  if (HKV > 0) {
    const int page = page_of(table, width, seq_slot[row_seq[row]], pos);
    cache_row = (size_t)page * HKV * KRK_PAGE + (pos % KRK_PAGE);
  }
  RopeLane t;
  if (cos_t) t = rope_lane(cos_t, sin_t, pos, D, sub);
  for (int base = 0; base < heads; base += U * groups) {  // the same trip count for every lane
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int head = base + u * groups + group;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (head < heads) raw[u] = *reinterpret_cast<const uint4*>(src_row + (size_t)head * D);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base + u * groups >= heads) break;  // no lane of the block has a head left
      const int head = base + u * groups + group;
      const bool is_q = head < HQ, is_v = head >= HQ + HKV;
      const uint4 done = norm_rope_piece(raw[u], lph, D, eps, is_v ? nullptr : (is_q ? q_gain : k_gain), gain_f32, sub,
                                         cos_t && !is_v, t);
      if (head < heads && !bad) {
        bf16* dst = src_row + (size_t)head * D;
        if (!is_q) {
          const int kh = (head - HQ) % HKV;
          dst = (is_v ? v_cache : k_cache) + (cache_row + (size_t)kh * KRK_PAGE) * D + 8 * sub;
        }
        *reinterpret_cast<uint4*>(dst) = done;
      }
    }
  }
}

}  // namespace

// from this many rows on, the block-per-row kernel; below it the flat one, whose few blocks start sooner
constexpr int ROW_KERNEL_MIN_ROWS = 256;

// gains may be null (no q/k norm); cos/sin may be null (no rotation); the cache
// pointers are unused when HKV == 0. rot: the rotated width (even, <= D; the tables are [positions, rot/2]).
KRK_API int krk_qk_norm_rope_write(void* qkv, const void* q_gain, const void* k_gain, int gain_f32, const void* cos_t,
                                   const void* sin_t, const int* row_seq, const int* row_pos, const int* seq_slot,
                                   const int* table, int width, void* k_cache, void* v_cache, int rows, int HQ, int HKV,
                                   int D, int rot, float eps, int n_pos, int* error, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (D % 2 || D > 4096) return -2;
  if (!cos_t) rot = D;
  if (rot % 2 || rot <= 0 || rot > D) return -2;
  const long long items = (long long)rows * (HQ + 2 * HKV);
  const bool gains_aligned = gain_f32 || ((((uintptr_t)q_gain) | ((uintptr_t)k_gain)) & 15) == 0;  // 16-byte gain loads
  if (dtype == KRK_DTYPE_BF16 && gains_aligned && rot == D && (D == 16 || D == 32 || D == 64 || D == 128 || D == 256)) {
    if (rows >= ROW_KERNEL_MIN_ROWS)
      return (int)launch_pdl(qk_norm_rope_write_row_kernel, dim3((unsigned)rows), dim3(256), 0, stream, (bf16*)qkv, q_gain,
                             k_gain, gain_f32, (const bf16*)cos_t, (const bf16*)sin_t, row_seq, row_pos, seq_slot, table,
                             width, (bf16*)k_cache, (bf16*)v_cache, HQ, HKV, D, eps, n_pos, error);
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
        table, width, (float*)k_cache, (float*)v_cache, rows, HQ, HKV, D, rot, eps, n_pos, error);
  return (int)launch_pdl(qk_norm_rope_write_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
        (bf16*)qkv, q_gain, k_gain, gain_f32, (const bf16*)cos_t, (const bf16*)sin_t, row_seq, row_pos, seq_slot, table,
        width, (bf16*)k_cache, (bf16*)v_cache, rows, HQ, HKV, D, rot, eps, n_pos, error);
}
