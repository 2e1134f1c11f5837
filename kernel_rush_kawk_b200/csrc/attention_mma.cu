// Causal grouped-query attention over the paged cache on the tensor cores
// (mma.sync m16n8k16, bfloat16 in, float32 accumulate): one kernel for steps that
// bring many tokens per sequence (prefill, chunks), one for single-token steps
// (decode, split over the keys), and the merge of the splits.
//
// Numerics follow the reference's decode kernel (engine/kernels/attention.py:9-11,
// 104-122 of willzeng274/kernel-rush-kawk): scores and softmax statistics in
// float32, probabilities rounded to bfloat16 before P.V, output accumulated in
// float32 and divided by the sum once at the end. A query at position p sees keys
// max(0, p - window + 1)..p (window 0: from key 0). As there (attention.py:70-73),
// all G = HQ / HKV query heads of a kv head share one read of K and V: the rows of
// a tile are (token, group member) pairs, row R -> token R / G, head kh * G + R % G.
//
// A key block is one cache page (64 positions), contiguous in memory for one kv
// head; blocks are brought to shared memory with cp.async, two stages.
//
// Compiled once per head size: -DKRK_HEAD_DIM=<D>, D a multiple of 16 up to 256.
#include <cooperative_groups.h>

#define KRK_TRACE_OWNER  // with -DKRK_TRACE this file keeps a timeline buffer of its own
#include "mma.cuh"
#include "tcgen05.cuh"  // mbarriers with bounded waits and TMA tile loads, for the TMA-fed single-token kernel

#ifndef KRK_HEAD_DIM
#error "compile with -DKRK_HEAD_DIM=<head size>"
#endif

#if KRK_HEAD_DIM % 16 == 0 && KRK_HEAD_DIM <= 256

namespace {

constexpr int D = KRK_HEAD_DIM;
constexpr int DP = D + 8;            // shared-memory row pitch (elements): 16 bytes of padding
constexpr int KSTEPS = D / 16;       // k-steps of Q.K^T
constexpr int DTILES = D / 8;        // n-tiles of P.V
constexpr int THREADS = 128;
// A page of keys or values in shared memory. Where a row is a power-of-two number (at least eight) of
// 16-byte pieces, rows are packed and piece c of key k sits at piece c ^ (k & 7), which spreads the eight
// rows of an ldmatrix over all banks without padding; other head sizes pad each row by 16 bytes instead.
constexpr bool KV_SWIZZLE = (D == 64 || D == 128 || D == 256);
constexpr int KVP = KV_SWIZZLE ? D : DP;  // row pitch of a page in shared memory (elements)
constexpr int TILE_ELEMS = KRK_PAGE * KVP;
__device__ __forceinline__ int kv_off(int key, int piece) {
  return key * KVP + ((KV_SWIZZLE ? (piece ^ (key & 7)) : piece) << 3);
}
// The same page as TMA writes it with the 128-byte swizzle: D / 64 sub-tiles of [64 keys][128 bytes], piece c of
// key k of a sub-tile at piece c ^ (k & 7). Head sizes that are multiples of 64 only.
constexpr bool TMA_PAGES = (D % 64 == 0);
constexpr int SUB_ELEMS = KRK_PAGE * 64;  // elements of one sub-tile (8 KB)
template <bool TMA>
__device__ __forceinline__ int page_off(int key, int piece) {
  if (TMA) return (piece >> 3) * SUB_ELEMS + key * 64 + (((piece & 7) ^ (key & 7)) << 3);
  return kv_off(key, piece);
}
constexpr float LOG2E = 1.4426950408889634f;

// Copy one page [64][D] of one kv head to shared memory [64][DP], all threads of the block.
__device__ __forceinline__ void load_page(bf16* dst, const bf16* __restrict__ src) {
  constexpr int CHUNKS = KRK_PAGE * (D / 8);
  for (int i = threadIdx.x; i < CHUNKS; i += THREADS) {
    const int key = i / (D / 8), ch = i % (D / 8);
    cp_async_16(dst + kv_off(key, ch), src + key * D + ch * 8);
  }
}

// S[16 x (8*NTILES)] = Q[16 x D] . K^T for keys key0 .. key0 + 8*NTILES - 1 of the tile in shared memory.
template <int NTILES, bool TMA = false>
__device__ __forceinline__ void qk_tile(float (&s)[NTILES][4], const uint32_t (&qf)[KSTEPS][4], const bf16* ks, int key0,
                                        int lane) {
  // even and odd k-steps accumulate apart and are added at the end: two chains of KSTEPS / 2 dependent MMAs
  // per n-tile instead of one of KSTEPS
  float odd[NTILES][4];
#pragma unroll
  for (int n = 0; n < NTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) s[n][c] = odd[n][c] = 0.f;
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
    for (int n = 0; n < NTILES; n += 2) {
      uint32_t b0, b1, b2, b3;
      const bf16* p = ks + page_off<TMA>(key0 + n * 8 + ((lane >> 4) << 3) + (lane & 7), kk * 2 + ((lane >> 3) & 1));
      ldmatrix_x4(b0, b1, b2, b3, p);
      if (kk & 1) {
        mma_bf16_16816(odd[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
        mma_bf16_16816(odd[n + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
      } else {
        mma_bf16_16816(s[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
        mma_bf16_16816(s[n + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
      }
    }
  }
#pragma unroll
  for (int n = 0; n < NTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) s[n][c] += odd[n][c];
}

// O[16 x D] += P[16 x (8*NTILES)] . V for the same keys; p holds probabilities (float) in S's layout.
template <int NTILES, bool TMA = false>
__device__ __forceinline__ void pv_tile(float (&o)[DTILES][4], const float (&p)[NTILES][4], const bf16* vs, int key0,
                                        int lane) {
#pragma unroll
  for (int kk = 0; kk < NTILES / 2; ++kk) {  // 16 keys per step
    const uint32_t a0 = pack_bf16x2(p[2 * kk][0], p[2 * kk][1]);
    const uint32_t a1 = pack_bf16x2(p[2 * kk][2], p[2 * kk][3]);
    const uint32_t a2 = pack_bf16x2(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    const uint32_t a3 = pack_bf16x2(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int n = 0; n < DTILES; n += 2) {
      uint32_t b0, b1, b2, b3;
      const bf16* q = vs + page_off<TMA>(key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, n + (lane >> 4));
      ldmatrix_x4_trans(b0, b1, b2, b3, q);
      mma_bf16_16816(o[n], a0, a1, a2, a3, b0, b1);
      mma_bf16_16816(o[n + 1], a0, a1, a2, a3, b2, b3);
    }
  }
}

// Load the A fragments of one 16-row tile of queries; row r of the tile is at qrow[r half] (null: zero row).
__device__ __forceinline__ void load_q(uint32_t (&qf)[KSTEPS][4], const bf16* q_lo, const bf16* q_hi, int lane) {
  const int t = lane & 3;
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    const int d = kk * 16 + 2 * t;
    qf[kk][0] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + d) : 0u;
    qf[kk][1] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + d) : 0u;
    qf[kk][2] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + d + 8) : 0u;
    qf[kk][3] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + d + 8) : 0u;
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One online-softmax update of a thread's two rows over NTILES*8 keys. s is in log2
// units already (scaled by scale*log2(e)) and masked with -inf where invisible.
template <int NTILES>
__device__ __forceinline__ void softmax_update(float (&s)[NTILES][4], float (&m)[2], float (&l)[2], float (&o)[DTILES][4]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = -INFINITY;
#pragma unroll
    for (int n = 0; n < NTILES; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * h], s[n][2 * h + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = fast_exp2(m[h] - m_safe);
    float sum = 0.f;
#pragma unroll
    for (int n = 0; n < NTILES; ++n) {
      s[n][2 * h] = fast_exp2(s[n][2 * h] - m_safe);
      s[n][2 * h + 1] = fast_exp2(s[n][2 * h + 1] - m_safe);
      sum += s[n][2 * h] + s[n][2 * h + 1];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l[h] = l[h] * alpha + sum;
    m[h] = m_new;
#pragma unroll
    for (int n = 0; n < DTILES; ++n) {
      o[n][2 * h] *= alpha;
      o[n][2 * h + 1] *= alpha;
    }
  }
}

// ---------------------------------------------------------------------------------
// Many tokens per sequence. Block = (row tile of 64, kv head, sequence); warp w owns
// rows 16w..16w+15 of the tile and walks all key blocks the tile can see.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_qlen, const int* __restrict__ cu_q, const int* __restrict__ table,
                         int width, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, float scale_log2,
                         int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);  // [2 stages][K, V][64][DP]
  const int seq = blockIdx.z, kh = blockIdx.y;
  const int tile = gridDim.x - 1 - blockIdx.x;  // long tiles first
  const int G = HQ / HKV;
  const int q_len = seq_qlen[seq];
  const int n_rows = q_len * G;
  if (tile * 64 >= n_rows) return;
  const int start = seq_start[seq], slot = seq_slot[seq], row0 = cu_q[seq];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;

  // this thread's two rows
  int tok[2], pos[2], lo[2];
  const bf16* qp[2];
  bf16* op[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = tile * 64 + warp * 16 + g + 8 * h;
    const bool ok = R < n_rows;
    tok[h] = ok ? R / G : -1;
    const int head = kh * G + (ok ? R % G : 0);
    pos[h] = ok ? start + tok[h] : -1;  // -1: sees nothing
    lo[h] = (ok && window > 0) ? max(0, pos[h] - window + 1) : 0;
    qp[h] = ok ? qkv + (size_t)(row0 + tok[h]) * q_stride + (size_t)head * D : nullptr;
    op[h] = ok ? out + (size_t)(row0 + tok[h]) * HQ * D + (size_t)head * D : nullptr;
  }
  uint32_t qf[KSTEPS][4];
  load_q(qf, qp[0], qp[1], lane);
  // the least position and the greatest window start among the warp's rows (an invalid row sees nothing)
  int warp_min_pos = min(pos[0], pos[1]), warp_max_lo = max(lo[0], lo[1]);
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) {
    warp_min_pos = min(warp_min_pos, __shfl_xor_sync(0xffffffffu, warp_min_pos, o2));
    warp_max_lo = max(warp_max_lo, __shfl_xor_sync(0xffffffffu, warp_max_lo, o2));
  }

  // key blocks the tile can see
  const int last_tok = min(q_len - 1, (tile * 64 + 63) / G);
  const int first_tok = (tile * 64) / G;
  const int j_hi = (start + last_tok) / KRK_PAGE;
  const int j_lo = window > 0 ? max(0, start + first_tok - window + 1) / KRK_PAGE : 0;
  const size_t page_stride = (size_t)HKV * KRK_PAGE * D;
  const size_t head_off = (size_t)kh * KRK_PAGE * D;

  auto issue = [&](int j, int stage) {
    const int page = table[(size_t)slot * width + j % width];
    bf16* ks = smem + (size_t)stage * 2 * TILE_ELEMS;
    load_page(ks, k_cache + (size_t)page * page_stride + head_off);
    load_page(ks + TILE_ELEMS, v_cache + (size_t)page * page_stride + head_off);
    cp_async_commit();
  };

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  issue(j_lo, 0);
  for (int j = j_lo; j <= j_hi; ++j) {
    const int stage = (j - j_lo) & 1;
    if (j + 1 <= j_hi) {
      issue(j + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* ks = smem + (size_t)stage * 2 * TILE_ELEMS;
    const bf16* vs = ks + TILE_ELEMS;
    float s[8][4];
    qk_tile<8>(s, qf, ks, 0, lane);
    const int key_base = j * KRK_PAGE;
    // a block that every row of the warp sees whole needs no mask (most blocks of a long prompt)
    const bool whole = key_base + KRK_PAGE - 1 <= warp_min_pos && key_base >= warp_max_lo;
    if (whole) {
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[n][c] *= scale_log2;
    } else {
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = key_base + n * 8 + 2 * t4 + (c & 1);
          const int h = c >> 1;
          s[n][c] = (key <= pos[h] && key >= lo[h]) ? s[n][c] * scale_log2 : -INFINITY;
        }
    }
    softmax_update<8>(s, m, l, o);
    pv_tile<8>(o, s, vs, 0, lane);
    __syncthreads();  // the stage is free for the load after next
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!op[h]) continue;
    const float inv = 1.0f / l[h];
#pragma unroll
    for (int n = 0; n < DTILES; ++n)
      *reinterpret_cast<uint32_t*>(op[h] + n * 8 + 2 * t4) = pack_bf16x2(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
  }
}

// ---------------------------------------------------------------------------------
// One token per sequence. Block = (key split, kv head x row tile, sequence). The block
// brings whole pages to shared memory; warp w works on keys 16w..16w+15 of each page
// with running statistics of its own; the four warps merge at the end and the block
// writes one partial (m, l, o[D]) per row, which the merge kernel combines.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(float* __restrict__ part, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                        const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                        const int* __restrict__ table, int width, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, float scale_log2, int window, int row_tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  grid_launch_dependents();
  grid_dependency_wait();
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int kh = blockIdx.y / row_tiles, rt = blockIdx.y % row_tiles;
  const int seq = blockIdx.z;
  const int G = HQ / HKV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int pos = seq_start[seq], slot = seq_slot[seq];  // the new token sits at `pos`, its key is cached
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int j_first = lo / KRK_PAGE, j_last = pos / KRK_PAGE;
  const int n_blocks = j_last - j_first + 1;
  const int per = (n_blocks + n_splits - 1) / n_splits;
  const int j_lo = j_first + split * per, j_hi = min(j_last, j_lo + per - 1);

  const bf16* qp[2];
  int head[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = rt * 16 + g + 8 * h;
    head[h] = r < G ? kh * G + r : -1;
    qp[h] = r < G ? qkv + (size_t)seq * q_stride + (size_t)head[h] * D : nullptr;
  }
  uint32_t qf[KSTEPS][4];
  load_q(qf, qp[0], qp[1], lane);

  const size_t page_stride = (size_t)HKV * KRK_PAGE * D;
  const size_t head_off = (size_t)kh * KRK_PAGE * D;
  auto issue = [&](int j, int stage) {
    const int page = table[(size_t)slot * width + j % width];
    bf16* ks = smem + (size_t)stage * 2 * TILE_ELEMS;
    load_page(ks, k_cache + (size_t)page * page_stride + head_off);
    load_page(ks + TILE_ELEMS, v_cache + (size_t)page * page_stride + head_off);
    cp_async_commit();
  };

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  if (j_lo <= j_hi) issue(j_lo, 0);
  for (int j = j_lo; j <= j_hi; ++j) {
    const int stage = (j - j_lo) & 1;
    if (j + 1 <= j_hi) {
      issue(j + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* ks = smem + (size_t)stage * 2 * TILE_ELEMS;
    const bf16* vs = ks + TILE_ELEMS;
    const int key0 = warp * 16;
    float s[2][4];
    qk_tile<2>(s, qf, ks, key0, lane);
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = j * KRK_PAGE + key0 + n * 8 + 2 * t4 + (c & 1);
        s[n][c] = (key <= pos && key >= lo) ? s[n][c] * scale_log2 : -INFINITY;
      }
    softmax_update<2>(s, m, l, o);
    pv_tile<2>(o, s, vs, key0, lane);
    __syncthreads();
  }

  // merge the four warps: through shared memory, in warp order
  float* red = reinterpret_cast<float*>(smem_raw);  // [4 warps][16 rows][D + 2]; the page buffers are free now
  constexpr int RP = D + 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float* dst = red + ((size_t)warp * 16 + g + 8 * h) * RP;
    if (t4 == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
    for (int n = 0; n < DTILES; ++n) {
      dst[n * 8 + 2 * t4] = o[n][2 * h];
      dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
    }
  }
  __syncthreads();
  for (int r = warp; r < 16; r += 4) {
    const int row = rt * 16 + r;
    if (row >= G) continue;
    float mw[4], big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mw[w] = red[((size_t)w * 16 + r) * RP + D]; big = fmaxf(big, mw[w]); }
    const float safe = big == -INFINITY ? 0.f : big;
    float wgt[4], lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { wgt[w] = exp2f(mw[w] - safe); lsum += wgt[w] * red[((size_t)w * 16 + r) * RP + D + 1]; }
    float* dst = part + (((size_t)seq * HQ + kh * G + row) * n_splits + split) * RP;
    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * RP + d];
      dst[d] = acc;
    }
    if (lane == 0) { dst[D] = big; dst[D + 1] = lsum; }
  }
}

// out[seq, head, :] = sum_s w_s o_s / sum_s w_s l_s with w_s = 2^(m_s - max m): one warp per (seq, head).
__global__ void attention_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part, int n_items, int n_splits) {
  constexpr int RP = D + 2;
  grid_launch_dependents();
  grid_dependency_wait();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const float* src = part + (size_t)item * n_splits * RP;
  // statistics: lane s reads split s, s + 32, ...; all loads are independent
  float big = -INFINITY;
  for (int s = lane; s < n_splits; s += 32) big = fmaxf(big, src[(size_t)s * RP + D]);
  big = warp_max(big);
  float lsum = 0.f;
  for (int s = lane; s < n_splits; s += 32) lsum += exp2f(src[(size_t)s * RP + D] - big) * src[(size_t)s * RP + D + 1];
  lsum = warp_sum(lsum);
  float acc[(D + 31) / 32];
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int s = 0; s < n_splits; ++s) {
    const float w = exp2f(src[(size_t)s * RP + D] - big);
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] += w * src[(size_t)s * RP + d];
    }
  }
  const float inv = 1.0f / lsum;
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out[(size_t)item * D + d] = __float2bfloat16_rn(acc[i] * inv);
  }
}


// Page stages of the fused single-token kernel: two where the keys of a (sequence, kv head) are split over
// a cluster (three blocks share an SM), three where one block walks them all (many sequences: two blocks
// an SM, each with two pages in flight; at 64 sequences of 1,024 tokens 7 % faster than two stages and two
// splits, while at 8 sequences three stages were slower).
__host__ __device__ constexpr size_t fused_base_bytes(int stages) {
  return ((size_t)stages * 2 * TILE_ELEMS * sizeof(bf16) > (size_t)4 * 16 * (D + 2) * sizeof(float))
             ? (size_t)stages * 2 * TILE_ELEMS * sizeof(bf16) : (size_t)4 * 16 * (D + 2) * sizeof(float);
}
constexpr size_t PAGE_SMEM = (size_t)2 * 2 * TILE_ELEMS * sizeof(bf16);
constexpr size_t RED_SMEM = (size_t)4 * 16 * (D + 2) * sizeof(float);
constexpr size_t DECODE_SMEM = PAGE_SMEM > RED_SMEM ? PAGE_SMEM : RED_SMEM;

// ---------------------------------------------------------------------------------
// One token per sequence, everything between the QKV projection and the output
// projection in one launch: per-head q/k RMSNorm and rotation of the new token
// (rounding points of engine/kernels/rope.py:19-30 of the reference), the write of its
// key and value to the cache, attention over the cache, and the merge of the key
// splits. The splits of one (sequence, kv head, row tile) form a thread-block cluster;
// each block leaves its partial (m, l, o[D]) in its own shared memory and block 0 of
// the cluster reads the others' through distributed shared memory, so no partial
// result goes through global memory and no second kernel merges.
// ---------------------------------------------------------------------------------
// One head row of the new token: its values, gains and table entries are loaded first,
// all at once, and the arithmetic follows, so that a row costs one memory latency.
// Lane L owns the pairs (i, i + D/2) for i = L, L + 32, ...
struct HeadRow {
  static constexpr int PAIRS = (D / 2 + 31) / 32;
  float lo[PAIRS], hi[PAIRS], g_lo[PAIRS], g_hi[PAIRS], c[PAIRS], s[PAIRS];

  // the row's values: their addresses do not depend on the token's position
  __device__ __forceinline__ void load_values(const bf16* __restrict__ src, int lane) {
    constexpr int HALF = D / 2;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + 32 * p;
      const bool ok = i < HALF;
      lo[p] = ok ? __bfloat162float(src[i]) : 0.f;
      hi[p] = ok ? __bfloat162float(src[i + HALF]) : 0.f;
    }
  }
  // the norm's gains: weights, which no kernel writes
  __device__ __forceinline__ void load_gains(const void* gain, int gain_f32, int lane) {
    constexpr int HALF = D / 2;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + 32 * p;
      const bool ok = i < HALF;
      g_lo[p] = (ok && gain) ? load_gain<bf16>(gain, i, gain_f32) : 1.f;
      g_hi[p] = (ok && gain) ? load_gain<bf16>(gain, i + HALF, gain_f32) : 1.f;
    }
  }
  // the rotation's table row of the token's position
  __device__ __forceinline__ void load_angles(const bf16* __restrict__ cos_row, const bf16* __restrict__ sin_row, int lane) {
    constexpr int HALF = D / 2;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + 32 * p;
      const bool ok = i < HALF;
      c[p] = (ok && cos_row) ? __bfloat162float(cos_row[i]) : 1.f;
      s[p] = (ok && sin_row) ? __bfloat162float(sin_row[i]) : 0.f;
    }
  }

  // norm (if has_gain), rotation (if has_rope), rounded as the reference rounds; written to dst
  __device__ __forceinline__ void finish(bf16* dst, bool has_gain, bool has_rope, float eps, int lane) const {
    constexpr int HALF = D / 2;
    float sq = 0.f;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) sq += lo[p] * lo[p] + hi[p] * hi[p];
    sq = warp_sum(sq);
    const float r = rsqrtf(sq / (float)D + eps);
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + 32 * p;
      if (i >= HALF) continue;
      float y1 = lo[p], y2 = hi[p];
      if (has_gain) {
        y1 = round_to<bf16>(g_lo[p] * round_to<bf16>(y1 * r));
        y2 = round_to<bf16>(g_hi[p] * round_to<bf16>(y2 * r));
      }
      if (has_rope) {
        const float o1 = round_to<bf16>(y1 * c[p]) + round_to<bf16>(-y2 * s[p]);
        const float o2 = round_to<bf16>(y2 * c[p]) + round_to<bf16>(y1 * s[p]);
        y1 = o1;
        y2 = o2;
      }
      dst[i] = __float2bfloat16_rn(y1);
      dst[i + HALF] = __float2bfloat16_rn(y2);
    }
  }
};

template <int FSTAGES>
__global__ void __launch_bounds__(THREADS)
attention_decode_fused_kernel(bf16* __restrict__ out, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                              const void* __restrict__ q_gain, const void* __restrict__ k_gain, int gain_f32,
                              const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t, float eps,
                              const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                              const int* __restrict__ table, int width, bf16* __restrict__ k_cache,
                              bf16* __restrict__ v_cache, float scale_log2, int window, int row_tiles, int n_pos,
                              int inbox_rows, int* __restrict__ error) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);                       // page buffers, later the partials
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw + fused_base_bytes(FSTAGES));  // [16][DP] rotated queries
  bf16* kv_new = q_s + 16 * DP;                                         // [2][D] the new token's key and value
  float* inbox = reinterpret_cast<float*>(kv_new + 2 * D);              // [splits][inbox_rows][D + 2], used in block 0
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  KRK_TRACE_DECL
  KRK_TRACE_MARKS
  // "I have started": waited for only before the first write into another block's shared memory
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  grid_launch_dependents();
  const int n_splits = cluster.num_blocks(), split = cluster.block_rank();
  const int kh = blockIdx.y / row_tiles, rt = blockIdx.y % row_tiles;
  const int seq = blockIdx.z;
  const int G = HQ / HKV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  // What the kernel before this one does not write is read before the wait on it: the step's positions and
  // slots (uploaded, or written by the selection kernel, which lets no later kernel start before it has
  // ended), the page table, and the pages of earlier tokens, whose copies travel while that kernel finishes.
  int pos = __ldcg(seq_start + seq);
  const int slot = __ldcg(seq_slot + seq);
  if (pos < 0 || pos >= n_pos) {  // flagged and clamped: never an access out of range
    if (threadIdx.x == 0 && error) atomicExch(error, 2);
    pos = max(0, min(pos, n_pos - 1));
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int j_first = lo / KRK_PAGE, j_last = pos / KRK_PAGE;
  const int n_blocks = j_last - j_first + 1;
  const int per = (n_blocks + n_splits - 1) / n_splits;
  const int j_lo = j_first + split * per, j_hi = min(j_last, j_lo + per - 1);
  const bool owns_new = j_lo <= j_last && j_last <= j_hi;  // this block's keys include the new token's

  const size_t page_stride = (size_t)HKV * KRK_PAGE * D;
  const size_t head_off = (size_t)kh * KRK_PAGE * D;
  auto issue = [&](int j) {  // page j of this block's range into stage (j - j_lo) % FSTAGES; one group per call
    if (j <= j_hi) {
      const int page = table[(size_t)slot * width + j % width];
      bf16* ks = smem + (size_t)((j - j_lo) % FSTAGES) * 2 * TILE_ELEMS;
      load_page(ks, k_cache + (size_t)page * page_stride + head_off);
      load_page(ks + TILE_ELEMS, v_cache + (size_t)page * page_stride + head_off);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < FSTAGES - 1; ++i) issue(j_lo + i);
  // the page that takes the new token's key and value (read here, ahead of the wait, by the block that writes them)
  const int page_new = (owns_new && rt == 0) ? table[(size_t)slot * width + j_last % width] : 0;
  // The new token's rows. Warp w takes query rows w, w + 4, ... of this tile (rows beyond G
  // are zero); the key and value rows go to the warp with the fewest query rows, in every
  // block (only the block whose keys include the new token uses them). The gains and the
  // position's table rows are weights, which no kernel writes: they are requested before
  // the wait on the kernel that writes the rows, and all loads of a row are issued before
  // any arithmetic, so that after the wait the prologue costs one memory latency,
  // whatever the number of rows.
  const bf16* row = qkv + (size_t)seq * q_stride;
  const int q_rows = min(16, G - rt * 16);
  const int k_warp = q_rows % 4;
  constexpr int MAX_ROWS = 4;  // 16 rows over 4 warps
  HeadRow regs[MAX_ROWS];
  HeadRow k_regs;
  float v_regs[(D + 31) / 32];
  const bf16* cos_row = cos_t ? cos_t + (size_t)pos * (D / 2) : nullptr;
  const bf16* sin_row = sin_t ? sin_t + (size_t)pos * (D / 2) : nullptr;
#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i)
    if (warp + 4 * i < q_rows) {
      regs[i].load_gains(q_gain, gain_f32, lane);
      regs[i].load_angles(cos_row, sin_row, lane);
    }
  if (warp == k_warp) {
    k_regs.load_gains(k_gain, gain_f32, lane);
    k_regs.load_angles(cos_row, sin_row, lane);
  }
  KRK_TRACE_MARK(0)
  grid_dependency_wait();
  KRK_TRACE_READY
#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i) {
    const int r = warp + 4 * i;
    if (r < q_rows) regs[i].load_values(row + (size_t)(kh * G + rt * 16 + r) * D, lane);
  }
  if (warp == k_warp) {
    k_regs.load_values(row + (size_t)(HQ + kh) * D, lane);
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      v_regs[i] = d < D ? __bfloat162float(row[(size_t)(HQ + HKV + kh) * D + d]) : 0.f;
    }
  }

#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i) {
    const int r = warp + 4 * i;
    if (r < q_rows) {
      regs[i].finish(q_s + r * DP, q_gain != nullptr, cos_t != nullptr, eps, lane);
    } else if (r < 16) {
      for (int d = lane; d < D; d += 32) q_s[r * DP + d] = __float2bfloat16_rn(0.f);
    }
  }
  KRK_TRACE_MARK(1)
  if (owns_new && warp == k_warp) {
    k_regs.finish(kv_new, k_gain != nullptr, cos_t != nullptr, eps, lane);
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) kv_new[D + d] = __float2bfloat16_rn(v_regs[i]);
    }
    __syncwarp();
    if (rt == 0) {
      const size_t at = (size_t)page_new * page_stride + head_off + (size_t)(pos % KRK_PAGE) * D;
      for (int d = lane; d < D; d += 32) {
        k_cache[at + d] = kv_new[d];
        v_cache[at + d] = kv_new[D + d];
      }
    }
  }
  __syncthreads();

  uint32_t qf[KSTEPS][4];
  load_q(qf, q_s + g * DP, q_s + (g + 8) * DP, lane);
  KRK_TRACE_END(1)
#ifdef KRK_TRACE
  t_begin__ = krk_now();
#endif

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  for (int j = j_lo; j <= j_hi; ++j) {
    const int stage = (j - j_lo) % FSTAGES;
    issue(j + FSTAGES - 1);
    cp_async_wait<FSTAGES - 1>();      // all but the newest FSTAGES - 1 groups: page j has landed
    __syncthreads();
    bf16* ks = smem + (size_t)stage * 2 * TILE_ELEMS;
    bf16* vs = ks + TILE_ELEMS;
    if (j == j_last) {  // the page in shared memory predates this step's write: put the new row in
      for (int i = threadIdx.x; i < D; i += THREADS) {
        ks[kv_off(pos % KRK_PAGE, i >> 3) + (i & 7)] = kv_new[i];
        vs[kv_off(pos % KRK_PAGE, i >> 3) + (i & 7)] = kv_new[D + i];
      }
      __syncthreads();
    }
    const int key0 = warp * 16;
    float s[2][4];
    qk_tile<2>(s, qf, ks, key0, lane);
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = j * KRK_PAGE + key0 + n * 8 + 2 * t4 + (c & 1);
        s[n][c] = (key <= pos && key >= lo) ? s[n][c] * scale_log2 : -INFINITY;
      }
    softmax_update<2>(s, m, l, o);
    pv_tile<2>(o, s, vs, key0, lane);
    __syncthreads();
  }

  KRK_TRACE_MARK(2)
  cp_async_wait<0>();
  // Merge the four warps through shared memory, in warp order, and push the block's partial
  // (m, l, o[D]) per row straight into block 0's inbox through distributed shared memory.
  // One cluster barrier later block 0 holds every split's partial locally and merges them in
  // split order; the other blocks are done, and their shared memory is free for the blocks of the
  // kernel that follows. (The merge spread over the cluster, every block taking D / splits of the
  // head's dimensions with inboxes of a few KB and 16-byte pushes, was measured: a step of eight
  // sequences 2.09 -> 2.17 ms, of one 1.915 -> 1.947, because all blocks then stay to the end.)
  constexpr int RP = D + 2;
  float* red = reinterpret_cast<float*>(smem_raw);   // [4 warps][16 rows][RP]; the page buffers are free now
  float* inbox0 = cluster.map_shared_rank(inbox, 0);  // [splits][inbox_rows][RP] in block 0
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float* dst = red + ((size_t)warp * 16 + g + 8 * h) * RP;
    if (t4 == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
    for (int n = 0; n < DTILES; ++n) {
      dst[n * 8 + 2 * t4] = o[n][2 * h];
      dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
    }
  }
  __syncthreads();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every block of the cluster has started
  for (int r = warp; r < q_rows; r += 4) {
    float mw[4], big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mw[w] = red[((size_t)w * 16 + r) * RP + D]; big = fmaxf(big, mw[w]); }
    const float safe = big == -INFINITY ? 0.f : big;
    float wgt[4], lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { wgt[w] = exp2f(mw[w] - safe); lsum += wgt[w] * red[((size_t)w * 16 + r) * RP + D + 1]; }
    float* dst = inbox0 + ((size_t)split * inbox_rows + r) * RP;
    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * RP + d];
      dst[d] = acc;
    }
    if (lane == 0) { dst[D] = big; dst[D + 1] = lsum; }
  }
  KRK_TRACE_READY
  cluster.sync();  // every block's partial has arrived in block 0
  if (split == 0) {
    for (int r = warp; r < q_rows; r += 4) {
      const float* mine = inbox + (size_t)r * RP;
      const size_t step = (size_t)inbox_rows * RP;
      float big = -INFINITY;
      for (int s2 = 0; s2 < n_splits; ++s2) big = fmaxf(big, mine[s2 * step + D]);
      float lsum = 0.f;
      float acc[(D + 31) / 32];
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
      for (int s2 = 0; s2 < n_splits; ++s2) {
        const float w = exp2f(mine[s2 * step + D] - big);
        lsum += w * mine[s2 * step + D + 1];
#pragma unroll
        for (int i = 0; i < (D + 31) / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] += w * mine[s2 * step + d];
        }
      }
      const float inv = 1.0f / lsum;
      bf16* dst = out + ((size_t)seq * HQ + kh * G + rt * 16 + r) * D;
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dst[d] = __float2bfloat16_rn(acc[i] * inv);
      }
    }
  }
  KRK_TRACE_END(2)
  KRK_TRACE_MARKS_OUT(3)
}

template <int FSTAGES>
int launch_decode_fused(bf16* out, const bf16* qkv, int q_stride, int HQ, int HKV, const void* q_gain, const void* k_gain,
                        int gain_f32, const bf16* cos_t, const bf16* sin_t, float eps, const int* seq_slot,
                        const int* seq_start, const int* table, int width, bf16* k_cache, bf16* v_cache, int n_seqs,
                        float scale, int window, int splits, int n_pos, int* error, cudaStream_t stream) {
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  const int inbox_rows = G < 16 ? G : 16;
  const size_t smem = fused_base_bytes(FSTAGES) + (size_t)(16 * DP + 2 * D) * sizeof(bf16) +
                      (size_t)splits * inbox_rows * (D + 2) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  auto kern = attention_decode_fused_kernel<FSTAGES>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, HKV * row_tiles, n_seqs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = splits;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (splits > 8) {
    // Clusters of more than eight blocks have to be allowed per kernel, and a device (or a partition of one) need
    // not have room for one: asked once, with this launch's shape; -8 tells the caller to take eight.
    static int fits = -1;
    if (fits < 0) {
      int clusters = 0;
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess ||
          cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
      }
      fits = clusters > 0 ? 1 : 0;
    }
    if (!fits) return -8;
  }
  return (int)cudaLaunchKernelEx(&cfg, kern, out, qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32, cos_t, sin_t, eps,
                                 seq_slot, seq_start, table, width, k_cache, v_cache, scale * LOG2E, window, row_tiles,
                                 n_pos, inbox_rows, error);
}


#if KRK_HEAD_DIM % 64 == 0
// ---------------------------------------------------------------------------------
// The same single-token step for many sequences (one block walks all keys of its
// (sequence, kv head); no cluster), fed by TMA. A fifth warp is the producer: one
// thread requests pages as tiled bulk copies (128-byte swizzle, so ldmatrix stays free
// of bank conflicts) into a ring of units, a unit being one page of keys or one of
// values; each unit completes on an mbarrier of its own and is handed back on another
// as soon as the four consumer warps have read it, keys before values. With units of
// half a page-pair, all but one unit of the ring are in flight while one is computed
// on (five of six at head size 128, against two of three page-pairs with cp.async),
// and no consumer thread spends instructions on copying. A request under load takes
// some microseconds to arrive, so bytes in flight per SM are what bounds this kernel.
// ---------------------------------------------------------------------------------
constexpr int UNIT_ELEMS = KRK_PAGE * D;  // one page of keys (or of values) of one kv head
constexpr uint32_t UNIT_BYTES = UNIT_ELEMS * 2;
constexpr int TMA_THREADS = 160;          // four consumer warps and the producer warp
constexpr int TMA_MAX_WIDTH = 1024;       // page-table entries of a sequence that the block keeps in shared memory

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

__global__ void __launch_bounds__(TMA_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            bf16* __restrict__ out, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                            const void* __restrict__ q_gain, const void* __restrict__ k_gain, int gain_f32,
                            const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t, float eps,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                            const int* __restrict__ table, int width, bf16* __restrict__ k_cache,
                            bf16* __restrict__ v_cache, float scale_log2, int window, int row_tiles, int n_pos, int ring,
                            int inbox_rows, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  bf16* units = reinterpret_cast<bf16*>(base);                                // [ring][UNIT_ELEMS], later the partials
  bf16* q_s = reinterpret_cast<bf16*>(base + (size_t)ring * UNIT_BYTES);      // [16][DP] rotated queries
  bf16* kv_new = q_s + 16 * DP;                                               // [2][D] the new token's key and value
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(kv_new + 2 * D);           // [ring]
  uint64_t* empty_bar = full_bar + ring;                                      // [ring]
  int* pages = reinterpret_cast<int*>(empty_bar + ring);                      // [width] this block's key blocks
  float* inbox = reinterpret_cast<float*>(pages + ((width + 3) & ~3));        // [splits][inbox_rows][D + 2], used in block 0

  // The key blocks of a (sequence, kv head, row tile) may be split over the blocks of a thread-block cluster
  // (few sequences, long contexts: more blocks, each with a ring of its own in flight); the partials meet in
  // block 0's shared memory as in attention_decode_fused_kernel. "I have started" is waited for only before the
  // first write into another block's shared memory.
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int n_splits = cluster.num_blocks(), split = cluster.block_rank();
  if (n_splits > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  grid_launch_dependents();
  const int kh = blockIdx.y / row_tiles, rt = blockIdx.y % row_tiles;
  const int seq = blockIdx.z;
  const int G = HQ / HKV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  // read before the wait on the previous kernel, as in the cluster kernel: positions, slots, the page table
  int pos = __ldcg(seq_start + seq);
  const int slot = __ldcg(seq_slot + seq);
  if (pos < 0 || pos >= n_pos) {
    if (threadIdx.x == 0 && error) atomicExch(error, 2);
    pos = max(0, min(pos, n_pos - 1));
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int j_all = lo / KRK_PAGE, j_last = pos / KRK_PAGE;
  const int per = (j_last - j_all + 1 + n_splits - 1) / n_splits;
  const int j_first = j_all + split * per, j_end = min(j_last, j_first + per - 1);  // this block's key blocks; none if j_first > j_end
  const int n_blocks = max(0, j_end - j_first + 1);
  const int n_units = 2 * n_blocks;
  const bool owns_new = n_blocks > 0 && j_end == j_last;  // this block's keys include the new token's

  if (threadIdx.x == 0) {
    for (int r = 0; r < ring; ++r) {
      tc::mbar_init(full_bar + r, 1);
      tc::mbar_init(empty_bar + r, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 4) {
    // ---- producer ----
    for (int i = lane; i < n_blocks; i += 32) pages[i] = table[(size_t)slot * width + (j_first + i) % width];
    __syncwarp();
    if (lane == 0) {
      for (int u = 0; u < n_units; ++u) {
        const int r = u % ring;
        if (u >= ring && !tc::mbar_wait(empty_bar + r, (uint32_t)((u / ring) - 1) & 1)) {
          if (error) atomicExch(error, 19);
          break;
        }
        tc::mbar_expect_tx(full_bar + r, UNIT_BYTES);
        const int row = (pages[u >> 1] * HKV + kh) * KRK_PAGE;
        const CUtensorMap* map = (u & 1) ? &map_v : &map_k;
        bf16* dst = units + (size_t)r * UNIT_ELEMS;
#pragma unroll
        for (int h = 0; h < D / 64; ++h) tc::tma_load_2d(dst + h * SUB_ELEMS, map, full_bar + r, h * 64, row);
      }
    }
    if (n_splits == 1) return;
    // a split block's producer stays for the cluster's barriers, which count every thread
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    cluster.sync();
    return;
  }

  // ---- consumers: warps 0..3 ----
  // gains and the position's table rows are weights: requested before the wait on the kernel that writes the rows
  const size_t page_stride = (size_t)HKV * KRK_PAGE * D;
  const size_t head_off = (size_t)kh * KRK_PAGE * D;
  const bf16* row = qkv + (size_t)seq * q_stride;
  const int q_rows = min(16, G - rt * 16);
  const int k_warp = q_rows % 4;
  constexpr int MAX_ROWS = 4;
  HeadRow regs[MAX_ROWS];
  HeadRow k_regs;
  float v_regs[(D + 31) / 32];
  const bf16* cos_row = cos_t ? cos_t + (size_t)pos * (D / 2) : nullptr;
  const bf16* sin_row = sin_t ? sin_t + (size_t)pos * (D / 2) : nullptr;
#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i)
    if (warp + 4 * i < q_rows) {
      regs[i].load_gains(q_gain, gain_f32, lane);
      regs[i].load_angles(cos_row, sin_row, lane);
    }
  if (warp == k_warp) {
    k_regs.load_gains(k_gain, gain_f32, lane);
    k_regs.load_angles(cos_row, sin_row, lane);
  }
  grid_dependency_wait();
#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i) {
    const int r = warp + 4 * i;
    if (r < q_rows) regs[i].load_values(row + (size_t)(kh * G + rt * 16 + r) * D, lane);
  }
  if (warp == k_warp) {
    k_regs.load_values(row + (size_t)(HQ + kh) * D, lane);
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      v_regs[i] = d < D ? __bfloat162float(row[(size_t)(HQ + HKV + kh) * D + d]) : 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_ROWS; ++i) {
    const int r = warp + 4 * i;
    if (r < q_rows) {
      regs[i].finish(q_s + r * DP, q_gain != nullptr, cos_t != nullptr, eps, lane);
    } else if (r < 16) {
      for (int d = lane; d < D; d += 32) q_s[r * DP + d] = __float2bfloat16_rn(0.f);
    }
  }
  if (warp == k_warp) {
    k_regs.finish(kv_new, k_gain != nullptr, cos_t != nullptr, eps, lane);
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) kv_new[D + d] = __float2bfloat16_rn(v_regs[i]);
    }
    __syncwarp();
    if (rt == 0 && owns_new) {
      const int page = table[(size_t)slot * width + j_last % width];
      const size_t at = (size_t)page * page_stride + head_off + (size_t)(pos % KRK_PAGE) * D;
      for (int d = lane; d < D; d += 32) {
        k_cache[at + d] = kv_new[d];
        v_cache[at + d] = kv_new[D + d];
      }
    }
  }
  consumer_sync();

  uint32_t qf[KSTEPS][4];
  load_q(qf, q_s + g * DP, q_s + (g + 8) * DP, lane);
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  bool alive = true;  // false once a wait ran out: the flow stays the same for all warps, the results are void
  auto arrived = [&](int u) {
    if (alive && !tc::mbar_wait(full_bar + u % ring, (uint32_t)(u / ring) & 1)) {
      alive = false;
      if (lane == 0 && error) atomicExch(error, 19);
    }
  };
  auto hand_back = [&](int u) {
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(empty_bar + u % ring);
  };
  const int tid = threadIdx.x;  // 0..127 among the consumers
  for (int j = j_first; j <= j_end; ++j) {
    const int uk = 2 * (j - j_first), uv = uk + 1;
    bf16* ks = units + (size_t)(uk % ring) * UNIT_ELEMS;
    bf16* vs = units + (size_t)(uv % ring) * UNIT_ELEMS;
    arrived(uk);
    if (j == j_last) {  // the page in shared memory predates this step's write: put the new key in
      for (int i = tid; i < D; i += 128) ks[page_off<true>(pos % KRK_PAGE, i >> 3) + (i & 7)] = kv_new[i];
      consumer_sync();
    }
    const int key0 = warp * 16;
    float s[2][4];
    qk_tile<2, true>(s, qf, ks, key0, lane);
    hand_back(uk);
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = j * KRK_PAGE + key0 + n * 8 + 2 * t4 + (c & 1);
        s[n][c] = (key <= pos && key >= lo) ? s[n][c] * scale_log2 : -INFINITY;
      }
    softmax_update<2>(s, m, l, o);
    arrived(uv);
    if (j == j_last) {
      for (int i = tid; i < D; i += 128) vs[page_off<true>(pos % KRK_PAGE, i >> 3) + (i & 7)] = kv_new[D + i];
      consumer_sync();
    }
    pv_tile<2, true>(o, s, vs, key0, lane);
    hand_back(uv);
  }
  consumer_sync();  // every warp is done with the ring: it now holds the warps' partials

  constexpr int RP = D + 2;
  float* red = reinterpret_cast<float*>(base);  // [4 warps][16 rows][RP]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float* dst = red + ((size_t)warp * 16 + g + 8 * h) * RP;
    if (t4 == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
    for (int n = 0; n < DTILES; ++n) {
      dst[n * 8 + 2 * t4] = o[n][2 * h];
      dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
    }
  }
  consumer_sync();
  // the four warps' partials of a row, in warp order: straight to the output if the block has all keys, else into
  // block 0's inbox through distributed shared memory
  float* inbox0 = n_splits > 1 ? cluster.map_shared_rank(inbox, 0) : nullptr;
  if (n_splits > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every block has started
  for (int r = warp; r < q_rows; r += 4) {
    float mw[4], big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mw[w] = red[((size_t)w * 16 + r) * RP + D]; big = fmaxf(big, mw[w]); }
    const float safe = big == -INFINITY ? 0.f : big;
    float wgt[4], lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { wgt[w] = exp2f(mw[w] - safe); lsum += wgt[w] * red[((size_t)w * 16 + r) * RP + D + 1]; }
    if (n_splits == 1) {
      const float inv = 1.0f / lsum;
      bf16* dst = out + ((size_t)seq * HQ + kh * G + rt * 16 + r) * D;
      for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * RP + d];
        dst[d] = __float2bfloat16_rn(acc * inv);
      }
    } else {
      float* dst = inbox0 + ((size_t)split * inbox_rows + r) * RP;
      for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * RP + d];
        dst[d] = acc;
      }
      if (lane == 0) { dst[D] = big; dst[D + 1] = lsum; }
    }
  }
  if (n_splits == 1) return;
  cluster.sync();  // every block's partial has arrived in block 0
  if (split == 0) {
    for (int r = warp; r < q_rows; r += 4) {  // the splits' partials of a row, in split order
      const float* mine = inbox + (size_t)r * RP;
      const size_t step = (size_t)inbox_rows * RP;
      float big = -INFINITY;
      for (int s2 = 0; s2 < n_splits; ++s2) big = fmaxf(big, mine[s2 * step + D]);
      float lsum = 0.f;
      float acc[(D + 31) / 32];
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
      for (int s2 = 0; s2 < n_splits; ++s2) {
        const float w = exp2f(mine[s2 * step + D] - big);
        lsum += w * mine[s2 * step + D + 1];
#pragma unroll
        for (int i = 0; i < (D + 31) / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] += w * mine[s2 * step + d];
        }
      }
      const float inv = 1.0f / lsum;
      bf16* dst = out + ((size_t)seq * HQ + kh * G + rt * 16 + r) * D;
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dst[d] = __float2bfloat16_rn(acc[i] * inv);
      }
    }
  }
}

int launch_decode_tma(bf16* out, const bf16* qkv, int q_stride, int HQ, int HKV, const void* q_gain, const void* k_gain,
                      int gain_f32, const bf16* cos_t, const bf16* sin_t, float eps, const int* seq_slot,
                      const int* seq_start, const int* table, int width, bf16* k_cache, bf16* v_cache, int n_pages,
                      int n_seqs, float scale, int window, int splits, int n_pos, int* error, cudaStream_t stream) {
  if (width > TMA_MAX_WIDTH) return -2;
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  const int inbox_rows = G < 16 ? G : 16;
  const size_t inbox = splits > 1 ? (size_t)splits * inbox_rows * (D + 2) * sizeof(float) : 0;
  const size_t fixed = 1024 + (size_t)(16 * DP + 2 * D) * sizeof(bf16) + (size_t)((width + 3) & ~3) * sizeof(int) + 64 + inbox;
  // The ring takes what the blocks that share an SM leave one another: two blocks per SM when there are more
  // blocks than SMs, else one block with a ring of up to twelve units (bytes in flight are what bounds the kernel).
  int sms = 148;
  {
    static int sm_count = 0;
    if (!sm_count) {
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sm_count = 148;
    }
    sms = sm_count;
  }
  const long long blocks = (long long)splits * HKV * row_tiles * n_seqs;
  const size_t budget = blocks > sms ? 111 * 1024 : 220 * 1024;
  if (fixed + 2 * UNIT_BYTES > budget) return -2;
  int ring = (int)((budget - fixed) / (UNIT_BYTES + 16));
  ring = ring > 12 ? 12 : ring;
  if (ring < 2 || (size_t)ring * UNIT_BYTES < (size_t)4 * 16 * (D + 2) * sizeof(float)) return -2;
  const size_t smem = fixed + (size_t)ring * UNIT_BYTES + (size_t)2 * ring * 8;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)n_pages * HKV * KRK_PAGE;
  int rc = tc::make_map_bf16(&map_k, k_cache, rows, D, D, 64);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_v, v_cache, rows, D, D, 64);
  if (rc) return rc;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const float scale_log2 = scale * LOG2E;
  if (splits == 1)  // no cluster: the plain launch, whose blocks the device places as it likes
    return (int)launch_pdl(attention_decode_tma_kernel, dim3(1, HKV * row_tiles, n_seqs), dim3(TMA_THREADS), smem, stream,
                           map_k, map_v, out, qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32, cos_t, sin_t, eps, seq_slot,
                           seq_start, table, width, k_cache, v_cache, scale_log2, window, row_tiles, n_pos, ring, inbox_rows,
                           error);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, HKV * row_tiles, n_seqs);
  cfg.blockDim = dim3(TMA_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = splits;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (splits > 8) {
    // clusters of more than eight blocks have to be allowed per kernel, and a device need not have room for one:
    // asked once per shared-memory size; -8 tells the caller to take eight
    static int fits = -1;
    static size_t fits_smem = 0;
    if (fits < 0 || fits_smem != smem) {
      int clusters = 0;
      if (cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess ||
          cudaOccupancyMaxActiveClusters(&clusters, attention_decode_tma_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
      }
      fits = clusters > 0 ? 1 : 0;
      fits_smem = smem;
    }
    if (!fits) return -8;
  }
  return (int)cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel, map_k, map_v, out, qkv, q_stride, HQ, HKV, q_gain, k_gain,
                                 gain_f32, cos_t, sin_t, eps, seq_slot, seq_start, table, width, k_cache, v_cache, scale_log2,
                                 window, row_tiles, n_pos, ring, inbox_rows, error);
}
#endif  // head sizes that TMA pages serve

}  // namespace

// out [rows, HQ*D]; q rows are the first HQ*D elements of each qkv row (row stride q_stride elements).
KRK_API int krk_attention_prefill(void* out, const void* qkv, int q_stride, int HQ, int HKV, const int* seq_slot,
                                  const int* seq_start, const int* seq_qlen, const int* cu_q, const int* table,
                                  int width, const void* k_cache, const void* v_cache, int n_seqs, int max_q_len,
                                  float scale, int window, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  const int G = HQ / HKV;
  const long long tiles = ((long long)max_q_len * G + 63) / 64;
  if (tiles > 0x7fffffffLL || HKV > 65535 || n_seqs > 65535) return -3;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAGE_SMEM);
    configured = true;
  }
  dim3 grid((unsigned)tiles, HKV, n_seqs);
  attention_prefill_kernel<<<grid, THREADS, PAGE_SMEM, stream>>>(
      (bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, seq_slot, seq_start, seq_qlen, cu_q, table, width,
      (const bf16*)k_cache, (const bf16*)v_cache, scale * LOG2E, window);
  KRK_CHECK_LAUNCH();
  return 0;
}

// One token per sequence: row `seq` of qkv is sequence seq's token at position seq_start[seq].
// part: float32 scratch of n_seqs * HQ * splits * (D + 2) elements.
KRK_API int krk_attention_decode(void* out, const void* qkv, int q_stride, int HQ, int HKV, const int* seq_slot,
                                 const int* seq_start, const int* table, int width, const void* k_cache,
                                 const void* v_cache, int n_seqs, float scale, int window, int splits, void* part,
                                 cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  if (HKV * row_tiles > 65535 || n_seqs > 65535 || splits < 1) return -3;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
    configured = true;
  }
  dim3 grid(splits, HKV * row_tiles, n_seqs);
  cudaError_t e = launch_pdl(attention_decode_kernel, grid, dim3(THREADS), DECODE_SMEM, stream, (float*)part,
                             (const bf16*)qkv, q_stride, HQ, HKV, seq_slot, seq_start, table, width,
                             (const bf16*)k_cache, (const bf16*)v_cache, scale * LOG2E, window, row_tiles);
  if (e != cudaSuccess) return (int)e;
  const int items = n_seqs * HQ;
  e = launch_pdl(attention_merge_kernel, dim3((items + 3) / 4), dim3(128), 0, stream, (bf16*)out, (const float*)part,
                 items, splits);
  return (int)e;
}

#ifdef KRK_TRACE
KRK_API int krk_trace_dump(unsigned long long* host, unsigned int cap, unsigned int* count) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(count, krk_trace_count, sizeof(unsigned int));
  unsigned int n = *count < cap ? *count : cap;
  if (n > KRK_TRACE_CAP) n = KRK_TRACE_CAP;
  cudaMemcpyFromSymbol(host, krk_trace_buf, (size_t)n * 4 * sizeof(unsigned long long));
  unsigned int zero = 0;
  cudaMemcpyToSymbol(krk_trace_count, &zero, sizeof(unsigned int));
  return 0;
}
#endif

// One token per sequence, from the raw QKV rows to the attention output in one launch (see the
// kernel's text). qkv rows hold q heads, k heads, v heads; gains and tables may be null. splits:
// 1, 2, 4, 8 or 16 blocks per cluster (16 where the device has room for such a cluster, else 8). The keys and values of the new tokens are written to the cache.
KRK_API int krk_attention_decode_fused(void* out, const void* qkv, int q_stride, int HQ, int HKV, const void* q_gain,
                                       const void* k_gain, int gain_f32, const void* cos_t, const void* sin_t,
                                       float eps, const int* seq_slot, const int* seq_start, const int* table,
                                       int width, void* k_cache, void* v_cache, int n_seqs, float scale, int window,
                                       int splits, int n_pos, int* error, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  if (HKV * row_tiles > 65535 || n_seqs > 65535) return -3;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return -2;
  if (splits == 16) {
    const int rc = launch_decode_fused<2>((bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32,
                                          (const bf16*)cos_t, (const bf16*)sin_t, eps, seq_slot, seq_start, table, width,
                                          (bf16*)k_cache, (bf16*)v_cache, n_seqs, scale, window, splits, n_pos, error, stream);
    if (rc != -8) return rc;
    splits = 8;  // no room for a cluster of sixteen on this device
  }
  if (splits == 1)
    return launch_decode_fused<3>((bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32,
                                  (const bf16*)cos_t, (const bf16*)sin_t, eps, seq_slot, seq_start, table, width,
                                  (bf16*)k_cache, (bf16*)v_cache, n_seqs, scale, window, splits, n_pos, error, stream);
  return launch_decode_fused<2>((bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32,
                                (const bf16*)cos_t, (const bf16*)sin_t, eps, seq_slot, seq_start, table, width,
                                (bf16*)k_cache, (bf16*)v_cache, n_seqs, scale, window, splits, n_pos, error, stream);
}

// The same step with the blocks fed by TMA (see attention_decode_tma_kernel): one block per (sequence, kv head),
// or a cluster of `splits` blocks (1, 2, 4, 8 or 16; 8 where the device has no room for 16) that share its keys.
// n_pages: pages of the cache (for the TMA maps). Returns -2 for head sizes that are no multiple of 64, page
// tables wider than 1024 entries and shapes whose shared memory does not fit: the caller then takes the kernel above.
KRK_API int krk_attention_decode_fused_tma(void* out, const void* qkv, int q_stride, int HQ, int HKV, const void* q_gain,
                                           const void* k_gain, int gain_f32, const void* cos_t, const void* sin_t,
                                           float eps, const int* seq_slot, const int* seq_start, const int* table,
                                           int width, void* k_cache, void* v_cache, int n_pages, int n_seqs, float scale,
                                           int window, int splits, int n_pos, int* error, cudaStream_t stream) {
#if KRK_HEAD_DIM % 64 == 0
  if (n_seqs == 0) return 0;
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  if (HKV * row_tiles > 65535 || n_seqs > 65535) return -3;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return -2;
  int rc = launch_decode_tma((bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32, (const bf16*)cos_t,
                             (const bf16*)sin_t, eps, seq_slot, seq_start, table, width, (bf16*)k_cache, (bf16*)v_cache,
                             n_pages, n_seqs, scale, window, splits, n_pos, error, stream);
  if (rc == -8)  // no room for a cluster of sixteen on this device
    rc = launch_decode_tma((bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, q_gain, k_gain, gain_f32, (const bf16*)cos_t,
                           (const bf16*)sin_t, eps, seq_slot, seq_start, table, width, (bf16*)k_cache, (bf16*)v_cache,
                           n_pages, n_seqs, scale, window, 8, n_pos, error, stream);
  return rc;
#else
  return -2;
#endif
}

#endif  // head size served by the tensor-core kernels

// ---------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate: the partial results
// live in a fixed array of this library (see attention_noalloc.h for who needs this,
// the limits, and the rules on first call and on overlapping calls).
// ---------------------------------------------------------------------------------
#if KRK_HEAD_DIM % 16 == 0 && KRK_HEAD_DIM <= 256
#include <mutex>

#include "attention_noalloc.h"

static __device__ __align__(256) float krk_noalloc_scratch[KRK_NOALLOC_SCRATCH_BYTES / sizeof(float)];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// Device address of the array per device. In host code the array's name is only a
// handle for the runtime, not an address a kernel could use.
float* noalloc_scratch_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex noalloc_setup_lock;
}  // namespace

extern "C" __attribute__((visibility("default"))) const char* krk_attention_decode_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -3: return "the grid would be too large (too many kv heads or sequences), or splits < 1";
    case KRK_NOALLOC_BAD_SHAPE:
      return "HQ and HKV must be positive with HQ a multiple of HKV, width positive, and q_stride at least (HQ + 2 HKV) * head_dim";
    case KRK_NOALLOC_TOO_LARGE:
      return "n_seqs * HQ * splits * (head_dim + 2) floats exceed the library's fixed 4 MiB scratch; "
             "use fewer splits or sequences per call, or krk_attention_decode with a scratch buffer of your own";
    case KRK_NOALLOC_SETUP_FAILED: return "the device address of the scratch array could not be obtained";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
  }
}

extern "C" __attribute__((visibility("default"))) int krk_attention_decode_noalloc(
    void* out, const void* qkv, int q_stride, int HQ, int HKV, const int* seq_slot, const int* seq_start,
    const int* table, int width, const void* k_cache, const void* v_cache, int n_seqs, float scale, int window,
    int splits, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (n_seqs < 0 || HKV < 1 || HQ < 1 || HQ % HKV != 0 || width < 1 || q_stride < (HQ + 2 * HKV) * D) return KRK_NOALLOC_BAD_SHAPE;
  const int G = HQ / HKV;
  const int row_tiles = (G + 15) / 16;
  if (HKV * row_tiles > 65535 || n_seqs > 65535 || splits < 1) return -3;
  const unsigned long long need = (unsigned long long)n_seqs * HQ * splits * (D + 2) * sizeof(float);
  if (need > KRK_NOALLOC_SCRATCH_BYTES) return KRK_NOALLOC_TOO_LARGE;

  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return KRK_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> guard(noalloc_setup_lock);  // host threads may call at the same time
  if (noalloc_scratch_ptr[device] == nullptr) {  // once per device, with that device current
    float* p = nullptr;
    err = cudaGetSymbolAddress((void**)&p, krk_noalloc_scratch);
    if (err != cudaSuccess) return (int)err;
    if (p == nullptr) return KRK_NOALLOC_SETUP_FAILED;
    err = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
    if (err != cudaSuccess) return (int)err;
    noalloc_scratch_ptr[device] = p;
  }
  float* part = noalloc_scratch_ptr[device];

  dim3 grid(splits, HKV * row_tiles, n_seqs);
  attention_decode_kernel<<<grid, THREADS, DECODE_SMEM, stream>>>(
      part, (const bf16*)qkv, q_stride, HQ, HKV, seq_slot, seq_start, table, width, (const bf16*)k_cache,
      (const bf16*)v_cache, scale * LOG2E, window, row_tiles);
  KRK_CHECK_LAUNCH();
  const int items = n_seqs * HQ;
  attention_merge_kernel<<<(items + 3) / 4, 128, 0, stream>>>((bf16*)out, part, items, splits);
  KRK_CHECK_LAUNCH();
  return 0;
}

#endif
