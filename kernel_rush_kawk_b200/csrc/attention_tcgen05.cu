// Causal grouped-query attention for steps that bring many tokens per sequence, on the
// 5th-generation tensor cores. A block owns two query tiles of 128 rows that share every K and V
// page it reads; S = Q K^T, P and O all live in tensor memory:
//
//   tensor memory (512 columns): S0 | S1 | O0 | O1. P_t, rounded to bfloat16, overwrites the first
//   64 columns of S_t (two keys per 32-bit column) and is the A operand of O_t += P_t V.
//   shared memory: Q0, Q1, and K and V double-buffered (128-byte swizzle, filled by TMA).
//
// Warps 0..7 run the softmax of tile 0 and of tile 1 in turn (thread = query row = tensor-memory lane,
// and one half of the block's keys: warps w and w + 4 share their rows); lane 0 of warp 8 issues every
// MMA (lane 0 of warp 9 the TMA loads), in the order
//   ... PV0(j-1) QK0(j) PV1(j-1) QK1(j) PV0(j) QK0(j+1) ...
// so that while one tile's rows are in the softmax the tensor core works for the other tile. A tile's
// next MMAs wait for its softmax, so all eight warps on one tile (half the time per block) shorten the
// chain that bounds the kernel: softmax of a block, its P V, the next block's Q K^T.
// Per key block of 128 keys (two cache pages) and tile:
//   S = Q K^T                                   [issuer]   -> s_full
//   row max; p = exp2(S*c - m) rounded to bfloat16 -> tensor memory  [softmax]  -> p_ready
//   O += P V   (V as an MN-major B operand)     [issuer]
// O stays in tensor memory across key blocks. The reference maximum m of a row moves only when the
// row's maximum has grown by more than 2^8 since it was set (then the warp rescales its O rows in
// tensor memory); until then p <= 2^8, which float32 sums and bfloat16 probabilities hold without
// loss. The final division by the row's sum undoes the choice of m exactly as with a running maximum.
//
// Numerics as in the other attention kernels of this library (and the reference's,
// engine/kernels/attention.py:9-11,104-122 of willzeng274/kernel-rush-kawk): scores, maxima and sums
// in float32, probabilities rounded to bfloat16 before P.V, the output accumulated in float32. A
// query at position p sees keys max(0, p - window + 1)..p. The rows of a tile are (token, group
// member) pairs of one kv head, row R -> token R / G, head kh * G + R % G, so all G query heads of a
// kv head share one read of K and V (attention.py:70-73). Every barrier wait is bounded.
//
// Compiled once per head size, for head sizes 64 and 128: -DKRK_HEAD_DIM=<D>.
#include "tcgen05.cuh"

#ifndef KRK_HEAD_DIM
#error "compile with -DKRK_HEAD_DIM=<head size>"
#endif

#if KRK_HEAD_DIM == 64 || KRK_HEAD_DIM == 128

namespace {

using namespace tc;

constexpr int D = KRK_HEAD_DIM;
constexpr int ROWS = 128;              // query rows per tile
constexpr int PAIR = 2 * ROWS;         // query rows per block
constexpr int KEYS = 128;              // keys per block iteration: two pages
constexpr int HALF = KEYS / 2;         // score columns a softmax thread holds at a time
constexpr int DB = D / 64;             // 64-wide blocks of the head dimension
constexpr int THREADS = 320;           // 8 softmax warps, the warp that issues the MMAs, the warp that loads
constexpr uint32_t SUB = 128 * 128;    // bytes of a [128 rows x 64 bf16] swizzled sub-tile
constexpr uint32_t TILE_BYTES = DB * SUB;  // a Q, K or V tile
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_O = 256;       // O_t starts at column 256 + t * D; S_t at t * 128
constexpr float LOG2E = 1.4426950408889634f;
constexpr int PAGE_IDS = 1024;         // page-table entries a block keeps in shared memory (64 K keys)
constexpr float RESCALE_STEP = 8.f;    // in log2 units: the reference maximum moves when outgrown by 2^8

enum Bar { K_FULL = 0, V_FULL = 2, K_FREE = 4, V_FREE = 6, S_FULL = 8, P_READY = 10, O_DONE = 12, Q_FULL = 14, N_BARS = 15 };

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of the 16-byte piece `chunk` (8 elements) of row `r` inside a swizzled [128 x 64] sub-tile
__device__ __forceinline__ uint32_t swz(int r, int chunk) { return (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4); }

struct TileRange {
  int lo, hi;  // key blocks the tile can see; lo > hi: the tile has no rows
  __device__ __forceinline__ bool has(int j) const { return j >= lo && j <= hi; }
};

__device__ __forceinline__ TileRange tile_range(int row_begin, int n_rows, int G, int q_len, int start, int window) {
  TileRange t;
  if (row_begin >= n_rows) { t.lo = 1; t.hi = 0; return t; }
  const int first_tok = row_begin / G;
  const int last_tok = min(q_len - 1, (row_begin + ROWS - 1) / G);
  t.lo = window > 0 ? max(0, start + first_tok - window + 1) / KEYS : 0;
  t.hi = (start + last_tok) / KEYS;
  return t;
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_o, int q_by_tma, bf16* __restrict__ out, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_qlen, const int* __restrict__ cu_q, const int* __restrict__ table,
                         int width, float scale_log2, int window, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                    // two tiles
  unsigned char* k_s = q_s + 2 * TILE_BYTES;    // two stages
  unsigned char* v_s = k_s + 2 * TILE_BYTES;    // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  int* pages_s = reinterpret_cast<int*>(tmem_slot + 2);  // [PAGE_IDS] the block's page-table entries, from page 2 * j_lo on
  float* xchg = reinterpret_cast<float*>(pages_s + PAGE_IDS);  // [2 copies][2 halves][ROWS] partial row maxima of the softmax warps
  float* xsum = xchg + 4 * ROWS;                               // [2 tiles][2 halves][ROWS] their partial row sums
  volatile int* gave_up = reinterpret_cast<volatile int*>(xsum + 4 * ROWS);  // [4] per pair of softmax warps

  // blockIdx.x counts (row pair, kv head) with the pair as the slow index, descending: blocks start in
  // launch order, so the pairs with the most key blocks, of every kv head, run first and the short ones
  // fill the tail
  const int seq = blockIdx.y, kh = blockIdx.x % HKV;
  const int pair = gridDim.x / HKV - 1 - blockIdx.x / HKV;
  const int G = HQ / HKV;
  const int q_len = seq_qlen[seq];
  const int n_rows = q_len * G;
  if (pair * PAIR >= n_rows) return;
  const int start = seq_start[seq], slot = seq_slot[seq], row0 = cu_q[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const TileRange r0 = tile_range(pair * PAIR, n_rows, G, q_len, start, window);
  const TileRange r1 = tile_range(pair * PAIR + ROWS, n_rows, G, q_len, start, window);
  const int j_lo = r0.lo;                                   // tile 0 exists and starts no later than tile 1
  const int j_hi = r1.lo <= r1.hi ? max(r0.hi, r1.hi) : r0.hi;
  const int n = j_hi - j_lo + 1;

  // TMA loads: the first ones by the issuer (warp 8, lane 0) before the block's first barrier, the rest by the loader
  auto load_tile = [&](unsigned char* dst, const CUtensorMap* map, uint64_t* bar, int i) {
    mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      // from shared memory: a load from the page table here would stand between the issuing thread's MMAs
      const int at = 2 * i + half;
      const int page = at < PAGE_IDS ? pages_s[at] : table[(size_t)slot * width + (2 * (j_lo + i) + half) % width];
      const int row = (page * HKV + kh) * KRK_PAGE;
#pragma unroll
      for (int h = 0; h < DB; ++h) tma_load_2d(dst + h * SUB + half * (64 * 128), map, bar, h * 64, row);
    }
  };
  auto load_k = [&](int i) { load_tile(k_s + (i & 1) * TILE_BYTES, &map_k, bars + K_FULL + (i & 1), i); };
  auto load_v = [&](int i) { load_tile(v_s + (i & 1) * TILE_BYTES, &map_v, bars + V_FULL + (i & 1), i); };

  if (warp == 8) {
    // The block's first loads in the order of what they wait for: the error word and the page-table entries are
    // requested together, the query tiles (which need neither) go out before either has arrived.
    // A block of this step that gave up on a wait (codes from 3 on): the others do no work. The host reads and
    // clears the word at the end of every step, so a flag never outlives the step that raised it.
    const int error_now = *reinterpret_cast<volatile int*>(error);
    int page_here[PAGE_IDS / 32 > 4 ? 4 : PAGE_IDS / 32];  // the first 128 entries, one load per lane and round
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = lane + 32 * q;
      page_here[q] = i < min(2 * n, PAGE_IDS) ? table[(size_t)slot * width + (2 * j_lo + i) % width] : 0;
    }
    if (lane == 0) {
      for (int i = 0; i < N_BARS; ++i) mbar_init(bars + i, (i == P_READY || i == P_READY + 1) ? 2 * ROWS : 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      for (int i = 0; i < 4; ++i) gave_up[i] = 0;
      if (q_by_tma) {
        // a query tile is a box of 128 / G tokens x G heads x 64 dims per 64-wide block of the head: its rows
        // land in (token, group member) order, which is the tile's row order
        const int tiles_here = r1.lo <= r1.hi ? 2 : 1;
        mbar_expect_tx(bars + Q_FULL, tiles_here * TILE_BYTES);
        for (int t = 0; t < tiles_here; ++t)
#pragma unroll
          for (int h = 0; h < DB; ++h)
            tma_load_3d(q_s + t * TILE_BYTES + h * SUB, &map_q, bars + Q_FULL, h * 64, kh * G, row0 + (pair * PAIR + t * ROWS) / G);
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (lane + 32 * q < min(2 * n, PAGE_IDS)) pages_s[lane + 32 * q] = page_here[q];
    for (int i = lane + 128; i < min(2 * n, PAGE_IDS); i += 32) pages_s[i] = table[(size_t)slot * width + (2 * j_lo + i) % width];
    __syncwarp();
    if (lane == 0) {
      tmem_slot[1] = (uint32_t)(error_now >= 3);
      load_k(0);
      load_v(0);
      if (n > 1) load_k(1);
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (!q_by_tma) {
    // the query tiles by hand: row r, 16-byte piece c -> swizzled K-major sub-tiles; rows past the end are zero
    for (int i = threadIdx.x; i < PAIR * (D / 8); i += THREADS) {
      const int r = i / (D / 8), c = i % (D / 8);
      const int R = pair * PAIR + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (R < n_rows) v = *reinterpret_cast<const uint4*>(qkv + (size_t)(row0 + R / G) * q_stride + (size_t)(kh * G + R % G) * D + c * 8);
      *reinterpret_cast<uint4*>(q_s + (r / ROWS) * TILE_BYTES + (c / 8) * SUB + swz(r % ROWS, c % 8)) = v;
    }
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool dead = tmem_slot[1] != 0;

  if (dead) {
    // nothing to do
  } else if (warp == 8) {
    if (lane == 0) {
      // ---- issuer: TMA loads and MMAs ----
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KEYS >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      bool ok = true;
      auto give_up = [&](int code) { atomicExch(error, code); ok = false; };
      auto qk = [&](int t, int i) {  // S_t = Q_t K_i^T
        const unsigned char* q = q_s + t * TILE_BYTES;
        const unsigned char* k = k_s + (i & 1) * TILE_BYTES;
#pragma unroll
        for (int h = 0; h < DB; ++h)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem + t * 128, umma_desc_sw128(q + h * SUB + kk * 32, 16, 1024),
                      umma_desc_sw128(k + h * SUB + kk * 32, 16, 1024), idesc_s, (h > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bars + S_FULL + t);
      };
      auto pv = [&](int t, int i, bool first) {  // O_t (+)= P_t V_i, 16 keys (8 columns of P) per instruction
        const unsigned char* v = v_s + (i & 1) * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ++ks)
          umma_bf16_tmem_a(tmem + TMEM_O + t * D, tmem + t * 128 + ks * 8, umma_desc_sw128(v + ks * 16 * 128, SUB, 1024),
                           idesc_o, (first && ks == 0) ? 0u : 1u);
      };
      const TileRange rng[2] = {r0, r1};
      if (q_by_tma && !mbar_wait(bars + Q_FULL, 0)) give_up(14);
      if (ok && !mbar_wait(bars + K_FULL, 0)) give_up(6);
      if (ok) {
        tc_fence_after();
        if (r0.has(j_lo)) qk(0, 0);
        if (r1.has(j_lo)) qk(1, 0);
        umma_commit(bars + K_FREE);
      }
      for (int i = 0; i < n && ok; ++i) {
        const int j = j_lo + i, b = i & 1;
        bool v_ready = false, k_ready = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (rng[t].has(j)) {
            if (!mbar_wait(bars + P_READY + t, (j - rng[t].lo) & 1)) { give_up(8); break; }
            if (!v_ready) {
              if (!mbar_wait(bars + V_FULL + b, (i >> 1) & 1)) { give_up(9); break; }
              v_ready = true;
            }
            tc_fence_after();
            pv(t, i, j == rng[t].lo);
            if (j == rng[t].hi) umma_commit(bars + O_DONE + t);
          }
          if (t == 1) umma_commit(bars + V_FREE + b);
          if (i + 1 < n) {
            if (rng[t].has(j + 1)) {
              if (!k_ready) {
                if (!mbar_wait(bars + K_FULL + ((i + 1) & 1), ((i + 1) >> 1) & 1)) { give_up(10); break; }
                k_ready = true;
              }
              tc_fence_after();
              qk(t, i + 1);
            }
            if (t == 1) umma_commit(bars + K_FREE + ((i + 1) & 1));
          }
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // ---- loader: the TMA loads after the first ones. A thread of its own: issuing a load takes the time of
      // several MMAs, and the issuer's instruction stream is what bounds the kernel.
      for (int i = 0; i < n; ++i) {
        if (i + 1 < n) {  // V of the next block goes where block i - 1's was
          if (i >= 1 && !mbar_wait(bars + V_FREE + ((i + 1) & 1), ((i - 1) >> 1) & 1)) { atomicExch(error, 7); break; }
          load_v(i + 1);
        }
        if (i + 2 < n) {  // K of block i + 2 goes where block i's was
          if (!mbar_wait(bars + K_FREE + (i & 1), (i >> 1) & 1)) { atomicExch(error, 11); break; }
          load_k(i + 2);
        }
      }
    }
  } else {
    // ---- softmax: all eight warps work on one tile at a time, tile 0 and tile 1 in turn. Thread = query row r of
    // both tiles (its tensor-memory lane) and one half of a block's keys: warps w and w + 4 share the rows
    // 32 (w & 3) .. + 31 and exchange their partial row maxima (and, at the end, sums) through shared memory.
    // A tile's block is through the softmax in half the time, which is what the other tile's MMAs wait for.
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const TileRange rng[2] = {r0, r1};
    bool valid[2];
    int tok[2], pos[2], lo[2];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int R = pair * PAIR + t * ROWS + r;
      valid[t] = R < n_rows;
      tok[t] = valid[t] ? R / G : 0;
      pos[t] = valid[t] ? start + tok[t] : -1;  // -1: sees nothing
      lo[t] = (valid[t] && window > 0) ? max(0, pos[t] - window + 1) : 0;
    }
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
    bool ok = true, stores_pending = false;
    uint32_t step = 0;
    for (int j = j_lo; j <= j_hi && ok; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j < rng[t].lo || j > rng[t].hi) continue;  // the same for every thread of the block
        const uint32_t c = (uint32_t)(j - rng[t].lo);
        const int key0 = j * KEYS + half * HALF;  // this thread's first key
        const uint32_t tmem_s = tmem + t * 128 + lane_addr;
        const uint32_t tmem_o = tmem + TMEM_O + t * D + lane_addr;
        float* xm = xchg + (step & 1) * 2 * ROWS;  // [half][row], two copies used in turn
        ++step;
        // the row sees keys first..first + span of its half: (unsigned)(i - first) <= span; none of them: no i passes
        const bool whole = key0 + HALF - 1 <= pos[t] && key0 >= lo[t];
        const bool none = pos[t] < max(lo[t], key0);
        const unsigned first = none ? (unsigned)HALF : (unsigned)max(lo[t] - key0, 0);
        const unsigned span = none ? 0u : (unsigned)(pos[t] - key0) - first;
        // tensor-memory loads and stores are warp-wide, and the two warps of a row meet at a barrier that has no
        // time limit: a warp that gives up says so in shared memory and both leave after the barrier
        const bool arrived = __all_sync(0xffffffffu, mbar_wait(bars + S_FULL + t, c & 1));
        uint32_t s[HALF];
        float mx = -INFINITY;
        if (arrived) {
          tc_fence_after();
#pragma unroll
          for (int q = 0; q < HALF / 32; ++q) tmem_ld_32x32(tmem_s + HALF * half + 32 * q, *reinterpret_cast<uint32_t(*)[32]>(s + 32 * q));
          tmem_wait_ld();
          if (whole) {
#pragma unroll
            for (int i = 0; i < HALF; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
          } else {
#pragma unroll
            for (int i = 0; i < HALF; ++i)
              if ((unsigned)i - first <= span) mx = fmaxf(mx, __uint_as_float(s[i]));
          }
          xm[half * ROWS + r] = mx;
        } else if (lane == 0) {
          atomicExch(error, 12);
          gave_up[quad] = 1;
        }
        pair_sync();
        if (gave_up[quad]) { ok = false; break; }
        mx = fmaxf(mx, xm[(half ^ 1) * ROWS + r]);
        const float m_new = fmaxf(m[t], mx * scale_log2);
        const bool outgrown = m[t] != -INFINITY && m_new - m[t] > RESCALE_STEP;
        if (__any_sync(0xffffffffu, outgrown)) {
          // the warp moves its rows' reference maxima (its partner, with the same rows and maxima, decides the
          // same) and scales its half of the columns of O; the block's P.V has not been issued and the one
          // before it is complete (S of this block came after it), so nothing else touches these rows of O
          const float alpha = m[t] == -INFINITY ? 1.f : fast_exp2(m[t] - m_new);
#pragma unroll
          for (int c0 = 0; c0 < D / 2; c0 += 32) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + half * (D / 2) + c0, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + half * (D / 2) + c0, o);
          }
          l[t] *= alpha;
          m[t] = m_new;
        } else if (m[t] == -INFINITY) {
          m[t] = m_new;  // no key seen before this block: O and l are still zero
        }
        const float m_safe = m[t] == -INFINITY ? 0.f : m[t];
        float sum = 0.f;
        uint32_t pk[HALF / 2];
        if (whole) {
#pragma unroll
          for (int i = 0; i < HALF; i += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), scale_log2, -m_safe));
            const float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), scale_log2, -m_safe));
            sum += p0 + p1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            pk[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
        } else {
#pragma unroll
          for (int i = 0; i < HALF; i += 2) {
            const float p0 = ((unsigned)i - first <= span) ? fast_exp2(fmaf(__uint_as_float(s[i]), scale_log2, -m_safe)) : 0.f;
            const float p1 = ((unsigned)(i + 1) - first <= span) ? fast_exp2(fmaf(__uint_as_float(s[i + 1]), scale_log2, -m_safe)) : 0.f;
            sum += p0 + p1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            pk[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        l[t] += sum;
        __syncwarp();  // rows that see their whole half and rows at its edge took different paths
        // P's second half lands on score columns of the partner warp, which holds them in registers since the barrier
        tmem_st_32x32(tmem_s + (HALF / 2) * half, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bars + P_READY + t);
      }
    }
    // the row's sum is the two halves' sums; every thread comes here exactly once, whatever happened before
    xsum[half * ROWS + r] = l[0];
    xsum[2 * ROWS + half * ROWS + r] = l[1];
    pair_sync();
    l[0] += xsum[(half ^ 1) * ROWS + r];
    l[1] += xsum[2 * ROWS + (half ^ 1) * ROWS + r];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (rng[t].lo > rng[t].hi) continue;  // the same for every thread of the block
      // O_t, divided by the row sums and rounded, goes through shared memory: a thread holds half a row, and rows
      // are 2 * D bytes apart at best in the output. It is staged in the tile's query buffer, which its MMAs are
      // done with, in the query tile's own layout (128-byte swizzle), and leaves as the query tile came: one
      // tiled store per 64-wide block of the head when the tile is whole, else 16-byte pieces by all threads,
      // consecutive threads storing consecutive pieces (the rows of a token lie side by side in the output).
      const bool fine = ok && __all_sync(0xffffffffu, mbar_wait(bars + O_DONE + t, 0));
      unsigned char* stage = q_s + t * TILE_BYTES;
      if (fine) {
        tc_fence_after();
        const uint32_t tmem_o = tmem + TMEM_O + t * D + lane_addr;
        const float inv = valid[t] ? 1.0f / l[t] : 0.f;
#pragma unroll
        for (int c0 = 0; c0 < D / 2; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + half * (D / 2) + c0, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 pk;
            __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              pp[e] = __floats2bfloat162_rn(__uint_as_float(o[c + 2 * e]) * inv, __uint_as_float(o[c + 2 * e + 1]) * inv);
            const int piece = (half * (D / 2) + c0 + c) / 8;
            *reinterpret_cast<uint4*>(stage + (piece / 8) * SUB + swz(r, piece % 8)) = pk;
          }
        }
        fence_async_smem();
      } else if (lane == 0) {
        if (ok) atomicExch(error, 13);
        gave_up[quad] = 1;
      }
      asm volatile("bar.sync 5, 256;" ::: "memory");  // the eight softmax warps
      if (gave_up[0] | gave_up[1] | gave_up[2] | gave_up[3]) continue;
      const int row_begin = pair * PAIR + t * ROWS;
      if (q_by_tma && row_begin + ROWS <= n_rows) {
        if (threadIdx.x == 0) {
#pragma unroll
          for (int h = 0; h < DB; ++h) tma_store_3d(&map_o, stage + h * SUB, h * 64, kh * G, row0 + row_begin / G);
          tma_store_commit();
          stores_pending = true;
        }
      } else {
#pragma unroll
        for (int k = 0; k < ROWS * (D / 8) / 256; ++k) {
          const int p = threadIdx.x + 256 * k;
          const int row = p / (D / 8), piece = p % (D / 8);
          const int R = row_begin + row;
          if (R < n_rows)
            *reinterpret_cast<uint4*>(out + (size_t)(row0 + R / G) * HQ * D + (size_t)(kh * G + R % G) * D + piece * 8) =
                *reinterpret_cast<const uint4*>(stage + (piece / 8) * SUB + swz(row, piece % 8));
        }
      }
    }
    if (stores_pending) tma_store_wait_read();  // shared memory is given up when the block ends
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

constexpr size_t SMEM_BYTES = 6 * TILE_BYTES + 1024 + N_BARS * 8 + 64 + PAGE_IDS * sizeof(int) + 8 * ROWS * sizeof(float) + 16;

}  // namespace

// Same arguments as krk_attention_prefill plus the cache's number of pages and the number of rows of qkv
// (for the TMA maps) and the device error word. The keys and values of the step's own rows must be in the cache already.
KRK_API int krk_attention_prefill_tcgen05(void* out, const void* qkv, int q_stride, int HQ, int HKV,
                                          const int* seq_slot, const int* seq_start, const int* seq_qlen,
                                          const int* cu_q, const int* table, int width, const void* k_cache,
                                          const void* v_cache, int n_pages, int n_seqs, int max_q_len, int total_rows,
                                          float scale, int window, int* error, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  const int G = HQ / HKV;
  const long long tiles = ((long long)max_q_len * G + PAIR - 1) / PAIR;
  if (tiles * HKV > 0x7fffffffLL || n_seqs > 65535) return -3;
  if ((q_stride % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15)) return -2;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)n_pages * HKV * KRK_PAGE;
  int rc = make_map_bf16(&map_k, k_cache, rows, D, D, 64);
  if (rc) return rc;
  rc = make_map_bf16(&map_v, v_cache, rows, D, D, 64);
  if (rc) return rc;
  // the query tiles come by TMA when a tile is a whole number of tokens (the group size divides 128)
  const int q_by_tma = (ROWS % G == 0) ? 1 : 0;
  CUtensorMap map_q = map_k;
  if (q_by_tma) {
    rc = make_map_bf16_3d(&map_q, qkv, D, HQ, total_rows, D, q_stride, G, ROWS / G);
    if (rc) return rc;
  }
  CUtensorMap map_o = map_k;
  if (q_by_tma) {
    rc = make_map_bf16_3d(&map_o, out, D, HQ, total_rows, D, (long long)HQ * D, G, ROWS / G);
    if (rc) return rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((unsigned)(tiles * HKV), n_seqs, 1);
  attention_tcgen05_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(
      map_k, map_v, map_q, map_o, q_by_tma, (bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, seq_slot, seq_start, seq_qlen, cu_q, table, width,
      scale * LOG2E, window, error);
  KRK_CHECK_LAUNCH();
  return 0;
}

#endif  // head sizes served by this kernel
