// Causal grouped-query attention for steps that bring many tokens per sequence, on the
// 5th-generation tensor cores: S = Q K^T and O_j = P V run as tcgen05.mma with their results
// in tensor memory; K and V pages arrive by TMA; the softmax runs in four warps, one query
// row per thread.
//
// Numerics as in the other attention kernels of this library (and the reference's,
// engine/kernels/attention.py:9-11,104-122 of willzeng274/kernel-rush-kawk): scores and
// running max / sum in float32, probabilities rounded to bfloat16 before P.V, the output
// accumulated in float32 (here in registers, one row per thread) and divided by the sum once
// at the end. A query at position p sees keys max(0, p - window + 1)..p. The rows of a tile
// are (token, group member) pairs of one kv head, row R -> token R / G, head kh * G + R % G,
// so all G query heads of a kv head share one read of K and V (attention.py:70-73).
//
// Block = 160 threads. Warps 0..3: softmax and output accumulation, thread t owns row t and
// tensor-memory lane t. Warp 4: allocates tensor memory; its lane 0 issues TMA loads and MMAs.
// Per key block of 128 keys (two cache pages):
//   TMA K, V -> shared memory (128-byte swizzle)             [issuer]
//   S = Q K^T          (tcgen05.mma, K-major A and B)          [issuer]   -> s_full
//   p = exp2(S*c - m)  rounded to bfloat16, written to shared
//       memory over the K tile, which S no longer needs        [softmax]  -> p_ready
//   O_j = P V          (tcgen05.mma, V as an MN-major B)       [issuer]   -> o_full
//   o = o * alpha + O_j (tcgen05.ld)                           [softmax]
// Two blocks share an SM (96 KB of shared memory and 256 tensor-memory columns each at head
// size 128), so one block's softmax overlaps the other's MMAs. Every barrier wait is bounded.
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
constexpr int ROWS = 128;              // query rows per block
constexpr int KEYS = 128;              // keys per block iteration: two pages
constexpr int DB = D / 64;             // 64-wide blocks of the head dimension
constexpr int THREADS = 160;
constexpr uint32_t SUB = 128 * 128;    // bytes of a [128 rows x 64 bf16] swizzled sub-tile
constexpr uint32_t Q_BYTES = DB * SUB, K_BYTES = DB * SUB, V_BYTES = DB * SUB, P_BYTES = 2 * SUB;
constexpr uint32_t KP_BYTES = K_BYTES > P_BYTES ? K_BYTES : P_BYTES;  // P overwrites K
constexpr uint32_t TMEM_COLS = (128 + D) <= 256 ? 256 : 512;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of the 16-byte piece `chunk` (8 elements) of row `r` inside a swizzled [128 x 64] sub-tile
__device__ __forceinline__ uint32_t swz(int r, int chunk) { return (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4); }

__global__ void __launch_bounds__(THREADS, 2)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         bf16* __restrict__ out, const bf16* __restrict__ qkv, int q_stride, int HQ, int HKV,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_qlen, const int* __restrict__ cu_q, const int* __restrict__ table,
                         int width, float scale_log2, int window, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;
  unsigned char* k_s = q_s + Q_BYTES;   // K, then P
  unsigned char* v_s = k_s + KP_BYTES;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(v_s + V_BYTES);
  uint64_t* s_full = kv_full + 1;
  uint64_t* p_ready = kv_full + 2;
  uint64_t* o_full = kv_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_full + 4);

  // blockIdx.x counts (tile, kv head) pairs with the tile as the slow index, descending: blocks start in
  // launch order, so the tiles with the most key blocks, of every kv head, run first and the short ones
  // fill the tail
  const int seq = blockIdx.y, kh = blockIdx.x % HKV;
  const int tile = gridDim.x / HKV - 1 - blockIdx.x / HKV;
  const int G = HQ / HKV;
  const int q_len = seq_qlen[seq];
  const int n_rows = q_len * G;
  if (tile * ROWS >= n_rows) return;
  const int start = seq_start[seq], slot = seq_slot[seq], row0 = cu_q[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the query tile: row r, 16-byte piece c -> swizzled K-major sub-tiles; rows past the end are zero
  for (int i = threadIdx.x; i < ROWS * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    const int R = tile * ROWS + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < n_rows) v = *reinterpret_cast<const uint4*>(qkv + (size_t)(row0 + R / G) * q_stride + (size_t)(kh * G + R % G) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + (c / 8) * SUB + swz(r, c % 8)) = v;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = *tmem_slot;        // S: columns 0..127
  const uint32_t tmem_o = tmem_s + 128;      // O_j: columns 128..128+D-1

  // key blocks this tile can see
  const int first_tok = (tile * ROWS) / G;
  const int last_tok = min(q_len - 1, (tile * ROWS + ROWS - 1) / G);
  const int jb_lo = window > 0 ? max(0, start + first_tok - window + 1) / KEYS : 0;
  const int jb_hi = (start + last_tok) / KEYS;

  if (warp == 4) {
    if (lane == 0) {
      // ---- issuer: TMA loads and MMAs ----
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KEYS >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
      bool ok = true;
      for (int jb = jb_lo; jb <= jb_hi && ok; ++jb) {
        const uint32_t it = (uint32_t)(jb - jb_lo);
        if (it > 0 && !mbar_wait(o_full, (it - 1) & 1)) { atomicExch(error, 6); ok = false; break; }  // K/P and V are free
        mbar_expect_tx(kv_full, K_BYTES + V_BYTES);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int page = table[(size_t)slot * width + (2 * jb + half) % width];
          const int row = (page * HKV + kh) * KRK_PAGE;
#pragma unroll
          for (int h = 0; h < DB; ++h) {
            tma_load_2d(k_s + h * SUB + half * (64 * 128), &map_k, kv_full, h * 64, row);
            tma_load_2d(v_s + h * SUB + half * (64 * 128), &map_v, kv_full, h * 64, row);
          }
        }
        if (!mbar_wait(kv_full, it & 1)) { atomicExch(error, 7); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < DB; ++h)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_s, umma_desc_sw128(q_s + h * SUB + kk * 32, 16, 1024),
                      umma_desc_sw128(k_s + h * SUB + kk * 32, 16, 1024), idesc_s, (h > 0 || kk > 0) ? 1u : 0u);
        umma_commit(s_full);
        if (!mbar_wait(p_ready, it & 1)) { atomicExch(error, 8); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ++ks)  // 16 keys per instruction
          umma_bf16(tmem_o, umma_desc_sw128(k_s + (ks / 4) * SUB + (ks % 4) * 32, 16, 1024),
                    umma_desc_sw128(v_s + ks * 16 * 128, SUB, 1024), idesc_o, ks > 0 ? 1u : 0u);
        umma_commit(o_full);
      }
    }
  } else {
    // ---- softmax and accumulation: thread t owns row t ----
    const int r = threadIdx.x;
    const int R = tile * ROWS + r;
    const bool valid = R < n_rows;
    const int tok = valid ? R / G : 0;
    const int pos = valid ? start + tok : -1;  // -1: sees nothing
    const int lo = (valid && window > 0) ? max(0, pos - window + 1) : 0;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int jb = jb_lo; jb <= jb_hi && ok; ++jb) {
      const uint32_t it = (uint32_t)(jb - jb_lo);
      const int key0 = jb * KEYS;
      if (!mbar_wait(s_full, it & 1)) { if (lane == 0) atomicExch(error, 9); ok = false; break; }
      tc_fence_after();
      const bool whole = key0 + KEYS - 1 <= pos && key0 >= lo;  // the row sees every key of the block
      // pass 1: the row's maximum
      float mx = -INFINITY;
#pragma unroll
      for (int c0 = 0; c0 < KEYS; c0 += 32) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, s);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (whole) {
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(s[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c0 + j;
            if (key <= pos && key >= lo) mx = fmaxf(mx, __uint_as_float(s[j]));
          }
        }
      }
      const float m_new = fmaxf(m, mx * scale_log2);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_safe);
      // pass 2: probabilities, their sum, P into shared memory (over the K tile)
      float sum = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < KEYS; c0 += 32) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, s);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float p[32];
        if (whole) {
#pragma unroll
          for (int j = 0; j < 32; ++j) p[j] = fast_exp2(fmaf(__uint_as_float(s[j]), scale_log2, -m_safe));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c0 + j;
            p[j] = (key <= pos && key >= lo) ? fast_exp2(fmaf(__uint_as_float(s[j]), scale_log2, -m_safe)) : 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) sum += p[j];
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // four 16-byte pieces of 8 keys
          uint4 pk;
          __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) pp[e] = __floats2bfloat162_rn(p[8 * q + 2 * e], p[8 * q + 2 * e + 1]);
          const int chunk = (c0 + 8 * q) / 8;  // 0..15 over the 128 keys
          *reinterpret_cast<uint4*>(k_s + (chunk / 8) * SUB + swz(r, chunk % 8)) = pk;
        }
      }
      l = l * alpha + sum;
      m = m_new;
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      if (!mbar_wait(o_full, it & 1)) { if (lane == 0) atomicExch(error, 10); ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_o + lane_addr + c0, t);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c0 + j] = o[c0 + j] * alpha + __uint_as_float(t[j]);
      }
      tc_fence_before();
    }
    if (valid && ok) {
      const float inv = 1.0f / l;
      bf16* dst = out + (size_t)(row0 + tok) * HQ * D + (size_t)(kh * G + R % G) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 pk;
        __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) pp[e] = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(dst + c) = pk;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
  }
}

constexpr size_t SMEM_BYTES = Q_BYTES + KP_BYTES + V_BYTES + 1024 + 64;

}  // namespace

// Same arguments as krk_attention_prefill plus the cache's number of pages (for the TMA maps) and the
// device error word. The keys and values of the step's own rows must be in the cache already.
KRK_API int krk_attention_prefill_tcgen05(void* out, const void* qkv, int q_stride, int HQ, int HKV,
                                          const int* seq_slot, const int* seq_start, const int* seq_qlen,
                                          const int* cu_q, const int* table, int width, const void* k_cache,
                                          const void* v_cache, int n_pages, int n_seqs, int max_q_len, float scale,
                                          int window, int* error, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  const int G = HQ / HKV;
  const long long tiles = ((long long)max_q_len * G + ROWS - 1) / ROWS;
  if (tiles * HKV > 0x7fffffffLL || n_seqs > 65535) return -3;
  if ((q_stride % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15)) return -2;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)n_pages * HKV * KRK_PAGE;
  int rc = make_map_bf16(&map_k, k_cache, rows, D, D, 64);
  if (rc) return rc;
  rc = make_map_bf16(&map_v, v_cache, rows, D, D, 64);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((unsigned)(tiles * HKV), n_seqs, 1);
  attention_tcgen05_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(
      map_k, map_v, (bf16*)out, (const bf16*)qkv, q_stride, HQ, HKV, seq_slot, seq_start, seq_qlen, cu_q, table, width,
      scale * LOG2E, window, error);
  KRK_CHECK_LAUNCH();
  return 0;
}

#endif  // head sizes served by this kernel
