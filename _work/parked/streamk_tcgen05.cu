// out[M, N] = x[M, K] * W[N, K]^T for a batch of up to 128 rows on the 5th-generation tensor
// cores, built for steps that bring 17 to 128 tokens: such a product is weight streaming, so the
// kernel is organised around keeping every SM's memory pipe full and equally loaded.
//
// The weights are the 128-row operand ("swap A and B"): a tile is 128 rows of W (output features)
// by 64 of K, the batch rows are the narrow operand (16, 32, 64 or 128 wide), the accumulator
// [128 features x batch rows] lives in tensor memory. The work, (feature tile, k-block) units, is
// dealt to one block per SM in equal contiguous ranges, whatever the number of tiles ("stream-K");
// a block whose range covers a tile only in part writes its float32 partial to scratch memory,
// and the block that arrives last at a tile adds the parts in their fixed order and finishes the
// tile. So results do not depend on which block came last. TMA brings the tiles into a ring of
// shared-memory stages as deep as shared memory allows; the weights of the first ring-full are
// requested before the wait on the previous kernel (they are written by no kernel). Two
// accumulators in tensor memory alternate, so the read-back of one range overlaps the products of
// the next.
//
// Epilogues: plain (bfloat16 or float32 out) and SwiGLU (rows n and I + n of W are gate and up; out
// = round(round(silu(round(g))) * round(u)), engine/kernels/gemm.py:108-113 of
// willzeng274/kernel-rush-kawk, whose fused kernels serve up to 32 rows, gateup64.py 64).
//
// Block = 192 threads: warp 0 drives TMA, warp 1 owns tensor memory and issues the MMAs, warps
// 2..5 read accumulators back. Every wait is bounded; one that runs out sets the error word.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int TILE_N = 128;   // weight rows (output features) per tile: the MMA's M
constexpr int BK = 64;        // k per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 16;
constexpr uint32_t W_BYTES = TILE_N * BK * 2;

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// the block that owns unit u when U units are dealt to P blocks as [c * U / P, (c + 1) * U / P)
__host__ __device__ __forceinline__ long long owner_of(long long u, long long U, long long P) { return (u * P + P - 1) / U; }

template <int MT, bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(THREADS)
streamk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TOut* __restrict__ out, float* __restrict__ part, int* __restrict__ counters, int M, int N, int K,
               int stages, int up_row_offset, int max_parts, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int NACC = SWIGLU ? 2 : 1;
  constexpr uint32_t X_BYTES = MT * BK * 2;
  constexpr uint32_t STAGE_BYTES = NACC * W_BYTES + X_BYTES;
  constexpr uint32_t ACC_COLS = NACC * MT;                               // columns of one accumulator set
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;  // two sets; 32, 64, 128, 256 or 512
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + (size_t)stages * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* acc_full = empty_bar + MAX_STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* ok_s = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2]: did the wait for this range succeed
  volatile int* last_s = ok_s + 2;                                        // is this block the last at its tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long KB = (K + BK - 1) / BK;
  const long long T = (N + TILE_N - 1) / TILE_N;
  const long long U = T * KB, P = gridDim.x, c = blockIdx.x;
  const long long lo = c * U / P, hi = (c + 1) * U / P;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();  // the next kernel may begin (it waits for this one's results itself)

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ----
      auto load_w = [&](long long u, int s) {
        const int tile = (int)(u / KB), kb = (int)(u % KB);
        unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(full_bar + s, STAGE_BYTES);
        tma_load_2d(stage, &map_w, full_bar + s, kb * BK, tile * TILE_N);
        if (SWIGLU) tma_load_2d(stage + W_BYTES, &map_w, full_bar + s, kb * BK, up_row_offset + tile * TILE_N);
      };
      auto load_x = [&](long long u, int s) {
        tma_load_2d(tiles + (size_t)s * STAGE_BYTES + NACC * W_BYTES, &map_x, full_bar + s, (int)(u % KB) * BK, 0);
      };
      const long long first_fill = (hi - lo) < stages ? (hi - lo) : stages;
      for (long long i = 0; i < first_fill; ++i) load_w(lo + i, (int)i);   // weights: written by no kernel
      grid_dependency_wait();                                                // the batch rows come from the previous one
      for (long long i = 0; i < first_fill; ++i) load_x(lo + i, (int)i);
      for (long long i = first_fill; i < hi - lo; ++i) {
        const int s = (int)(i % stages);
        if (!mbar_wait(empty_bar + s, (uint32_t)((i / stages) - 1) & 1)) { atomicExch(error, 15); break; }
        load_w(lo + i, s);
        load_x(lo + i, s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc = umma_idesc(TILE_N, MT);
      int q = -1, buf = 0;
      for (long long i = 0; i < hi - lo; ++i) {
        const long long u = lo + i;
        const int kb = (int)(u % KB);
        const int s = (int)(i % stages);
        const bool first = (i == 0) || kb == 0;
        if (first) {
          ++q;
          buf = q & 1;
          if (q >= 2 && !mbar_wait(acc_empty + buf, (uint32_t)((q >> 1) - 1) & 1)) { atomicExch(error, 16); break; }
          tc_fence_after();
        }
        if (!mbar_wait(full_bar + s, (uint32_t)(i / stages) & 1)) { atomicExch(error, 17); break; }
        tc_fence_after();
        unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
        const uint64_t w_desc = umma_desc(stage);
        const uint64_t w2_desc = umma_desc(stage + W_BYTES);
        const uint64_t x_desc = umma_desc(stage + NACC * W_BYTES);
        const uint32_t acc = tmem_base + (uint32_t)buf * ACC_COLS;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
          const uint32_t accumulate = (first && k == 0) ? 0u : 1u;
          umma_bf16(acc, w_desc + adv, x_desc + adv, idesc, accumulate);
          if (SWIGLU) umma_bf16(acc + MT, w2_desc + adv, x_desc + adv, idesc, accumulate);
        }
        umma_commit(empty_bar + s);
        if (i == hi - lo - 1 || kb == (int)KB - 1) umma_commit(acc_full + buf);
      }
    }
  } else {
    // ---- read-back: warp w owns lanes 32 * (w % 4) .. + 31 of tensor memory = features of the tile ----
    grid_dependency_wait();  // whoever read this output buffer before has finished
    const int quarter = warp & 3;
    const int et = (quarter << 5) + lane;        // 0..127: this thread's feature within the tile
    int q = 0;
    for (long long u = lo; u < hi; ++q) {
      const long long tile = u / KB;
      const long long end = (tile + 1) * KB < hi ? (tile + 1) * KB : hi;
      const bool whole = (u == tile * KB) && (end == (tile + 1) * KB);
      const int buf = q & 1;
      if (et == 0) ok_s[buf] = mbar_wait(acc_full + buf, (uint32_t)(q >> 1) & 1) ? 1 : 0;
      epilogue_sync();
      if (!ok_s[buf]) {
        if (et == 0) atomicExch(error, 18);
        break;
      }
      tc_fence_after();
      const int n = (int)tile * TILE_N + et;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_COLS;

      auto finish = [&](int c0, const float (&g)[16], const float (&up)[16]) {  // 16 batch rows of this feature
        if (n >= N) return;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = c0 + j;
          if (row < M) {
            float v = g[j];
            if (SWIGLU) {
              const float gate = round_to<bf16>(v);
              v = round_to<bf16>(gate / (1.0f + __expf(-gate))) * round_to<bf16>(up[j]);
            }
            out[(size_t)row * N + n] = from_float<TOut>(v);
          }
        }
      };

      const long long first_cta = owner_of(tile * KB, U, P);
      float* mine = part + ((size_t)tile * max_parts + (size_t)(c - first_cta)) * (NACC * MT * TILE_N);
#pragma unroll 1
      for (int c0 = 0; c0 < MT; c0 += 16) {
        uint32_t gr[16], ur[16];
        tmem_ld_32x32_x16(taddr + c0, gr);
        if (SWIGLU) tmem_ld_32x32_x16(taddr + MT + c0, ur);
        tmem_wait_ld();
        float g[16], up[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          g[j] = __uint_as_float(gr[j]);
          up[j] = SWIGLU ? __uint_as_float(ur[j]) : 0.f;
        }
        if (whole) {
          finish(c0, g, up);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __stcg(mine + (size_t)(c0 + j) * TILE_N + et, g[j]);
            if (SWIGLU) __stcg(mine + (size_t)(MT + c0 + j) * TILE_N + et, up[j]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty + buf);  // this accumulator set may be overwritten
      if (!whole) {
        const int n_parts = (int)(owner_of((tile + 1) * KB - 1, U, P) - first_cta) + 1;
        __threadfence();
        epilogue_sync();
        if (et == 0) {
          const int before = atomicAdd(counters + tile, 1);
          *last_s = (before == n_parts - 1) ? 1 : 0;
          if (before == n_parts - 1) counters[tile] = 0;  // everyone has been: ready for the next launch
        }
        epilogue_sync();
        if (*last_s) {
          // Add the parts in their order, whoever came last. For this every thread takes four neighbouring
          // features and every fourth batch row (the scratch tile is [batch row][128 features] per accumulator),
          // and four rows at a time, so that many 16-byte loads are in flight together.
          __threadfence();
          const float* base = part + (size_t)tile * max_parts * (NACC * MT * TILE_N);
          const int f4 = (et & 31) * 4, r_first = et >> 5;
          const int n4 = (int)tile * TILE_N + f4;
          constexpr int ROWS_AT_ONCE = 4;
#pragma unroll 1
          for (int r0 = r_first; r0 < MT; r0 += 4 * ROWS_AT_ONCE) {
            float4 g[ROWS_AT_ONCE], up[ROWS_AT_ONCE];
#pragma unroll
            for (int i = 0; i < ROWS_AT_ONCE; ++i) g[i] = up[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < n_parts; ++p) {
              const float* src = base + (size_t)p * (NACC * MT * TILE_N) + f4;
#pragma unroll
              for (int i = 0; i < ROWS_AT_ONCE; ++i) {
                const int r = r0 + 4 * i;
                if (r < MT) {
                  const float4 a = __ldcg(reinterpret_cast<const float4*>(src + (size_t)r * TILE_N));
                  g[i].x += a.x; g[i].y += a.y; g[i].z += a.z; g[i].w += a.w;
                  if (SWIGLU) {
                    const float4 b = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(MT + r) * TILE_N));
                    up[i].x += b.x; up[i].y += b.y; up[i].z += b.z; up[i].w += b.w;
                  }
                }
              }
            }
#pragma unroll
            for (int i = 0; i < ROWS_AT_ONCE; ++i) {
              const int r = r0 + 4 * i;
              if (r >= MT || r >= M || n4 >= N) continue;
              float v[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
              const float uu[4] = {up[i].x, up[i].y, up[i].z, up[i].w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (SWIGLU) {
                  const float gate = round_to<bf16>(v[e]);
                  v[e] = round_to<bf16>(gate / (1.0f + __expf(-gate))) * round_to<bf16>(uu[e]);
                }
              TOut* dst = out + (size_t)r * N + n4;
              if (n4 + 3 < N && (((uintptr_t)dst) & (4 * sizeof(TOut) - 1)) == 0) {
                if (sizeof(TOut) == 4) {
                  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                  uint2 pk;
                  __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
                  pp[0] = __floats2bfloat162_rn(v[0], v[1]);
                  pp[1] = __floats2bfloat162_rn(v[2], v[3]);
                  *reinterpret_cast<uint2*>(dst) = pk;
                }
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (n4 + e < N) dst[e] = from_float<TOut>(v[e]);
              }
            }
          }
        }
        epilogue_sync();  // last_s is free for the next range
      }
      u = end;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

struct Plan {
  int blocks, stages, max_parts, tiles;
  size_t smem, part_floats;
};

template <int MT, bool SWIGLU>
Plan plan_for(int N, int K, int sms) {
  constexpr int NACC = SWIGLU ? 2 : 1;
  constexpr size_t STAGE = (size_t)NACC * W_BYTES + (size_t)MT * BK * 2;
  Plan p;
  const long long KB = (K + BK - 1) / BK, T = (N + TILE_N - 1) / TILE_N, U = T * KB;
  p.tiles = (int)T;
  p.blocks = (int)(U < sms ? U : sms);
  int stages = (int)((200 * 1024) / STAGE);
  p.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
  p.smem = (size_t)p.stages * STAGE + 1024 + (2 * MAX_STAGES + 4) * 8 + 64;
  const long long per = U / p.blocks;  // the shortest range
  p.max_parts = (int)((KB + per - 1) / per) + 1;
  p.part_floats = (size_t)T * p.max_parts * NACC * MT * TILE_N;
  return p;
}

int sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <int MT, bool SWIGLU, typename TOut>
int launch(void* out, const void* x, const void* W, float* part, size_t part_floats, int* counters, int n_counters, int M,
           int N, int K, int* error, cudaStream_t stream) {
  const Plan p = plan_for<MT, SWIGLU>(N, K, sm_count());
  if (p.part_floats > part_floats || p.tiles > n_counters) return -8;
  CUtensorMap map_w, map_x;
  int rc = make_map_bf16(&map_w, W, SWIGLU ? 2LL * N : N, K, K, TILE_N);
  if (rc) return rc;
  rc = make_map_bf16(&map_x, x, M, K, K, MT);
  if (rc) return rc;
  auto kern = streamk_kernel<MT, SWIGLU, TOut>;
  static size_t configured = 0;
  if (p.smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    if (e != cudaSuccess) return (int)e;
    configured = p.smem;
  }
  return (int)launch_pdl(kern, dim3(p.blocks), dim3(THREADS), p.smem, stream, map_w, map_x, (TOut*)out, part, counters, M, N, K,
                         p.stages, N, p.max_parts, error);
}

template <bool SWIGLU, typename TOut>
int pick_mt(void* out, const void* x, const void* W, float* part, size_t part_floats, int* counters, int n_counters, int M,
            int N, int K, int* error, cudaStream_t stream) {
  if (M <= 16) return launch<16, SWIGLU, TOut>(out, x, W, part, part_floats, counters, n_counters, M, N, K, error, stream);
  if (M <= 32) return launch<32, SWIGLU, TOut>(out, x, W, part, part_floats, counters, n_counters, M, N, K, error, stream);
  if (M <= 64) return launch<64, SWIGLU, TOut>(out, x, W, part, part_floats, counters, n_counters, M, N, K, error, stream);
  return launch<128, SWIGLU, TOut>(out, x, W, part, part_floats, counters, n_counters, M, N, K, error, stream);
}

}  // namespace

// What a product of these sizes needs from its caller: floats of scratch for the partial tiles (returned)
// and zeroed int counters, one per feature tile (*n_counters). The kernel leaves the counters zero.
KRK_API long long krk_streamk_scratch(int M, int N, int K, int swiglu, int* n_counters) {
  const int sms = sm_count();
  Plan p;
  if (swiglu) p = M <= 16 ? plan_for<16, true>(N, K, sms) : M <= 32 ? plan_for<32, true>(N, K, sms) : M <= 64 ? plan_for<64, true>(N, K, sms) : plan_for<128, true>(N, K, sms);
  else p = M <= 16 ? plan_for<16, false>(N, K, sms) : M <= 32 ? plan_for<32, false>(N, K, sms) : M <= 64 ? plan_for<64, false>(N, K, sms) : plan_for<128, false>(N, K, sms);
  if (n_counters) *n_counters = p.tiles;
  return (long long)p.part_floats;
}

// out [M, N] (bfloat16, or float32 with out_f32) = x [M, K] * W^T; x and W bfloat16, contiguous rows; with
// swiglu W is [2N, K] (gate rows, then up rows) and out the activated product. M <= 128, K a multiple of 8,
// 16-byte aligned bases. part / counters: scratch as krk_streamk_scratch says (counters zeroed once).
KRK_API int krk_streamk_linear(void* out, const void* x, const void* W, void* part, long long part_floats, int* counters,
                               int n_counters, int M, int N, int K, int swiglu, int out_f32, int* error,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 128 || K <= 0 || K % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return -2;
  float* p = (float*)part;
  if (swiglu) {
    if (out_f32) return -4;
    return pick_mt<true, bf16>(out, x, W, p, (size_t)part_floats, counters, n_counters, M, N, K, error, stream);
  }
  if (out_f32) return pick_mt<false, float>(out, x, W, p, (size_t)part_floats, counters, n_counters, M, N, K, error, stream);
  return pick_mt<false, bf16>(out, x, W, p, (size_t)part_floats, counters, n_counters, M, N, K, error, stream);
}
