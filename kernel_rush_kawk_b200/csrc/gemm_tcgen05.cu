// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores:
// TMA brings 128x64 tiles of A and W into shared memory (128-byte swizzle), one elected
// thread issues tcgen05.mma with the accumulator in tensor memory, four warps read it back
// with tcgen05.ld for the epilogue. Weights are [out, in], y = x W^T, float32 accumulate,
// bfloat16 output, as in the reference's prefill products (engine/model.py:295,299,301 of
// willzeng274/kernel-rush-kawk, which calls cuBLAS there).
//
// Epilogues: plain; SwiGLU (the block computes the gate tile and the up tile of the same
// columns, rows n and I + n of W, and writes round(round(silu(round(g))) * round(u)),
// engine/kernels/gemm.py:108-113 of the reference), which saves writing and re-reading the
// [M, 2I] product.
//
// Block = 192 threads: warp 0 drives TMA, warp 1 owns tensor memory and issues the MMAs,
// warps 2..5 are the epilogue (each reads the 32 lanes of tensor memory its warp id maps
// to). One 128x128 output tile per block (two accumulators with SwiGLU). A ring of
// shared-memory stages connects the roles through mbarriers. Every wait is bounded: a wait
// that runs out sets the error word and the block leaves, after freeing its tensor memory.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64;                // tile rows and depth; BK * 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t A_BYTES = BM * BK * 2;

template <bool SWIGLU, int BN, int STAGES, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    TOut* __restrict__ C, int M, int N, int K, int ldc, int up_row_offset, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int NB = SWIGLU ? 2 : 1;                       // weight tiles per stage
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + NB * B_BYTES;
  constexpr uint32_t TMEM_COLS = NB * BN <= 128 ? 128 : NB * BN <= 256 ? 256 : 512;  // a power of two
  constexpr int WBOX = (BN % 128 == 0) ? 128 : BN / 2;     // rows of a weight box (192- and 224-wide tiles: two boxes)
  // 1024-byte alignment of every tile: the 128-byte swizzle pattern repeats every 8 rows of 128 bytes
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // this warp owns the tensor memory: allocate, publish the base address
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES && !mbar_wait(empty_bar + s, ((kb / STAGES) - 1) & 1)) { atomicExch(error, 3); break; }
      unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
      mbar_expect_tx(full_bar + s, STAGE_BYTES);
      tma_load_2d(stage, &map_a, full_bar + s, kb * BK, m0);
#pragma unroll
      for (int h = 0; h < BN / WBOX; ++h) {
        tma_load_2d(stage + A_BYTES + h * (WBOX * BK * 2), &map_w, full_bar + s, kb * BK, n0 + WBOX * h);
        if (SWIGLU)
          tma_load_2d(stage + A_BYTES + B_BYTES + h * (WBOX * BK * 2), &map_w, full_bar + s, kb * BK,
                      up_row_offset + n0 + WBOX * h);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = umma_idesc(BM, BN);  // N up to 256 in one instruction
    bool ok = true;
    for (int kb = 0; kb < k_blocks && ok; ++kb) {
      const int s = kb % STAGES;
      if (!mbar_wait(full_bar + s, (kb / STAGES) & 1)) { atomicExch(error, 4); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
      const uint64_t a_desc = umma_desc(stage);
      const uint64_t b_desc = umma_desc(stage + A_BYTES);
      const uint64_t b2_desc = umma_desc(stage + A_BYTES + B_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);  // 32 bytes per k-step inside the swizzled row
        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
        umma_bf16(tmem_base, a_desc + adv, b_desc + adv, idesc, acc);
        if (SWIGLU) umma_bf16(tmem_base + BN, a_desc + adv, b2_desc + adv, idesc, acc);
      }
      umma_commit(empty_bar + s);  // the stage is free once these MMAs have read it
    }
    umma_commit(acc_bar);  // the accumulator is complete (arrives even after a failed wait, so the epilogue moves on)
  } else if (warp >= 2) {
    // ---- epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of the accumulator ----
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    const bool ok = mbar_wait(acc_bar, 0);
    if (!ok && lane == 0) atomicExch(error, 5);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t g[32], u[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        tmem_ld_32x32(taddr, g);
        if (SWIGLU) tmem_ld_32x32(taddr + BN, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < M) {
          TOut* dst = C + (size_t)row * ldc + n0 + c0;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(g[j]);
            if (SWIGLU) {
              const float gj = round_to<bf16>(v[j]);
              v[j] = round_to<bf16>(gj / (1.0f + __expf(-gj))) * round_to<bf16>(__uint_as_float(u[j]));
            }
          }
          constexpr int PER16 = 16 / sizeof(TOut);  // elements per 16-byte store
          if (n0 + c0 + 32 <= N && (ldc % PER16) == 0 && ((uintptr_t)C & 15) == 0) {
            if (sizeof(TOut) == 4) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int q = 0; q < 4; ++q) pp[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + j) = pk;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c0 + j < N) dst[j] = from_float<TOut>(v[j]);
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <bool SWIGLU, int BN, int STAGES, typename TOut>
int launch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc, int* error,
           cudaStream_t stream) {
  constexpr int NB = SWIGLU ? 2 : 1;
  constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + NB * BN * BK * 2) + 1024 + (2 * STAGES + 1) * 8 + 16;
  CUtensorMap map_a, map_w;
  int rc = make_map_bf16(&map_a, A, M, K, lda, BM);
  if (rc) return rc;
  rc = make_map_bf16(&map_w, W, SWIGLU ? 2 * N : N, K, ldw, (BN % 128 == 0) ? 128 : BN / 2);
  if (rc) return rc;
  auto kern = gemm_tcgen05_kernel<SWIGLU, BN, STAGES, TOut>;
  static bool configured = false;  // one flag per instantiation of this template
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  kern<<<grid, THREADS, SMEM, stream>>>(map_a, map_w, (TOut*)C, M, N, K, ldc, N, error);
  KRK_CHECK_LAUNCH();
  return 0;
}

}  // namespace

// C [M, N] bfloat16 (row stride ldc) = A [M, K] (row stride lda) * W^T, W [N, K] (row stride ldw); with
// swiglu, W is [2N, K] (gate rows, then up rows) and C receives the activated product. Needs K, lda and
// ldw multiples of 8 and 16-byte aligned base addresses (the TMA's rules). error: device word that a
// barrier wait which ran out sets to 3, 4 or 5.
KRK_API int krk_gemm_tcgen05(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                             int swiglu, int variant, int out_f32, int* error, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)C & 3))
    return -2;
  // variant: 0 = 128x256 tile, one block per SM (with swiglu: 128x128 gate + 128x128 up);
  //          1 = 128x128 tile, three stages, two blocks per SM
  if (out_f32) {  // float32 output (output-head logits); no activation
    if (swiglu) return -4;
    // One tile per block and one block per SM: the time is rounds of blocks x tile width. A vocabulary that leaves
    // the last round of 256-wide tiles nearly empty is served faster by narrower tiles that fill their rounds
    // (151,936 columns at up to 128 rows: 594 tiles of 256 = five rounds, 679 of 224 = five shorter ones).
    int sms = 148;
    {
      int dev = 0;
      if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long row_tiles = (M + BM - 1) / BM;
    auto cost = [&](int bn) { return ((row_tiles * ((N + bn - 1) / bn) + sms - 1) / sms) * bn; };
    if (cost(224) < cost(256) && cost(224) <= cost(192))
      return launch<false, 224, 4, float>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
    if (cost(192) < cost(256)) return launch<false, 192, 4, float>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
    return launch<false, 256, 4, float>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
  }
  if (swiglu) return launch<true, 128, 4, bf16>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
  if (variant == 1) return launch<false, 128, 3, bf16>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
  return launch<false, 256, 4, bf16>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
}

// A wait that runs out, for the tests of the error path: one thread waits, with a short limit, on a
// barrier at which nothing ever arrives, then reports as every bounded wait of these kernels does:
// it writes its code into the error word and returns. Nothing faults and nothing spins without limit.
namespace {
__global__ void wait_runs_out_kernel(int* error, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!tc::mbar_wait(&bar, 0, limit_ns)) atomicExch(error, 21);
  }
}
}  // namespace

KRK_API int krk_selftest_wait_runs_out(int* error, int limit_us, cudaStream_t stream) {
  if (limit_us < 1 || limit_us > 100000) return -2;
  wait_runs_out_kernel<<<1, 32, 0, stream>>>(error, (unsigned long long)limit_us * 1000ull);
  KRK_CHECK_LAUNCH();
  return 0;
}
