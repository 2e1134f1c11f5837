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
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64;      // tile; BK * 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr long long SPIN_LIMIT = 1LL << 24;     // polls of a barrier before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity; false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (long long i = 0; i < SPIN_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// start address, stride between 8-row groups = 1024 bytes, descriptor version 1, swizzle mode 2.
__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);  // bits 0..13: address / 16
  d |= (uint64_t)1 << 16;                                  // bits 16..29: leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                        // bits 32..45: stride byte offset / 16
  d |= (uint64_t)1 << 46;                                  // bits 46..47: descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                                  // bits 61..63: 128-byte swizzle
  return d;
}

// Instruction descriptor: bfloat16 A and B, both K-major, float32 accumulator, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

template <bool SWIGLU, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ C, int M, int N, int K, int ldc, int up_row_offset, int* __restrict__ error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int NB = SWIGLU ? 2 : 1;                       // weight tiles per stage
  constexpr uint32_t STAGE_BYTES = A_BYTES + NB * B_BYTES;
  constexpr uint32_t TMEM_COLS = SWIGLU ? 256 : 128;
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
      tma_load_2d(stage + A_BYTES, &map_w, full_bar + s, kb * BK, n0);
      if (SWIGLU) tma_load_2d(stage + A_BYTES + B_BYTES, &map_w, full_bar + s, kb * BK, up_row_offset + n0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = umma_idesc(BM, BN);
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
          bf16* dst = C + (size_t)row * ldc + n0 + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float v0 = __uint_as_float(g[j]), v1 = __uint_as_float(g[j + 1]);
            if (SWIGLU) {
              const float g0 = round_to<bf16>(v0), g1 = round_to<bf16>(v1);
              v0 = round_to<bf16>(g0 / (1.0f + expf(-g0))) * round_to<bf16>(__uint_as_float(u[j]));
              v1 = round_to<bf16>(g1 / (1.0f + expf(-g1))) * round_to<bf16>(__uint_as_float(u[j + 1]));
            }
            const int col = n0 + c0 + j;
            if (col + 1 < N) {
              *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(v0, v1);
            } else if (col < N) {
              dst[j] = __float2bfloat16_rn(v0);
            }
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

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

// A row-major [rows, cols] bfloat16 matrix with row stride ld elements, read in boxes of 128 rows x 64 columns.
int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  EncodeTiled fn = encode_fn();
  if (!fn) return -6;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -7;
}

template <bool SWIGLU>
int launch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc, int* error,
           cudaStream_t stream) {
  constexpr int STAGES = SWIGLU ? 4 : 6;
  constexpr int NB = SWIGLU ? 2 : 1;
  constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + NB * B_BYTES) + 1024 + (2 * STAGES + 1) * 8 + 16;
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, A, M, K, lda);
  if (rc) return rc;
  rc = make_map(&map_w, W, SWIGLU ? 2 * N : N, K, ldw);
  if (rc) return rc;
  auto kern = gemm_tcgen05_kernel<SWIGLU, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  kern<<<grid, THREADS, SMEM, stream>>>(map_a, map_w, (bf16*)C, M, N, K, ldc, N, error);
  KRK_CHECK_LAUNCH();
  return 0;
}

}  // namespace

// C [M, N] bfloat16 (row stride ldc) = A [M, K] (row stride lda) * W^T, W [N, K] (row stride ldw); with
// swiglu, W is [2N, K] (gate rows, then up rows) and C receives the activated product. Needs K, lda and
// ldw multiples of 8 and 16-byte aligned base addresses (the TMA's rules). error: device word that a
// barrier wait which ran out sets to 3, 4 or 5.
KRK_API int krk_gemm_tcgen05(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                             int swiglu, int* error, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || (ldc & 1) || ((uintptr_t)C & 3))
    return -2;
  return swiglu ? launch<true>(C, A, W, M, N, K, lda, ldw, ldc, error, stream)
                : launch<false>(C, A, W, M, N, K, lda, ldw, ldc, error, stream);
}
