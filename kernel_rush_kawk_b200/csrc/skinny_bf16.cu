// Decode-time matrix product for few rows: out[M, N] = act(x)[M, K] * W[N, K]^T,
// bfloat16, M <= 16, with the residual add and RMSNorm folded into the prologue
// and SwiGLU into the epilogue.
//
// At decode the projections are pure weight streaming (the reference says so of
// its own skinny kernel, engine/kernels/gemm.py:1-10 of willzeng274/kernel-rush-kawk).
// Here the weights are the 16-row operand of the tensor-core instruction ("swap
// A and B"): a warp owns 16 output features (rows of W) and a slice of K; each
// lane reads 16 contiguous bytes of a weight row straight from global memory into
// the A fragment, the batch rows are the 8-wide B operand. The K index inside a
// 32-wide chunk is permuted identically for both operands (a dot product does not
// care), which is what lets one 16-byte load fill a fragment. No weight byte goes
// through shared memory. The warps of a block split K and reduce through shared
// memory in a fixed order, so results are reproducible.
//
// Prologue (gain != null): s = round(x + branch) (new residual stream, written by
// block 0), r = rsqrt(mean(s^2) + eps), a = round(gain * round(s * r)), as the
// reference's fused kernels compute it (gemm.py:22-51). Epilogue (swiglu): rows
// n and N + n of W are gate and up; out = round(round(silu(round(g))) * round(u))
// (gemm.py:108-113).
//
// A product with few output features (N of some thousands) has too few 16-row tiles to keep
// every SM's memory pipe full: what bounds a block is the bytes it has in flight, and one block
// of eight warps per SM holds 64 KB. Such products split K as well: the KSPLIT blocks of a
// thread-block cluster stream a quarter of K each for the same tile, five small blocks share an
// SM, and the partial sums meet in the first block's shared memory (distributed shared memory,
// added in block order, so the result does not depend on timing).
#include <cooperative_groups.h>

#define KRK_TRACE_OWNER  // with -DKRK_TRACE this file keeps the timeline buffer
#include "mma.cuh"

namespace {

constexpr int CHUNK = 32;        // k values per fragment load
constexpr int RING_LOADS = 8;    // 16-row tile chunks in flight per thread (32 bytes each); DEEP doubles it
// With two batch tiles whose rows ride in the ring (9 to 16 rows, no prologue) a stage is a third larger, and
// at 8 loads an 8-warp block takes 131 KB of shared memory: one block per SM. Six keep two blocks per SM;
// a decode step at 16 sequences of the 4B shape: 2.79 ms against 3.08 ms with 8 (and 2.96 / 3.06 / 3.30 ms
// with 5 / 7 / 4; the library product: 2.83 ms).
constexpr int RING_LOADS_TWO_TILES = 6;
// five 4-warp blocks of a K-split product share an SM: 40 KB each with the ring, the reduction buffer and the inbox
constexpr int RING_LOADS_KSPLIT = 6, RING_LOADS_KSPLIT_TWO_TILES = 4;
template <int NT, bool NORM, bool DEEP, int KSPLIT = 1, int RING = 0>
__host__ __device__ constexpr int ring_loads() {
  return RING > 0 ? RING : (KSPLIT > 1) ? (NT == 2 ? RING_LOADS_KSPLIT_TWO_TILES : RING_LOADS_KSPLIT)
                      : (NT == 2 && !NORM) ? RING_LOADS_TWO_TILES : (DEEP ? 2 : 1) * RING_LOADS;
}

// NT: 8-row batch tiles (1 or 2). RT: 16-row weight tiles per block; with SWIGLU the
// block streams RT gate tiles and RT up tiles.
//
// Weight bytes travel global -> shared memory with cp.async into a ring that is
// private to each thread: a thread later reads back exactly the 16-byte pieces it
// copied itself, so the ring needs no barrier, only cp.async.wait_group. The first
// ring-full of copies is issued before anything else (before the wait on the
// previous kernel, before the norm prologue), so the memory system is busy from the
// block's first instruction.
template <int WARPS, int NT, int RT, bool SWIGLU, bool NORM, typename TOut, bool DEEP = false, int KSPLIT = 1, int RING = 0>
__global__ void __launch_bounds__(WARPS * 32)
skinny_kernel(TOut* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ W,
              const bf16* __restrict__ branch, const void* __restrict__ gain, int gain_f32, bf16* __restrict__ x_new,
              int M, int N, int K, float eps, int pitch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  KRK_TRACE_DECL
  constexpr int THREADS = WARPS * 32;
  constexpr int TILES = SWIGLU ? 2 * RT : RT;  // 16-row weight tiles this block streams
  constexpr int STAGES = ring_loads<NT, NORM, DEEP, KSPLIT, RING>() / TILES;
  constexpr int XSLOTS = NORM ? 0 : NT;          // without the prologue the batch rows ride in the ring too
  constexpr int SLOTS = TILES * 2 + XSLOTS;      // 16-byte pieces per thread and stage
  constexpr size_t RING_BYTES = (size_t)STAGES * SLOTS * THREADS * 16;
  uint4* ring = reinterpret_cast<uint4*>(smem_raw);                                 // [STAGES][SLOTS][THREADS]
  float* red = reinterpret_cast<float*>(smem_raw + RING_BYTES);                       // [WARPS][TILES*NT*4*32]
  constexpr size_t RED_BYTES = (size_t)WARPS * TILES * NT * 4 * 32 * sizeof(float);
  bf16* xs = reinterpret_cast<bf16*>(smem_raw + RING_BYTES + RED_BYTES);              // [M][pitch] when NORM
  float* inbox = reinterpret_cast<float*>(smem_raw + RING_BYTES + RED_BYTES);         // [KSPLIT - 1][outputs] (never with NORM)
  static_assert(KSPLIT == 1 || (!NORM && !SWIGLU), "K is split only for the plain product");
  if (KSPLIT > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // "I have started"

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ks = KSPLIT > 1 ? blockIdx.x % KSPLIT : 0;  // this block's part of K: its rank in the cluster

  // weight rows of this block's tiles, clamped so that edge tiles read valid memory
  const int n0 = (blockIdx.x / KSPLIT) * 16 * RT;
  const bf16* wrow[TILES][2];
#pragma unroll
  for (int s = 0; s < TILES; ++s) {
    const int tile_row = n0 + (s % RT) * 16 + (SWIGLU && s >= RT ? N : 0);
    const int limit = (SWIGLU && s >= RT ? 2 * N : N) - 1;
    wrow[s][0] = W + (size_t)min(tile_row + g, limit) * K + 8 * t;
    wrow[s][1] = W + (size_t)min(tile_row + g + 8, limit) * K + 8 * t;
  }
  const int n_chunks = K / CHUNK;
  const int per_block = (n_chunks + KSPLIT - 1) / KSPLIT;
  const int b_begin = ks * per_block, b_end = min(n_chunks, b_begin + per_block);
  const int per_warp = (max(0, b_end - b_begin) + WARPS - 1) / WARPS;
  const int c_begin = b_begin + warp * per_warp, c_end = min(b_end, c_begin + per_warp);
  const int nc = max(0, c_end - c_begin);

  // batch rows of the B fragments when they come from global memory (no prologue)
  const bf16* xsrc[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    xok[j] = m < M;
    xsrc[j] = x + (size_t)min(m, M - 1) * K + 8 * t;
  }

  const uint64_t stream_policy = l2_evict_first_policy();
  auto issue_w = [&](int i) {  // weights of chunk i of this warp's slice into stage i % STAGES
    if (i < nc) {
      uint4* dst = ring + ((size_t)(i % STAGES) * SLOTS) * THREADS + threadIdx.x;
      const size_t off = (size_t)(c_begin + i) * CHUNK;
#pragma unroll
      for (int s = 0; s < TILES; ++s) {
        cp_async_16_stream(dst + (s * 2 + 0) * THREADS, wrow[s][0] + off, stream_policy);
        cp_async_16_stream(dst + (s * 2 + 1) * THREADS, wrow[s][1] + off, stream_policy);
      }
    }
  };
  auto issue_x = [&](int i) {  // the batch rows' piece of chunk i (only without the prologue)
    if (!NORM && i < nc) {
      uint4* dst = ring + ((size_t)(i % STAGES) * SLOTS + TILES * 2) * THREADS + threadIdx.x;
      const size_t off = (size_t)(c_begin + i) * CHUNK;
#pragma unroll
      for (int j = 0; j < XSLOTS; ++j)
        if (xok[j]) cp_async_16(dst + j * THREADS, xsrc[j] + off);
    }
  };
  // Weights are written by no kernel: their copies start before the wait on the previous
  // kernel. Activations come from it: their copies start after the wait. One commit group
  // per stage, empty or not, so that group counting stays simple.
#pragma unroll
  for (int i = 0; i < STAGES; ++i) issue_w(i);
  // The next kernel's blocks may start at once: they prefetch their weights beside this kernel.
  // (Letting them in only after this kernel's streaming was measured: slower.)
  grid_launch_dependents();
  grid_dependency_wait();  // x, branch come from earlier kernels; x_new may still be read by them
  KRK_TRACE_READY
#pragma unroll
  for (int i = 0; i < STAGES; ++i) {
    issue_x(i);
    cp_async_commit();
  }

  if (NORM) {
    // All threads work on every batch row: thread c owns the 8-element pieces c, c + 256, ...
    // of a row. Pass 1: s = round(x + branch) into shared memory, partial sums of squares per
    // warp. Pass 2, after the warps' partials are added in warp order: normalise in place.
    float* partial = red;  // [8*NT][WARPS]; the reduction buffer is free until the main loop ends
    const int K8 = K / 8;
    float sq[8 * NT];
#pragma unroll
    for (int m = 0; m < 8 * NT; ++m) sq[m] = 0.f;
    for (int c = threadIdx.x; c < K8; c += THREADS) {
      const int k = c * 8;
      // the rows' loads are independent of one another: unrolled, they are all in flight together
#pragma unroll
      for (int m = 0; m < 8 * NT; ++m) {
        if (m < M) {
          uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * K + k);
          __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
          if (branch) {
            uint4 bv = *reinterpret_cast<const uint4*>(branch + (size_t)m * K + k);
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              xp[j] = __floats2bfloat162_rn(__low2float(xp[j]) + __low2float(bp[j]),
                                            __high2float(xp[j]) + __high2float(bp[j]));
            if (blockIdx.x == 0) *reinterpret_cast<uint4*>(x_new + (size_t)m * K + k) = xv;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = __low2float(xp[j]), b = __high2float(xp[j]);
            sq[m] += a * a + b * b;
          }
          *reinterpret_cast<uint4*>(xs + (size_t)m * pitch + k) = xv;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < 8 * NT; ++m) {
      const float v = warp_sum(sq[m]);
      if (lane == 0) partial[m * WARPS + warp] = v;
    }
    __syncthreads();
    for (int m = 0; m < M; ++m) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) total += partial[m * WARPS + w];
      const float r = rsqrtf(total / (float)K + eps);
      bf16* dst = xs + (size_t)m * pitch;
      for (int c = threadIdx.x; c < K8; c += THREADS) {
        const int k = c * 8;
        uint4 xv = *reinterpret_cast<uint4*>(dst + k);
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float n0 = round_to<bf16>(__low2float(xp[j]) * r), n1 = round_to<bf16>(__high2float(xp[j]) * r);
          xp[j] = __floats2bfloat162_rn(n0 * load_gain<bf16>(gain, k + 2 * j, gain_f32),
                                        n1 * load_gain<bf16>(gain, k + 2 * j + 1, gain_f32));
        }
        *reinterpret_cast<uint4*>(dst + k) = xv;
      }
    }
    __syncthreads();
  }

  // batch rows of the B fragments after the prologue: normalised rows in shared memory
  const bf16* xrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xrow[j] = xs + (size_t)(8 * j + g) * pitch + 8 * t;

  float acc[TILES][NT][4];
#pragma unroll
  for (int s = 0; s < TILES; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[s][j][c] = 0.f;

  for (int i = 0; i < nc; ++i) {
    cp_async_wait<STAGES - 1>();  // all but the newest STAGES-1 groups are complete: chunk i has landed
    const uint4* src = ring + ((size_t)(i % STAGES) * SLOTS) * THREADS + threadIdx.x;
    uint4 wa[TILES][2];
#pragma unroll
    for (int s = 0; s < TILES; ++s) {
      wa[s][0] = src[(s * 2 + 0) * THREADS];
      wa[s][1] = src[(s * 2 + 1) * THREADS];
    }
    const int c = c_begin + i;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      uint4 xb = make_uint4(0, 0, 0, 0);
      if (NORM) { if (xok[j]) xb = *reinterpret_cast<const uint4*>(xrow[j] + (size_t)c * CHUNK); }
      else if (xok[j]) xb = src[(TILES * 2 + j) * THREADS];
#pragma unroll
      for (int s = 0; s < TILES; ++s) {
        mma_bf16_16816(acc[s][j], wa[s][0].x, wa[s][1].x, wa[s][0].y, wa[s][1].y, xb.x, xb.y);
        mma_bf16_16816(acc[s][j], wa[s][0].z, wa[s][1].z, wa[s][0].w, wa[s][1].w, xb.z, xb.w);
      }
    }
    issue_w(i + STAGES);  // refill the stage just consumed (its values are in registers and used)
    issue_x(i + STAGES);
    cp_async_commit();
  }
  cp_async_wait<0>();

  // reduce over the warps in a fixed order
  constexpr int PER_WARP = TILES * NT * 4 * 32;
#pragma unroll
  for (int s = 0; s < TILES; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[warp * PER_WARP + ((s * NT + j) * 4 + c) * 32 + lane] = acc[s][j][c];
  __syncthreads();

  // outputs of this block: RT*16 features x NT*8 batch rows
  constexpr int OUTS = RT * 16 * NT * 8;
  if (KSPLIT > 1) {
    // every block of the cluster but the first adds its warps' parts and puts the sums into the first block's
    // inbox; one cluster barrier later the first block holds them all
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every block of the cluster has started
    if (ks != 0) {
      float* dst = cluster.map_shared_rank(inbox, 0) + (size_t)(ks - 1) * OUTS;
      for (int o = threadIdx.x; o < OUTS; o += THREADS) {
        const int m = o % (NT * 8), f = o / (NT * 8);
        const int tile = f / 16, r = f % 16;
        const int j = m / 8, col = m % 8;
        const int src_lane = (r % 8) * 4 + col / 2, reg = (r / 8) * 2 + (col & 1);
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[w * PER_WARP + ((tile * NT + j) * 4 + reg) * 32 + src_lane];
        dst[o] = v;
      }
    }
    cluster.sync();
  }
  for (int o = threadIdx.x; o < OUTS; o += THREADS) {
    const int m = o % (NT * 8), f = o / (NT * 8);  // batch row, feature within the block
    const int tile = f / 16, r = f % 16;
    const int j = m / 8, col = m % 8;
    // accumulator (row r, column col) of tile: lane = (r % 8) * 4 + col / 2, register (r / 8) * 2 + col % 2
    const int src_lane = (r % 8) * 4 + col / 2, reg = (r / 8) * 2 + (col & 1);
    float v = 0.f, v2 = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      v += red[w * PER_WARP + ((tile * NT + j) * 4 + reg) * 32 + src_lane];
      if (SWIGLU) v2 += red[w * PER_WARP + (((RT + tile) * NT + j) * 4 + reg) * 32 + src_lane];
    }
    if (KSPLIT > 1) {
      if (ks == 0) {
#pragma unroll
        for (int r = 0; r < KSPLIT - 1; ++r) v += inbox[r * OUTS + o];  // the other blocks' parts, in block order
      } else {
        continue;
      }
    }
    const int n = n0 + f;
    if (m < M && n < N) {
      if (SWIGLU) {
        const float gate = round_to<bf16>(v), up = round_to<bf16>(v2);
        v = round_to<bf16>(gate / (1.0f + expf(-gate))) * up;
      }
      out[(size_t)m * N + n] = from_float<TOut>(v);
    }
  }
  KRK_TRACE_END(K)
}

template <int WARPS, int NT, int RT, bool SWIGLU, bool NORM, typename TOut, bool DEEP = false, int KSPLIT = 1, int RING = 0>
int launch_warps(void* out, const void* x, const void* W, const void* branch, const void* gain, int gain_f32, void* x_new, int M,
           int N, int K, float eps, cudaStream_t stream) {
  constexpr int THREADS = WARPS * 32;
  constexpr int TILES = SWIGLU ? 2 * RT : RT;
  constexpr int STAGES = ring_loads<NT, NORM, DEEP, KSPLIT, RING>() / TILES;
  int pitch = 0;
  constexpr int SLOTS = TILES * 2 + (NORM ? 0 : NT);
  size_t smem = (size_t)STAGES * SLOTS * THREADS * 16 + (size_t)WARPS * TILES * NT * 4 * 32 * sizeof(float) +
                (size_t)(KSPLIT - 1) * RT * 16 * NT * 8 * sizeof(float);
  if (NORM) {
    const int pad_bytes = (64 - (K * 2) % 128 + 128) % 128;
    pitch = K + pad_bytes / 2;
    smem += (size_t)M * pitch * 2;
  }
  if (smem > 220 * 1024) return -2;
  auto kern = skinny_kernel<WARPS, NT, RT, SWIGLU, NORM, TOut, DEEP, KSPLIT, RING>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int blocks = (N + 16 * RT - 1) / (16 * RT);
  if (KSPLIT > 1) {  // the blocks of a cluster share a tile and split K
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks * KSPLIT);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KSPLIT;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    static const bool plain = getenv("KRK_NO_PDL") != nullptr;
    cfg.attrs = attr;
    cfg.numAttrs = plain ? 1 : 2;
    return (int)cudaLaunchKernelEx(&cfg, kern, (TOut*)out, (const bf16*)x, (const bf16*)W, (const bf16*)branch, gain, gain_f32,
                                   (bf16*)x_new, M, N, K, eps, pitch);
  }
  cudaError_t e = launch_pdl(kern, dim3(blocks), dim3(THREADS), smem, stream, (TOut*)out, (const bf16*)x, (const bf16*)W,
                             (const bf16*)branch, gain, gain_f32, (bf16*)x_new, M, N, K, eps, pitch);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

// Blocks of 8 warps hold more bytes in flight each; blocks of 4 warps are small enough for
// five of them to share an SM. With between two and five blocks per SM the small ones all
// fit at once (one wave, no straggling second wave of a few blocks); otherwise the large.
template <int NT, int RT, bool SWIGLU, bool NORM, typename TOut>
int launch(void* out, const void* x, const void* W, const void* branch, const void* gain, int gain_f32, void* x_new, int M,
           int N, int K, float eps, cudaStream_t stream) {
  const int blocks = (N + 16 * RT - 1) / (16 * RT);
  // Between two and three blocks per SM: small blocks, but with rings as deep as three of them fit beside one
  // another, since what bounds a block is the bytes it has in flight (with the norm prologue, one or two rows:
  // fourteen loads; a step of one sequence of the 4B shape, alternating runs: 1.913 ms against 1.925 with twelve
  // and 1.919 with ten; without the prologue the depth makes no difference inside a step: eight loads against
  // eleven at eight rows, six against eight at sixteen, each within 0.3 %).
  if constexpr (!SWIGLU && RT == 1) {
    if (blocks > 2 * 148 && blocks <= 3 * 148)
      return launch_warps<4, NT, RT, SWIGLU, NORM, TOut, false, 1, (NORM ? 14 : NT == 1 ? 11 : 8)>(
          out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  }
  if (blocks > 2 * 148 && blocks <= 5 * 148)
    return launch_warps<4, NT, RT, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  // few tiles (about one per SM): split K four ways over a cluster, so that four to five small blocks an SM
  // have their bytes in flight instead of one large one
  if constexpr (!SWIGLU && !NORM && RT == 1) {
    if (blocks * 4 <= 5 * 148 && K >= 4 * 4 * CHUNK * 4)
      return launch_warps<4, NT, RT, SWIGLU, NORM, TOut, false, 4>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps,
                                                                    stream);
  }
  // (a ring twice as deep for kernels of about one block per SM was measured: slower, because the
  // next kernel's blocks then no longer fit beside it to prefetch their weights)
  return launch_warps<8, NT, RT, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
}

template <int NT, bool SWIGLU, bool NORM, typename TOut>
int pick_rt(void* out, const void* x, const void* W, const void* branch, const void* gain, int gain_f32, void* x_new,
            int M, int N, int K, float eps, cudaStream_t stream) {
  // two row tiles per block when that still leaves a few blocks for each of the 148 SMs
  if (!SWIGLU && N >= 16 * 2 * 296)
    return launch<NT, 2, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  return launch<NT, 1, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
}

template <bool SWIGLU, bool NORM, typename TOut>
int pick_nt(void* out, const void* x, const void* W, const void* branch, const void* gain, int gain_f32, void* x_new,
            int M, int N, int K, float eps, cudaStream_t stream) {
  if (M <= 8) return pick_rt<1, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  return pick_rt<2, SWIGLU, NORM, TOut>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
}

}  // namespace

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

// out [M, N] (bfloat16 or float32), x [M, K] bfloat16 contiguous, W [N, K] ([2N, K] with swiglu) bfloat16
// contiguous; branch, gain, x_new may be null (see the file text). Needs M <= 16 and K % 32 == 0.
KRK_API int krk_skinny_linear(void* out, const void* x, const void* W, const void* branch, const void* gain,
                              void* x_new, int gain_f32, void* reserved, int M, int N, int K, float eps, int swiglu,
                              int out_dtype, cudaStream_t stream) {
  (void)reserved;
  if (M == 0 || N == 0) return 0;
  if (M > 16 || K % CHUNK || K <= 0) return -2;
  if (branch && !gain) return -2;
  const bool norm = gain != nullptr;
  if (swiglu) {
    if (out_dtype != KRK_DTYPE_BF16) return -4;
    return norm ? pick_nt<true, true, bf16>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream)
                : pick_nt<true, false, bf16>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  }
  if (out_dtype == KRK_DTYPE_F32)
    return norm ? pick_nt<false, true, float>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream)
                : pick_nt<false, false, float>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
  return norm ? pick_nt<false, true, bf16>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream)
              : pick_nt<false, false, bf16>(out, x, W, branch, gain, gain_f32, x_new, M, N, K, eps, stream);
}
