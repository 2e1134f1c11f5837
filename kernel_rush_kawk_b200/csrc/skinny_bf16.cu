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
#include "mma.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int CHUNK = 32;   // k values per fragment load
constexpr int LOADS = 8;    // 16-row tile chunks in flight per warp

// NT: 8-row batch tiles (1 or 2). STREAMS: weight row tiles per block: 1, 2 (two
// row tiles), or gate+up when SWIGLU.
template <int NT, int RT, bool SWIGLU, bool NORM, typename TOut>
__global__ void __launch_bounds__(THREADS)
skinny_kernel(TOut* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ W,
              const bf16* __restrict__ branch, const void* __restrict__ gain, int gain_f32, bf16* __restrict__ x_new,
              int M, int N, int K, float eps, int pitch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TILES = SWIGLU ? 2 * RT : RT;  // 16-row weight tiles this block streams
  constexpr int UNROLL = LOADS / TILES;
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                      // [8*NT][pitch] when NORM
  float* red = reinterpret_cast<float*>(smem_raw + (NORM ? (size_t)8 * NT * pitch * 2 : 0));  // [WARPS][TILES*NT*4*32]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  if (NORM) {
    // one warp per batch row: add, statistics, normalise, into shared memory
    for (int m = warp; m < 8 * NT; m += WARPS) {
      bf16* dst = xs + (size_t)m * pitch;
      if (m >= M) {
        for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
        continue;
      }
      float sq = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * K + k);
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
        if (branch) {
          uint4 bv = *reinterpret_cast<const uint4*>(branch + (size_t)m * K + k);
          const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            xp[j] = __floats2bfloat162_rn(__low2float(xp[j]) + __low2float(bp[j]), __high2float(xp[j]) + __high2float(bp[j]));
          if (blockIdx.x == 0) *reinterpret_cast<uint4*>(x_new + (size_t)m * K + k) = xv;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = __low2float(xp[j]), b = __high2float(xp[j]);
          sq += a * a + b * b;
        }
        *reinterpret_cast<uint4*>(dst + k) = xv;
      }
      sq = warp_sum(sq);
      const float r = rsqrtf(sq / (float)K + eps);
      for (int k = lane * 8; k < K; k += 256) {
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

  // weight rows of this block's tiles, clamped so that edge tiles read valid memory
  const int n0 = blockIdx.x * 16 * RT;
  const bf16* wrow[TILES][2];
#pragma unroll
  for (int s = 0; s < TILES; ++s) {
    const int tile_row = n0 + (s % RT) * 16 + (SWIGLU && s >= RT ? N : 0);
    const int limit = (SWIGLU && s >= RT ? 2 * N : N) - 1;
    wrow[s][0] = W + (size_t)min(tile_row + g, limit) * K + 8 * t;
    wrow[s][1] = W + (size_t)min(tile_row + g + 8, limit) * K + 8 * t;
  }
  // batch rows of the B fragments
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    xok[j] = NORM || m < M;
    xrow[j] = NORM ? xs + (size_t)m * pitch + 8 * t : x + (size_t)min(m, M - 1) * K + 8 * t;
  }

  float acc[TILES][NT][4];
#pragma unroll
  for (int s = 0; s < TILES; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[s][j][c] = 0.f;

  const int n_chunks = K / CHUNK;
  const int per_warp = (n_chunks + WARPS - 1) / WARPS;
  const int c_begin = warp * per_warp, c_end = min(n_chunks, c_begin + per_warp);

  for (int c0 = c_begin; c0 < c_end; c0 += UNROLL) {
    uint4 wa[UNROLL][TILES][2];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = min(c0 + u, c_end - 1);  // a repeated chunk is loaded but not used
#pragma unroll
      for (int s = 0; s < TILES; ++s) {
        wa[u][s][0] = ld_stream_16(wrow[s][0] + (size_t)c * CHUNK);
        wa[u][s][1] = ld_stream_16(wrow[s][1] + (size_t)c * CHUNK);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (c0 + u < c_end) {
        const int c = c0 + u;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint4 xb = make_uint4(0, 0, 0, 0);
          if (xok[j]) xb = *reinterpret_cast<const uint4*>(xrow[j] + (size_t)c * CHUNK);
#pragma unroll
          for (int s = 0; s < TILES; ++s) {
            mma_bf16_16816(acc[s][j], wa[u][s][0].x, wa[u][s][1].x, wa[u][s][0].y, wa[u][s][1].y, xb.x, xb.y);
            mma_bf16_16816(acc[s][j], wa[u][s][0].z, wa[u][s][1].z, wa[u][s][0].w, wa[u][s][1].w, xb.z, xb.w);
          }
        }
      }
    }
  }

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
    const int n = n0 + f;
    if (m < M && n < N) {
      if (SWIGLU) {
        const float gate = round_to<bf16>(v), up = round_to<bf16>(v2);
        v = round_to<bf16>(gate / (1.0f + expf(-gate))) * up;
      }
      out[(size_t)m * N + n] = from_float<TOut>(v);
    }
  }
}

template <int NT, int RT, bool SWIGLU, bool NORM, typename TOut>
int launch(void* out, const void* x, const void* W, const void* branch, const void* gain, int gain_f32, void* x_new, int M,
           int N, int K, float eps, cudaStream_t stream) {
  constexpr int TILES = SWIGLU ? 2 * RT : RT;
  int pitch = 0;
  size_t smem = (size_t)WARPS * TILES * NT * 4 * 32 * sizeof(float);
  if (NORM) {
    const int pad_bytes = (64 - (K * 2) % 128 + 128) % 128;
    pitch = K + pad_bytes / 2;
    smem += (size_t)8 * NT * pitch * 2;
  }
  if (smem > 200 * 1024) return -2;
  auto kern = skinny_kernel<NT, RT, SWIGLU, NORM, TOut>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int blocks = (N + 16 * RT - 1) / (16 * RT);
  kern<<<blocks, THREADS, smem, stream>>>((TOut*)out, (const bf16*)x, (const bf16*)W, (const bf16*)branch, gain,
                                          gain_f32, (bf16*)x_new, M, N, K, eps, pitch);
  KRK_CHECK_LAUNCH();
  return 0;
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
