// Token selection over float32 logits: greedy, or temperature sampling.
//
// Greedy is the reference's rule: argmax over the vocabulary, the lowest index
// winning an exact tie (engine/engine.py:193,196 of willzeng274/kernel-rush-kawk).
// Temperature sampling (not in the reference) uses the Gumbel-max form
//   token = argmax_i( logit_i / temperature - log(-log(u_i)) ),
// a draw from softmax(logits / temperature), with u_i from a 32-bit mixing hash of
// (seed, request, step, i): u_i = ((hash >> 9) + 0.5) / 2^23, exact in float32 and
// strictly inside (0, 1). One block per row.
#include "common.cuh"

namespace {

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

__global__ void select_tokens_kernel(int* __restrict__ tokens, const float* __restrict__ logits, int vocab,
                                     float temperature, uint32_t seed, const int* __restrict__ requests,
                                     uint32_t step, int* __restrict__ feed_tokens, int* __restrict__ feed_pos,
                                     int* __restrict__ feed_start) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * vocab;
  const bool sample = temperature > 0.f;
  uint32_t key = 0;
  if (sample) key = mix32(mix32(mix32(seed) ^ (uint32_t)requests[row]) ^ step);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = x[i];
    if (sample) {
      const uint32_t h = mix32(key ^ ((uint32_t)i * 0x9E3779B9u));
      const float u = ((float)(h >> 9) + 0.5f) * (1.0f / 8388608.0f);
      v = v / temperature - logf(-logf(u));
    }
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int n_warps = blockDim.x >> 5;
    bv = lane < n_warps ? best_v[lane] : -INFINITY;
    bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      const int tok = bi == 0x7fffffff ? 0 : bi;
      tokens[row] = tok;
      if (feed_tokens) {  // feed the next single-token step on the device: its token, its position
        feed_tokens[row] = tok;
        feed_pos[row] += 1;
        feed_start[row] += 1;
      }
    }
  }
}

}  // namespace

// feed_*: null, or the token / row position / sequence start arrays of a single-token step's batch
// description, which then describe the next step: token = the selected one, positions + 1.
KRK_API int krk_select_tokens(int* tokens, const float* logits, int rows, int vocab, float temperature, unsigned seed,
                              const int* requests, unsigned step, int* feed_tokens, int* feed_pos, int* feed_start,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  select_tokens_kernel<<<rows, 1024, 0, stream>>>(tokens, logits, vocab, temperature, seed, requests, step,
                                                  feed_tokens, feed_pos, feed_start);
  KRK_CHECK_LAUNCH();
  return 0;
}
