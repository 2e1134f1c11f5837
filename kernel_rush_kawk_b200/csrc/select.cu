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

// Order-preserving map from float to unsigned: a < b  <=>  key(a) < key(b).
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Phase 1: block (chunk, row) scans its share of the row and folds its best (value,
// index) into packed[row] with a 64-bit atomic max of (ordered value, ~index): the
// maximum is the largest value and, among equals, the lowest index, in whatever order
// the blocks arrive. packed[row] must be 0 on entry; phase 2 leaves it 0 again.
__global__ void select_scan_kernel(unsigned long long* __restrict__ packed, const float* __restrict__ logits, int vocab,
                                   float temperature, uint32_t seed, const int* __restrict__ requests, uint32_t step) {
  __shared__ unsigned long long best_s[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.y;
  const float* x = logits + (size_t)row * vocab;
  const bool sample = temperature > 0.f;
  uint32_t key = 0;
  if (sample) key = mix32(mix32(mix32(seed) ^ (uint32_t)requests[row]) ^ step);
  const int per = (((vocab + gridDim.x - 1) / gridDim.x) + 3) & ~3;  // a multiple of four: chunks start on 16 bytes
  const int begin = blockIdx.x * per, end = min(vocab, begin + per);
  unsigned long long best = 0;
  auto take = [&](float v, int i) {
    if (sample) {
      const uint32_t h = mix32(key ^ ((uint32_t)i * 0x9E3779B9u));
      const float u = ((float)(h >> 9) + 0.5f) * (1.0f / 8388608.0f);
      v = v / temperature - logf(-logf(u));
    }
    const unsigned long long cand = ((unsigned long long)ordered_bits(v) << 32) | (uint32_t)(~(uint32_t)i);
    best = cand > best ? cand : best;
  };
  if ((vocab & 3) == 0 && ((uintptr_t)logits & 15) == 0) {  // rows start on 16 bytes: four logits per load
    for (int i = begin + 4 * threadIdx.x; i < end; i += 4 * blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      take(v.x, i);
      take(v.y, i + 1);
      take(v.z, i + 2);
      take(v.w, i + 3);
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) take(x[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) best_s[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? best_s[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if (lane == 0 && best) atomicMax(packed + row, best);
  }
}

// Phase 2: one thread per row turns packed[row] into the token, optionally feeds the
// next single-token step, and clears packed[row].
__global__ void select_finish_kernel(int* __restrict__ tokens, unsigned long long* __restrict__ packed, int rows,
                                     int* __restrict__ feed_tokens, int* __restrict__ feed_pos,
                                     int* __restrict__ feed_start) {
  // No early start for the kernels behind this one: it writes the next step's tokens and positions, and
  // kernels of that step read the positions before their own wait on their predecessor.
  grid_dependency_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const unsigned long long best = packed[row];
  packed[row] = 0ull;
  const int tok = best ? (int)(~(uint32_t)(best & 0xffffffffull)) : 0;
  tokens[row] = tok;
  if (feed_tokens) {  // feed the next single-token step on the device: its token, its position
    feed_tokens[row] = tok;
    feed_pos[row] += 1;
    feed_start[row] += 1;
  }
}

}  // namespace

// packed: 64-bit scratch, one word per row, zero before the first call (each call leaves it zero).
// feed_*: null, or the token / row position / sequence start arrays of a single-token step's batch
// description, which then describe the next step: token = the selected one, positions + 1.
KRK_API int krk_select_tokens(int* tokens, const float* logits, int rows, int vocab, float temperature, unsigned seed,
                              const int* requests, unsigned step, int* feed_tokens, int* feed_pos, int* feed_start,
                              void* packed, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows > 65535) return -3;
  const int chunks = max(1, min(64, vocab / 2048));
  cudaError_t e = launch_pdl(select_scan_kernel, dim3(chunks, rows), dim3(256), 0, stream, (unsigned long long*)packed,
                             logits, vocab, temperature, (uint32_t)seed, requests, (uint32_t)step);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(select_finish_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, tokens,
                 (unsigned long long*)packed, rows, feed_tokens, feed_pos, feed_start);
  return (int)e;
}
