// Shared device helpers: element types, rounding, vector access, reductions.
//
// Every kernel of this library is instantiated for two element types: float
// (the true 32-bit path) and __nv_bfloat16 (the serving path). round_to<T>(x)
// rounds a float to T's precision and returns it as float; it is the identity
// for float. The places where it is applied are the places where the
// reference's BF16 path rounds (engine/kernels/rmsnorm.py:30-45,
// add_rmsnorm.py:21-29, rope.py:19-30, swiglu.py:21-24 of
// willzeng274/kernel-rush-kawk).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define KRK_PAGE 64  // cache positions per page

#define KRK_DTYPE_F32 0
#define KRK_DTYPE_BF16 1

#define KRK_API extern "C" __attribute__((visibility("default")))

#define KRK_CHECK_LAUNCH()                         \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch. Every kernel of this library is launched with the
// attribute that lets it start while its predecessor in the stream drains. A kernel
// calls grid_dependency_wait() before it touches anything another kernel produced (or
// still reads); only loads of weights, which no kernel writes, may come before it.
// grid_launch_dependents() lets the next kernel in the stream begin its own prologue.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Optional timeline for performance work (compile with -DKRK_TRACE): blocks record global
// timer stamps into a buffer of the library that krk_trace_dump copies out.
#if defined(KRK_TRACE) && defined(KRK_TRACE_OWNER)
#define KRK_TRACE_CAP (1 << 20)
static __device__ unsigned long long krk_trace_buf[KRK_TRACE_CAP * 4];
static __device__ unsigned int krk_trace_count;
__device__ __forceinline__ unsigned long long krk_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define KRK_TRACE_DECL unsigned long long t_begin__ = krk_now(), t_ready__ = 0;
#define KRK_TRACE_READY t_ready__ = krk_now();
#define KRK_TRACE_END(kind)                                                  \
  if (threadIdx.x == 0) {                                                    \
    unsigned int i__ = atomicAdd(&krk_trace_count, 1u);                      \
    if (i__ < KRK_TRACE_CAP) {                                               \
      krk_trace_buf[4 * i__] = ((unsigned long long)(kind) << 32) | blockIdx.x | (blockIdx.y << 16); \
      krk_trace_buf[4 * i__ + 1] = t_begin__;                                \
      krk_trace_buf[4 * i__ + 2] = t_ready__;                                \
      krk_trace_buf[4 * i__ + 3] = krk_now();                                \
    }                                                                        \
  }
#define KRK_TRACE_MARKS unsigned long long mark__[6] = {0, 0, 0, 0, 0, 0};
#define KRK_TRACE_MARK(i) mark__[i] = krk_now();
#define KRK_TRACE_REC(kind, a, b, c)                                         \
  if (threadIdx.x == 0) {                                                    \
    unsigned int i__ = atomicAdd(&krk_trace_count, 1u);                      \
    if (i__ < KRK_TRACE_CAP) {                                               \
      krk_trace_buf[4 * i__] = ((unsigned long long)(kind) << 32) | blockIdx.x | (blockIdx.y << 16); \
      krk_trace_buf[4 * i__ + 1] = (a);                                      \
      krk_trace_buf[4 * i__ + 2] = (b);                                      \
      krk_trace_buf[4 * i__ + 3] = (c);                                      \
    }                                                                        \
  }
#define KRK_TRACE_MARKS_OUT(kind)                                            \
  KRK_TRACE_REC(kind, mark__[0], mark__[1], mark__[2])                       \
  KRK_TRACE_REC((kind) + 1, mark__[3], mark__[4], mark__[5])
#else
#define KRK_TRACE_DECL
#define KRK_TRACE_READY
#define KRK_TRACE_END(kind)
#define KRK_TRACE_MARKS
#define KRK_TRACE_MARK(i)
#define KRK_TRACE_MARKS_OUT(kind)
#endif

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  static const bool plain = getenv("KRK_NO_PDL") != nullptr;  // measurement switch: ordinary stream order
  cfg.attrs = attr;
  cfg.numAttrs = plain ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ float round_to(float v) { return to_float<T>(from_float<T>(v)); }

// A norm's gain may be stored in 32-bit even on the bfloat16 path.
template <typename T>
__device__ __forceinline__ float load_gain(const void* g, int i, int gain_f32) {
  return gain_f32 ? reinterpret_cast<const float*>(g)[i] : to_float<T>(reinterpret_cast<const T*>(g)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 32 floats of shared memory. Safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < n_warps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Page of position `pos` for cache slot `slot`: table is [slots, width].
__device__ __forceinline__ int page_of(const int* __restrict__ table, int width, int slot, int pos) {
  return table[(size_t)slot * width + (pos / KRK_PAGE) % width];
}
