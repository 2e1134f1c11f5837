// Row kernels bound by memory traffic: embedding gather, RMSNorm with the
// residual add folded in, SwiGLU, row gather.
//
// RMSNorm: v = mean(x^2); n = round(x * rsqrt(v + eps)); y = round(n * w) -- the
// value is rounded to the element type BEFORE the weight multiply, which is what
// the reference computes (engine/kernels/rmsnorm.py:30-45 of
// willzeng274/kernel-rush-kawk). With a branch: s = round(x + branch) is written
// out as the new residual stream and normalised (engine/kernels/add_rmsnorm.py:
// 21-29). Squares, mean and rsqrt are float32. One block per row; the row is
// held in shared memory as float so that global memory is read once.
#include "common.cuh"

namespace {

template <typename T> struct Pack4;
template <> struct Pack4<float> {
  typedef float4 raw;
  static __device__ __forceinline__ void unpack(const raw& r, float* f) { f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
  static __device__ __forceinline__ raw pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Pack4<bf16> {
  typedef uint2 raw;
  static __device__ __forceinline__ void unpack(const raw& r, float* f) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
  }
  static __device__ __forceinline__ raw pack(const float* f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
    raw r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    return r;
  }
};

// out = norm(x [+ branch]) * gain; x_new = round(x + branch) when branch is given.
template <typename T, bool VEC>
__global__ void rmsnorm_kernel(T* __restrict__ out, T* x_new, const T* x, const T* __restrict__ branch,
                               const void* __restrict__ gain, int gain_f32, int H, float eps) {
  extern __shared__ float row_s[];  // H floats
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * H;
  float sq = 0.f;
  if (VEC) {
    typedef typename Pack4<T>::raw raw;
    const raw* xv = reinterpret_cast<const raw*>(x + base);
    const raw* bv = branch ? reinterpret_cast<const raw*>(branch + base) : nullptr;
    raw* nv = reinterpret_cast<raw*>(x_new + base);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float f[4];
      Pack4<T>::unpack(xv[i], f);
      if (bv) {
        float g[4];
        Pack4<T>::unpack(bv[i], g);
#pragma unroll
        for (int j = 0; j < 4; ++j) f[j] = round_to<T>(f[j] + g[j]);
        nv[i] = Pack4<T>::pack(f);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) { row_s[4 * i + j] = f[j]; sq += f[j] * f[j]; }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float f = to_float<T>(x[base + i]);
      if (branch) {
        f = round_to<T>(f + to_float<T>(branch[base + i]));
        x_new[base + i] = from_float<T>(f);
      }
      row_s[i] = f;
      sq += f * f;
    }
  }
  const float total = block_sum(sq, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  if (VEC) {
    typedef typename Pack4<T>::raw raw;
    raw* ov = reinterpret_cast<raw*>(out + base);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float f[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) f[j] = round_to<T>(row_s[4 * i + j] * rstd) * load_gain<T>(gain, 4 * i + j, gain_f32);
      ov[i] = Pack4<T>::pack(f);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      out[base + i] = from_float<T>(round_to<T>(row_s[i] * rstd) * load_gain<T>(gain, i, gain_f32));
  }
}

// bfloat16 rows of up to 8192 elements (a multiple of 8): one 16-byte piece per thread, the
// row stays in registers, global memory is read and written exactly once.
__global__ void rmsnorm_bf16x8_kernel(bf16* __restrict__ out, bf16* x_new, const bf16* x, const bf16* __restrict__ branch,
                                      const void* __restrict__ gain, int gain_f32, int H, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * H;
  const int k = threadIdx.x * 8;
  const bool on = k < H;
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = 0.f;
  if (on) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + base + k);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    if (branch) {
      uint4 bv = *reinterpret_cast<const uint4*>(branch + base + k);
      const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
      uint4 sv;
      __nv_bfloat162* sp = reinterpret_cast<__nv_bfloat162*>(&sv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sp[j] = __hadd2_rn(xp[j], bp[j]);  // the 32-bit sum of two bfloat16 values, rounded once
        f[2 * j] = __low2float(sp[j]);
        f[2 * j + 1] = __high2float(sp[j]);
      }
      *reinterpret_cast<uint4*>(x_new + base + k) = sv;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { f[2 * j] = __low2float(xp[j]); f[2 * j + 1] = __high2float(xp[j]); }
    }
  }
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) sq += f[j] * f[j];
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
  if (on) {
    uint4 ov;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
    if (gain_f32) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        op[j] = __floats2bfloat162_rn(round_to<bf16>(f[2 * j] * rstd) * load_gain<bf16>(gain, k + 2 * j, 1),
                                      round_to<bf16>(f[2 * j + 1] * rstd) * load_gain<bf16>(gain, k + 2 * j + 1, 1));
    } else {
      const uint4 gv = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(gain) + k);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        op[j] = __hmul2_rn(__floats2bfloat162_rn(f[2 * j] * rstd, f[2 * j + 1] * rstd), reinterpret_cast<const __nv_bfloat162*>(&gv)[j]);
    }
    *reinterpret_cast<uint4*>(out + base + k) = ov;
  }
}

template <typename T>
int launch_rmsnorm(void* out, void* x_new, const void* x, const void* branch, const void* gain, int gain_f32, int rows,
                   int H, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (sizeof(T) == 2 && H % 8 == 0 && H <= 8192 && (gain_f32 || ((uintptr_t)gain & 15) == 0)) {  // 16-byte gain loads
    const int threads = ((H / 8 + 31) / 32) * 32;
    return (int)launch_pdl(rmsnorm_bf16x8_kernel, dim3(rows), dim3(threads), 0, stream, (bf16*)out, (bf16*)x_new,
                           (const bf16*)x, (const bf16*)branch, gain, gain_f32, H, eps);
  }
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 220 * 1024) return -2;  // a row must fit in shared memory
  int threads = H / 4 >= 1024 ? 1024 : (H / 4 >= 512 ? 512 : (H / 4 >= 256 ? 256 : 128));
  const bool vec = (H % 4 == 0);
  auto kern = vec ? rmsnorm_kernel<T, true> : rmsnorm_kernel<T, false>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaError_t e = launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (T*)out, (T*)x_new, (const T*)x,
                             (const T*)branch, gain, gain_f32, H, eps);
  return (int)e;
}

// out[r] = table[ids[r]] ; an id outside [0, n_table_rows) sets *error and yields zeros.
template <typename T>
__global__ void gather_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids, int H,
                              int n_table_rows, int* error) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int id = ids[r];
  const bool bad = id < 0 || id >= n_table_rows;
  if (bad && threadIdx.x == 0 && error) atomicExch(error, 1);
  const T* src = table + (size_t)(bad ? 0 : id) * H;
  T* dst = out + (size_t)r * H;
  const bool vec = ((size_t)H * sizeof(T)) % 16 == 0;
  if (vec) {
    const int n = (int)((size_t)H * sizeof(T) / 16);
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < n; i += blockDim.x) d[i] = bad ? make_uint4(0, 0, 0, 0) : s[i];
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = bad ? from_float<T>(0.f) : src[i];
  }
}

// out[r, i] = round(round(silu(g)) * u), g = gu[r, i], u = gu[r, I + i]
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int I) {
  const size_t r = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const float g = to_float<T>(gu[r * 2 * I + i]);
  const float u = to_float<T>(gu[r * 2 * I + I + i]);
  const float s = round_to<T>(g / (1.0f + expf(-g)));
  out[r * I + i] = from_float<T>(s * u);
}

// bfloat16, I a multiple of 8: eight gate and eight up values per thread; blockIdx.x is the row.
// silu runs in 32-bit with the fast exponential and reciprocal (a few units in the last place of a float,
// far below the bfloat16 rounding that follows); the product of the two rounded factors is one packed
// bfloat16 multiply, which rounds the exact product as the unpacked form does.
__global__ void swiglu_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int I) {
  const size_t r = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= I) return;
  const uint4 gv = *reinterpret_cast<const uint4*>(gu + r * 2 * I + i);
  const uint4 uv = *reinterpret_cast<const uint4*>(gu + r * 2 * I + I + i);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float g0 = __low2float(gp[j]), g1 = __high2float(gp[j]);
    const __nv_bfloat162 silu = __floats2bfloat162_rn(__fdividef(g0, 1.0f + __expf(-g0)), __fdividef(g1, 1.0f + __expf(-g1)));
    op[j] = __hmul2_rn(silu, up[j]);
  }
  *reinterpret_cast<uint4*>(out + r * I + i) = ov;
}

}  // namespace

KRK_API int krk_rmsnorm(void* out, void* x_new, const void* x, const void* branch, const void* gain, int gain_f32,
                        int rows, int H, float eps, int dtype, cudaStream_t stream) {
  return dtype == KRK_DTYPE_F32 ? launch_rmsnorm<float>(out, x_new, x, branch, gain, gain_f32, rows, H, eps, stream)
                                : launch_rmsnorm<bf16>(out, x_new, x, branch, gain, gain_f32, rows, H, eps, stream);
}

KRK_API int krk_gather_rows(void* out, const void* table, const int* ids, int rows, int H, int n_table_rows, int* error,
                            int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(gather_kernel<float>, dim3(rows), dim3(128), 0, stream, (float*)out, (const float*)table, ids,
                           H, n_table_rows, error);
  return (int)launch_pdl(gather_kernel<bf16>, dim3(rows), dim3(128), 0, stream, (bf16*)out, (const bf16*)table, ids, H,
                         n_table_rows, error);
}

KRK_API int krk_swiglu(void* out, const void* gu, int rows, int I, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (dtype == KRK_DTYPE_BF16 && I % 8 == 0) {
    const int chunks = (I / 8 + 255) / 256;
    if (chunks > 65535) return -3;
    swiglu_bf16x8_kernel<<<dim3(rows, chunks), 256, 0, stream>>>((bf16*)out, (const bf16*)gu, I);
    KRK_CHECK_LAUNCH();
    return 0;
  }
  if ((I + 255) / 256 > 65535) return -3;
  dim3 grid(rows, (I + 255) / 256);
  if (dtype == KRK_DTYPE_F32)
    swiglu_kernel<float><<<grid, 256, 0, stream>>>((float*)out, (const float*)gu, I);
  else
    swiglu_kernel<bf16><<<grid, 256, 0, stream>>>((bf16*)out, (const bf16*)gu, I);
  KRK_CHECK_LAUNCH();
  return 0;
}
