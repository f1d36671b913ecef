// Guidance and scheduler steps on the device, each one pass (or two) over the latents.
//
//   cfg_renorm_euler   guided = uncond + g (cond - uncond); s = clamp(||cond|| / (||guided|| + 1e-8),
//                      renorm_min, 1) over the WHOLE tensor; z += s guided dt. Two launches: the first
//                      accumulates both squared norms (double precision, per-block partials, the last
//                      block to finish folds them in fixed order and writes s), the second applies.
//   cfg_rownorm_euler  the same with one ratio per row of the last dimension, no clamp
//                      (s = ||cond_row|| / (||guided_row|| + eps), 0 when the denominator is 0): one
//                      block per row, one launch.
//   lincomb            out = sum_i coef_i x_i for up to eight fp32 tensors: the update of multistep
//                      solvers (UniPC, DPM-Solver++) written as ONE kernel instead of a chain of
//                      tensor ops that each re-read the latents.
//
// cond / uncond are bf16 or fp32, z and the lincomb operands fp32. Reference counterparts:
// src/HartsyInference.Cuda/Kernels/dit/dit_f32.cu (dit_cfg_renorm_reduce_f32:323,
// dit_cfg_renorm_finalize_f32:365, dit_cfg_renorm_euler_f32:404, dit_cfg_normalized_euler_f32:433) and
// the tensor-op UniPC update of src/HartsyInference.Diffusion/Schedulers/FlowUniPCMultistepScheduler.cs.
#include "common.cuh"

namespace b200 {

template <typename T>
__device__ __forceinline__ float g_load(const T* p, long long i);
template <>
__device__ __forceinline__ float g_load<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float g_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

constexpr int kNormBlocks = 592;        // 4 per SM

__device__ __forceinline__ double block_sum_d(double v, double* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  double t = l < nw ? red[l] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// scratch: [0] scale (float), [1] block counter (u32), then 2 * gridDim doubles of partials (8-byte aligned)
template <typename T>
__global__ void __launch_bounds__(256) cfg_renorm_reduce_kernel(const T* __restrict__ cond, const T* __restrict__ uncond,
                                                                long long n, float g, float renorm_min,
                                                                uint32_t* scratch) {
  __shared__ double red[8];
  __shared__ bool last;
  double c2 = 0.0, g2 = 0.0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float c = g_load<T>(cond, i), u = g_load<T>(uncond, i);
    const float v = u + g * (c - u);
    c2 += static_cast<double>(c) * c;
    g2 += static_cast<double>(v) * v;
  }
  c2 = block_sum_d(c2, red);
  g2 = block_sum_d(g2, red);
  double* part = reinterpret_cast<double*>(scratch + 2);
  if (threadIdx.x == 0) {
    part[2 * blockIdx.x] = c2;
    part[2 * blockIdx.x + 1] = g2;
    __threadfence();
    last = atomicAdd(scratch + 1, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  double a = 0.0, b = 0.0;
  for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += blockDim.x) {     // fixed order per thread, then a tree
    a += __ldcg(part + 2 * i);
    b += __ldcg(part + 2 * i + 1);
  }
  a = block_sum_d(a, red);
  b = block_sum_d(b, red);
  if (threadIdx.x == 0) {
    double ratio = sqrt(a) / (sqrt(b) + 1.0e-8);
    if (ratio < static_cast<double>(renorm_min)) ratio = renorm_min;      // branches, not fmin / fmax: a NaN stays a NaN
    else if (ratio > 1.0) ratio = 1.0;
    *reinterpret_cast<float*>(scratch) = static_cast<float>(ratio);
    scratch[1] = 0;                                                       // ready for the next call
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cfg_renorm_apply_kernel(float* __restrict__ z, const T* __restrict__ cond,
                                                               const T* __restrict__ uncond, long long n, float g, float dt,
                                                               const float* __restrict__ scale) {
  const float s = *scale * dt;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float c = g_load<T>(cond, i), u = g_load<T>(uncond, i);
    z[i] += (u + g * (c - u)) * s;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cfg_rownorm_euler_kernel(float* __restrict__ z, const T* __restrict__ cond,
                                                                const T* __restrict__ uncond, long long rows, int dim,
                                                                float g, float dt, float eps) {
  __shared__ double red[8];
  __shared__ float ratio;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * dim;
    double c2 = 0.0, g2 = 0.0;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float c = g_load<T>(cond, base + d), u = g_load<T>(uncond, base + d);
      const float v = u + g * (c - u);
      c2 += static_cast<double>(c) * c;
      g2 += static_cast<double>(v) * v;
    }
    c2 = block_sum_d(c2, red);
    g2 = block_sum_d(g2, red);
    if (threadIdx.x == 0) {
      const double den = sqrt(g2) + static_cast<double>(eps);
      ratio = den > 0.0 ? static_cast<float>(sqrt(c2) / den) : 0.f;
    }
    __syncthreads();
    const float s = ratio * dt;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float c = g_load<T>(cond, base + d), u = g_load<T>(uncond, base + d);
      z[base + d] += (u + g * (c - u)) * s;
    }
    __syncthreads();
  }
}

struct LincombArgs {
  const float* x[8];
  float coef[8];
  int terms;
};

__global__ void __launch_bounds__(256) lincomb_kernel(float* out, const LincombArgs a, long long n4, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < 8; ++t)
      if (t < a.terms) {
        const float4 v = *reinterpret_cast<const float4*>(a.x[t] + 4 * i);
        acc.x += a.coef[t] * v.x; acc.y += a.coef[t] * v.y; acc.z += a.coef[t] * v.z; acc.w += a.coef[t] * v.w;
      }
    *reinterpret_cast<float4*>(out + 4 * i) = acc;
  }
  if (blockIdx.x == 0 && threadIdx.x < static_cast<unsigned>(n - 4 * n4)) {      // tail of fewer than four values
    const long long i = 4 * n4 + threadIdx.x;
    float acc = 0.f;
    for (int t = 0; t < a.terms; ++t) acc += a.coef[t] * a.x[t][i];
    out[i] = acc;
  }
}

}  // namespace b200

using namespace b200;

static int guidance_err() {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(1000 + static_cast<int>(e));
}

B200_API long long b200_cfg_renorm_scratch_bytes() { return 8 + 16ll * kNormBlocks; }

// `scratch`: b200_cfg_renorm_scratch_bytes() bytes, 8-byte aligned, zeroed once. The scale used is left in
// its first float.
B200_API int b200_cfg_renorm_euler(float* z, const void* cond, const void* uncond, int bf16, long long n, float guidance,
                                   float dt, float renorm_min, void* scratch, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 7) != 0) return -2;
  long long want = (n + 255) / 256;
  const int grid = static_cast<int>(want < kNormBlocks ? want : kNormBlocks);
  uint32_t* s = static_cast<uint32_t*>(scratch);
  if (bf16) {
    auto c = static_cast<const __nv_bfloat16*>(cond), u = static_cast<const __nv_bfloat16*>(uncond);
    cfg_renorm_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(c, u, n, guidance, renorm_min, s);
    cfg_renorm_apply_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(z, c, u, n, guidance, dt, reinterpret_cast<const float*>(s));
  } else {
    auto c = static_cast<const float*>(cond), u = static_cast<const float*>(uncond);
    cfg_renorm_reduce_kernel<float><<<grid, 256, 0, stream>>>(c, u, n, guidance, renorm_min, s);
    cfg_renorm_apply_kernel<float><<<grid, 256, 0, stream>>>(z, c, u, n, guidance, dt, reinterpret_cast<const float*>(s));
  }
  return guidance_err();
}

B200_API int b200_cfg_rownorm_euler(float* z, const void* cond, const void* uncond, int bf16, long long rows, int dim,
                                    float guidance, float dt, float eps, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return 0;
  const int grid = static_cast<int>(rows < 4 * 148 * 4 ? rows : 4 * 148 * 4);
  if (bf16)
    cfg_rownorm_euler_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(z, static_cast<const __nv_bfloat16*>(cond),
                                                                     static_cast<const __nv_bfloat16*>(uncond), rows, dim,
                                                                     guidance, dt, eps);
  else
    cfg_rownorm_euler_kernel<float><<<grid, 256, 0, stream>>>(z, static_cast<const float*>(cond),
                                                             static_cast<const float*>(uncond), rows, dim, guidance, dt, eps);
  return guidance_err();
}

// out (fp32, 16-byte aligned like every operand) = sum_i coefs[i] * xs[i], 1 <= terms <= 8. out may alias an operand.
B200_API int b200_lincomb(float* out, const float* const* xs, const float* coefs, int terms, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (terms < 1 || terms > 8) return -2;
  LincombArgs a{};
  a.terms = terms;
  for (int i = 0; i < terms; ++i) {
    if ((reinterpret_cast<uintptr_t>(xs[i]) & 15) != 0) return -3;
    a.x[i] = xs[i];
    a.coef[i] = coefs[i];
  }
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0) return -3;
  const long long n4 = n / 4;
  long long want = (n4 + 255) / 256;
  if (want < 1) want = 1;
  lincomb_kernel<<<static_cast<int>(want < 1184 ? want : 1184), 256, 0, stream>>>(out, a, n4, n);
  return guidance_err();
}
