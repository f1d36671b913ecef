// Int8 activation quantisation for W8A8 linears (tcgen05 kind::i8 GEMM, dtype 3 of b200_gemm), with
// the two optional transforms the int8 checkpoint formats ask for on the activation side:
//   * SmoothQuant: x_j *= inv_smooth[j] per input channel before quantisation;
//   * ConvRot: every contiguous group of G input channels (G a power of four) is rotated by the
//     normalised regular Hadamard matrix H = kron(h4, ..., h4), because the stored weight is
//     W H^T: (x H)(W H^T)^T = x W^T. The rotation is a radix-4 butterfly in shared memory,
//     log4(G) stages, each output = half of (sum of its four inputs - twice the mirrored one).
// One block per token row: load (+ smooth) -> rotate -> absmax -> quantise; scale = absmax / 127.
//
// Reference: src/HartsyInference.Cuda/Kernels/dequant/w8a8.cu (w8a8_quant_rowwise_f16, two-phase
// per-row quantisation), dequant/convrot.cu (activation rotation), src/HartsyInference.Core/Tensors/
// Int8ConvRotCodec.cs:118-145 (the butterfly and its normalisation).
#include "common.cuh"

namespace b200 {

constexpr int kW8Threads = 256;

__global__ void __launch_bounds__(kW8Threads) quant_int8_rows_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                                                                      float* __restrict__ scale,
                                                                      const float* __restrict__ inv_smooth, long long ldx,
                                                                      long long ldq, int cols, int group) {
  extern __shared__ float row[];          // [cols]
  __shared__ float red[kW8Threads / 32];
  const long long r = blockIdx.x;
  const __nv_bfloat16* xr = x + r * ldx;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = __bfloat162float(xr[i]);
    if (inv_smooth) v *= inv_smooth[i];
    row[i] = v;
  }
  __syncthreads();
  if (group > 1) {
    // radix-4 butterflies: at stride s the element index is (block, digit, lane) with digit in 0..3
    for (int stride = 1; stride < group; stride *= 4) {
      const int quads = cols / 4;
      for (int t = threadIdx.x; t < quads; t += blockDim.x) {
        const int lane = t % stride, blk = t / stride;          // blk counts spans of 4 * stride
        float* a = row + static_cast<long long>(blk) * 4 * stride + lane;
        const float v0 = a[0], v1 = a[stride], v2 = a[2 * stride], v3 = a[3 * stride];
        const float sum = v0 + v1 + v2 + v3;
        a[0] = 0.5f * (sum - 2.f * v3);
        a[stride] = 0.5f * (sum - 2.f * v2);
        a[2 * stride] = 0.5f * (sum - 2.f * v1);
        a[3 * stride] = 0.5f * (sum - 2.f * v0);
      }
      __syncthreads();
    }
  }
  float amax = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < kW8Threads / 32; ++w) amax = fmaxf(amax, red[w]);
  const float sc = amax > 0.f ? amax / 127.f : 1.f;
  const float inv = amax > 0.f ? 127.f / amax : 0.f;
  if (threadIdx.x == 0) scale[r] = sc;
  int8_t* qr = q + r * ldq;
  for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int iv = i + e < cols ? max(-127, min(127, __float2int_rn(row[i + e] * inv))) : 0;
      word |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(iv))) << (8 * e);
    }
    *reinterpret_cast<uint32_t*>(qr + i) = word;
  }
}

}  // namespace b200

using namespace b200;

// x [rows][ldx] bf16 -> q [rows][ldq] int8 and scale [rows] fp32 (dequantisation scale). cols % 4 == 0;
// ldq % 4 == 0; convrot_group: 0 / 1 = no rotation, else a power of four dividing cols;
// inv_smooth: [cols] fp32 or null.
B200_API int b200_quant_int8_rows(const void* x, void* q, float* scale, const float* inv_smooth, long long rows, int cols,
                                  long long ldx, long long ldq, int convrot_group, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols <= 0 || cols % 4 != 0 || ldq % 4 != 0 || cols > 48 * 1024) return -2;
  if (convrot_group > 1) {
    int g = convrot_group;
    while (g > 1 && g % 4 == 0) g /= 4;
    if (g != 1 || cols % convrot_group != 0) return -2;
  }
  const size_t smem = static_cast<size_t>(cols) * 4;
  static PerDeviceOnce configured;
  if (configured.first_time() &&
      cudaFuncSetAttribute(quant_int8_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
    return -4;
  quant_int8_rows_kernel<<<static_cast<unsigned>(rows), kW8Threads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<int8_t*>(q), scale, inv_smooth, ldx, ldq, cols, convrot_group);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
