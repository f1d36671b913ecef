// GGUF block-quantised weights on the device: Q8_0 and Q4_K stay in their file layout in HBM
// (8.5 and 4.5 bits per weight) and are consumed directly.
//
//  * gguf_gemv:     y[m][n] = sum_k x[m][k] * W[n][k] for 1..16 tokens. Activations are quantised
//                   once per call to int8 in blocks of 32 (scale + block sum, the Q8_1 form); one
//                   warp per output row walks the row's quant blocks with coalesced 4-byte loads
//                   and integer dot products (dp4a), so decode reads each weight bit exactly once.
//  * gguf_dequant:  blocks -> bf16 [n][k], for token counts where the tensor-core GEMM wins; the
//                   caller then runs the ordinary GEMM on the scratch copy.
//
// Q8_0 block (34 bytes, 32 weights):   fp16 d, int8 q[32];                 w = d * q
// Q4_K block (144 bytes, 256 weights): fp16 d, fp16 dmin, 12 bytes of 6-bit (scale, min) pairs
//   for eight sub-blocks of 32, 128 bytes of nibbles (bytes 32 c .. 32 c + 31 hold sub-block 2 c in
//   the low and 2 c + 1 in the high nibbles);                               w = d * sc * q - dmin * m
//
// Reference: the m <= 8 fused GEMV ladder of src/HartsyInference.Cuda/CudaBackend.cs:1911-2047
// (dp4a Q8_1 path) and src/HartsyInference.Cuda/Kernels/lm/ (dequant_gemv kernels);
// block geometry as in src/HartsyInference.ModelAssets/Gguf/Codecs/Codec_Q8_0.cs, Codec_Q4_K.cs.
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

constexpr int kGgmlQ8_0 = 8;
constexpr int kGgmlQ4_K = 12;
constexpr int kMaxGemvTokens = 16;

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// ---- activation quantisation: x bf16 [m][k] -> q int8 [m][k], d fp32 [m][k/32], s fp32 [m][k/32]
// (s = sum of the ORIGINAL values of the block, needed by formats with a minimum term).
__global__ void quant_q8_1_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int8_t* __restrict__ q,
                                  float* __restrict__ d, float* __restrict__ s, int m, int k) {
  const int blocks = k >> 5;
  const long long gid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;   // one warp per block
  const int lane = threadIdx.x & 31;
  if (gid >= static_cast<long long>(m) * blocks) return;
  const int row = static_cast<int>(gid / blocks), b = static_cast<int>(gid % blocks);
  const float v = __bfloat162float(x[row * ldx + b * 32 + lane]);
  const float amax = warp_max(fabsf(v));
  const float sum = warp_sum(v);
  const float scale = amax / 127.f;
  const float inv = scale > 0.f ? 1.f / scale : 0.f;
  q[static_cast<long long>(row) * k + b * 32 + lane] = static_cast<int8_t>(__float2int_rn(v * inv));
  if (lane == 0) {
    d[static_cast<long long>(row) * blocks + b] = scale;
    s[static_cast<long long>(row) * blocks + b] = sum;
  }
}

struct GemvParams {
  const uint8_t* w;        // [n][k / block * block_bytes]
  const int8_t* xq;        // [m][k]
  const float* xd;         // [m][k / 32]
  const float* xs;         // [m][k / 32]
  __nv_bfloat16* out;      // [m][ldc]
  const __nv_bfloat16* bias;
  int m, n, k;
  long long ldc;
};

// One warp per output row. Consecutive lanes read consecutive 4-byte words of the row so that
// loads coalesce; a Q8_0 block has 8 words of weights, so a warp covers 4 blocks per pass.
template <int kTokens>
__global__ void __launch_bounds__(256) gemv_q8_0_kernel(const GemvParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.n) return;
  const int blocks = p.k >> 5;
  const uint8_t* row = p.w + static_cast<long long>(warp) * blocks * 34;
  float acc[kTokens];
#pragma unroll
  for (int t = 0; t < kTokens; ++t) acc[t] = 0.f;
  const int sub = lane & 7;                  // word within the block
  for (int b = lane >> 3; b < blocks; b += 4) {
    const uint8_t* blk = row + b * 34;
    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(blk));
    // the block starts on a 2-byte boundary only: assemble the word from two 16-bit loads
    const uint16_t lo = *reinterpret_cast<const uint16_t*>(blk + 2 + sub * 4);
    const uint16_t hi = *reinterpret_cast<const uint16_t*>(blk + 4 + sub * 4);
    const int wq = static_cast<int>(static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16));
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      if (t < p.m) {
        const int xq = *reinterpret_cast<const int*>(p.xq + static_cast<long long>(t) * p.k + b * 32 + sub * 4);
        const int dot = __dp4a(wq, xq, 0);
        acc[t] = fmaf(d * p.xd[static_cast<long long>(t) * blocks + b], static_cast<float>(dot), acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const float v = warp_sum(acc[t]);
    if (lane == 0 && t < p.m) {
      const float b = p.bias ? __bfloat162float(p.bias[warp]) : 0.f;
      p.out[static_cast<long long>(t) * p.ldc + warp] = __float2bfloat16(v + b);
    }
  }
}

__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* sc, int& s, int& m) {
  if (j < 4) {
    s = sc[j] & 63;
    m = sc[j + 4] & 63;
  } else {
    s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
    m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
  }
}

// Q4_K: lane l reads nibble word l of the super-block (bytes 4 l .. 4 l + 3 of qs): chunk
// c = l / 8 (64 weights), byte offset o = (l % 8) * 4; its low nibbles are weights
// c * 64 + o .. o + 3 of sub-block 2 c, its high nibbles the same positions of sub-block 2 c + 1.
template <int kTokens>
__global__ void __launch_bounds__(256) gemv_q4_k_kernel(const GemvParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.n) return;
  const int sblocks = p.k >> 8;
  const int xblocks = p.k >> 5;
  const uint8_t* row = p.w + static_cast<long long>(warp) * sblocks * 144;
  float acc[kTokens];
#pragma unroll
  for (int t = 0; t < kTokens; ++t) acc[t] = 0.f;
  const int c = lane >> 3, o = (lane & 7) * 4;
  for (int sb = 0; sb < sblocks; ++sb) {
    const uint8_t* blk = row + sb * 144;          // 144 = 16 * 9: every super-block is 16-byte aligned
    const uint32_t dd = *reinterpret_cast<const uint32_t*>(blk);
    const float d = half_bits_to_float(static_cast<uint16_t>(dd & 0xffff));
    const float dmin = half_bits_to_float(static_cast<uint16_t>(dd >> 16));
    int s0, m0, s1, m1;
    q4k_scale_min(2 * c, blk + 4, s0, m0);
    q4k_scale_min(2 * c + 1, blk + 4, s1, m1);
    const uint32_t qw = *reinterpret_cast<const uint32_t*>(blk + 16 + lane * 4);
    const int qlo = static_cast<int>(qw & 0x0F0F0F0Fu), qhi = static_cast<int>((qw >> 4) & 0x0F0F0F0Fu);
    const int xb0 = sb * 8 + 2 * c;               // activation block of sub-block 2 c
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      if (t < p.m) {
        const int8_t* xq = p.xq + static_cast<long long>(t) * p.k + sb * 256 + c * 64 + o;
        const int x0 = *reinterpret_cast<const int*>(xq), x1 = *reinterpret_cast<const int*>(xq + 32);
        const float dx0 = p.xd[static_cast<long long>(t) * xblocks + xb0];
        const float dx1 = p.xd[static_cast<long long>(t) * xblocks + xb0 + 1];
        acc[t] = fmaf(d * s0 * dx0, static_cast<float>(__dp4a(qlo, x0, 0)), acc[t]);
        acc[t] = fmaf(d * s1 * dx1, static_cast<float>(__dp4a(qhi, x1, 0)), acc[t]);
        // the minimum term needs the block sums once per sub-block: lanes with o == 0 add it
        if (o == 0) {
          acc[t] -= dmin * (m0 * p.xs[static_cast<long long>(t) * xblocks + xb0] +
                            m1 * p.xs[static_cast<long long>(t) * xblocks + xb0 + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const float v = warp_sum(acc[t]);
    if (lane == 0 && t < p.m) {
      const float b = p.bias ? __bfloat162float(p.bias[warp]) : 0.f;
      p.out[static_cast<long long>(t) * p.ldc + warp] = __float2bfloat16(v + b);
    }
  }
}

// ---- dequantisation to bf16 (one thread per 8 output values)
__global__ void dequant_q8_0_kernel(const uint8_t* __restrict__ w, __nv_bfloat16* __restrict__ out, long long total8) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const long long blk = i >> 2;
  const int part = static_cast<int>(i & 3);
  const uint8_t* b = w + blk * 34;
  const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b));
  const int8_t* q = reinterpret_cast<const int8_t*>(b + 2 + part * 8);
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) ow[j] = pack_bf16x2(d * q[2 * j], d * q[2 * j + 1]);
  *reinterpret_cast<uint4*>(out + i * 8) = o;
}

__global__ void dequant_q4_k_kernel(const uint8_t* __restrict__ w, __nv_bfloat16* __restrict__ out, long long total8) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const long long sb = i >> 5;                  // 32 groups of 8 values per super-block
  const int g = static_cast<int>(i & 31);       // values g * 8 .. g * 8 + 7
  const int j = g >> 2;                         // sub-block (32 values)
  const int off = (g & 3) * 8;                  // position inside the sub-block
  const uint8_t* b = w + sb * 144;
  const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b));
  const float dmin = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b + 2));
  int s, m;
  q4k_scale_min(j, b + 4, s, m);
  const uint8_t* qs = b + 16 + (j >> 1) * 32 + off;
  const int shift = (j & 1) * 4;
  const float ds = d * s, mm = dmin * m;
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int t = 0; t < 4; ++t)
    ow[t] = pack_bf16x2(ds * ((qs[2 * t] >> shift) & 0xF) - mm, ds * ((qs[2 * t + 1] >> shift) & 0xF) - mm);
  *reinterpret_cast<uint4*>(out + i * 8) = o;
}

template <int kTokens>
int launch_gemv(int type, const GemvParams& p, cudaStream_t stream) {
  const int blocks = (p.n * 32 + 255) / 256;
  if (type == kGgmlQ8_0) gemv_q8_0_kernel<kTokens><<<blocks, 256, 0, stream>>>(p);
  else gemv_q4_k_kernel<kTokens><<<blocks, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}

}  // namespace b200

using namespace b200;

// Bytes of one row of k values in ggml type `type` (0 if the type has no device kernels here).
B200_API long long b200_gguf_row_bytes(int type, int k) {
  if (type == kGgmlQ8_0 && k % 32 == 0) return static_cast<long long>(k / 32) * 34;
  if (type == kGgmlQ4_K && k % 256 == 0) return static_cast<long long>(k / 256) * 144;
  return 0;
}

// Scratch for the quantised activations of b200_gguf_gemv: int8 [m][k] + 2 x fp32 [m][k / 32].
B200_API long long b200_gguf_gemv_workspace_bytes(int m, int k) {
  return static_cast<long long>(m) * k + 2ll * m * (k / 32) * 4 + 256;
}

// out[m][n] (bf16, row pitch ldc) = x[m][k] (bf16, row pitch ldx) * W^T + bias, W in ggml type `type`.
B200_API int b200_gguf_gemv(const void* x, long long ldx, const void* w, int type, void* out, long long ldc,
                            const void* bias, int m, int n, int k, void* workspace, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m > kMaxGemvTokens) return -8;
  if (b200_gguf_row_bytes(type, k) == 0 || workspace == nullptr) return -2;
  int8_t* xq = static_cast<int8_t*>(workspace);
  const long long off = (static_cast<long long>(m) * k + 255) / 256 * 256;
  float* xd = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + off);
  float* xs = xd + static_cast<long long>(m) * (k / 32);
  const long long warps = static_cast<long long>(m) * (k / 32);
  quant_q8_1_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, xq, xd, xs, m, k);
  GemvParams p{static_cast<const uint8_t*>(w), xq, xd, xs, static_cast<__nv_bfloat16*>(out),
               static_cast<const __nv_bfloat16*>(bias), m, n, k, ldc};
  if (m == 1) return launch_gemv<1>(type, p, stream);
  if (m <= 2) return launch_gemv<2>(type, p, stream);
  if (m <= 4) return launch_gemv<4>(type, p, stream);
  if (m <= 8) return launch_gemv<8>(type, p, stream);
  return launch_gemv<16>(type, p, stream);
}

// Blocks -> bf16 [n][k] (contiguous).
B200_API int b200_gguf_dequant(const void* w, int type, void* out, long long n, int k, cudaStream_t stream) {
  if (b200_gguf_row_bytes(type, k) == 0) return -2;
  const long long total8 = n * k / 8;
  if (total8 == 0) return 0;
  const unsigned blocks = static_cast<unsigned>((total8 + 255) / 256);
  if (type == kGgmlQ8_0)
    dequant_q8_0_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(w), static_cast<__nv_bfloat16*>(out), total8);
  else
    dequant_q4_k_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(w), static_cast<__nv_bfloat16*>(out), total8);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
