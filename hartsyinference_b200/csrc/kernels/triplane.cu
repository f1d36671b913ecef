// Triplane radiance-field decode in one kernel: for every query point the three feature planes are
// sampled bilinearly (grid_sample semantics: align_corners = false, zero padding) and the 3 C
// features run through the SiLU MLP (3 C -> H, `mid` x (H -> H), H -> 4) without ever leaving the SM:
// the weights sit in shared memory, the activations of a point in one thread's registers. Points
// are either given explicitly or generated from a res^3 lattice over [-R, R]^3 (x outermost, z
// innermost, end points included), so a 256^3 density field needs no coordinate buffer.
//
// Plane p of a point (x, y, z) scaled to [-1, 1]: p = 0 samples at (x, y), p = 1 at (x, z), p = 2 at
// (y, z); the first coordinate indexes the plane's width, the second its height. Output per point:
// [density_raw, r_raw, g_raw, b_raw] (density activation exp(raw + bias) and colour sigmoid are the
// caller's, as in the model definition).
//
// The reference runs this as a grid-sample kernel followed by ten Linear + SiLU launches per chunk of
// 131072 points (src/HartsyInference.Cuda/Kernels/dit/dit_f32.cu:1179 triplane_grid_sample_f32;
// src/HartsyInference.ThreeD/Models/TripoSr/TriplaneNerfDecoder.cs:118-139).
#include "common.cuh"

namespace b200 {

constexpr int kTriHidden = 64;
constexpr int kTriThreads = 128;

struct TriplaneParams {
  const float* planes;     // [3][C][H][W]
  int c, h, w;
  const float* coords;     // [count][3] in [-R, R], or null: lattice
  long long first;         // lattice: flat index of the first point
  int res;                 // lattice resolution per axis
  float radius;
  long long count;
  const float* w_in;       // [64][3C]
  const float* b_in;       // [64]
  const float* w_mid;      // [mid][64][64]
  const float* b_mid;      // [mid][64]
  int mid;
  const float* w_out;      // [4][64]
  const float* b_out;      // [4]
  float* out;              // [count][4]
};

__device__ __forceinline__ float tri_silu(float x) { return x / (1.f + __expf(-x)); }

// h_out[o] = silu(b[o] + sum_i w[o][i] * h_in[i]) for 64 x 64 weights in shared memory
__device__ __forceinline__ void tri_layer64(const float* __restrict__ w, const float* __restrict__ b, const float (&in)[kTriHidden],
                                            float (&out)[kTriHidden]) {
#pragma unroll
  for (int o = 0; o < kTriHidden; ++o) {
    float acc = b[o];
    const float4* wr = reinterpret_cast<const float4*>(w + o * kTriHidden);
#pragma unroll
    for (int i4 = 0; i4 < kTriHidden / 4; ++i4) {
      const float4 ww = wr[i4];
      acc = fmaf(ww.x, in[4 * i4], acc);
      acc = fmaf(ww.y, in[4 * i4 + 1], acc);
      acc = fmaf(ww.z, in[4 * i4 + 2], acc);
      acc = fmaf(ww.w, in[4 * i4 + 3], acc);
    }
    out[o] = tri_silu(acc);
  }
}

__global__ void __launch_bounds__(kTriThreads) triplane_nerf_kernel(const TriplaneParams p) {
  extern __shared__ float smem[];
  const int feat = 3 * p.c;
  float* s_win = smem;                                   // [64][feat]
  float* s_bin = s_win + kTriHidden * feat;              // [64]
  float* s_wmid = s_bin + kTriHidden;                    // [mid][64][64]
  float* s_bmid = s_wmid + p.mid * kTriHidden * kTriHidden;
  float* s_wout = s_bmid + p.mid * kTriHidden;           // [4][64]
  float* s_bout = s_wout + 4 * kTriHidden;               // [4]
  for (int i = threadIdx.x; i < kTriHidden * feat; i += blockDim.x) s_win[i] = p.w_in[i];
  for (int i = threadIdx.x; i < kTriHidden; i += blockDim.x) s_bin[i] = p.b_in[i];
  for (int i = threadIdx.x; i < p.mid * kTriHidden * kTriHidden; i += blockDim.x) s_wmid[i] = p.w_mid[i];
  for (int i = threadIdx.x; i < p.mid * kTriHidden; i += blockDim.x) s_bmid[i] = p.b_mid[i];
  for (int i = threadIdx.x; i < 4 * kTriHidden; i += blockDim.x) s_wout[i] = p.w_out[i];
  if (threadIdx.x < 4) s_bout[threadIdx.x] = p.b_out[threadIdx.x];
  __syncthreads();

  const long long plane_elems = static_cast<long long>(p.h) * p.w;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < p.count;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    float pos[3];
    if (p.coords != nullptr) {
      pos[0] = p.coords[idx * 3]; pos[1] = p.coords[idx * 3 + 1]; pos[2] = p.coords[idx * 3 + 2];
    } else {
      const long long g = p.first + idx;
      const int iz = static_cast<int>(g % p.res), iy = static_cast<int>((g / p.res) % p.res);
      const int ix = static_cast<int>(g / (static_cast<long long>(p.res) * p.res));
      const float step = p.res > 1 ? 2.f * p.radius / (p.res - 1) : 0.f;
      pos[0] = -p.radius + ix * step; pos[1] = -p.radius + iy * step; pos[2] = -p.radius + iz * step;
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) pos[a] /= p.radius;

    // ---- first layer fused with the sampling: h[o] += w_in[o][plane * C + ch] * feature
    float h0[kTriHidden];
#pragma unroll
    for (int o = 0; o < kTriHidden; ++o) h0[o] = s_bin[o];
    for (int pl = 0; pl < 3; ++pl) {
      const float gx = pl == 2 ? pos[1] : pos[0];
      const float gy = pl == 0 ? pos[1] : pos[2];
      const float fx = ((gx + 1.f) * p.w - 1.f) * 0.5f, fy = ((gy + 1.f) * p.h - 1.f) * 0.5f;
      const float x0f = floorf(fx), y0f = floorf(fy);
      const int x0 = static_cast<int>(x0f), y0 = static_cast<int>(y0f);
      const float tx = fx - x0f, ty = fy - y0f;
      const bool vx0 = x0 >= 0 && x0 < p.w, vx1 = x0 + 1 >= 0 && x0 + 1 < p.w;
      const bool vy0 = y0 >= 0 && y0 < p.h, vy1 = y0 + 1 >= 0 && y0 + 1 < p.h;
      const float w00 = (vx0 && vy0) ? (1.f - tx) * (1.f - ty) : 0.f, w01 = (vx1 && vy0) ? tx * (1.f - ty) : 0.f;
      const float w10 = (vx0 && vy1) ? (1.f - tx) * ty : 0.f, w11 = (vx1 && vy1) ? tx * ty : 0.f;
      const int cx0 = min(max(x0, 0), p.w - 1), cx1 = min(max(x0 + 1, 0), p.w - 1);
      const int cy0 = min(max(y0, 0), p.h - 1), cy1 = min(max(y0 + 1, 0), p.h - 1);
      const float* base = p.planes + static_cast<long long>(pl) * p.c * plane_elems;
      for (int ch = 0; ch < p.c; ++ch) {
        const float* pc = base + ch * plane_elems;
        const float f = w00 * __ldg(pc + cy0 * p.w + cx0) + w01 * __ldg(pc + cy0 * p.w + cx1) +
                        w10 * __ldg(pc + cy1 * p.w + cx0) + w11 * __ldg(pc + cy1 * p.w + cx1);
        const float* wc = s_win + pl * p.c + ch;
#pragma unroll
        for (int o = 0; o < kTriHidden; ++o) h0[o] = fmaf(wc[o * feat], f, h0[o]);
      }
    }
#pragma unroll
    for (int o = 0; o < kTriHidden; ++o) h0[o] = tri_silu(h0[o]);

    // ---- hidden layers, ping-pong between two register arrays
    float h1[kTriHidden];
    int l = 0;
    for (; l + 1 < p.mid; l += 2) {
      tri_layer64(s_wmid + l * kTriHidden * kTriHidden, s_bmid + l * kTriHidden, h0, h1);
      tri_layer64(s_wmid + (l + 1) * kTriHidden * kTriHidden, s_bmid + (l + 1) * kTriHidden, h1, h0);
    }
    if (l < p.mid) {
      tri_layer64(s_wmid + l * kTriHidden * kTriHidden, s_bmid + l * kTriHidden, h0, h1);
#pragma unroll
      for (int o = 0; o < kTriHidden; ++o) h0[o] = h1[o];
    }
    float4 res;
    float* rp = reinterpret_cast<float*>(&res);
#pragma unroll
    for (int o = 0; o < 4; ++o) {
      float acc = s_bout[o];
#pragma unroll
      for (int i = 0; i < kTriHidden; ++i) acc = fmaf(s_wout[o * kTriHidden + i], h0[i], acc);
      rp[o] = acc;
    }
    *reinterpret_cast<float4*>(p.out + idx * 4) = res;
  }
}

}  // namespace b200

using namespace b200;

// planes [3][C][H][W] fp32; coords [count][3] fp32 or null (lattice of `res` points per axis over
// [-radius, radius]^3 starting at flat index `first`); MLP weights fp32 row-major ([out][in]), hidden
// width 64; out [count][4] fp32.
B200_API int b200_triplane_nerf(const float* planes, int c, int h, int w, const float* coords, long long first, int res,
                                float radius, long long count, const float* w_in, const float* b_in, const float* w_mid,
                                const float* b_mid, int mid, const float* w_out, const float* b_out, float* out,
                                cudaStream_t stream) {
  if (count <= 0) return 0;
  if (c <= 0 || h <= 0 || w <= 0 || mid < 0 || radius <= 0.f || (coords == nullptr && res < 1)) return -2;
  const size_t smem = (static_cast<size_t>(kTriHidden) * 3 * c + kTriHidden + static_cast<size_t>(mid) * kTriHidden * (kTriHidden + 1) +
                       4 * kTriHidden + 4) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  static PerDeviceOnce configured;
  if (configured.first_time() &&
      cudaFuncSetAttribute(triplane_nerf_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
    return -4;
  TriplaneParams p{};
  p.planes = planes; p.c = c; p.h = h; p.w = w; p.coords = coords; p.first = first; p.res = res; p.radius = radius;
  p.count = count; p.w_in = w_in; p.b_in = b_in; p.w_mid = w_mid; p.b_mid = b_mid; p.mid = mid; p.w_out = w_out;
  p.b_out = b_out; p.out = out;
  long long blocks = (count + kTriThreads - 1) / kTriThreads;
  const long long cap = 148ll * 8;
  if (blocks > cap) blocks = cap;
  triplane_nerf_kernel<<<static_cast<unsigned>(blocks), kTriThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
