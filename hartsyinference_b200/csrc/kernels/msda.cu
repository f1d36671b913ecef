// Multi-scale deformable attention (Deformable DETR / RT-DETR / Grounding DINO decoders), one kernel
// for what the module does between its linear layers:
//
//   weights  = softmax over the L x P sampling points of a (query, head)
//   location = reference point (+ offset / P x box size / 2 for 4-d references, + offset / level
//              size for 2-d references)
//   out[q, head, :] = sum over points of weight x bilinear sample of the level's value map
//
// One warp per (batch, query, head). The first L x P lanes each own one sampling point (softmax
// across them by shuffles, location and corner arithmetic once per point); then the warp walks the
// points and every lane gathers ITS channels of the four corners, so each corner read is one
// coalesced row of the value tensor [B][S][heads][D]. Zero padding outside the map, pixel centres at
// half-integers (grid_sample with align_corners = False).
//
// Reference counterpart: src/HartsyInference.Cuda/Kernels/vision/msda.cu (one thread per output
// channel, weights and locations prepared by separate kernels).
#include "common.cuh"

namespace b200 {

struct MsdaParams {
  const void* value;          // [B][S][heads][D] bf16 or fp32
  const float* offsets;       // [B][Q][heads][L][P][2]
  const float* logits;        // [B][Q][heads][L][P]
  const float* ref;           // [B][Q][ref_dim] (ref_dim 4: cx, cy, w, h; 2: x, y; one reference for all levels)
                              // or [B][Q][L][ref_dim] when ref_per_level
  const int* shapes;          // [L][2] height, width
  const int* starts;          // [L] first row of each level in S
  void* out;                  // [B][Q][heads * D], dtype of value
  int batch, rows, queries, heads, dim, levels, points, ref_dim, ref_per_level;
};

template <typename T>
__device__ __forceinline__ float msda_load(const T* p);
template <>
__device__ __forceinline__ float msda_load<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float msda_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void msda_store(T* p, float v);
template <>
__device__ __forceinline__ void msda_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void msda_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(256) msda_kernel(const MsdaParams p) {
  const int lane = threadIdx.x & 31;
  const long long unit = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);   // (b, q, head)
  const long long units = static_cast<long long>(p.batch) * p.queries * p.heads;
  if (unit >= units) return;
  const int head = static_cast<int>(unit % p.heads);
  const long long bq = unit / p.heads;
  const int b = static_cast<int>(bq / p.queries);
  const int np = p.levels * p.points;

  // ---- this lane's sampling point: softmax weight, pixel coordinates, level
  float w = 0.f, px = 0.f, py = 0.f;
  int lh = 1, lw = 1, ls = 0;
  const bool mine = lane < np;
  float logit = -INFINITY;
  if (mine) {
    const int level = lane / p.points;
    logit = p.logits[unit * np + lane];
    lh = p.shapes[2 * level];
    lw = p.shapes[2 * level + 1];
    ls = p.starts[level];
    const float ox = p.offsets[(unit * np + lane) * 2], oy = p.offsets[(unit * np + lane) * 2 + 1];
    const float* r = p.ref + (p.ref_per_level ? (bq * p.levels + level) : bq) * p.ref_dim;
    float x, y;
    if (p.ref_dim == 4) {
      x = r[0] + ox / p.points * r[2] * 0.5f;
      y = r[1] + oy / p.points * r[3] * 0.5f;
    } else {
      x = r[0] + ox / lw;
      y = r[1] + oy / lh;
    }
    px = x * lw - 0.5f;
    py = y * lh - 0.5f;
  }
  const float mx = warp_max(logit);
  const float e = mine ? __expf(logit - mx) : 0.f;
  const float sum = warp_sum(e);
  w = e / sum;

  // ---- gather: every lane accumulates its channels
  const T* value = static_cast<const T*>(p.value) + static_cast<long long>(b) * p.rows * p.heads * p.dim + head * p.dim;
  const long long row_stride = static_cast<long long>(p.heads) * p.dim;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};      // channels lane, lane + 32, lane + 64, lane + 96
  for (int i = 0; i < np; ++i) {
    const float wi = __shfl_sync(0xffffffffu, w, i);
    const float xi = __shfl_sync(0xffffffffu, px, i), yi = __shfl_sync(0xffffffffu, py, i);
    const int hi = __shfl_sync(0xffffffffu, lh, i), wd = __shfl_sync(0xffffffffu, lw, i);
    const int si = __shfl_sync(0xffffffffu, ls, i);
    const float fx = floorf(xi), fy = floorf(yi);
    const int x0 = static_cast<int>(fx), y0 = static_cast<int>(fy);
    const float ax = xi - fx, ay = yi - fy;
    if (x0 < -1 || y0 < -1 || x0 >= wd || y0 >= hi) continue;     // all four corners outside (uniform per warp)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int yy = y0 + (c >> 1), xx = x0 + (c & 1);
      if (yy < 0 || yy >= hi || xx < 0 || xx >= wd) continue;
      const float cw = wi * ((c & 1) ? ax : 1.f - ax) * ((c >> 1) ? ay : 1.f - ay);
      const T* src = value + (static_cast<long long>(si) + static_cast<long long>(yy) * wd + xx) * row_stride;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int ch = lane + 32 * k;
        if (ch < p.dim) acc[k] += cw * msda_load<T>(src + ch);
      }
    }
  }
  T* out = static_cast<T*>(p.out) + unit * p.dim;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int ch = lane + 32 * k;
    if (ch < p.dim) msda_store<T>(out + ch, acc[k]);
  }
}

}  // namespace b200

using namespace b200;

// value / out: bf16 (value_bf16 = 1) or fp32; offsets, logits, ref: fp32. At most 32 sampling points
// per (query, head) and 128 channels per head.
B200_API int b200_msda(const void* value, int value_bf16, const float* offsets, const float* logits, const float* ref,
                       int ref_dim, int ref_per_level, const int* shapes, const int* starts, void* out, int batch, int rows,
                       int queries, int heads, int dim, int levels, int points, cudaStream_t stream) {
  if (batch <= 0 || queries <= 0) return 0;
  if (levels * points > 32 || levels * points <= 0 || dim > 128 || dim <= 0 || (ref_dim != 2 && ref_dim != 4)) return -2;
  MsdaParams p{value, offsets, logits, ref, shapes, starts, out, batch, rows, queries, heads, dim, levels, points, ref_dim,
               ref_per_level};
  const long long units = static_cast<long long>(batch) * queries * heads;
  const unsigned grid = static_cast<unsigned>((units + 7) / 8);
  if (value_bf16) msda_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else msda_kernel<float><<<grid, 256, 0, stream>>>(p);
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));
}
