// Selective scan of Mamba-style state-space layers.
//   h_t = exp(dt_t * A) .* h_{t-1} + (dt_t * x_t) * B_t        (h: [channels][N])
//   y_t = <h_t, C_t> + D * x_t
// One thread owns one channel: its N (<= 32) state values stay in registers for the whole token
// run, B_t and C_t (shared by all channels) are staged through shared memory per block of tokens.
// The recurrence is sequential in t by definition; parallelism comes from channels x sequences.
// Decode runs with T = 1. The state is fp32 and updated in place.
//
// Reference: the scan of src/HartsyInference.LLM/Ssm/ (CPU loop / per-op GPU kernels).
#include "common.cuh"

namespace b200 {

constexpr int kScanMaxState = 32;
constexpr int kScanTokenBlock = 32;

struct ScanParams {
  const __nv_bfloat16* x;    // [T][Di]
  const float* dt;           // [T][Di] (after softplus)
  const float* a;            // [Di][N]  (negative)
  const __nv_bfloat16* b;    // [T][N]
  const __nv_bfloat16* c;    // [T][N]
  const float* d;            // [Di]
  float* state;              // [Di][N]
  __nv_bfloat16* y;          // [T][Di]
  int tokens, channels, n;
};

__global__ void __launch_bounds__(128) selective_scan_kernel(const ScanParams p) {
  __shared__ float sb[kScanTokenBlock][kScanMaxState];
  __shared__ float sc[kScanTokenBlock][kScanMaxState];
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = ch < p.channels;
  float h[kScanMaxState], a[kScanMaxState];
#pragma unroll
  for (int i = 0; i < kScanMaxState; ++i) {
    const bool on = active && i < p.n;
    h[i] = on ? p.state[static_cast<long long>(ch) * p.n + i] : 0.f;
    a[i] = on ? p.a[static_cast<long long>(ch) * p.n + i] : 0.f;
  }
  const float dskip = active ? p.d[ch] : 0.f;
  for (int t0 = 0; t0 < p.tokens; t0 += kScanTokenBlock) {
    const int nt = min(kScanTokenBlock, p.tokens - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * p.n; i += blockDim.x) {
      const int tt = i / p.n, j = i - tt * p.n;
      sb[tt][j] = __bfloat162float(p.b[static_cast<long long>(t0 + tt) * p.n + j]);
      sc[tt][j] = __bfloat162float(p.c[static_cast<long long>(t0 + tt) * p.n + j]);
    }
    __syncthreads();
    if (!active) continue;
    for (int tt = 0; tt < nt; ++tt) {
      const long long at = static_cast<long long>(t0 + tt) * p.channels + ch;
      const float xv = __bfloat162float(p.x[at]);
      const float dtv = p.dt[at];
      const float dx = dtv * xv;
      float acc = dskip * xv;
#pragma unroll
      for (int i = 0; i < kScanMaxState; ++i) {
        if (i < p.n) {
          h[i] = fmaf(__expf(dtv * a[i]), h[i], dx * sb[tt][i]);
          acc = fmaf(h[i], sc[tt][i], acc);
        }
      }
      p.y[at] = __float2bfloat16(acc);
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < kScanMaxState; ++i)
      if (i < p.n) p.state[static_cast<long long>(ch) * p.n + i] = h[i];
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_selective_scan(const void* x, const float* dt, const float* a, const void* b, const void* c,
                                 const float* d, float* state, void* y, int tokens, int channels, int n,
                                 cudaStream_t stream) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (n < 1 || n > kScanMaxState) return -2;
  ScanParams p{static_cast<const __nv_bfloat16*>(x), dt, a, static_cast<const __nv_bfloat16*>(b),
               static_cast<const __nv_bfloat16*>(c), d, state, static_cast<__nv_bfloat16*>(y), tokens, channels, n};
  selective_scan_kernel<<<(channels + 127) / 128, 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
