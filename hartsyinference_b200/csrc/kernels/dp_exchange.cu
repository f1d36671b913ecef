// Token exchange of the data-parallel-attention / expert-parallel decode layout (DeepSeek-V3 style
// MLA + MoE models): every rank runs the attention of its own L = T / W requests with all heads, the
// expert layer runs over all T rows on every rank with that rank's experts, and the two collectives
// in between are done by the kernels that produce and consume the data, over peer memory:
//
//   dp_norm_gather      residual add + RMSNorm of the L local rows, stored into EVERY rank's
//                       gathered-activation buffer [T][H] (peer stores), together with the latent-cache
//                       row each local request wrote in this layer (so that every rank's cache stays
//                       complete and any rank can serve any request in a later step);
//   dp_gather_wait      waits (bounded) for the W sources and writes the other ranks' latent rows into
//                       the local cache; the expert layer's kernels follow in stream order;
//   dp_combine_scatter  the expert combine (sum_k w[t][k] * y[slot(t, k)] + shared-expert / dense
//                       partial) stored straight into the slot [source][row] of the rank that owns
//                       the token: the "reduce-scatter" is W stores of L rows per rank;
//   dp_reduce_norm      waits for the W sources, sums the W slots of each local row in fixed order
//                       into the residual stream and applies the next RMSNorm.
//
// Flags are cumulative counters in the symmetric heap (one call adds one), call numbers live in
// device memory, so the kernels are CUDA-graph capturable and nothing is reset between calls. A rank
// writes a peer's gather buffer for call c + 1 only after that peer's dp_reduce_norm of call c, which
// needs this rank's scatter of call c, which follows this rank's last read of its gather buffer of
// call c in stream order; the same argument with the roles swapped covers the scatter slots. Every
// wait is bounded and reports into the status word.
//
// Reference counterpart: src/HartsyInference.LLM/Transformer/MoeFeedForward.cs:88-161 (host routing
// with a device-to-host copy per layer, per-expert gather / GEMM / scatter-add on one device).
#include "comm.cuh"

namespace b200 {

constexpr int kDpLatRow = 576;                       // latent 512 + rotary 64
constexpr int kDpFlagGather = 0, kDpFlagScatter = 8; // per rank: arrivals from source s
// local counters: [0] gather calls completed, [1] CTAs of dp_norm_gather done, [2] CTAs of
// dp_gather_wait finished, [4] scatter calls completed, [5] CTAs of dp_combine_scatter done,
// [6] CTAs of dp_reduce_norm finished
constexpr int kDpMaxVec = 4;                         // 16-byte vectors per thread: hidden <= 256 * 4 * 8

struct DpGatherArgs {
  const __nv_bfloat16* a;        // [L][H] output of the attention block (may be null: res is used as it is)
  __nv_bfloat16* res;            // [L][H] residual stream, updated in place
  const __nv_bfloat16* norm_w;   // [H]
  const __nv_bfloat16* cache;    // this layer's latent cache [slots][576] (may be null)
  const long long* slots;        // [L] cache slot of each local row (< 0: none)
  __nv_bfloat16* g[8];           // rank d's gathered activations [T][H]
  __nv_bfloat16* gl[8];          // rank d's gathered latent rows [T][576]
  uint32_t* flags[8];
  uint32_t* ctr;
  int rows, hidden, rank, world;
  float eps;
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) ow[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  return o;
}

// Sum over the block of one float per thread (256 threads).
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += red[i];
  __syncthreads();
  return s;
}

// The last CTA of a launch adds one to word `which + rank` of every rank's flags. The barrier orders
// every thread's peer stores before thread 0, whose system-scope fence then covers them all.
__device__ __forceinline__ void dp_arrive(uint32_t* ctr_done, uint32_t* const* flags, int which, int rank, int world) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(ctr_done, 1u) == gridDim.x - 1) {
      atomicExch(ctr_done, 0u);
      fence_acq_rel_sys();
      for (int i = 0; i < world; ++i) {
        const int d = (rank + i) % world;
        red_relaxed_sys_add(flags[d] + which + rank, 1u);
      }
    }
  }
}

// grid = local rows, 256 threads
__global__ void __launch_bounds__(256) dp_norm_gather_kernel(const DpGatherArgs p) {
  __shared__ float red[8];
  const int r = blockIdx.x, tid = threadIdx.x;
  const int vecs = p.hidden / 8;
  const long long grow = static_cast<long long>(p.rank) * p.rows + r;
  float v[kDpMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kDpMaxVec; ++i) {
    const int c = tid + i * 256;
    if (c < vecs) {
      const long long at = static_cast<long long>(r) * p.hidden + c * 8;
      unpack8(*reinterpret_cast<const uint4*>(p.res + at), v[i]);
      if (p.a != nullptr) {
        float a[8];
        unpack8(*reinterpret_cast<const uint4*>(p.a + at), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += a[j];
        // the stream is kept in bf16: normalise what is stored
        const uint4 o = pack8(v[i]);
        *reinterpret_cast<uint4*>(p.res + at) = o;
        unpack8(o, v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float inv = rsqrtf(block_sum_256(ss, red) / p.hidden + p.eps);
#pragma unroll
  for (int i = 0; i < kDpMaxVec; ++i) {
    const int c = tid + i * 256;
    if (c < vecs) {
      float w[8];
      unpack8(*reinterpret_cast<const uint4*>(p.norm_w + c * 8), w);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= inv * w[j];
      const uint4 o = pack8(v[i]);
      for (int k = 0; k < p.world; ++k) {
        const int d = (p.rank + k) % p.world;       // own copy first, then the neighbours in turn
        *reinterpret_cast<uint4*>(p.g[d] + grow * p.hidden + c * 8) = o;
      }
    }
  }
  if (p.cache != nullptr && tid < kDpLatRow / 8) {
    const long long slot = p.slots[r];
    if (slot >= 0) {
      const uint4 o = *reinterpret_cast<const uint4*>(p.cache + slot * kDpLatRow + tid * 8);
      for (int k = 0; k < p.world; ++k) {
        const int d = (p.rank + k) % p.world;
        *reinterpret_cast<uint4*>(p.gl[d] + grow * kDpLatRow + tid * 8) = o;
      }
    }
  }
  dp_arrive(p.ctr + 1, p.flags, kDpFlagGather, p.rank, p.world);
}

struct DpWaitArgs {
  const __nv_bfloat16* gl;       // local gathered latent rows [T][576]
  __nv_bfloat16* cache;          // may be null
  const long long* slots;        // [T] cache slot of every row (< 0: none)
  const uint32_t* flags_local;
  uint32_t* ctr;
  int rows_total, rows_local, rank;
  long long wait_budget;
  DeviceStatus* status;
};

// grid = all rows, 96 threads. Row t came from rank t / L.
__global__ void __launch_bounds__(96) dp_gather_wait_kernel(const DpWaitArgs p) {
  __shared__ int s_ok;
  const int t = blockIdx.x, tid = threadIdx.x;
  const int src = t / p.rows_local;
  uint32_t call = 0;
  if (tid == 0) {
    call = *reinterpret_cast<volatile uint32_t*>(p.ctr) + 1u;
    s_ok = wait_flag_geq(p.flags_local + kDpFlagGather + src, call, p.wait_budget) ? 1 : 0;
    if (!s_ok) report_status(p.status, kWaitTimeout, kKernelDpExchange, 1, static_cast<uint32_t>(src));
  }
  __syncthreads();
  if (s_ok && src != p.rank && p.cache != nullptr && tid < kDpLatRow / 8) {
    const long long slot = p.slots[t];
    if (slot >= 0)     // the row arrived as a peer's stores after this SM may have cached the line: read past L1
      *reinterpret_cast<uint4*>(p.cache + slot * kDpLatRow + tid * 8) =
          ld_relaxed_sys_v4(p.gl + static_cast<long long>(t) * kDpLatRow + tid * 8);
  }
  if (tid == 0) {
    // the last block to finish closes the call: every block has read the call counter by now
    __threadfence();
    if (atomicAdd(p.ctr + 2, 1u) == gridDim.x - 1) {
      p.ctr[2] = 0;
      *reinterpret_cast<volatile uint32_t*>(p.ctr) = call;
      __threadfence();
    }
  }
}

struct DpScatterArgs {
  const __nv_bfloat16* y;        // expert outputs by slot (may be null when top_k == 0)
  const int* slot_of;            // [T][top_k], < 0: the expert lives on another rank
  const float* topk_w;           // [T][top_k]
  const __nv_bfloat16* shared;   // [T][dim] partial sum to start from (shared expert / dense block), may be null
  __nv_bfloat16* slots[8];       // rank d's slots [W][L][dim]
  uint32_t* flags[8];
  uint32_t* ctr;
  int top_k, dim, rows_local, rank, world;
};

// grid = all rows, 128 threads
__global__ void __launch_bounds__(128) dp_combine_scatter_kernel(const DpScatterArgs p) {
  const int t = blockIdx.x;
  const int d = t / p.rows_local, lr = t - d * p.rows_local;
  __nv_bfloat16* dst = p.slots[d] + (static_cast<long long>(p.rank) * p.rows_local + lr) * p.dim;
  for (int c = threadIdx.x * 8; c < p.dim; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (p.shared != nullptr) unpack8(*reinterpret_cast<const uint4*>(p.shared + static_cast<long long>(t) * p.dim + c), acc);
    for (int k = 0; k < p.top_k; ++k) {
      const int slot = p.slot_of[t * p.top_k + k];
      if (slot < 0) continue;
      const float w = p.topk_w[t * p.top_k + k];
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.y + static_cast<long long>(slot) * p.dim + c), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * f[i];
    }
    *reinterpret_cast<uint4*>(dst + c) = pack8(acc);
  }
  dp_arrive(p.ctr + 5, p.flags, kDpFlagScatter, p.rank, p.world);
}

struct DpReduceArgs {
  const __nv_bfloat16* slots;    // local [W][L][H]
  __nv_bfloat16* res;            // [L][H] residual stream, updated in place
  const __nv_bfloat16* norm_w;   // [H]
  __nv_bfloat16* h;              // [L][H] normalised output
  const uint32_t* flags_local;
  uint32_t* ctr;
  int rows, hidden, world;
  float eps;
  long long wait_budget;
  DeviceStatus* status;
};

// grid = local rows, 256 threads
__global__ void __launch_bounds__(256) dp_reduce_norm_kernel(const DpReduceArgs p) {
  __shared__ float red[8];
  __shared__ int s_ok;
  const int r = blockIdx.x, tid = threadIdx.x;
  const int vecs = p.hidden / 8;
  uint32_t call = 0;
  if (tid == 0) {
    call = *reinterpret_cast<volatile uint32_t*>(p.ctr + 4) + 1u;
    int ok = 1;
    for (int s = 0; s < p.world && ok; ++s) {
      ok = wait_flag_geq(p.flags_local + kDpFlagScatter + s, call, p.wait_budget) ? 1 : 0;
      if (!ok) report_status(p.status, kWaitTimeout, kKernelDpExchange, 2, static_cast<uint32_t>(s));
    }
    s_ok = ok;
  }
  __syncthreads();
  float v[kDpMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kDpMaxVec; ++i) {
    const int c = tid + i * 256;
    if (c < vecs) {
      const long long at = static_cast<long long>(r) * p.hidden + c * 8;
      unpack8(*reinterpret_cast<const uint4*>(p.res + at), v[i]);
      if (s_ok) {
        for (int s = 0; s < p.world; ++s) {       // fixed order: the result does not depend on arrival order
          float f[8];
          unpack8(ld_relaxed_sys_v4(p.slots + (static_cast<long long>(s) * p.rows + r) * p.hidden + c * 8), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += f[j];
        }
      }
      const uint4 o = pack8(v[i]);
      *reinterpret_cast<uint4*>(p.res + at) = o;
      unpack8(o, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float inv = rsqrtf(block_sum_256(ss, red) / p.hidden + p.eps);
#pragma unroll
  for (int i = 0; i < kDpMaxVec; ++i) {
    const int c = tid + i * 256;
    if (c < vecs) {
      float w[8];
      unpack8(*reinterpret_cast<const uint4*>(p.norm_w + c * 8), w);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= inv * w[j];
      *reinterpret_cast<uint4*>(p.h + static_cast<long long>(r) * p.hidden + c * 8) = pack8(v[i]);
    }
  }
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.ctr + 6, 1u) == gridDim.x - 1) {
      p.ctr[6] = 0;
      *reinterpret_cast<volatile uint32_t*>(p.ctr + 4) = call;
      __threadfence();
    }
  }
}

}  // namespace b200

using namespace b200;

static int dp_last_error() {
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));
}

// Pointer tables have `world` entries (index = rank) into the symmetric heap. `flags`: 16 u32 per
// rank, `ctr`: 8 local u32, all zeroed once. hidden: a multiple of 8, at most 8192.
B200_API int b200_dp_norm_gather(const void* a, void* res, const void* norm_w, const void* cache, const long long* slots,
                                 void* const* g, void* const* gl, void* const* flags, void* ctr, int rows, int hidden,
                                 int rank, int world, float eps, cudaStream_t stream) {
  if (world < 1 || world > 8 || rows <= 0 || hidden % 8 || hidden > 256 * kDpMaxVec * 8) return -2;
  DpGatherArgs p{};
  p.a = static_cast<const __nv_bfloat16*>(a);
  p.res = static_cast<__nv_bfloat16*>(res);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.slots = slots;
  for (int d = 0; d < world; ++d) {
    p.g[d] = static_cast<__nv_bfloat16*>(g[d]);
    p.gl[d] = static_cast<__nv_bfloat16*>(gl[d]);
    p.flags[d] = static_cast<uint32_t*>(flags[d]);
  }
  p.ctr = static_cast<uint32_t*>(ctr);
  p.rows = rows; p.hidden = hidden; p.rank = rank; p.world = world; p.eps = eps;
  dp_norm_gather_kernel<<<rows, 256, 0, stream>>>(p);
  return dp_last_error();
}

B200_API int b200_dp_gather_wait(const void* gl_local, void* cache, const long long* slots_all, const void* flags_local,
                                 void* ctr, int rows_total, int rows_local, int rank, long long wait_budget_cycles,
                                 void* status, cudaStream_t stream) {
  if (rows_total <= 0 || rows_local <= 0 || rows_total % rows_local) return -2;
  DpWaitArgs p{};
  p.gl = static_cast<const __nv_bfloat16*>(gl_local);
  p.cache = static_cast<__nv_bfloat16*>(cache);
  p.slots = slots_all;
  p.flags_local = static_cast<const uint32_t*>(flags_local);
  p.ctr = static_cast<uint32_t*>(ctr);
  p.rows_total = rows_total; p.rows_local = rows_local; p.rank = rank;
  p.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  p.status = static_cast<DeviceStatus*>(status);
  dp_gather_wait_kernel<<<rows_total, 96, 0, stream>>>(p);
  return dp_last_error();
}

B200_API int b200_dp_combine_scatter(const void* y, const int* slot_of, const float* topk_w, const void* shared, int top_k,
                                     int dim, void* const* slots, void* const* flags, void* ctr, int rows_total,
                                     int rows_local, int rank, int world, cudaStream_t stream) {
  if (world < 1 || world > 8 || rows_total != rows_local * world || dim % 8) return -2;
  if (top_k > 0 && (y == nullptr || slot_of == nullptr || topk_w == nullptr)) return -3;
  DpScatterArgs p{};
  p.y = static_cast<const __nv_bfloat16*>(y);
  p.slot_of = slot_of;
  p.topk_w = topk_w;
  p.shared = static_cast<const __nv_bfloat16*>(shared);
  for (int d = 0; d < world; ++d) {
    p.slots[d] = static_cast<__nv_bfloat16*>(slots[d]);
    p.flags[d] = static_cast<uint32_t*>(flags[d]);
  }
  p.ctr = static_cast<uint32_t*>(ctr);
  p.top_k = top_k; p.dim = dim; p.rows_local = rows_local; p.rank = rank; p.world = world;
  dp_combine_scatter_kernel<<<rows_total, 128, 0, stream>>>(p);
  return dp_last_error();
}

B200_API int b200_dp_reduce_norm(const void* slots_local, void* res, const void* norm_w, void* h, const void* flags_local,
                                 void* ctr, int rows, int hidden, int world, float eps, long long wait_budget_cycles,
                                 void* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || rows <= 0 || hidden % 8 || hidden > 256 * kDpMaxVec * 8) return -2;
  DpReduceArgs p{};
  p.slots = static_cast<const __nv_bfloat16*>(slots_local);
  p.res = static_cast<__nv_bfloat16*>(res);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  p.h = static_cast<__nv_bfloat16*>(h);
  p.flags_local = static_cast<const uint32_t*>(flags_local);
  p.ctr = static_cast<uint32_t*>(ctr);
  p.rows = rows; p.hidden = hidden; p.world = world; p.eps = eps;
  p.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  p.status = static_cast<DeviceStatus*>(status);
  dp_reduce_norm_kernel<<<rows, 256, 0, stream>>>(p);
  return dp_last_error();
}
