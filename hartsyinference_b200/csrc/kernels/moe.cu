// Mixture-of-experts routing, dispatch and combine on the device (no host round trip).
//
//  * moe_route:    scores = softmax or sigmoid of the router logits; plain top-k, or DeepSeek-V3
//                  group-limited selection (selection score = sigmoid + per-expert bias, group
//                  score = sum of its two best, keep the best `topk_group` groups, top-k inside
//                  them; the mixing weight is the raw sigmoid, renormalised with +1e-20, times
//                  the routed scaling factor). Ties resolve to the lowest expert index.
//  * moe_dispatch: for the experts [e0, e0 + e_local) owned by this rank, give every (token, k)
//                  pair a slot in its expert's fixed-capacity block and copy the token row there.
//                  Slots that get no token keep whatever they held: GEMM rows are independent and
//                  the combine step reads assigned slots only.
//  * moe_combine:  out[t] = sum_k w[t][k] * y[slot(t, k)] in fixed k order (deterministic).
//
// Replaces the reference's host-side router with one D2H copy per MoE layer
// (src/HartsyInference.LLM/Transformer/MoeFeedForward.cs: Route:186-233, RouteGroupLimited:240-312,
// Forward:88-161 gather / GEMM / scatter-add per expert) and lm_scatter_add_weighted_rows_f32:152,
// dit_moe_topk_gate_f32:924.
#include "common.cuh"

namespace b200 {

constexpr int kMaxExpertsPerLane = 16;   // up to 512 experts, one warp per token

struct RouteParams {
  const void* logits;       // [T][E] fp32, or bf16 when logits_bf16 is set
  int logits_bf16;
  const float* bias;        // [E] selection bias (may be null)
  int* topk_ids;            // [T][k]
  float* topk_w;            // [T][k]
  int tokens, experts, top_k, n_group, topk_group;
  int sigmoid;              // 1 = sigmoid scoring, 0 = softmax
  int norm_topk;            // renormalise the selected weights
  float scale;              // routed scaling factor
};

__global__ void moe_route_kernel(const RouteParams p) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= p.tokens) return;
  const int per = (p.experts + 31) / 32;
  float score[kMaxExpertsPerLane], sel[kMaxExpertsPerLane];
  // expert e lives in lane e % 32, slot e / 32
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = lane + 32 * i;
    const long long at = static_cast<long long>(t) * p.experts + e;
    score[i] = e >= p.experts ? -INFINITY
               : p.logits_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.logits)[at])
                               : static_cast<const float*>(p.logits)[at];
    mx = fmaxf(mx, score[i]);
  }
  if (p.sigmoid) {
    for (int i = 0; i < per; ++i) score[i] = (lane + 32 * i) < p.experts ? 1.f / (1.f + __expf(-score[i])) : -INFINITY;
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = 0; i < per; ++i) {
      score[i] = (lane + 32 * i) < p.experts ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
    for (int i = 0; i < per; ++i) score[i] = (lane + 32 * i) < p.experts ? score[i] / sum : -INFINITY;
  }
  for (int i = 0; i < per; ++i) {
    const int e = lane + 32 * i;
    sel[i] = e < p.experts ? score[i] + (p.bias ? p.bias[e] : 0.f) : -INFINITY;
  }
  // group-limited masking
  if (p.n_group > 1 && p.topk_group < p.n_group) {
    const int gsize = p.experts / p.n_group;
    // group score = sum of the two best selection scores of the group; computed by letting lane g
    // own group g (n_group <= 32)
    float gscore = -INFINITY;
    for (int g = 0; g < p.n_group; ++g) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int i = 0; i < per; ++i) {
        const int e = lane + 32 * i;
        if (e < p.experts && e / gsize == g) {
          if (sel[i] > b1) { b2 = b1; b1 = sel[i]; } else if (sel[i] > b2) b2 = sel[i];
        }
      }
      // merge the per-lane top-2 across the warp
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      if (lane == g) gscore = b1 + (b2 == -INFINITY ? 0.f : b2);
    }
    // keep the best topk_group groups (ties -> lowest group index)
    uint32_t keep = 0;
    for (int r = 0; r < p.topk_group; ++r) {
      float v = (keep >> lane) & 1 ? -INFINITY : gscore;
      int idx = lane;
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      keep |= 1u << idx;
    }
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      if (e < p.experts && !((keep >> (e / gsize)) & 1)) sel[i] = -INFINITY;
    }
  }
  // iterative top-k over the selection scores
  float wsum = 0.f;
  float my_w = 0.f;   // lane r keeps the r-th weight (top_k <= 32)
  int my_id = 0;
  for (int r = 0; r < p.top_k; ++r) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    float raw = 0.f;
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      if (e < p.experts && (sel[i] > v || (sel[i] == v && e < idx))) { v = sel[i]; idx = e; raw = score[i]; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      const float orw = __shfl_xor_sync(0xffffffffu, raw, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; raw = orw; }
    }
    if ((idx & 31) == lane) sel[idx >> 5] = -INFINITY;   // remove from further rounds
    if (lane == r) { my_w = raw; my_id = idx; }
    wsum += raw;
  }
  if (lane < p.top_k) {
    float w = my_w;
    if (p.norm_topk) w = w / (wsum + 1e-20f);
    p.topk_ids[static_cast<long long>(t) * p.top_k + lane] = my_id;
    p.topk_w[static_cast<long long>(t) * p.top_k + lane] = w * p.scale;
  }
}

// counts[e_local] must be zero on entry. slot_of[t][k] = e_local * capacity + position, or -1 when
// the expert is not local or its block is full.
// Tokens are taken in chunks of `chunk_tokens`: expert e keeps one block of `capacity` slots per
// chunk (block index e * chunks + c), so a block can never overflow when capacity >= chunk_tokens.
__global__ void moe_assign_kernel(const int* __restrict__ topk_ids, int* __restrict__ slot_of,
                                  int* __restrict__ counts, int pairs, int top_k, int e0, int e_local,
                                  int capacity, int chunks, int chunk_tokens) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = topk_ids[i] - e0;
  int slot = -1;
  if (e >= 0 && e < e_local) {
    const int blk = e * chunks + (i / top_k) / chunk_tokens;
    const int pos = atomicAdd(counts + blk, 1);
    if (pos < capacity) slot = blk * capacity + pos;
  }
  slot_of[i] = slot;
}

// ---- variable-size dispatch: experts get as many blocks of `cap` slots as their token count needs
// pass 1: position of every (token, k) pair inside its expert
__global__ void moe_count_kernel(const int* __restrict__ topk_ids, int* __restrict__ pos_of, int* __restrict__ counts,
                                 int pairs, int e0, int e_local) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = topk_ids[i] - e0;
  pos_of[i] = (e >= 0 && e < e_local) ? atomicAdd(counts + e, 1) : -1;
}
// pass 2 (one block): block_start[e] = sum of ceil(count / cap) over earlier experts; block list
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ block_start,
                                int* __restrict__ block_group, int* __restrict__ dyn_blocks, int e_local, int cap,
                                int max_blocks) {
  __shared__ int s_start[1025];
  const int tid = threadIdx.x;
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      s_start[e] = acc;
      acc += (counts[e] + cap - 1) / cap;
    }
    s_start[e_local] = acc;
    *dyn_blocks = acc < max_blocks ? acc : max_blocks;
  }
  __syncthreads();
  for (int e = tid; e < e_local; e += blockDim.x) {
    block_start[e] = s_start[e];
    for (int b = s_start[e]; b < s_start[e + 1] && b < max_blocks; ++b) block_group[b] = e;
  }
}
// pass 3: copy rows into their slots
__global__ void moe_scatter_dynamic_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xs,
                                           const int* __restrict__ topk_ids, const int* __restrict__ pos_of,
                                           const int* __restrict__ block_start, int* __restrict__ slot_of,
                                           int top_k, int dim, int e0, int cap, int max_blocks) {
  const int pair = blockIdx.x;
  const int pos = pos_of[pair];
  int slot = -1;
  if (pos >= 0) {
    const int blk = block_start[topk_ids[pair] - e0] + pos / cap;
    if (blk < max_blocks) slot = blk * cap + pos % cap;
  }
  if (threadIdx.x == 0) slot_of[pair] = slot;
  if (slot < 0) return;
  const int t = pair / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * dim);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<long long>(slot) * dim);
  for (int i = threadIdx.x; i < (dim >> 3); i += blockDim.x) dst[i] = src[i];
}

// Copies token rows into their slots (bf16 rows of `dim`, 16-byte vectors). One block per pair.
__global__ void moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xs,
                                   const int* __restrict__ slot_of, int top_k, int dim) {
  const int pair = blockIdx.x;
  const int slot = slot_of[pair];
  if (slot < 0) return;
  const int t = pair / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * dim);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<long long>(slot) * dim);
  for (int i = threadIdx.x; i < (dim >> 3); i += blockDim.x) dst[i] = src[i];
}

// out[t] (+)= sum_k w[t][k] * y[slot_of[t][k]]; `accumulate` adds to what is already in out (shared
// expert, other ranks' partial sums). One block per token.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_of,
                                   const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ out,
                                   int top_k, int dim, int accumulate) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (accumulate) {
      const uint4 raw = *reinterpret_cast<const uint4*>(out + static_cast<long long>(t) * dim + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] = f.x; acc[2 * i + 1] = f.y; }
    }
    for (int k = 0; k < top_k; ++k) {
      const int slot = slot_of[t * top_k + k];
      if (slot < 0) continue;
      const float w = topk_w[t * top_k + k];
      const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<long long>(slot) * dim + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += w * f.x; acc[2 * i + 1] += w * f.y; }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) ow[i] = pack_bf16x2(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * dim + c) = o;
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_moe_route(const void* logits, int logits_bf16, const float* bias, int* topk_ids, float* topk_w, int tokens,
                            int experts, int top_k, int n_group, int topk_group, int sigmoid, int norm_topk,
                            float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts > 32 * kMaxExpertsPerLane || top_k > 32 || n_group > 32 || (n_group > 1 && experts % n_group)) return -2;
  RouteParams p{logits, logits_bf16, bias, topk_ids, topk_w, tokens, experts, top_k, n_group < 1 ? 1 : n_group,
                topk_group < 1 ? 1 : topk_group, sigmoid, norm_topk, scale};
  const int block = 128;
  moe_route_kernel<<<(tokens * 32 + block - 1) / block, block, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}

B200_API int b200_moe_dispatch(const void* x, void* xs, const int* topk_ids, int* slot_of, int* counts, int tokens,
                               int top_k, int dim, int e0, int e_local, int capacity, int chunks, int chunk_tokens,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim % 8 || chunks < 1 || chunk_tokens < 1 || tokens > chunks * chunk_tokens) return -2;
  const int pairs = tokens * top_k;
  if (cudaMemsetAsync(counts, 0, sizeof(int) * e_local * chunks, stream) != cudaSuccess) return -3;
  moe_assign_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(topk_ids, slot_of, counts, pairs, top_k, e0, e_local,
                                                             capacity, chunks, chunk_tokens);
  moe_scatter_kernel<<<pairs, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(xs),
                                                slot_of, top_k, dim);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}

// Variable-size dispatch. Every local expert receives ceil(tokens_for_it / cap) blocks of `cap`
// slots, packed back to back: the grouped GEMM then runs only over blocks that hold tokens and the
// MMA N dimension is `cap`, not a worst-case capacity. Worst case blocks: ceil(T k / cap) + e_local
// (= max_blocks, the size of xs / block_group). scratch: int[2 * e_local + T * k] (counts,
// block_start, positions). Outputs: slot_of [T][k], block_group [max_blocks], dyn_blocks [1].
B200_API int b200_moe_dispatch_dynamic(const void* x, void* xs, const int* topk_ids, int* slot_of, int* scratch,
                                       int* block_group, int* dyn_blocks, int tokens, int top_k, int dim, int e0,
                                       int e_local, int cap, int max_blocks, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim % 8 || e_local > 1024 || cap < 1) return -2;
  const int pairs = tokens * top_k;
  int* counts = scratch;
  int* block_start = scratch + e_local;
  int* pos_of = scratch + 2 * e_local;
  if (cudaMemsetAsync(counts, 0, sizeof(int) * e_local, stream) != cudaSuccess) return -3;
  moe_count_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(topk_ids, pos_of, counts, pairs, e0, e_local);
  moe_plan_kernel<<<1, 256, 0, stream>>>(counts, block_start, block_group, dyn_blocks, e_local, cap, max_blocks);
  moe_scatter_dynamic_kernel<<<pairs, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                        static_cast<__nv_bfloat16*>(xs), topk_ids, pos_of, block_start,
                                                        slot_of, top_k, dim, e0, cap, max_blocks);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}

B200_API int b200_moe_combine(const void* y, const int* slot_of, const float* topk_w, void* out, int tokens,
                              int top_k, int dim, int accumulate, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim % 8) return -2;
  moe_combine_kernel<<<tokens, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), slot_of, topk_w,
                                                 static_cast<__nv_bfloat16*>(out), top_k, dim, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
