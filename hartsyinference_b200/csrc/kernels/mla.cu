// Multi-head latent attention (DeepSeek-V2/V3) over a paged LATENT cache.
//
// The cache keeps, per token, the 512 normalised latent values c_kv followed by the 64 rotated
// shared key values k_pe (576 bf16 = 1152 bytes per token and layer, against 128 heads x (192 + 128)
// values for an expanded K/V cache). Queries are "absorbed": q_abs[h] = [W_uk[h]^T q_nope[h], q_pe[h]]
// (576 values), so attention is multi-query over the latent rows and the per-head value projection
// W_uv[h] is applied to the 512-wide result afterwards. Both per-head projections run on the
// column-batched grouped GEMM.
//
//  * mla_prep:    RMSNorm of the latent part, interleaved-pair RoPE of k_pe, write of the cache row;
//                 RoPE of every head's q_pe into the tail of its absorbed query.
//  * mla_attn:    one CTA per (query row, group of 16 heads, KV split): scores over 576 dims, online
//                 softmax, output over the first 512 dims of the SAME shared-memory tile (each KV
//                 tile is read from HBM once and serves as K and as V). The four warps split the 64
//                 tokens of a tile for the scores and the 512 output columns for P.V.
//  * mla_combine: merges the KV splits.
//
// Every query row carries its own kv length and block-table row, so a prefill chunk runs as rows
// with causal lengths. Reference behaviour: src/HartsyInference.LLM/Transformer/MlaAttention.cs
// (expanded K/V per head, contiguous KV cache, scalar attention).
#include "common.cuh"
#include "mma_sync.cuh"

namespace b200 {

constexpr int kLat = 512;            // latent width (also the value width)
constexpr int kRopeDim = 64;
constexpr int kRow = kLat + kRopeDim;        // 576
constexpr int kPitch = (kRow + 8) * 2;       // bytes per shared-memory row: 1168 (4-bank skew per row)
constexpr int kMlaTile = 64;
constexpr int kMlaThreads = 128;
constexpr int kPPitch = (kMlaTile + 8) * 2;  // 144 bytes
constexpr int kMaxPagesPerTile = 8;          // page >= 8 tokens

struct MlaPrepParams {
  const __nv_bfloat16* kv;          // [T][576] output of the kv_a projection
  const __nv_bfloat16* kv_norm_w;   // [512]
  const __nv_bfloat16* q;           // [T][heads * q_stride]: per head [nope][rope 64]
  __nv_bfloat16* q_abs;             // [T][heads][576]; this kernel writes [512, 576)
  __nv_bfloat16* cache;             // [slots][576]
  const int* positions;             // [T]
  const long long* slot_mapping;    // [T], < 0 = do not write
  const float* inv_freq;            // [32]
  int tokens, heads, q_stride, q_rope_off;
  float eps, rope_mscale;
};

__global__ void __launch_bounds__(128) mla_prep_kernel(const MlaPrepParams p) {
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  __shared__ float red[4];
  __shared__ float cs[32], sn[32];
  const float pos = static_cast<float>(p.positions[t]);
  if (tid < 32) {
    float s, c;
    sincosf(pos * p.inv_freq[tid], &s, &c);
    cs[tid] = c * p.rope_mscale;
    sn[tid] = s * p.rope_mscale;
  }
  // grid.y deals the heads' q_pe rotation in chunks of 16; the latent row is the first chunk's work
  if (blockIdx.y == 0) {
  // latent RMSNorm: 4 values per thread
  const __nv_bfloat16* row = p.kv + static_cast<long long>(t) * kRow;
  float v[4];
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(row + tid * 4);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / kLat + p.eps);
  const long long slot = p.slot_mapping ? p.slot_mapping[t] : -1;
  if (slot >= 0) {
    __nv_bfloat16* dst = p.cache + slot * kRow;
    uint2 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __bfloat162float(p.kv_norm_w[tid * 4 + i]);
    ow[0] = pack_bf16x2(v[0] * inv * w[0], v[1] * inv * w[1]);
    ow[1] = pack_bf16x2(v[2] * inv * w[2], v[3] * inv * w[3]);
    *reinterpret_cast<uint2*>(dst + tid * 4) = o;
    if (tid < 32) {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + kLat + 2 * tid));
      *reinterpret_cast<uint32_t*>(dst + kLat + 2 * tid) =
          pack_bf16x2(x.x * cs[tid] - x.y * sn[tid], x.x * sn[tid] + x.y * cs[tid]);
    }
  }
  } else {
    __syncthreads();     // the rotation table
  }
  // q_pe of this block's heads
  const int h0 = blockIdx.y * 16, h1 = min(p.heads, h0 + 16);
  for (int i = h0 * 32 + tid; i < h1 * 32; i += blockDim.x) {
    const int h = i >> 5, j = i & 31;
    const __nv_bfloat16* src = p.q + (static_cast<long long>(t) * p.heads + h) * p.q_stride + p.q_rope_off + 2 * j;
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
    __nv_bfloat16* dst = p.q_abs + (static_cast<long long>(t) * p.heads + h) * kRow + kLat + 2 * j;
    *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(x.x * cs[j] - x.y * sn[j], x.x * sn[j] + x.y * cs[j]);
  }
}

struct MlaAttnParams {
  const __nv_bfloat16* q;       // [rows][heads][576]
  const __nv_bfloat16* cache;   // [pages][page][576]
  __nv_bfloat16* out;           // [rows][heads][512]
  float* part_o;                // [rows][heads][splits][512]
  float* part_ml;               // [rows][heads][splits][2]
  const int* block_table;       // [seqs][table_stride]
  const int* kv_lens;           // [rows]
  const int* row_seq;           // [rows] or null (row r uses block-table row r)
  int rows, heads, page, page_shift, table_stride, splits;
  float scale_log2;
};

// kSets groups of four warps share one CTA and one staged KV tile; each group owns 16 heads of the
// same query row (with many heads per row, as in the data-parallel attention layout, every tile that
// is read from memory then serves 32 heads instead of 16, and eight warps hide each other's latencies).
template <int kSets>
struct MlaSmem {
  uint8_t kv[2][kMlaTile * kPitch];
  uint8_t q[kSets][16 * kPitch];
  uint8_t pmat[kSets][16 * kPPitch];
  float red_max[kSets][4][16];
  float red_sum[kSets][4][16];
  int pages[2][kMaxPagesPerTile];
};

__device__ __forceinline__ void mla_load_tile(uint32_t dst, const MlaAttnParams& p, const int* pages,
                                              int tok0, int kv_len) {
  // 64 tokens x 72 chunks of 16 bytes
  for (int i = threadIdx.x; i < kMlaTile * (kRow / 8); i += blockDim.x) {
    const int token = i / (kRow / 8), chunk = i - token * (kRow / 8);
    const int pos = tok0 + token;
    const bool valid = pos < kv_len;
    const int pg = valid ? pages[token >> p.page_shift] : 0;
    const __nv_bfloat16* src = p.cache + (static_cast<long long>(pg) * p.page + (pos & (p.page - 1))) * kRow + chunk * 8;
    cp_async_16(dst + token * kPitch + chunk * 16, valid ? src : p.cache, valid);
  }
}

template <int kSets>
__global__ void __launch_bounds__(kMlaThreads * kSets) mla_attn_kernel(const MlaAttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  MlaSmem<kSets>& sm = *reinterpret_cast<MlaSmem<kSets>*>(smem_raw);
  const int row_q = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31;
  const int set = kSets > 1 ? tid >> 7 : 0;      // which group of four warps
  const int warp = (tid >> 5) & 3;               // warp inside its group
  const int hg = blockIdx.x * kSets + set;
  const int kv_len = p.kv_lens[row_q];
  const int seq = p.row_seq ? p.row_seq[row_q] : row_q;
  const int* table = p.block_table + static_cast<long long>(seq) * p.table_stride;
  const int n_tiles = (kv_len + kMlaTile - 1) / kMlaTile;
  const int per = (n_tiles + p.splits - 1) / p.splits;
  const int t0 = split * per, t1 = min(n_tiles, t0 + per);
  const int heads_here = max(0, min(16, p.heads - hg * 16));
  const int pages_per_tile = kMlaTile >> p.page_shift;

  const uint32_t kv_s[2] = {smem_u32(sm.kv[0]), smem_u32(sm.kv[1])};
  const uint32_t q_s = smem_u32(sm.q[set]), p_s = smem_u32(sm.pmat[set]);
  uint8_t* pmat = sm.pmat[set];
  float (*red_max)[16] = sm.red_max[set];
  float (*red_sum)[16] = sm.red_sum[set];

  // Q rows of the CTA's head groups (zero rows for heads past the end)
  for (int i = tid; i < kSets * 16 * (kRow / 8); i += kMlaThreads * kSets) {
    const int hh = i / (kRow / 8), chunk = i - hh * (kRow / 8);
    const int head = blockIdx.x * kSets * 16 + hh;
    const bool valid = head < p.heads;
    const __nv_bfloat16* src = p.q + (static_cast<long long>(row_q) * p.heads + (valid ? head : 0)) * kRow + chunk * 8;
    cp_async_16(smem_u32(sm.q[0]) + hh * kPitch + chunk * 16, src, valid);
  }
  auto stage_pages = [&](int tile, int buf) {
    if (tid < pages_per_tile) {
      const int first = (tile * kMlaTile) >> p.page_shift;
      const int idx = first + tid;
      const int last = (kv_len - 1) >> p.page_shift;
      sm.pages[buf][tid] = idx <= last ? table[idx] : 0;
    }
  };
  if (t0 < t1) stage_pages(t0, 0);
  __syncthreads();
  if (t0 < t1) mla_load_tile(kv_s[0], p, sm.pages[0], t0 * kMlaTile, kv_len);
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int r0 = lane >> 2, tq = lane & 3;

  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    if (t + 1 < t1) {
      stage_pages(t + 1, buf ^ 1);
      __syncthreads();
      mla_load_tile(kv_s[buf ^ 1], p, sm.pages[buf ^ 1], (t + 1) * kMlaTile, kv_len);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // ---- scores of this warp's 16 tokens
    // two accumulator sets over alternate k steps: four independent chains of 18 tensor-core
    // instructions instead of two of 36 (the chain latency is what a warp waits on here)
    float s[2][4], s_odd[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = s_odd[i][j] = 0.f;
    {
      const int mi = lane >> 3;
      const uint32_t q_lane = q_s + (lane & 15) * kPitch + (lane >> 4) * 16;
      const uint32_t k_lane = kv_s[buf] + (warp * 16 + (lane & 7) + 8 * (mi >> 1)) * kPitch + (mi & 1) * 16;
#pragma unroll 6
      for (int kk = 0; kk < kRow / 16; kk += 2) {
        uint32_t a[4], a2[4], b0, b1, b2, b3, c0, c1, c2, c3;
        ldmatrix_x4(q_lane + kk * 32, a[0], a[1], a[2], a[3]);
        ldmatrix_x4(k_lane + kk * 32, b0, b1, b2, b3);
        ldmatrix_x4(q_lane + kk * 32 + 32, a2[0], a2[1], a2[2], a2[3]);
        ldmatrix_x4(k_lane + kk * 32 + 32, c0, c1, c2, c3);
        mma_bf16_16816(s[0], a, b0, b1);
        mma_bf16_16816(s[1], a, b2, b3);
        mma_bf16_16816(s_odd[0], a2, c0, c1);
        mma_bf16_16816(s_odd[1], a2, c2, c3);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] += s_odd[i][j];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = t * kMlaTile + warp * 16 + nt * 8 + tq * 2 + (j & 1);
        const float x = key < kv_len ? s[nt][j] * p.scale_log2 : -INFINITY;
        s[nt][j] = x;
        mx[j >> 1] = fmaxf(mx[j >> 1], x);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if (tq == 0) { red_max[warp][r0] = mx[0]; red_max[warp][r0 + 8] = mx[1]; }
    __syncthreads();
    float alpha[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r0 + 8 * r;
      const float tm = fmaxf(fmaxf(red_max[0][rr], red_max[1][rr]), fmaxf(red_max[2][rr], red_max[3][rr]));
      const float mnew = fmaxf(m_run[r], tm);
      msafe[r] = mnew == -INFINITY ? 0.f : mnew;
      alpha[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] - msafe[r]);
      m_run[r] = mnew;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float e[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        e[j] = exp2f(s[nt][j] - msafe[j >> 1]);
        rs[j >> 1] += e[j];
      }
      const int col = warp * 16 + nt * 8 + tq * 2;
      *reinterpret_cast<uint32_t*>(pmat + r0 * kPPitch + col * 2) = pack_bf16x2(e[0], e[1]);
      *reinterpret_cast<uint32_t*>(pmat + (r0 + 8) * kPPitch + col * 2) = pack_bf16x2(e[2], e[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    }
    if (tq == 0) { red_sum[warp][r0] = rs[0]; red_sum[warp][r0 + 8] = rs[1]; }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r0 + 8 * r;
      l_run[r] = l_run[r] * alpha[r] + red_sum[0][rr] + red_sum[1][rr] + red_sum[2][rr] + red_sum[3][rr];
    }
    // ---- O[:, warp * 128 ...] += P V
#pragma unroll
    for (int kk = 0; kk < kMlaTile / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(p_s + (lane & 15) * kPPitch + (kk * 2 + (lane >> 4)) * 16, a[0], a[1], a[2], a[3]);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        const int mi = lane >> 3;
        const int token = kk * 16 + (lane & 7) + 8 * (mi & 1);
        const int chunk = warp * 16 + np * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(kv_s[buf] + token * kPitch + chunk * 16, b0, b1, b2, b3);
        mma_bf16_16816(o[np * 2], a, b0, b1);
        mma_bf16_16816(o[np * 2 + 1], a, b2, b3);
      }
    }
    __syncthreads();   // the tile, P and the reduction slots are reused by the next iteration
  }
  cp_async_wait<0>();

  // ---- epilogue
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int h = r0 + 8 * r;
    if (h >= heads_here) continue;
    const long long rh = static_cast<long long>(row_q) * p.heads + hg * 16 + h;
    if (p.splits == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* dst = p.out + rh * kLat + warp * 128 + tq * 2;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<uint32_t*>(dst + nt * 8) = pack_bf16x2(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    } else {
      float* dst = p.part_o + (rh * p.splits + split) * kLat + warp * 128 + tq * 2;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * r], o[nt][2 * r + 1]);
      if (warp == 0 && tq == 0) {
        p.part_ml[(rh * p.splits + split) * 2] = m_run[r];
        p.part_ml[(rh * p.splits + split) * 2 + 1] = l_run[r];
      }
    }
  }
}

// One block of 128 threads per (row, head): out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s.
__global__ void mla_combine_kernel(const MlaAttnParams p) {
  const long long rh = blockIdx.x;
  const float* ml = p.part_ml + rh * p.splits * 2;
  float big = -INFINITY;
  for (int s = 0; s < p.splits; ++s) big = fmaxf(big, ml[2 * s]);
  float den = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < p.splits; ++s) {
    const float m = ml[2 * s];
    if (m == -INFINITY) continue;
    const float wgt = exp2f(m - big);
    den += wgt * ml[2 * s + 1];
    const float4 v = *reinterpret_cast<const float4*>(p.part_o + (rh * p.splits + s) * kLat + threadIdx.x * 4);
    acc[0] += wgt * v.x; acc[1] += wgt * v.y; acc[2] += wgt * v.z; acc[3] += wgt * v.w;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint2 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
  ow[0] = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  ow[1] = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(p.out + rh * kLat + threadIdx.x * 4) = o;
}

}  // namespace b200

using namespace b200;

B200_API int b200_mla_prep(const void* kv, const void* kv_norm_w, const void* q, void* q_abs, void* cache,
                           const int* positions, const long long* slot_mapping, const float* inv_freq, int tokens,
                           int heads, int q_stride, int q_rope_off, float eps, float rope_mscale,
                           cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_stride % 2 || q_rope_off % 2) return -2;
  MlaPrepParams p{static_cast<const __nv_bfloat16*>(kv), static_cast<const __nv_bfloat16*>(kv_norm_w),
                  static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(q_abs),
                  static_cast<__nv_bfloat16*>(cache), positions, slot_mapping, inv_freq, tokens, heads, q_stride,
                  q_rope_off, eps, rope_mscale};
  mla_prep_kernel<<<dim3(tokens, heads > 16 ? (heads + 15) / 16 : 1), 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}

// Head groups of 16 that one CTA serves: two once a row has more than one group.
static int mla_sets(int heads) { return heads > 16 ? 2 : 1; }

B200_API int b200_mla_pick_splits(int rows, int heads, int max_kv_len) {
  const int per_cta = 16 * mla_sets(heads);
  const int ctas = rows * ((heads + per_cta - 1) / per_cta);
  const int tiles = (max_kv_len + kMlaTile - 1) / kMlaTile;
  int s = (2 * 148 + ctas - 1) / ctas;
  if (s > tiles) s = tiles;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

B200_API long long b200_mla_workspace_bytes(int rows, int heads, int splits) {
  if (splits <= 1) return 0;
  return static_cast<long long>(rows) * heads * splits * (kLat + 2) * 4;
}

B200_API int b200_mla_attn(const void* q, const void* cache, void* out, const int* block_table,
                           const int* kv_lens, const int* row_seq, int rows, int heads, int page,
                           int table_stride, int splits, void* workspace, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  int shift = 0;
  while ((1 << shift) < page) ++shift;
  if ((1 << shift) != page || page < 8 || page > kMlaTile) return -2;
  if (splits < 1) splits = 1;
  if (splits > 1 && workspace == nullptr) return -3;
  MlaAttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = static_cast<float*>(workspace);
  p.part_ml = p.part_o ? p.part_o + static_cast<long long>(rows) * heads * splits * kLat : nullptr;
  p.block_table = block_table;
  p.kv_lens = kv_lens;
  p.row_seq = row_seq;
  p.rows = rows; p.heads = heads; p.page = page; p.page_shift = shift; p.table_stride = table_stride;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  static PerDeviceOnce configured;
  const int smem1 = static_cast<int>(sizeof(MlaSmem<1>)), smem2 = static_cast<int>(sizeof(MlaSmem<2>));
  if (configured.first_time()) {
    if (cudaFuncSetAttribute(mla_attn_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1) != cudaSuccess ||
        cudaFuncSetAttribute(mla_attn_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) != cudaSuccess)
      return -4;
  }
  if (mla_sets(heads) == 2) {
    mla_attn_kernel<2><<<dim3((heads + 31) / 32, rows, splits), kMlaThreads * 2, smem2, stream>>>(p);
  } else {
    mla_attn_kernel<1><<<dim3((heads + 15) / 16, rows, splits), kMlaThreads, smem1, stream>>>(p);
  }
  if (splits > 1) mla_combine_kernel<<<rows * heads, 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
