// Attention over a paged or contiguous KV store, bf16 in / fp32 softmax / bf16 out.
//
//  * decode:  one query token per sequence; the G query heads that share a KV head form the rows
//             of the score tile, the four warps of a CTA split each 64-token KV tile, optional
//             split-KV across CTAs with a combine kernel (flash-decoding).
//  * prefill: 64 query tokens of one head per CTA (16 per warp), causal or full, KV read either
//             through the block table (chunked prefill with a cached prefix) or from contiguous
//             [tokens][heads][d] tensors (DiT self/cross attention).
//
// K/V pages are read straight from the page pool through the block table; nothing is gathered
// into a contiguous scratch first. This replaces the reference's per-sequence page gather plus
// scalar flash kernels (src/HartsyInference.LLM/Transformer/PagedKvCache.cs:116-169,
// src/HartsyInference.Cuda/Kernels/lm/flash_attn_f32.cu, flash_attn_f32_split.cu,
// flash_attn_v2_tf32.cu). Supported per-call options follow the reference's attention oracle
// (src/HartsyInference.Core/Backends/AttentionReference.cs): GQA, causal, sliding window,
// logit soft-cap.
//
// The score and PV products use warp-level mma.sync (m16n8k16, bf16): with one to sixteen query
// rows per KV head the kernel is bound by KV bandwidth, not by tensor throughput, and a 128-row
// tcgen05 tile would be mostly padding.
#include "common.cuh"
#include "mma_sync.cuh"

namespace b200 {

constexpr int kTileTokens = 64;
constexpr int kAttnThreads = 128;

struct AttnParams {
  const __nv_bfloat16* q;       // decode: [seqs][hq][d]; prefill: [total_q][hq][d]
  const __nv_bfloat16* k;       // paged: [pages][hkv][page][d]; contiguous: [total_kv][hkv][d]
  const __nv_bfloat16* v;
  __nv_bfloat16* out;           // same layout as q
  const int* block_table;       // [seqs][max_pages]
  const int* kv_lens;           // [seqs] keys visible to the last query token
  const int* cu_q;              // prefill: [seqs + 1] offsets into q (null -> one sequence)
  const int* cu_kv;             // contiguous prefill: [seqs + 1] offsets into k/v
  float* ws_o;                  // split partials [seqs][hq][splits][d]
  float* ws_ml;                 // [seqs][hq][splits][2]
  int seqs, hq, hkv, max_pages, page, page_shift, splits;
  int q_len_single, kv_len_single;   // used when cu_q / kv_lens are null
  int causal, window;           // window <= 0: unlimited
  float scale_log2;             // softmax scale * log2(e)
  float softcap;                // 0 = off; scores = cap * tanh(scores / cap) (pre-scale units)
  float scale;                  // plain softmax scale (needed with softcap)
  // decode, head dim 128, split path: the combine kernel also emits the output as e4m3 with one
  // scale per head (= one 1x128 group of the following linear's input), saving a quantise kernel
  uint8_t* out_q;               // [seqs][hq * d] or null
  void* out_scale;              // fp32 [seqs][hq], or blocked UE8M0 bytes when sf_tile_rows > 0
  int sf_tile_rows;
};

// Shared-memory tile: [64 tokens][D] bf16, row pitch D * 2 bytes, 16-byte chunks XOR-swizzled with
// (token & 7) so that ldmatrix rows of consecutive tokens hit different banks.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int token, int chunk) {
  return static_cast<uint32_t>(token * (D * 2) + ((chunk ^ (token & 7)) << 4));
}

// Loads one 64-token K or V tile through the block table. The tile's page ids were staged in
// shared memory (`pg`, 64 / page entries) an iteration earlier, so no cp.async waits on a
// dependent global load of the table; page sizes are powers of two (8..64), so token -> (page,
// offset) is a shift and a mask.
template <int D>
__device__ __forceinline__ void load_tile_paged(uint32_t smem_base, const __nv_bfloat16* pool,
                                                const int* pg, int kv_head, int hkv, int page_shift,
                                                int tok0, int kv_len) {
  constexpr int kChunks = D / 8;
  const int page_mask = (1 << page_shift) - 1;
  for (int i = threadIdx.x; i < kTileTokens * kChunks; i += kAttnThreads) {
    const int t = i / kChunks, c = i % kChunks;
    const bool valid = tok0 + t < kv_len;
    const __nv_bfloat16* src = pool;
    if (valid) {
      const long long pgi = pg[t >> page_shift];
      src = pool + (((pgi * hkv + kv_head) << page_shift) + (t & page_mask)) * D + c * 8;
    }
    cp_async_16(smem_base + tile_off<D>(t, c), src, valid);
  }
}
// Stages the page ids of tile `tile` into ring slot (tile & 3). Tiles start on page boundaries
// because 64 is a multiple of every supported page size.
__device__ __forceinline__ void stage_pages(int (*ring)[8], const int* table, int tile, int n_tiles,
                                            int page_shift, int kv_len) {
  const int per_tile = kTileTokens >> page_shift;
  if (tile < n_tiles && threadIdx.x < per_tile) {
    const int first = (tile * kTileTokens) >> page_shift;
    const int idx = first + threadIdx.x;
    const int last_page = (kv_len - 1) >> page_shift;
    ring[tile & 3][threadIdx.x] = idx <= last_page ? table[idx] : 0;
  }
}
template <int D>
__device__ __forceinline__ void load_tile_linear(uint32_t smem_base, const __nv_bfloat16* base,
                                                 long long row_stride, int tok0, int kv_len) {
  constexpr int kChunks = D / 8;
  for (int i = threadIdx.x; i < kTileTokens * kChunks; i += kAttnThreads) {
    const int t = i / kChunks, c = i % kChunks;
    const int tok = tok0 + t;
    const bool valid = tok < kv_len;
    const __nv_bfloat16* src = valid ? base + tok * row_stride + c * 8 : base;
    cp_async_16(smem_base + tile_off<D>(t, c), src, valid);
  }
}

// Per-warp flash-attention state for 16 query rows: thread (g = lane / 4, t = lane % 4) owns rows g
// and g + 8.
template <int D>
struct WarpState {
  float o[D / 8][4];
  float m[2], l[2];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// Processes NG groups of 16 tokens starting at tile-local token `t_begin` for this warp.
//   qf: Q fragments [D/16][4]; row_limit[r]: first masked key position for the thread's row r
//   (keys >= limit are masked), row_start[r]: first visible key (sliding window).
template <int D, int NG>
__device__ __forceinline__ void warp_tile(WarpState<D>& st, const uint32_t (&qf)[D / 16][4],
                                          uint32_t k_smem, uint32_t v_smem, int t_begin,
                                          int tok0, const int (&row_limit)[2],
                                          const int (&row_start)[2], const AttnParams& p) {
  const int lane = threadIdx.x & 31;
  const int tq = lane & 3;
  float s[NG * 2][4];
#pragma unroll
  for (int i = 0; i < NG * 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
  // S = Q K^T
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      const int mi = lane >> 3;
      const int token = t_begin + gi * 16 + (lane & 7) + 8 * (mi >> 1);
      const int chunk = kk * 2 + (mi & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(k_smem + tile_off<D>(token, chunk), b0, b1, b2, b3);
      mma_bf16_16816(s[gi * 2], qf[kk], b0, b1);
      mma_bf16_16816(s[gi * 2 + 1], qf[kk], b2, b3);
    }
  }
  // scale, soft-cap, mask; running max
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NG * 2; ++nt) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = j >> 1;
      const int key = tok0 + t_begin + nt * 8 + tq * 2 + (j & 1);
      float x = s[nt][j];
      if (p.softcap > 0.f) x = p.softcap * tanhf(x * p.scale / p.softcap) * (p.scale_log2 / p.scale);
      else x *= p.scale_log2;
      if (key >= row_limit[r] || key < row_start[r]) x = -INFINITY;
      s[nt][j] = x;
      mx[r] = fmaxf(mx[r], x);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float alpha[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float mnew = fmaxf(st.m[r], mx[r]);
    msafe[r] = mnew == -INFINITY ? 0.f : mnew;
    alpha[r] = st.m[r] == -INFINITY ? 0.f : exp2f(st.m[r] - msafe[r]);
    st.m[r] = mnew;
  }
  float rs[2] = {0.f, 0.f};
  uint32_t pf[NG][4];
#pragma unroll
  for (int nt = 0; nt < NG * 2; ++nt) {
    float e[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[j] = exp2f(s[nt][j] - msafe[j >> 1]);
      rs[j >> 1] += e[j];
    }
    // A fragment of P for the 16-token group nt / 2: (a0, a1) from the even n-tile, (a2, a3)
    // from the odd one
    pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(e[0], e[1]);
    pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(e[2], e[3]);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    st.l[r] = st.l[r] * alpha[r] + rs[r];
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    st.o[i][0] *= alpha[0];
    st.o[i][1] *= alpha[0];
    st.o[i][2] *= alpha[1];
    st.o[i][3] *= alpha[1];
  }
  // O += P V
#pragma unroll
  for (int gi = 0; gi < NG; ++gi) {
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      const int mi = lane >> 3;
      const int token = t_begin + gi * 16 + (lane & 7) + 8 * (mi & 1);
      const int chunk = np * 2 + (mi >> 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(v_smem + tile_off<D>(token, chunk), b0, b1, b2, b3);
      mma_bf16_16816(st.o[np * 2], pf[gi], b0, b1);
      mma_bf16_16816(st.o[np * 2 + 1], pf[gi], b2, b3);
    }
  }
}

// ------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------
template <int D, int kStages>
__global__ void __launch_bounds__(kAttnThreads)
attn_decode_kernel(const AttnParams p) {
  pdl_wait();
  pdl_trigger();
  constexpr int kTileBytes = kTileTokens * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int G = p.hq / p.hkv;
  const int kv_len = p.kv_lens[seq];
  const int n_tiles = (kv_len + kTileTokens - 1) / kTileTokens;
  const int tiles_per_split = (n_tiles + p.splits - 1) / p.splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(n_tiles, tile_begin + tiles_per_split);
  const int* table = p.block_table + static_cast<long long>(seq) * p.max_pages;
  const uint32_t smem_base = smem_u32(smem);

  // Q fragments: row = query head within the group (rows >= G are zero)
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* qb = p.q + (static_cast<long long>(seq) * p.hq + kvh * G) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c0 = kk * 16 + tq * 2;
      qf[kk][0] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * D + c0) : 0u;
      qf[kk][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * D + c0) : 0u;
      qf[kk][2] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * D + c0 + 8) : 0u;
      qf[kk][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * D + c0 + 8) : 0u;
    }
  }
  WarpState<D> st;
  st.init();
  const int lim[2] = {kv_len, kv_len};
  const int start_key = p.window > 0 ? max(0, kv_len - p.window) : 0;
  const int start[2] = {start_key, start_key};

  __shared__ int pg_ring[4][8];
  auto issue = [&](int tile, int stage) {
    if (tile < tile_end) {
      const uint32_t kb = smem_base + stage * 2 * kTileBytes;
      load_tile_paged<D>(kb, p.k, pg_ring[tile & 3], kvh, p.hkv, p.page_shift, tile * kTileTokens, kv_len);
      load_tile_paged<D>(kb + kTileBytes, p.v, pg_ring[tile & 3], kvh, p.hkv, p.page_shift,
                         tile * kTileTokens, kv_len);
    }
    cp_async_commit();
  };
  stage_pages(pg_ring, table, tile_begin, tile_end, p.page_shift, kv_len);
  stage_pages(pg_ring, table, tile_begin + 1, tile_end, p.page_shift, kv_len);
  stage_pages(pg_ring, table, tile_begin + 2, tile_end, p.page_shift, kv_len);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(tile_begin + i, i);
  int stage = 0;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    // page ids of tile + 3 are read by issue() in a later iteration, after two barriers
    stage_pages(pg_ring, table, tile + 3, tile_end, p.page_shift, kv_len);
    issue(tile + kStages - 1, (stage + kStages - 1) % kStages);
    cp_async_wait<kStages - 1>();
    __syncthreads();
    const uint32_t kb = smem_base + stage * 2 * kTileBytes;
    warp_tile<D, 1>(st, qf, kb, kb + kTileBytes, warp * 16, tile * kTileTokens, lim, start, p);
    __syncthreads();
    stage = (stage + 1) % kStages;
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps' partial states through shared memory
  float* so = reinterpret_cast<float*>(smem);                    // [4][16][D]
  float* sml = so + 4 * 16 * D;                                  // [4][16][2]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int c = i * 8 + tq * 2;
    so[(warp * 16 + g) * D + c] = st.o[i][0];
    so[(warp * 16 + g) * D + c + 1] = st.o[i][1];
    so[(warp * 16 + g + 8) * D + c] = st.o[i][2];
    so[(warp * 16 + g + 8) * D + c + 1] = st.o[i][3];
  }
  if (tq == 0) {
    sml[(warp * 16 + g) * 2] = st.m[0];
    sml[(warp * 16 + g) * 2 + 1] = st.l[0];
    sml[(warp * 16 + g + 8) * 2] = st.m[1];
    sml[(warp * 16 + g + 8) * 2 + 1] = st.l[1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
    const int r = i / D, c = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sml[(w * 16 + r) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sml[(w * 16 + r) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      acc += so[(w * 16 + r) * D + c] * f;
      ll += sml[(w * 16 + r) * 2 + 1] * f;
    }
    const int head = kvh * G + r;
    if (p.splits == 1) {
      p.out[(static_cast<long long>(seq) * p.hq + head) * D + c] =
          __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const long long base = (static_cast<long long>(seq) * p.hq + head) * p.splits + split;
      p.ws_o[base * D + c] = acc;
      if (c == 0) {
        p.ws_ml[base * 2] = mm;
        p.ws_ml[base * 2 + 1] = ll;
      }
    }
  }
}

template <int D>
__global__ void attn_combine_kernel(const AttnParams p) {
  pdl_wait();
  pdl_trigger();
  const int seq = blockIdx.x, head = blockIdx.y;
  const long long base = (static_cast<long long>(seq) * p.hq + head) * p.splits;
  float mm = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, p.ws_ml[(base + s) * 2]);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f, ll = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = p.ws_ml[(base + s) * 2];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      acc += p.ws_o[(base + s) * D + c] * f;
      ll += p.ws_ml[(base + s) * 2 + 1] * f;
    }
    const __nv_bfloat16 o = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    if (p.out) p.out[(static_cast<long long>(seq) * p.hq + head) * D + c] = o;
    if (D == 128 && p.out_q) {
      // blockDim == D: every thread holds one value of the head; the head is one quantisation group
      __shared__ float wmax[4];
      const float v = __bfloat162float(o);
      float amax = warp_max(fabsf(v));
      if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
      float sc = fmaxf(amax, 1e-12f) / 448.f, inv = 1.f / sc;
      uint32_t eb = 127;
      if (p.sf_tile_rows > 0) {
        // UE8M0: the smallest power of two >= amax / 448
        const uint32_t bits = __float_as_uint(amax / 448.f);
        int e = static_cast<int>(bits >> 23) - 127 + ((bits & 0x7fffffu) != 0 ? 1 : 0);
        e = max(-126, min(126, e));
        eb = static_cast<uint32_t>(e + 127);
        inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
      }
      p.out_q[(static_cast<long long>(seq) * p.hq + head) * D + c] =
          static_cast<uint8_t>(__nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3));
      if (c == 0) {
        if (p.sf_tile_rows > 0) {
          // blocked layout: row tiles of sf_tile_rows, K groups of four 128-wide blocks, row r of a
          // tile at word (r % 32) * 4 + r / 32, K block kb at byte kb % 4
          const int kgroups = (p.hq * D + 511) >> 9;
          const int tile = seq / p.sf_tile_rows, r = seq - tile * p.sf_tile_rows;
          const long long blk = static_cast<long long>(tile) * kgroups + (head >> 2);
          static_cast<uint8_t*>(p.out_scale)[(blk * 128 + (r & 31) * 4 + (r >> 5)) * 4 + (head & 3)] =
              static_cast<uint8_t>(eb);
        } else {
          static_cast<float*>(p.out_scale)[static_cast<long long>(seq) * p.hq + head] = sc;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// prefill / full attention
// ------------------------------------------------------------------------------------------
template <int D, bool kPaged>
__global__ void __launch_bounds__(kAttnThreads)
attn_prefill_kernel(const AttnParams p) {
  constexpr int kStages = 2;
  constexpr int kTileBytes = kTileTokens * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int qt = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int G = p.hq / p.hkv;
  const int kvh = head / G;
  const int q_off = p.cu_q ? p.cu_q[seq] : 0;
  const int q_len = p.cu_q ? p.cu_q[seq + 1] - q_off : p.q_len_single;
  const int kv_len = p.kv_lens ? p.kv_lens[seq] : p.kv_len_single;
  if (qt * 64 >= q_len) return;
  const int ctx = kv_len - q_len;   // keys that precede the first query token
  const uint32_t smem_base = smem_u32(smem);

  const int row0 = qt * 64 + warp * 16 + g;   // this thread's rows: row0, row0 + 8
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* qb = p.q + (static_cast<long long>(q_off) * p.hq + head) * D;
    const long long rs = static_cast<long long>(p.hq) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c0 = kk * 16 + tq * 2;
      qf[kk][0] = row0 < q_len ? *reinterpret_cast<const uint32_t*>(qb + row0 * rs + c0) : 0u;
      qf[kk][1] = row0 + 8 < q_len ? *reinterpret_cast<const uint32_t*>(qb + (row0 + 8) * rs + c0) : 0u;
      qf[kk][2] = row0 < q_len ? *reinterpret_cast<const uint32_t*>(qb + row0 * rs + c0 + 8) : 0u;
      qf[kk][3] = row0 + 8 < q_len ? *reinterpret_cast<const uint32_t*>(qb + (row0 + 8) * rs + c0 + 8) : 0u;
    }
  }
  WarpState<D> st;
  st.init();
  int lim[2], start[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int pos = ctx + row0 + 8 * r;   // absolute position of the query row
    lim[r] = p.causal ? min(kv_len, pos + 1) : kv_len;
    start[r] = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
  }
  // keys needed by this CTA: up to the last row's position when causal
  const int last_pos = ctx + min(q_len, qt * 64 + 64) - 1;
  const int kv_needed = p.causal ? min(kv_len, last_pos + 1) : kv_len;
  const int n_tiles = (kv_needed + kTileTokens - 1) / kTileTokens;
  int tile0 = 0;
  if (p.window > 0) tile0 = max(0, ctx + qt * 64 + 1 - p.window) / kTileTokens;

  const int* table = kPaged ? p.block_table + static_cast<long long>(seq) * p.max_pages : nullptr;
  const int kv_off = (!kPaged && p.cu_kv) ? p.cu_kv[seq] : 0;
  const long long kv_rs = static_cast<long long>(p.hkv) * D;
  const __nv_bfloat16* kbase = kPaged ? p.k : p.k + (static_cast<long long>(kv_off) * p.hkv + kvh) * D;
  const __nv_bfloat16* vbase = kPaged ? p.v : p.v + (static_cast<long long>(kv_off) * p.hkv + kvh) * D;

  __shared__ int pg_ring[4][8];
  auto issue = [&](int tile, int stage) {
    if (tile < n_tiles) {
      const uint32_t kb = smem_base + stage * 2 * kTileBytes;
      if (kPaged) {
        load_tile_paged<D>(kb, p.k, pg_ring[tile & 3], kvh, p.hkv, p.page_shift, tile * kTileTokens, kv_needed);
        load_tile_paged<D>(kb + kTileBytes, p.v, pg_ring[tile & 3], kvh, p.hkv, p.page_shift,
                           tile * kTileTokens, kv_needed);
      } else {
        load_tile_linear<D>(kb, kbase, kv_rs, tile * kTileTokens, kv_needed);
        load_tile_linear<D>(kb + kTileBytes, vbase, kv_rs, tile * kTileTokens, kv_needed);
      }
    }
    cp_async_commit();
  };
  if (kPaged) {
    stage_pages(pg_ring, table, tile0, n_tiles, p.page_shift, kv_needed);
    stage_pages(pg_ring, table, tile0 + 1, n_tiles, p.page_shift, kv_needed);
    __syncthreads();
  }
  issue(tile0, 0);
  int stage = 0;
  for (int tile = tile0; tile < n_tiles; ++tile) {
    if (kPaged) stage_pages(pg_ring, table, tile + 2, n_tiles, p.page_shift, kv_needed);
    issue(tile + 1, stage ^ 1);
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kb = smem_base + stage * 2 * kTileBytes;
    // a warp whose rows all lie before this tile (causal) still runs: masked scores cost nothing
    // in correctness and keep the barrier pattern uniform
    warp_tile<D, 4>(st, qf, kb, kb + kTileBytes, 0, tile * kTileTokens, lim, start, p);
    __syncthreads();
    stage ^= 1;
  }
  cp_async_wait<0>();
  static_assert(kStages == 2, "double buffered");

  __nv_bfloat16* ob = p.out + (static_cast<long long>(q_off) * p.hq + head) * D;
  const long long rs = static_cast<long long>(p.hq) * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + 8 * r;
    if (row < q_len) {
      const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + tq * 2;
        *reinterpret_cast<uint32_t*>(ob + row * rs + c) =
            pack_bf16x2(st.o[i][2 * r] * inv, st.o[i][2 * r + 1] * inv);
      }
    }
  }
}

}  // namespace b200

using namespace b200;

B200_API long long b200_attn_decode_workspace_bytes(int seqs, int hq, int d, int splits) {
  return splits > 1 ? static_cast<long long>(seqs) * hq * splits * (d + 2) * 4 : 0;
}

static int g_decode_stages = 2;

// Number of KV splits for a decode batch, from a wave model fitted to B200 timings: the grid runs
// in waves of (148 SMs x resident CTAs) and a CTA costs its tiles plus about four tiles' worth of
// prologue and merge, so the estimate is waves x (ceil(tiles / splits) + 4); ties go to fewer
// splits (less partial traffic and a cheaper combine). Measured with the two-tile ring, 64-token
// tiles, 2304-token contexts (CTAs before splitting: best splits, time): 16: 12, 13.5 us;
// 64: 6, 24.9 us; 128: 3, 40.4 us; 256: 3 or 1, 76-78 us; 512: 2, 132 us (8192 tokens: 4, 388 us;
// 512 tokens: 1, 41 us); 1024: 1, 238 us.
B200_API int b200_attn_decode_pick_splits(int seqs, int hkv, int max_kv_len) {
  const int ctas = seqs * hkv > 0 ? seqs * hkv : 1;
  const int tiles = (max_kv_len + kTileTokens - 1) / kTileTokens;
  const int slots = 148 * (g_decode_stages == 2 ? 3 : 2);
  int best = 1;
  long long best_cost = -1;
  for (int sp = 1; sp <= 16 && sp <= tiles; ++sp) {
    const long long waves = (static_cast<long long>(ctas) * sp + slots - 1) / slots;
    const long long cost = waves * ((tiles + sp - 1) / sp + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = sp; }
  }
  return best;
}


// Depth of the decode kernel's K/V staging ring: 3 (two CTAs per SM at head dim 128) or 2 (three).
B200_API void b200_attn_set_decode_stages(int stages) { g_decode_stages = stages == 2 ? 2 : 3; }

B200_API int b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                              const int* block_table, const int* kv_lens, int seqs, int hq, int hkv,
                              int d, int page, int max_pages, int splits, void* workspace,
                              float scale, float softcap, int window, void* out_q, void* out_scale,
                              int sf_tile_rows, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (out_q != nullptr && (d != 128 || splits <= 1 || out_scale == nullptr)) return -6;   // combine kernel only
  if (d != 64 && d != 128) return -2;
  if (hq % hkv != 0 || hq / hkv > 16) return -3;
  if (splits > 1 && !workspace) return -5;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k_cache);
  p.v = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.kv_lens = kv_lens;
  p.seqs = seqs; p.hq = hq; p.hkv = hkv; p.max_pages = max_pages; p.page = page;
  p.page_shift = page == 8 ? 3 : page == 16 ? 4 : page == 32 ? 5 : page == 64 ? 6 : -1;
  if (p.page_shift < 0) return -4;
  p.splits = splits < 1 ? 1 : splits;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap;
  p.out_q = static_cast<uint8_t*>(out_q);
  p.out_scale = out_scale;
  p.sf_tile_rows = sf_tile_rows;
  if (p.splits > 1) {
    p.ws_o = static_cast<float*>(workspace);
    p.ws_ml = p.ws_o + static_cast<long long>(seqs) * hq * p.splits * d;
  }
  dim3 grid(seqs, hkv, p.splits);
  // staging ring depth: 3 tiles (two CTAs per SM at d = 128) or 2 tiles (three CTAs per SM)
  const int stages = g_decode_stages == 2 ? 2 : 3;
  const int smem = stages * 2 * kTileTokens * d * 2;
  static PerDeviceOnce attr_set[2][2];
  PerDeviceOnce& once = attr_set[d == 128 ? 1 : 0][stages - 2];
  auto launch = [&](auto kernel) {
    if (once.first_time()) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    launch_pdl(kernel, grid, dim3(kAttnThreads), smem, stream, p);
  };
  if (d == 128) {
    if (stages == 2) launch(attn_decode_kernel<128, 2>); else launch(attn_decode_kernel<128, 3>);
  } else {
    if (stages == 2) launch(attn_decode_kernel<64, 2>); else launch(attn_decode_kernel<64, 3>);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -static_cast<int>(e) - 300;
  if (p.splits > 1) {
    dim3 cg(seqs, hq);
    if (d == 128) launch_pdl(attn_combine_kernel<128>, cg, dim3(128), 0, stream, p);
    else launch_pdl(attn_combine_kernel<64>, cg, dim3(64), 0, stream, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return -static_cast<int>(e) - 400;
  }
  return 0;
}

// Prefill / full attention. paged != 0: k, v are page pools read through block_table and kv_lens;
// else k, v are contiguous [tokens][hkv][d] with optional cu_kv offsets.
B200_API int b200_attn_prefill(const void* q, const void* k, const void* v, void* out,
                               const int* block_table, const int* kv_lens, const int* cu_q,
                               const int* cu_kv, int seqs, int max_q_len, int q_len_single,
                               int kv_len_single, int hq, int hkv, int d, int page, int max_pages,
                               int paged, int causal, int window, float scale, float softcap,
                               cudaStream_t stream) {
  if (seqs <= 0 || max_q_len <= 0) return 0;
  if (d != 64 && d != 128) return -2;
  if (hq % hkv != 0) return -3;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.kv_lens = kv_lens;
  p.cu_q = cu_q;
  p.cu_kv = cu_kv;
  p.seqs = seqs; p.hq = hq; p.hkv = hkv; p.max_pages = max_pages; p.page = page; p.splits = 1;
  p.page_shift = page == 8 ? 3 : page == 16 ? 4 : page == 32 ? 5 : page == 64 ? 6 : -1;
  if (paged && p.page_shift < 0) return -4;
  p.q_len_single = q_len_single; p.kv_len_single = kv_len_single;
  p.causal = causal; p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap;
  dim3 grid((max_q_len + 63) / 64, hq, seqs);
  const int smem = 2 * 2 * kTileTokens * d * 2;
#define LAUNCH_PREFILL(DD, PG)                                                                   \
  do {                                                                                           \
    static PerDeviceOnce once;                                                                   \
    if (once.first_time())                                                                       \
      cudaFuncSetAttribute(attn_prefill_kernel<DD, PG>,                                          \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                   \
    attn_prefill_kernel<DD, PG><<<grid, kAttnThreads, smem, stream>>>(p);                        \
  } while (0)
  if (d == 128) {
    if (paged) LAUNCH_PREFILL(128, true); else LAUNCH_PREFILL(128, false);
  } else {
    if (paged) LAUNCH_PREFILL(64, true); else LAUNCH_PREFILL(64, false);
  }
#undef LAUNCH_PREFILL
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 300;
}
