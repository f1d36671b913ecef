// Dense (non-causal) attention on the 5th-generation tensor cores, head dim 128, bf16.
//
// For the DiT families every block attends over the whole joint sequence (thousands to tens of
// thousands of tokens), so attention is compute bound and the warp-level mma.sync kernel leaves
// most of the tensor throughput unused. Here one CTA owns 128 query rows of one head and walks
// the keys in tiles of 128:
//
//   warp 0      TMA producer: Q tile once, then K tile [128 keys x 128] and V^T tile [128 dims x
//               128 keys] per step into a two-stage ring (128B-swizzled, K-major)
//   warp 1      one thread issues tcgen05.mma: S_j = Q K_j^T into TMEM (two S buffers, so S_{j+1}
//               is computed while the softmax warps work on S_j), then O_j = P_j V_j into a second
//               pair of TMEM buffers
//   warps 2..5  softmax: thread r owns query row r (TMEM lane r): reads its S row with tcgen05.ld,
//               keeps the running maximum / sum, writes P_j (bf16) into shared memory in the
//               layout of an MMA A operand, and accumulates O in registers as
//               O = O * alpha + (P_j V_j) read back from TMEM. No shuffles: a row never leaves
//               its thread.
//
// V is consumed transposed ([head dim][keys], keys contiguous) so that both MMAs use K-major
// operands; the transpose is a small kernel of its own in front (V is read once per call, the
// attention reads it S_q / 128 times).
#include "common.cuh"

namespace b200 {

constexpr int kAtD = 128;
constexpr int kAtTile = 128;            // queries per CTA and keys per step
constexpr int kAtThreads = 192;
constexpr int kAtTileBytes = 128 * 128 * 2;   // one [128 x 128] bf16 tile = two swizzle atoms of 16 KB

struct AttnTcBarriers {
  uint64_t q_full;
  uint64_t kv_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty;
  uint64_t pv_full[2], pv_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct AttnTcParams {
  __nv_bfloat16* out;     // [batch * sq][ld] (ld = heads * 128)
  long long ld;
  int sq, sk, heads, batch;
  float scale_log2;       // softmax scale * log2(e)
  DeviceStatus* status;
};

__global__ void __launch_bounds__(kAtThreads, 1)
attn_tc_kernel(const AttnTcParams p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_vt) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;                                  // 32 KB
  uint8_t* sk[2] = {smem + kAtTileBytes, smem + 2 * kAtTileBytes};
  uint8_t* sv[2] = {smem + 3 * kAtTileBytes, smem + 4 * kAtTileBytes};
  uint8_t* sp = smem + 5 * kAtTileBytes;               // P tile
  AttnTcBarriers* bars = reinterpret_cast<AttnTcBarriers*>(smem + 6 * kAtTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int n_tiles = (p.sk + kAtTile - 1) / kAtTile;
  const int q_row0 = b * p.sq + qt * kAtTile;          // row in the [batch * sq] matrix
  const int k_row0 = b * p.sk;
  const int vt_row0 = (b * p.heads + head) * kAtD;     // row in the [batch * heads * 128][sk] matrix

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->kv_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4);
      mbar_init(&bars->pv_full[i], 1);
      mbar_init(&bars->pv_empty[i], 4);
    }
    mbar_init(&bars->p_full, 4);
    mbar_init(&bars->p_empty, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_vt);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  constexpr uint32_t kIdesc = make_idesc(128, 128, kFmtBf16, kFmtBf16);

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->q_full, kAtTileBytes);
      tma_load_2d(sq, &tm_q, &bars->q_full, head * kAtD, q_row0);
      tma_load_2d(sq + kAtTileBytes / 2, &tm_q, &bars->q_full, head * kAtD + 64, q_row0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&bars->kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 11, blockIdx.x);
          break;
        }
        mbar_arrive_expect_tx(&bars->kv_full[s], 2 * kAtTileBytes);
        tma_load_2d(sk[s], &tm_k, &bars->kv_full[s], head * kAtD, k_row0 + j * kAtTile);
        tma_load_2d(sk[s] + kAtTileBytes / 2, &tm_k, &bars->kv_full[s], head * kAtD + 64, k_row0 + j * kAtTile);
        tma_load_2d(sv[s], &tm_vt, &bars->kv_full[s], j * kAtTile, vt_row0);
        tma_load_2d(sv[s] + kAtTileBytes / 2, &tm_vt, &bars->kv_full[s], j * kAtTile + 64, vt_row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait(&bars->kv_full[s], (j >> 1) & 1, abort_flag)) return false;
        if (!mbar_wait(&bars->s_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + s * 128;
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          const uint64_t ad = make_desc_sw128(smem_u32(sq + a * (kAtTileBytes / 2)));
          const uint64_t bd = make_desc_sw128(smem_u32(sk[s] + a * (kAtTileBytes / 2)));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_bf16_ss(d_tmem, ad + 2 * k, bd + 2 * k, kIdesc, (a | k) != 0);
        }
        tc_commit(&bars->s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(&bars->p_full, j & 1, abort_flag) ||
            !mbar_wait(&bars->pv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + 256 + s * 128;
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          const uint64_t ad = make_desc_sw128(smem_u32(sp + a * (kAtTileBytes / 2)));
          const uint64_t bd = make_desc_sw128(smem_u32(sv[s] + a * (kAtTileBytes / 2)));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_bf16_ss(d_tmem, ad + 2 * k, bd + 2 * k, kIdesc, (a | k) != 0);
        }
        tc_commit(&bars->pv_full[s]);
        tc_commit(&bars->kv_empty[s]);
        tc_commit(&bars->p_empty);
      }
      if (!ok) report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 12, blockIdx.x);
    }
  } else {
    // ---------------------------------------------------------------- softmax / output warps
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // query row inside the tile = TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float o[kAtD];
#pragma unroll
    for (int i = 0; i < kAtD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    bool ok = true;
    auto consume_pv = [&](int j, float alpha) {
      const int s = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_full[s], (j >> 1) & 1, abort_flag))) return false;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_base + 256 + s * 128 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(r[i]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pv_empty[s]);
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], (j >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const int key0 = j * kAtTile;
      const bool tail = key0 + kAtTile > p.sk;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_base + s * 128 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]);
          if (tail && key0 + c * 32 + i >= p.sk) v = -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m_run == -INFINITY ? 0.f : exp2f(m_run - m_safe);
      m_run = m_new;
      // P of the previous step must have been consumed by its MMA before the tile is overwritten
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->p_empty, (j & 1) ^ 1, abort_flag))) { ok = false; break; }
      // pass 2: probabilities -> shared memory (A-operand layout: two atoms of 64 keys, 128-byte
      // rows, 16-byte chunks XOR-swizzled with the row index), row sum
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_base + s * 128 + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_safe));
          float bq = exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_safe));
          if (tail) {
            if (key0 + c * 32 + i >= p.sk) a = 0.f;
            if (key0 + c * 32 + i + 1 >= p.sk) bq = 0.f;
          }
          sum += a + bq;
          packed[i >> 1] = pack_bf16x2(a, bq);
        }
        uint8_t* atom = sp + (c >> 1) * (kAtTileBytes / 2) + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c & 1) * 4 + q4;                 // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      l_run = l_run * alpha + sum;
      // S buffer free for the tile after next; P visible to the tensor core
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->s_empty[s]);
        mbar_arrive(&bars->p_full);
      }
      // fold in the previous step's P V while the tensor core works on this step
      if (j > 0) ok = consume_pv(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (ok && n_tiles > 0) ok = consume_pv(n_tiles - 1, alpha_prev);
    if (!ok) {
      if (lane == 0) report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 13, blockIdx.x);
    } else {
      const int q_idx = qt * kAtTile + row;
      if (q_idx < p.sq) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.out + static_cast<long long>(q_row0 + row) * p.ld + head * kAtD;
#pragma unroll
        for (int i = 0; i < kAtD; i += 8) {
          uint4 v;
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int t = 0; t < 4; ++t) w[t] = pack_bf16x2(o[i + 2 * t] * inv, o[i + 2 * t + 1] * inv);
          *reinterpret_cast<uint4*>(dst + i) = v;
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// v [batch * sk][ld] (head h at columns h * 128 ...) -> vt [batch * heads * 128][sk_pad]
__global__ void transpose_v_kernel(const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ vt, long long ld,
                                   int sk, int sk_pad, int heads) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int bh = blockIdx.z, b = bh / heads, h = bh % heads;
  const int key0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int key = key0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x)
      tile[i][j] = key < sk ? v[(static_cast<long long>(b) * sk + key) * ld + h * kAtD + d0 + j] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const long long row = (static_cast<long long>(bh) * kAtD + d0 + i) * sk_pad;
    for (int j = threadIdx.x; j < 64; j += blockDim.x)
      if (key0 + j < sk_pad) vt[row + key0 + j] = tile[j][i];
  }
}

}  // namespace b200

namespace b200 {
// defined in gemm_tcgen05.cu
int make_kmajor_map(CUtensorMap* out, const void* base, int elem_bytes, long long rows, long long k,
                    long long ld, int box_rows);
}  // namespace b200

using namespace b200;

static inline int attn_tc_sk_pad(int sk) { return (sk + 63) / 64 * 64; }

// Scratch for the transposed V: [batch * heads * 128][sk rounded up to 64] bf16.
B200_API long long b200_attn_tc_workspace_bytes(int batch, int heads, int sk) {
  return static_cast<long long>(batch) * heads * kAtD * attn_tc_sk_pad(sk) * 2;
}

// Dense attention, head dim 128, bf16: q [batch * sq][heads * 128], k / v [batch * sk][heads * 128]
// (contiguous), out like q. softmax(q k^T * scale) v per (batch, head).
B200_API int b200_attn_tc(const void* q, const void* k, const void* v, void* out, int batch, int sq, int sk,
                          int heads, float scale, void* vt_scratch, void* status, cudaStream_t stream) {
  if (batch <= 0 || sq <= 0 || sk <= 0) return 0;
  if (vt_scratch == nullptr) return -2;
  const long long ld = static_cast<long long>(heads) * kAtD;
  const int sk_pad = attn_tc_sk_pad(sk);
  dim3 tgrid((sk_pad + 63) / 64, kAtD / 64, batch * heads);
  transpose_v_kernel<<<tgrid, dim3(32, 8), 0, stream>>>(static_cast<const __nv_bfloat16*>(v),
                                                        static_cast<__nv_bfloat16*>(vt_scratch), ld, sk, sk_pad, heads);
  CUtensorMap tq, tk, tv;
  int rc = make_kmajor_map(&tq, q, 2, static_cast<long long>(batch) * sq, ld, ld, 128);
  if (rc) return rc;
  rc = make_kmajor_map(&tk, k, 2, static_cast<long long>(batch) * sk, ld, ld, 128);
  if (rc) return rc;
  rc = make_kmajor_map(&tv, vt_scratch, 2, static_cast<long long>(batch) * heads * kAtD, sk_pad, sk_pad, 128);
  if (rc) return rc;
  AttnTcParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld = ld;
  p.sq = sq; p.sk = sk; p.heads = heads; p.batch = batch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<DeviceStatus*>(status);
  const int smem = 6 * kAtTileBytes + static_cast<int>(sizeof(AttnTcBarriers)) + 1024;
  static PerDeviceOnce configured;
  if (configured.first_time()) {
    if (cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
  }
  dim3 grid((sq + kAtTile - 1) / kAtTile, heads, batch);
  attn_tc_kernel<<<grid, kAtThreads, smem, stream>>>(p, tq, tk, tv);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
