// Dense (non-causal) flash attention on the 5th-generation tensor cores, head dim 128, for the
// long joint sequences of the DiT families (thousands to tens of thousands of tokens), in two
// operand modes of one kernel:
//   bf16   S = Q K^T with tcgen05.mma.kind::f16
//   int8   "SageAttention": Q quantised to int8 with one scale per row, K with one scale per tile of
//          128 keys after its per-head mean over the sequence has been removed (softmax cannot see
//          a vector added to every key), S = Q8 K8^T with tcgen05.mma.kind::i8 (s32 accumulators);
//          the dequantisation is one fused multiply-add inside the exponent; P V stays bf16.
//          Replaces the reference's five-launch host sequence around sage_attn_int8_v1
//          (src/HartsyInference.Cuda/Kernels/attention/sage_attn_int8_v1.cu:394-480, sage_attn_int8.cu
//          sage_k_mean_f32 / sage_quant_q_int8_f32 / sage_quant_k_int8_f32; CudaBackend.cs:7623-7695)
//          and its cuDNN SDPA path (CudnnSdpa.cs).
//
// One CTA owns TWO tiles of 128 query rows of one head and walks the keys in tiles of 128:
//   warp 0       TMA producer: both Q tiles once, then K tile [128 keys x 128] and V^T tile [128
//                dims x 128 keys] per step into separate rings
//   warp 1       one thread issues every tcgen05.mma. TMEM holds S0 | S1 | O0 | O1 (4 x 128 columns).
//                Per key tile j and query tile t: O_t += P_t(j) V_j with P_t read from TMEM (it lives in
//                the first 64 columns of S_t, written there by the softmax warps), directly
//                followed by S_t(j+1) = Q_t K_{j+1}^T, so the two query tiles alternate on the tensor
//                core and each one's softmax overlaps the other one's matrix products
//   warps 4..7   softmax of query tile 0; warps 8..11 softmax of query tile 1 (warps 2, 3 idle, so
//                that each role is a whole warp group and registers can be moved between the
//                groups with setmaxnreg). Thread r owns query
//                row r (TMEM lane r): reads its S row (tcgen05.ld), applies scale (and the int8
//                dequantisation), keeps running maximum / sum in the exp2 domain, writes P as bf16
//                pairs back into TMEM (tcgen05.st). O is never read back during the loop: the
//                running maximum is only raised (and O rescaled in TMEM) when it would grow by
//                more than 2^8, otherwise the stale maximum keeps being used, which is exact
//                because the final division by the row sum uses the same maximum.
//
// V is consumed transposed ([head dim][keys], keys contiguous) so that both MMAs use K-major
// operands; the transpose (and the int8 quantisation) is a small kernel of its own in front.
#include "comm.cuh"

namespace b200 {

constexpr int kFaD = 128;
constexpr int kFaTile = 128;              // rows of one query tile and keys per step
constexpr int kFaThreads = 384;           // warp group 0: producer, MMA (+ 2 idle warps); groups 1, 2: softmax of tile 0, 1
constexpr float kFaRescaleGap = 8.f;      // raise the running maximum only beyond this many powers of two

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct FaBarriers {
  uint64_t q_full;
  uint64_t k_full[3], k_empty[3];
  uint64_t v_full[3], v_empty[3];
  uint64_t s_full[2];        // S_t(j) is in TMEM
  uint64_t p_ready[2];       // P_t(j) is in TMEM (and O_t rescaled if needed): 4 warp arrivals
  uint64_t o_done[2];        // O_t += P_t(j) V_j has completed
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct FaParams {
  __nv_bfloat16* out;        // [batch * sq][ld_out]
  long long ld_out;
  int sq, sk, heads, batch;
  float scale_log2;          // softmax scale * log2(e)
  // int8 mode: q_scale [batch * heads][sq_pad] (one per query row), k_scale [batch * heads][key tiles]
  const float* q_scale;
  const float* k_scale;
  int sq_pad;
  DeviceStatus* status;
  // Segmented operands (the sequence-parallel exchange below): the key buffers hold `nseg`
  // segments of `seg_pad` rows (a multiple of 128) of which the first `seg_len` are real; segment
  // s was written by rank s and is complete once seg_flags[s] has reached seg_target. The walk
  // over the keys starts with segment `seg_first` (this rank's own, which arrives first). Query
  // rows use the same layout; the output rows of query segment s go to out_seg[s] (rank s's
  // buffer, row = index inside the segment, column offset out_col0). A plain call has one segment
  // and no flags.
  int n_tiles, tiles_per_seg, nseg, seg_len, seg_first, seg_pad;
  int seg_mode;
  int q_seg_base;            // segment index of query row 0 (context-parallel form: the queries are this rank's only)
  int pull;                  // 1: segment s of K / V^T stays in rank s's memory and is read from there, tile by tile,
                             // through the tensor maps of FaPeerMaps (rows / columns counted inside the segment)
  const uint32_t* seg_flags;
  uint32_t seg_target;
  long long wait_budget;
  __nv_bfloat16* out_seg[8];
  long long out_col0;
  uint32_t* done_flags[8];   // rank s's "outputs have arrived" counter
  uint32_t* done_ctr;        // CTAs of this launch that have finished
};

// K and V^T tensor maps per source rank for the pull form (ring-style context parallelism without
// copies: the TMA unit loads each key / value tile straight from the owner's memory over NVLink; plain
// tiled loads, no cluster multicast).
struct FaPeerMaps {
  CUtensorMap k[8];
  CUtensorMap vt[8];
};

// Buffer tile (index into the segmented key buffers) and number of real keys of walk step j.
__device__ __forceinline__ void fa_key_tile(const FaParams& p, int j, int& buf_tile, int& valid, int& seg) {
  const int sg = j / p.tiles_per_seg, lt = j - sg * p.tiles_per_seg;
  seg = p.seg_first + sg;
  if (seg >= p.nseg) seg -= p.nseg;
  buf_tile = seg * p.tiles_per_seg + lt;
  valid = min(kFaTile, p.seg_len - lt * kFaTile);
}

template <bool kI8>
__global__ void __launch_bounds__(kFaThreads, 1)
attn_fa_kernel(const FaParams p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_vt,
               const __grid_constant__ FaPeerMaps peers) {
  constexpr int kQkTileBytes = kI8 ? 128 * 128 : 128 * 128 * 2;   // one Q or K tile
  constexpr int kQkAtoms = kI8 ? 1 : 2;                           // 128-byte-wide swizzle atoms per tile
  constexpr int kVTileBytes = 128 * 128 * 2;
  constexpr int kStages = kI8 ? 3 : 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;                                           // two Q tiles
  uint8_t* sk = sq + 2 * kQkTileBytes;                          // K ring
  uint8_t* sv = sk + kStages * kQkTileBytes;                    // V^T ring
  FaBarriers* bars = reinterpret_cast<FaBarriers*>(sv + kStages * kVTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt2 = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int n_tiles = p.n_tiles;
  const int q_row0 = b * p.sq + qt2 * 2 * kFaTile;     // row of the CTA's first query in [batch * sq]
  const int k_row0 = b * p.sk;
  const int vt_row0 = (b * p.heads + head) * kFaD;     // row in the [batch * heads * 128][sk_pad] matrix
  const int col0 = head * kFaD;                        // element (= byte for int8) column of the head
  // the second query tile may lie completely past the end of the sequence
  const bool tile1 = qt2 * 2 * kFaTile + kFaTile < p.sq;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_ready[t], 4);
      mbar_init(&bars->o_done[t], 1);
    }
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
  constexpr uint32_t kIdescS = kI8 ? make_idesc(128, 128, kFmtS8, kFmtS8, 2) : make_idesc(128, 128, kFmtBf16, kFmtBf16);
  constexpr uint32_t kIdescPV = make_idesc(128, 128, kFmtBf16, kFmtBf16);

  // The softmax threads keep a whole score row in registers; the producer and MMA warps need few.
  // Registers move between the warp groups accordingly (launch: 168 per thread).
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int nq = tile1 ? 2 : 1;
      bool ok = true;
      // a segment written by a peer: its flag first, then a proxy fence, because the loads below
      // are issued by the TMA unit and the peer's data arrived as ordinary stores
      auto wait_segment = [&](int seg) {
        if (p.seg_flags == nullptr) return true;
        if (!wait_flag_geq(p.seg_flags + seg, p.seg_target, p.wait_budget)) {
          *abort_flag = 1;
          return false;
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
        return true;
      };
      if (p.seg_mode) {
        const int first = qt2 * 2 * kFaTile, last = first + nq * kFaTile - 1;
        for (int seg = first / p.seg_pad; seg <= last / p.seg_pad && ok; ++seg) ok = wait_segment(seg + p.q_seg_base);
      }
      if (ok) {
        mbar_arrive_expect_tx(&bars->q_full, nq * kQkTileBytes);
        for (int t = 0; t < nq; ++t)
          for (int a = 0; a < kQkAtoms; ++a)
            tma_load_2d(sq + t * kQkTileBytes + a * (kQkTileBytes / kQkAtoms), &tm_q, &bars->q_full,
                        col0 + a * 64, q_row0 + t * kFaTile);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
        int bt, valid, seg;
        fa_key_tile(p, j, bt, valid, seg);
        if (p.seg_mode && j % p.tiles_per_seg == 0 && !wait_segment(seg)) { ok = false; break; }
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        // pull form: the tile is read from its owner's buffers (tile index inside the segment)
        const CUtensorMap* mk = p.pull ? &peers.k[seg] : &tm_k;
        const CUtensorMap* mv = p.pull ? &peers.vt[seg] : &tm_vt;
        const int tile_at = p.pull ? bt - seg * p.tiles_per_seg : bt;
        mbar_arrive_expect_tx(&bars->k_full[s], kQkTileBytes);
        for (int a = 0; a < kQkAtoms; ++a)
          tma_load_2d(sk + s * kQkTileBytes + a * (kQkTileBytes / kQkAtoms), mk, &bars->k_full[s],
                      col0 + a * 64, k_row0 + tile_at * kFaTile);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars->v_full[s], kVTileBytes);
        tma_load_2d(sv + s * kVTileBytes, mv, &bars->v_full[s], tile_at * kFaTile, vt_row0);
        tma_load_2d(sv + s * kVTileBytes + kVTileBytes / 2, mv, &bars->v_full[s], tile_at * kFaTile + 64, vt_row0);
      }
      if (!ok) report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 21, blockIdx.x);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const int nq = tile1 ? 2 : 1;
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      // S_t(j) = Q_t K_j^T into TMEM columns [t * 128, t * 128 + 128)
      auto issue_s = [&](int t, int j) {
        const int s = j % kStages;
        const uint32_t d_tmem = tmem_base + t * 128;
#pragma unroll
        for (int a = 0; a < kQkAtoms; ++a) {
          const uint64_t ad = make_desc_sw128(smem_u32(sq + t * kQkTileBytes + a * (kQkTileBytes / kQkAtoms)));
          const uint64_t bd = make_desc_sw128(smem_u32(sk + s * kQkTileBytes + a * (kQkTileBytes / kQkAtoms)));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (kI8) mma_i8_ss(d_tmem, ad + 2 * k, bd + 2 * k, kIdescS, (a | k) != 0);
            else mma_bf16_ss(d_tmem, ad + 2 * k, bd + 2 * k, kIdescS, (a | k) != 0);
          }
        }
        tc_commit(&bars->s_full[t]);
      };
      if (ok) ok = mbar_wait(&bars->k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < nq; ++t) issue_s(t, 0);
        tc_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
        for (int t = 0; t < nq && ok; ++t) {
          if (!mbar_wait(&bars->p_ready[t], j & 1, abort_flag)) { ok = false; break; }
          if (t == 0 && !mbar_wait(&bars->v_full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          // O_t += P_t V_j: A = P_t in TMEM (64 columns of bf16 pairs), B = V^T tile (two atoms of 64 keys)
          const uint32_t d_tmem = tmem_base + 256 + t * 128;
          const uint32_t a_tmem = tmem_base + t * 128;
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            const uint64_t bd = make_desc_sw128(smem_u32(sv + s * kVTileBytes + a * (kVTileBytes / 2)));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_bf16_ts(d_tmem, a_tmem + (a * 4 + k) * 8, bd + 2 * k, kIdescPV, (j | a | k) != 0);
          }
          tc_commit(&bars->o_done[t]);
          if (t == nq - 1) tc_commit(&bars->v_empty[s]);
          if (j + 1 < n_tiles) {
            const int s1 = (j + 1) % kStages;
            if (t == 0 && !mbar_wait(&bars->k_full[s1], static_cast<uint32_t>(((j + 1) / kStages) & 1), abort_flag)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_s(t, j + 1);       // executes after the P_t V_j above: it overwrites the columns P_t lives in
            if (t == nq - 1) tc_commit(&bars->k_empty[s1]);
          }
        }
      }
      if (!ok) report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 22, blockIdx.x);
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ------------------------------------------------------------------------- softmax warps
    const int t = (warp >> 2) - 1;                        // query tile of this warp group
    const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;                  // query row inside the tile = TMEM lane
    const int q_idx = qt2 * 2 * kFaTile + t * kFaTile + row;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_col = lane_base + t * 128, o_col = lane_base + 256 + t * 128;
    // position of the row inside its query segment (a plain call has one segment of sq rows)
    const int q_seg = p.seg_mode ? q_idx / p.seg_pad : 0;
    const int q_local = q_idx - q_seg * p.seg_pad;
    const bool q_valid = p.seg_mode ? q_local < p.seg_len : q_idx < p.sq;
    if (t == 0 || tile1) {
      float m_run = -INFINITY, l_run = 0.f;
      float qs = p.scale_log2;
      bool ok = true;
      const float* ksc = kI8 ? p.k_scale + static_cast<long long>(b * p.heads + head) * n_tiles : nullptr;
      for (int j = 0; j < n_tiles && ok; ++j) {
        int bt, valid, seg;
        fa_key_tile(p, j, bt, valid, seg);
        if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[t], j & 1, abort_flag))) { ok = false; break; }
        tc_fence_after_sync();
        // scores -> exp2 domain: x = raw * c (bf16: c = scale; int8: c = q row scale * K tile scale * scale).
        // Both scales are read past the wait and around L1: in a segmented call a peer wrote them, and
        // they arrive with the segment.
        if (kI8 && j == 0)
          qs *= q_valid ? __ldcg(p.q_scale + static_cast<long long>(b * p.heads + head) * p.sq_pad + q_idx) : 0.f;
        const float c = kI8 ? qs * __ldcg(ksc + bt) : qs;
        const bool tail = valid < kFaTile;
        // the raw S row of this thread in two halves: the second half is in flight while the maximum
        // of the first is taken; eight independent running maxima keep the compare pipe busy instead
        // of one chain of 128 dependent compares
        uint32_t r[128];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld_32x32(s_col + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[cc * 32]));
        tmem_ld_wait();
#pragma unroll
        for (int cc = 2; cc < 4; ++cc) tmem_ld_32x32(s_col + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[cc * 32]));
        float mx;
        if (kI8) {
          int mi[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) mi[u] = tail && u >= valid ? -(1 << 22) : static_cast<int>(r[u]);
#pragma unroll
          for (int i = 8; i < 64; ++i) mi[i & 7] = max(mi[i & 7], tail && i >= valid ? -(1 << 22) : static_cast<int>(r[i]));
          tmem_ld_wait();
#pragma unroll
          for (int i = 64; i < 128; ++i) mi[i & 7] = max(mi[i & 7], tail && i >= valid ? -(1 << 22) : static_cast<int>(r[i]));
          mx = static_cast<float>(max(max(max(mi[0], mi[1]), max(mi[2], mi[3])), max(max(mi[4], mi[5]), max(mi[6], mi[7])))) * c;
        } else {
          float mf[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) mf[u] = tail && u >= valid ? -INFINITY : __uint_as_float(r[u]);
#pragma unroll
          for (int i = 8; i < 64; ++i) mf[i & 7] = fmaxf(mf[i & 7], tail && i >= valid ? -INFINITY : __uint_as_float(r[i]));
          tmem_ld_wait();
#pragma unroll
          for (int i = 64; i < 128; ++i) mf[i & 7] = fmaxf(mf[i & 7], tail && i >= valid ? -INFINITY : __uint_as_float(r[i]));
          mx = fmaxf(fmaxf(fmaxf(mf[0], mf[1]), fmaxf(mf[2], mf[3])), fmaxf(fmaxf(mf[4], mf[5]), fmaxf(mf[6], mf[7]))) * c;
        }
        if (tail) {
          // keys past the end: the most negative value the exponent path below maps far below any maximum
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i >= valid) r[i] = kI8 ? static_cast<uint32_t>(-(1 << 22)) : 0xff800000u;
        }
        // raise the running maximum only when it would grow by more than the gap (or on the first
        // tile); a warp decides together because the O rescale below is a warp-wide TMEM access
        const bool grow = mx > m_run + kFaRescaleGap;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_run, mx);
          const float alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run - m_new);
          if (j > 0) {
            // O_t must be complete up to tile j - 1 before it is rescaled
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->o_done[t], (j - 1) & 1, abort_flag))) { ok = false; break; }
            tc_fence_after_sync();
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t o[32];
              tmem_ld_32x32(o_col + cc * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32x32(o_col + cc * 32, o);
            }
            tmem_st_wait();
          }
          l_run *= alpha;
          m_run = m_new;
        }
        const float m_safe = m_run == -INFINITY ? 0.f : m_run;
        // p = 2^(raw * c - m): one fused multiply-add and one ex2 per score. int8: the s32 score is
        // turned into 12582912 + s by an integer add on its bits (exact for |s| < 2^22) and the
        // constant is folded into the subtrahend, so no conversion instruction is spent
        const float sub = kI8 ? fmaf(12582912.f, c, m_safe) : m_safe;
        float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t packed[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t r0 = r[cc * 64 + 2 * i], r1 = r[cc * 64 + 2 * i + 1];
            const float f0 = kI8 ? __uint_as_float(r0 + 0x4B400000u) : __uint_as_float(r0);
            const float f1 = kI8 ? __uint_as_float(r1 + 0x4B400000u) : __uint_as_float(r1);
            const float a = fast_exp2(fmaf(f0, c, -sub));
            const float bq = fast_exp2(fmaf(f1, c, -sub));
            sums[i & 3] += a + bq;
            packed[i] = pack_bf16x2(a, bq);
          }
          tmem_st_32x32(s_col + cc * 32, packed);      // P_t: columns [0, 64) of S_t
        }
        tmem_st_wait();
        l_run += (sums[0] + sums[1]) + (sums[2] + sums[3]);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[t]);
      }
      if (ok && n_tiles > 0)
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_done[t], (n_tiles - 1) & 1, abort_flag));
      if (!ok) {
        if (lane == 0) report_status(p.status, kWaitTimeout, kKernelAttnPrefill, 23, blockIdx.x);
      } else {
        tc_fence_after_sync();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.seg_mode
            ? p.out_seg[q_valid ? q_seg + p.q_seg_base : 0] + static_cast<long long>(q_local) * p.ld_out + p.out_col0 + col0
            : p.out + static_cast<long long>(q_row0 + t * kFaTile + row) * p.ld_out + col0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_col + c * 32, r);
          tmem_ld_wait();
          if (q_valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
              for (int u = 0; u < 4; ++u)
                w[u] = pack_bf16x2(__uint_as_float(r[i + 2 * u]) * inv, __uint_as_float(r[i + 2 * u + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
            }
          }
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
  if (p.done_ctr != nullptr && threadIdx.x == 0) {
    // the last CTA of the launch tells every rank that this rank's share of its output is there.
    // The softmax threads' stores to the peers are ordered before this thread by the barrier above;
    // one system-scope fence here then covers all of them (fences are cumulative), instead of one
    // fence per storing thread
    __threadfence_system();
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(p.done_ctr, 1u) == total - 1) {
      atomicExch(p.done_ctr, 0u);
      fence_acq_rel_sys();
      for (int s = 0; s < p.nseg; ++s) red_relaxed_sys_add(p.done_flags[s], 1u);
    }
  }
}

// v [batch * sk][ld] (head h at columns h * 128 ...) -> vt [batch * heads * 128][sk_pad], zero padded
__global__ void fa_transpose_v_kernel(const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ vt, long long ld,
                                      int sk, int sk_pad, int heads) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int bh = blockIdx.z, b = bh / heads, h = bh % heads;
  const int key0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int key = key0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x)
      tile[i][j] = key < sk ? v[(static_cast<long long>(b) * sk + key) * ld + h * kFaD + d0 + j] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const long long row = (static_cast<long long>(bh) * kFaD + d0 + i) * sk_pad;
    for (int j = threadIdx.x; j < 64; j += blockDim.x)
      if (key0 + j < sk_pad) vt[row + key0 + j] = tile[j][i];
  }
}

// ---- SageAttention preparation --------------------------------------------------------------
// Column sums of K per (batch, head): ksum [batch * heads][128] fp32 (zeroed by the caller), so that
// mean = ksum / sk. grid (chunks of 256 keys, batch * heads), 128 threads (one per dim).
__global__ void sage_k_sum_kernel(const __nv_bfloat16* __restrict__ k, float* __restrict__ ksum, long long ld, int sk,
                                  int heads) {
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int key0 = blockIdx.x * 256, key1 = min(sk, key0 + 256);
  float acc = 0.f;
  for (int key = key0; key < key1; ++key)
    acc += __bfloat162float(k[(static_cast<long long>(b) * sk + key) * ld + h * kFaD + threadIdx.x]);
  atomicAdd(ksum + static_cast<long long>(bh) * kFaD + threadIdx.x, acc);
}

// Row quantisation to int8: one warp per (row, head). x [batch * s][ld] bf16 -> out [batch * s][ld]
// int8 (same column layout), scale [batch * heads][s_pad] fp32 = max|row| / 127. `center` (optional,
// [batch * heads][128], with `center_div`) is subtracted first: the K mean.
__global__ void sage_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ out,
                                       float* __restrict__ scale, const float* __restrict__ center, float center_div,
                                       long long ld, int s, int s_pad, int heads, int batch) {
  const int lane = threadIdx.x & 31;
  const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(batch) * s * heads;
  if (w >= total) return;
  const int h = static_cast<int>(w % heads);
  const long long row = w / heads;                 // row in [batch * s]
  const int b = static_cast<int>(row / s), tok = static_cast<int>(row % s);
  const __nv_bfloat16* src = x + row * ld + h * kFaD + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float v[4];
  v[0] = __bfloat162float(hp[0].x); v[1] = __bfloat162float(hp[0].y);
  v[2] = __bfloat162float(hp[1].x); v[3] = __bfloat162float(hp[1].y);
  if (center) {
    const float* c = center + static_cast<long long>(b * heads + h) * kFaD + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] -= c[i] / center_div;
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float sc = fmaxf(amax, 1e-12f) / 127.f;
  const float inv = 1.f / sc;
  uint32_t q = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int iv = max(-127, min(127, __float2int_rn(v[i] * inv)));
    q |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(iv))) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(out + row * ld + h * kFaD + lane * 4) = q;
  if (lane == 0) scale[static_cast<long long>(b * heads + h) * s_pad + tok] = sc;
}

// K quantisation with one scale per tile of 128 keys: grid (key tiles, batch * heads), 256 threads;
// thread (row, half) handles 64 dims of one key. k [batch * sk][ld] bf16 -> out int8 (same layout),
// scale [batch * heads][key tiles] = max|tile - mean| / 127. `center` [batch * heads][128] holds the
// column sums of K (mean = center / sk).
__global__ void __launch_bounds__(256) sage_quant_k_tiles_kernel(const __nv_bfloat16* __restrict__ k,
                                                                 int8_t* __restrict__ out, float* __restrict__ scale,
                                                                 const float* __restrict__ center, long long ld, int sk,
                                                                 int heads) {
  __shared__ float wmax[8];
  const int tile = blockIdx.x, bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int n_tiles = gridDim.x;
  const int key = tile * kFaTile + (threadIdx.x >> 1), d0 = (threadIdx.x & 1) * 64;
  const bool valid = key < sk;
  float v[64];
  float amax = 0.f;
  const float inv_sk = 1.f / static_cast<float>(sk);
  if (valid) {
    const __nv_bfloat16* src = k + (static_cast<long long>(b) * sk + key) * ld + h * kFaD + d0;
    const float* c = center + static_cast<long long>(bh) * kFaD + d0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i * 8);
      const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(hp[u]);
        v[i * 8 + 2 * u] = f.x - c[i * 8 + 2 * u] * inv_sk;
        v[i * 8 + 2 * u + 1] = f.y - c[i * 8 + 2 * u + 1] * inv_sk;
        amax = fmaxf(amax, fmaxf(fabsf(v[i * 8 + 2 * u]), fabsf(v[i * 8 + 2 * u + 1])));
      }
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wmax[i]);
  const float sc = fmaxf(amax, 1e-12f) / 127.f;
  if (threadIdx.x == 0) scale[static_cast<long long>(bh) * n_tiles + tile] = sc;
  if (!valid) return;
  const float inv = 1.f / sc;
  int8_t* dst = out + (static_cast<long long>(b) * sk + key) * ld + h * kFaD + d0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 q;
    uint32_t* qw = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int iv = max(-127, min(127, __float2int_rn(v[i * 16 + w * 4 + e] * inv)));
        word |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(iv))) << (8 * e);
      }
      qw[w] = word;
    }
    *reinterpret_cast<uint4*>(dst + i * 16) = q;
  }
}


// ---- Ulysses exchange fused around the attention kernel ------------------------------------------
// Sequence parallelism: every rank holds `s_l` tokens of all heads and needs all tokens of its
// heads / world heads. Instead of three all-to-all collectives in front of the attention and one
// behind it, the quantisation kernel below stores its results straight into the destination rank's
// operand buffers (ordinary 16-byte peer stores into the symmetric heap) and raises one arrival
// counter per (destination, source); the attention kernel starts with its own segment, waits per
// segment for the others, and stores its output rows into the owning rank's output buffer. One
// tiny kernel in front of the consumer waits for the `world` output shares.
// Replaces the reference's exchange of K / V through a host-side rendezvous
// (src/HartsyInference.Diffusion/Utilities/CpKvExchange.cs:48-135, called from
// Models/Denoisers/DiTBlocks/WanVideoBlock.cs:193-195).
//
// Flag words of one rank (cumulative counters, one exchange adds one): [0, 8) operand segment of
// source s has arrived; [8, 16) K column sums of source s have arrived; [16] output shares.
constexpr int kUlyFlagArrive = 0, kUlyFlagKsum = 8, kUlyFlagDone = 16, kUlyFlagWords = 32;

struct UlyPush {
  int cp;                      // 1: context-parallel form (K / V of all heads to every rank, Q stays here)
  const __nv_bfloat16* q;      // local [s_l][heads * 128]
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int s_l, s_pad, heads, hl, rank, world;
  void* qbuf[8];               // rank d's Q operand [world * s_pad][hl * 128] (int8 or bf16)
  void* kbuf[8];
  __nv_bfloat16* vtbuf[8];     // rank d's V^T [hl * 128][world * s_pad]
  float* qscale[8];            // rank d's [hl][world * s_pad]
  float* kscale[8];            // rank d's [hl][world * tiles]
  const float* ksum_in;        // local [world][heads][128]: every rank's K column sums
  const uint32_t* flags_local;
  uint32_t* flags[8];          // rank d's flag words
  uint32_t* ctr;               // CTAs of this launch that have finished
  uint32_t target;
  float inv_total;             // 1 / (tokens of the whole sequence)
  long long wait_budget;
  DeviceStatus* status;
};

// Local column sums [heads][128] -> every rank's ksum_in[rank], then one arrival per destination.
struct UlyTabs {
  float* ksum_in[8];
  uint32_t* flags[8];
};
__global__ void __launch_bounds__(1024) uly_ksum_push_kernel(const float* __restrict__ ksum_local, const UlyTabs tabs, int n,
                                                             int rank, int world) {
  for (int d = 0; d < world; ++d) {
    float* dst = tabs.ksum_in[d] + static_cast<long long>(rank) * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = ksum_local[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    for (int d = 0; d < world; ++d) red_relaxed_sys_add(tabs.flags[d] + kUlyFlagKsum + rank, 1u);
  }
}

// grid (token tiles of 128, heads), 256 threads: thread (row, half) owns 64 dims of one token.
template <bool kI8>
__global__ void __launch_bounds__(256) uly_push_kernel(const UlyPush p) {
  __shared__ float mean[kFaD];
  __shared__ float wmax[8];
  __shared__ int wait_ok;
  __shared__ __align__(16) __nv_bfloat16 vtile[kFaTile][kFaD + 8];
  const int tile = blockIdx.x, head = blockIdx.y;
  // Ulysses: the head belongs to one destination rank. Context parallel: every rank gets K / V of every
  // head (p.hl == p.heads), the queries stay local (row = token, no segment offset).
  const int dst = p.cp ? p.rank : head / p.hl, hi = p.cp ? head : head - dst * p.hl;
  const bool pull = p.cp == 2;          // K / V^T stay in this rank's own region (peers read them from here)
  const int first_dst = pull ? p.rank : p.cp ? 0 : dst, last_dst = pull ? p.rank : p.cp ? p.world - 1 : dst;
  const int row = threadIdx.x >> 1, d0 = (threadIdx.x & 1) * 64;
  const int tok = tile * kFaTile + row;
  const bool valid = tok < p.s_l;
  const long long ld_in = static_cast<long long>(p.heads) * kFaD;
  const long long ld_out = static_cast<long long>(p.hl) * kFaD;
  const long long seg_row = (pull ? 0 : static_cast<long long>(p.rank) * p.s_pad) + tok;     // row in the destination K / V buffers
  const long long q_row = p.cp ? tok : seg_row;
  const long long q_rows = p.cp ? p.s_pad : static_cast<long long>(p.world) * p.s_pad;
  const int tiles = p.s_pad / kFaTile;

  if (kI8) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int s = 0; s < p.world && ok; ++s)
        ok = wait_flag_geq(p.flags_local + kUlyFlagKsum + s, p.target, p.wait_budget) ? 1 : 0;
      wait_ok = ok;
      if (!ok) report_status(p.status, kWaitTimeout, kKernelAllToAll, 1, blockIdx.x);
    }
    __syncthreads();
    if (threadIdx.x < kFaD) {
      float acc = 0.f;
      if (wait_ok)
        for (int s = 0; s < p.world; ++s)
          acc += __ldcg(p.ksum_in + (static_cast<long long>(s) * p.heads + head) * kFaD + threadIdx.x);
      mean[threadIdx.x] = acc * p.inv_total;
    }
    __syncthreads();
  }

  auto load64 = [&](const __nv_bfloat16* src, float (&out)[64]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i * 8);
      const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(hp[u]);
        out[i * 8 + 2 * u] = f.x;
        out[i * 8 + 2 * u + 1] = f.y;
      }
    }
  };
  auto store_q8 = [&](int8_t* dstp, const float (&v)[64], float inv) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q;
      uint32_t* qw = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int iv = max(-127, min(127, __float2int_rn(v[i * 16 + w * 4 + e] * inv)));
          word |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(iv))) << (8 * e);
        }
        qw[w] = word;
      }
      *reinterpret_cast<uint4*>(dstp + i * 16) = q;
    }
  };

  // ---- Q: one scale per row
  if (kI8) {
    float v[64];
    float amax = 0.f;
    if (valid) {
      load64(p.q + static_cast<long long>(tok) * ld_in + head * kFaD + d0, v);
#pragma unroll
      for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float sc = fmaxf(amax, 1e-12f) / 127.f;
    if (valid) {
      store_q8(static_cast<int8_t*>(p.qbuf[dst]) + q_row * ld_out + hi * kFaD + d0, v, 1.f / sc);
      if (d0 == 0) p.qscale[dst][static_cast<long long>(hi) * q_rows + q_row] = sc;
    }
  } else if (valid) {
    const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<long long>(tok) * ld_in + head * kFaD + d0);
    uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.qbuf[dst]) + q_row * ld_out + hi * kFaD + d0);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = src[i];
  }

  // ---- K: mean removed, one scale per tile of 128 keys
  if (kI8) {
    float v[64];
    float amax = 0.f;
    if (valid) {
      load64(p.k + static_cast<long long>(tok) * ld_in + head * kFaD + d0, v);
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        v[i] -= mean[d0 + i];
        amax = fmaxf(amax, fabsf(v[i]));
      }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = wmax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wmax[i]);
    const float sc = fmaxf(amax, 1e-12f) / 127.f;
    for (int d = first_dst; d <= last_dst; ++d) {
      if (threadIdx.x == 0) p.kscale[d][static_cast<long long>(hi) * p.world * tiles + p.rank * tiles + tile] = sc;
      if (valid) store_q8(static_cast<int8_t*>(p.kbuf[d]) + seg_row * ld_out + hi * kFaD + d0, v, 1.f / sc);
    }
  } else if (valid) {
    const uint4* src = reinterpret_cast<const uint4*>(p.k + static_cast<long long>(tok) * ld_in + head * kFaD + d0);
    uint4 kv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) kv[i] = src[i];
    for (int d = first_dst; d <= last_dst; ++d) {
      uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.kbuf[d]) + seg_row * ld_out + hi * kFaD + d0);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = kv[i];
    }
  }

  // ---- V: transposed through shared memory; rows past the end become zeros
  {
    uint4* srow = reinterpret_cast<uint4*>(&vtile[row][d0]);
    if (valid) {
      const uint4* src = reinterpret_cast<const uint4*>(p.v + static_cast<long long>(tok) * ld_in + head * kFaD + d0);
#pragma unroll
      for (int i = 0; i < 8; ++i) srow[i] = src[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) srow[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    // thread (dim, half) writes 64 consecutive tokens of one dim
    const int dim = threadIdx.x >> 1, t0 = (threadIdx.x & 1) * 64;
    const long long off = pull ? (static_cast<long long>(hi) * kFaD + dim) * p.s_pad + tile * kFaTile + t0
                               : (static_cast<long long>(hi) * kFaD + dim) * p.world * p.s_pad +
                                     static_cast<long long>(p.rank) * p.s_pad + tile * kFaTile + t0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 o;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int u = 0; u < 8; ++u) e[u] = vtile[t0 + i * 8 + u][dim];
      for (int d = first_dst; d <= last_dst; ++d) *reinterpret_cast<uint4*>(p.vtbuf[d] + off + i * 8) = o;
    }
  }

  // ---- arrival: the last CTA of the launch adds one to this rank's slot on every destination. The
  // barrier orders every thread's peer stores before thread 0, whose single system-scope fence then
  // covers them all (a fence per thread made the kernel wait on `membar` most of the time)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned total = gridDim.x * gridDim.y;
    if (atomicAdd(p.ctr, 1u) == total - 1) {
      atomicExch(p.ctr, 0u);
      fence_acq_rel_sys();
      for (int d = 0; d < p.world; ++d) red_relaxed_sys_add(p.flags[d] + kUlyFlagArrive + p.rank, 1u);
    }
  }
}

// One thread waits until *flag >= target, or reports that the wait ran out.
__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t target, long long budget, DeviceStatus* status,
                                 uint32_t kernel_id, uint32_t site) {
  if (threadIdx.x == 0 && !wait_flag_geq(flag, target, budget)) report_status(status, kWaitTimeout, kernel_id, site, 0);
}
}  // namespace b200

namespace b200 {
// defined in gemm_tcgen05.cu
int make_kmajor_map(CUtensorMap* out, const void* base, int elem_bytes, long long rows, long long k,
                    long long ld, int box_rows);
}  // namespace b200

using namespace b200;

static inline int fa_pad(int s, int to) { return (s + to - 1) / to * to; }
static int fa_launch(const FaParams& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, dim3 grid,
                     int int8, cudaStream_t stream, const FaPeerMaps* peers = nullptr);

// Scratch layout of one call: V^T [batch * heads * 128][sk_pad64] bf16, then (int8 mode) Q8
// [batch * sq][heads * 128], K8 [batch * sk][heads * 128], q scales [batch * heads][sq_pad128],
// K tile scales [batch * heads][key tiles] fp32, K sums [batch * heads][128] fp32.
struct FaScratch {
  long long vt, q8, k8, qs, ks, ksum, total;
};
static FaScratch fa_scratch(int batch, int heads, int sq, int sk, int int8) {
  FaScratch s{};
  auto up = [](long long v) { return (v + 255) / 256 * 256; };
  long long off = 0;
  s.vt = off; off = up(off + static_cast<long long>(batch) * heads * kFaD * fa_pad(sk, 64) * 2);
  if (int8) {
    s.q8 = off; off = up(off + static_cast<long long>(batch) * sq * heads * kFaD);
    s.k8 = off; off = up(off + static_cast<long long>(batch) * sk * heads * kFaD);
    s.qs = off; off = up(off + static_cast<long long>(batch) * heads * fa_pad(sq, 128) * 4);
    s.ks = off; off = up(off + static_cast<long long>(batch) * heads * (fa_pad(sk, 128) / 128) * 4);
    s.ksum = off; off = up(off + static_cast<long long>(batch) * heads * kFaD * 4);
  }
  s.total = off;
  return s;
}

B200_API long long b200_attn_fa_workspace_bytes(int batch, int heads, int sq, int sk, int int8) {
  return fa_scratch(batch, heads, sq, sk, int8).total;
}

// Dense attention, head dim 128: q [batch * sq][heads * 128], k / v [batch * sk][heads * 128] bf16
// (contiguous), out like q: softmax(q k^T * scale) v per (batch, head). int8 != 0: SageAttention
// (K mean removal, int8 Q K^T). `scratch`: b200_attn_fa_workspace_bytes bytes.
B200_API int b200_attn_fa(const void* q, const void* k, const void* v, void* out, int batch, int sq, int sk,
                          int heads, float scale, int int8, void* scratch, void* status, cudaStream_t stream) {
  if (batch <= 0 || sq <= 0 || sk <= 0) return 0;
  if (scratch == nullptr) return -2;
  const long long ld = static_cast<long long>(heads) * kFaD;
  const FaScratch sc = fa_scratch(batch, heads, sq, sk, int8);
  uint8_t* base = static_cast<uint8_t*>(scratch);
  const int sk_pad64 = fa_pad(sk, 64);
  dim3 tgrid((sk_pad64 + 63) / 64, kFaD / 64, batch * heads);
  fa_transpose_v_kernel<<<tgrid, dim3(32, 8), 0, stream>>>(static_cast<const __nv_bfloat16*>(v),
                                                           reinterpret_cast<__nv_bfloat16*>(base + sc.vt), ld, sk,
                                                           sk_pad64, heads);
  FaParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld_out = ld;
  p.sq = sq; p.sk = sk; p.heads = heads; p.batch = batch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<DeviceStatus*>(status);
  p.n_tiles = fa_pad(sk, 128) / 128;
  p.tiles_per_seg = p.n_tiles;
  p.nseg = 1;
  p.seg_len = sk;
  p.seg_pad = p.n_tiles * 128;
  CUtensorMap tq, tk, tv;
  int rc;
  if (int8) {
    const int sq_pad = fa_pad(sq, 128), n_tiles = fa_pad(sk, 128) / 128;
    float* ksum = reinterpret_cast<float*>(base + sc.ksum);
    float* qs = reinterpret_cast<float*>(base + sc.qs);
    float* ks = reinterpret_cast<float*>(base + sc.ks);
    if (cudaMemsetAsync(ksum, 0, static_cast<size_t>(batch) * heads * kFaD * 4, stream) != cudaSuccess) return -3;
    sage_k_sum_kernel<<<dim3((sk + 255) / 256, batch * heads), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(k), ksum, ld, sk, heads);
    const long long wq = static_cast<long long>(batch) * sq * heads;
    sage_quant_rows_kernel<<<static_cast<unsigned>((wq + 7) / 8), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), reinterpret_cast<int8_t*>(base + sc.q8), qs, nullptr, 1.f, ld, sq, sq_pad,
        heads, batch);
    sage_quant_k_tiles_kernel<<<dim3(n_tiles, batch * heads), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(k), reinterpret_cast<int8_t*>(base + sc.k8), ks, ksum, ld, sk, heads);
    p.q_scale = qs;
    p.k_scale = ks;
    p.sq_pad = sq_pad;
    rc = make_kmajor_map(&tq, base + sc.q8, 1, static_cast<long long>(batch) * sq, ld, ld, 128);
    if (rc) return rc;
    rc = make_kmajor_map(&tk, base + sc.k8, 1, static_cast<long long>(batch) * sk, ld, ld, 128);
    if (rc) return rc;
  } else {
    rc = make_kmajor_map(&tq, q, 2, static_cast<long long>(batch) * sq, ld, ld, 128);
    if (rc) return rc;
    rc = make_kmajor_map(&tk, k, 2, static_cast<long long>(batch) * sk, ld, ld, 128);
    if (rc) return rc;
  }
  rc = make_kmajor_map(&tv, base + sc.vt, 2, static_cast<long long>(batch) * heads * kFaD, sk_pad64, sk_pad64, 128);
  if (rc) return rc;
  return fa_launch(p, tq, tk, tv, dim3((sq + 2 * kFaTile - 1) / (2 * kFaTile), heads, batch), int8, stream);
}

static int fa_launch(const FaParams& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, dim3 grid,
                     int int8, cudaStream_t stream, const FaPeerMaps* peers) {
  static const FaPeerMaps no_peers{};
  const FaPeerMaps& pm = peers ? *peers : no_peers;
  const int qk_tile = int8 ? 128 * 128 : 128 * 128 * 2;
  const int stages = int8 ? 3 : 2;
  const int smem = 2 * qk_tile + stages * (qk_tile + 128 * 128 * 2) + static_cast<int>(sizeof(FaBarriers)) + 1024;
  static PerDeviceOnce configured[2];
  if (int8) {
    if (configured[1].first_time() &&
        cudaFuncSetAttribute(attn_fa_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -4;
    attn_fa_kernel<true><<<grid, kFaThreads, smem, stream>>>(p, tq, tk, tv, pm);
  } else {
    if (configured[0].first_time() &&
        cudaFuncSetAttribute(attn_fa_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -4;
    attn_fa_kernel<false><<<grid, kFaThreads, smem, stream>>>(p, tq, tk, tv, pm);
  }
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));   // the CUDA error number stays readable
}

// ---- host side of the fused exchange --------------------------------------------------------------
// Bytes of one rank's exchange region, and where its parts sit (the same on every rank).
struct UlyLayout {
  long long flags, ctr, ksum_in, ksum_local, qbuf, kbuf, vtbuf, qscale, kscale, out, total;
};
static UlyLayout uly_layout(int s_l, int heads, int world, int int8, int cp = 0) {
  UlyLayout l{};
  auto up = [](long long v) { return (v + 1023) / 1024 * 1024; };
  const int s_pad = fa_pad(s_l, 128), hl = cp ? heads : heads / world;
  const long long rows = cp == 2 ? s_pad : static_cast<long long>(world) * s_pad;     // K / V^T rows held per rank
  const long long q_rows = cp ? s_pad : rows;
  long long off = 0;
  l.flags = off; off = up(off + kUlyFlagWords * 4);
  l.ctr = off; off = up(off + 64);
  l.ksum_in = off; off = up(off + static_cast<long long>(world) * heads * kFaD * 4);
  l.ksum_local = off; off = up(off + static_cast<long long>(heads) * kFaD * 4);
  l.qbuf = off; off = up(off + q_rows * hl * kFaD * (int8 ? 1 : 2));
  l.kbuf = off; off = up(off + rows * hl * kFaD * (int8 ? 1 : 2));
  l.vtbuf = off; off = up(off + rows * hl * kFaD * 2);
  l.qscale = off; off = up(off + static_cast<long long>(hl) * q_rows * 4);
  l.kscale = off; off = up(off + static_cast<long long>(hl) * (rows / 128) * 4);
  l.out = off; off = up(off + static_cast<long long>(s_pad) * heads * kFaD * 2);
  l.total = off;
  return l;
}

B200_API long long b200_ulysses_region_bytes(int s_l, int heads, int world, int int8) {
  if (world <= 0 || world > 8 || heads % world != 0) return -1;
  return uly_layout(s_l, heads, world, int8).total;
}
// Context-parallel form (any head count): every rank keeps its own queries and receives K / V of all heads.
B200_API long long b200_context_parallel_region_bytes(int s_l, int heads, int world, int int8) {
  if (world <= 0 || world > 8) return -1;
  return uly_layout(s_l, heads, world, int8, 1).total;
}
B200_API long long b200_context_parallel_out_offset(int s_l, int heads, int world, int int8) {
  return uly_layout(s_l, heads, world, int8, 1).out;
}
// Pull form (bf16 only): a rank's region holds its own K / V^T segment only; peers read it in place.
B200_API long long b200_ring_region_bytes(int s_l, int heads, int world) {
  if (world <= 0 || world > 8) return -1;
  return uly_layout(s_l, heads, world, 0, 2).total;
}
B200_API long long b200_ring_out_offset(int s_l, int heads, int world) { return uly_layout(s_l, heads, world, 0, 2).out; }
// Offset of the output [s_l][heads * 128] bf16 inside the region (the caller reads it after
// b200_ulysses_wait_outputs).
B200_API long long b200_ulysses_out_offset(int s_l, int heads, int world, int int8) {
  return uly_layout(s_l, heads, world, int8).out;
}

// One exchange + attention on this rank. q, k, v: local [s_l][heads * 128] bf16. `regions`: the base
// address of every rank's region in this process's address space (entry `rank` is local); regions
// must have been zeroed once. `epoch`: 1 for the first call on these regions, then 2, 3 ... (the
// same on every rank). The output lands in every rank's region at b200_ulysses_out_offset.
// `phases` selects the steps (bits: 1 K column sums, 2 operand push, 4 attention, 8 wait for the
// outputs); a rank passes 15. Tests that play every rank on one GPU run each phase for all ranks
// before the next one, so that no kernel ever waits for a later launch.
// Bit 16 selects the context-parallel form, for head counts the group size does not divide: every rank
// keeps its queries (and its output rows, [s_l][heads * 128] at b200_context_parallel_out_offset of its
// own region) and receives the K / V operands of all heads from every rank. world x the K / V bytes
// cross the links instead of (world - 1) / world of Q, K, V and the output, so the head-split form
// is the one to use whenever it applies.
B200_API int b200_ulysses_attention(const void* q, const void* k, const void* v, void* const* regions, int s_l, int heads,
                                    int rank, int world, float scale, int int8, unsigned epoch, int phases,
                                    long long wait_budget_cycles, void* status, cudaStream_t stream) {
  const int cp = (phases & 32) ? 2 : (phases & 16) ? 1 : 0;
  if (world <= 0 || world > 8 || (!cp && heads % world != 0) || s_l <= 0) return -2;
  if (cp == 2 && int8) return -6;      // the pull form reads bf16 operands (no per-tile scale tables on the peers)
  const UlyLayout l = uly_layout(s_l, heads, world, int8, cp);
  const int s_pad = fa_pad(s_l, 128), hl = cp ? heads : heads / world, tiles = s_pad / 128;
  const long long rows = static_cast<long long>(world) * s_pad;        // keys of the whole sequence
  const long long kv_rows = cp == 2 ? s_pad : rows;                    // rows of one rank's K / V^T buffers
  const long long q_rows = cp ? s_pad : rows;
  uint8_t* mine = static_cast<uint8_t*>(regions[rank]);
  const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;

  UlyPush u{};
  u.q = static_cast<const __nv_bfloat16*>(q);
  u.k = static_cast<const __nv_bfloat16*>(k);
  u.v = static_cast<const __nv_bfloat16*>(v);
  u.cp = cp;
  u.s_l = s_l; u.s_pad = s_pad; u.heads = heads; u.hl = hl; u.rank = rank; u.world = world;
  for (int d = 0; d < world; ++d) {
    uint8_t* r = static_cast<uint8_t*>(regions[d]);
    u.qbuf[d] = r + l.qbuf;
    u.kbuf[d] = r + l.kbuf;
    u.vtbuf[d] = reinterpret_cast<__nv_bfloat16*>(r + l.vtbuf);
    u.qscale[d] = reinterpret_cast<float*>(r + l.qscale);
    u.kscale[d] = reinterpret_cast<float*>(r + l.kscale);
    u.flags[d] = reinterpret_cast<uint32_t*>(r + l.flags);
  }
  u.ksum_in = reinterpret_cast<const float*>(mine + l.ksum_in);
  u.flags_local = reinterpret_cast<const uint32_t*>(mine + l.flags);
  u.ctr = reinterpret_cast<uint32_t*>(mine + l.ctr);
  u.target = epoch;
  u.inv_total = 1.f / (static_cast<float>(s_l) * world);
  u.wait_budget = budget;
  u.status = static_cast<DeviceStatus*>(status);

  if (int8 && (phases & 1)) {
    float* ksum_local = reinterpret_cast<float*>(mine + l.ksum_local);
    const int n = heads * kFaD;
    if (cudaMemsetAsync(ksum_local, 0, static_cast<size_t>(n) * 4, stream) != cudaSuccess) return -3;
    sage_k_sum_kernel<<<dim3((s_l + 255) / 256, heads), 128, 0, stream>>>(u.k, ksum_local, static_cast<long long>(heads) * kFaD,
                                                                         s_l, heads);
    UlyTabs tabs{};
    for (int d = 0; d < world; ++d) {
      tabs.ksum_in[d] = reinterpret_cast<float*>(static_cast<uint8_t*>(regions[d]) + l.ksum_in);
      tabs.flags[d] = u.flags[d];
    }
    uly_ksum_push_kernel<<<1, 1024, 0, stream>>>(ksum_local, tabs, n, rank, world);
  }
  if (phases & 2) {
    if (int8) uly_push_kernel<true><<<dim3(tiles, heads), 256, 0, stream>>>(u);
    else uly_push_kernel<false><<<dim3(tiles, heads), 256, 0, stream>>>(u);
  }
  if (cudaGetLastError() != cudaSuccess) return -5;
  if ((phases & 12) == 0) return 0;

  FaParams p{};
  p.ld_out = static_cast<long long>(heads) * kFaD;
  p.sq = static_cast<int>(q_rows); p.sk = static_cast<int>(rows); p.heads = hl; p.batch = 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<DeviceStatus*>(status);
  p.q_scale = reinterpret_cast<const float*>(mine + l.qscale);
  p.k_scale = reinterpret_cast<const float*>(mine + l.kscale);
  p.sq_pad = static_cast<int>(q_rows);
  p.q_seg_base = cp ? rank : 0;
  p.pull = cp == 2 ? 1 : 0;
  p.n_tiles = world * tiles;
  p.tiles_per_seg = tiles;
  p.nseg = world;
  p.seg_len = s_l;
  p.seg_first = rank;
  p.seg_pad = s_pad;
  p.seg_mode = 1;
  p.seg_flags = reinterpret_cast<const uint32_t*>(mine + l.flags) + kUlyFlagArrive;
  p.seg_target = epoch;
  p.wait_budget = budget;
  p.out_col0 = cp ? 0 : static_cast<long long>(rank) * hl * kFaD;
  for (int d = 0; d < world; ++d) {
    uint8_t* r = static_cast<uint8_t*>(regions[d]);
    p.out_seg[d] = reinterpret_cast<__nv_bfloat16*>(r + l.out);
    p.done_flags[d] = reinterpret_cast<uint32_t*>(r + l.flags) + kUlyFlagDone;
  }
  p.done_ctr = reinterpret_cast<uint32_t*>(mine + l.ctr) + 4;
  CUtensorMap tq, tk, tv;
  const int eb = int8 ? 1 : 2;
  int rc = make_kmajor_map(&tq, mine + l.qbuf, eb, q_rows, static_cast<long long>(hl) * kFaD, static_cast<long long>(hl) * kFaD, 128);
  if (rc) return rc;
  rc = make_kmajor_map(&tk, mine + l.kbuf, eb, kv_rows, static_cast<long long>(hl) * kFaD, static_cast<long long>(hl) * kFaD, 128);
  if (rc) return rc;
  rc = make_kmajor_map(&tv, mine + l.vtbuf, 2, static_cast<long long>(hl) * kFaD, kv_rows, kv_rows, 128);
  if (rc) return rc;
  FaPeerMaps pm{};
  if (cp == 2 && (phases & 4)) {
    for (int d = 0; d < world; ++d) {
      uint8_t* r = static_cast<uint8_t*>(regions[d]);
      rc = make_kmajor_map(&pm.k[d], r + l.kbuf, eb, kv_rows, static_cast<long long>(hl) * kFaD, static_cast<long long>(hl) * kFaD, 128);
      if (rc) return rc;
      rc = make_kmajor_map(&pm.vt[d], r + l.vtbuf, 2, static_cast<long long>(hl) * kFaD, kv_rows, kv_rows, 128);
      if (rc) return rc;
    }
  }
  if (phases & 4) {
    rc = fa_launch(p, tq, tk, tv, dim3(static_cast<unsigned>((q_rows + 2 * kFaTile - 1) / (2 * kFaTile)), hl, 1), int8, stream,
                   cp == 2 ? &pm : nullptr);
    if (rc) return rc;
  }
  if (phases & 8)
    flag_wait_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(mine + l.flags) + kUlyFlagDone,
                                         epoch * static_cast<unsigned>(world), budget, static_cast<DeviceStatus*>(status),
                                         kKernelAllToAll, 2);
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));
}
