// Dense GEMM on the 5th-generation tensor cores: C = A * B^T with both operands K-major
// ("nn.Linear" orientation), bf16 or fp8-e4m3 inputs with 128-wide block scales, fp32
// accumulation in TMEM. Optionally fused with the all-reduce of a tensor-parallel group.
//
// Replaces the reference's cuBLASLt / cublasGemmEx ladder (src/HartsyInference.Cuda/
// CudaBackend.cs:1769-2425, LtGemmExecutor.cs, Fp8GemmExecutor.cs:110-111 which is per-tensor
// scaled), its mma.sync kernels (Kernels/dequant/int8_mma_gemm.cu, Ptx/hgemm_mma_sm80.ptx) and, in
// the fused form, the GEMM + NCCL all-reduce pairs of its tensor-parallel transformer
// (src/HartsyInference.LLM/Transformer/TensorParallelTransformer.cs:298,307).
//
// Structure of one CTA (320 threads, persistent over a static list of work items):
//   warp 0      TMA producer: one thread issues cp.async.bulk.tensor loads of 128 x 128-byte A
//               atoms and BN x 128-byte B atoms (one or two atoms per stage) into 128B-swizzled
//               shared memory
//   warp 1      allocates TMEM; one thread issues tcgen05.mma (M = 128, N = BN, K = 32 bytes) and
//               commits to the stage's "empty" barrier and to the accumulator's "full" barrier
//   warps 2..9  epilogue: tcgen05.ld of the accumulator quarter that belongs to the warp (two
//               warps per quarter split the columns), scale / bias / activation / gate /
//               residual, store
// The caller decides which operand is the activation: for small token counts the weight matrix is
// passed as A so that its rows fill the 128-row MMA dimension and the tokens become the narrow N
// dimension (`swap_out = 1` then stores C transposed).
//
// Work items. Output tiles are dealt round-robin to the CTAs. When the tile count is not a
// multiple of the grid, the tiles of the last, partial wave are split along K so that this wave
// also covers every SM (a bandwidth-bound GEMM otherwise loses up to half its throughput to wave
// quantisation). The CTAs of a split tile write fp32 partials to a scratch buffer and bump a
// counter; whoever arrives last sums the partials in split order (deterministic) and runs the
// epilogue. A GEMM with fewer tiles than SMs is split completely; its partials are summed by a
// second, machine-wide kernel (splitk_reduce_kernel) or, optionally, through the distributed
// shared memory of a thread-block cluster (measured slower, off by default).
//
// fp8 (128 x 128 weight blocks, 1 x 128 activation groups), two scale modes:
//   UE8M0  power-of-two scales in the blocked layout the tensor core reads: the producer brings the
//          512-byte scale-factor blocks of four K blocks in with bulk copies, the MMA thread moves
//          them to TMEM (tcgen05.cp) and issues tcgen05.mma.kind::mxf8f6f4.block_scale; the
//          accumulator never leaves TMEM during the K loop (same flow as bf16).
//   fp32   arbitrary scales: every 128-deep K block is accumulated into its own TMEM buffer (a ring
//          of up to eight); the epilogue warps pull the block out, multiply by
//          scale_a(row, kb) * scale_b(col, kb) and add into fp32 registers while the tensor core
//          already works on the next blocks.
//
// Further modes of the same kernel: grouped (stacked expert weights; fixed blocks per expert or a
// device-side block list for variable token counts), column-batched (per-head projections of one
// token block), shifted-row accumulation (convolution taps as row offsets of one padded matrix).
//
// Programmatic dependent launch: the grid may start while its predecessor still runs. In the
// small-token orientation the producer requests the first stages of WEIGHT tiles before
// griddepcontrol.wait and the activation tiles after it; every other role waits first.
#include "comm.cuh"

namespace b200 {

// Fused GEMM -> all-reduce (+ residual add + RMSNorm + fp8 quantisation) for the row-parallel
// linears of a tensor-parallel group, token counts up to 128. One kernel per linear:
//   1. the tcgen05 tiles of this rank's partial product are stored as bf16 into the rank's OWN
//      `part` buffer of the symmetric heap ([K splits][tokens][features]; a K split is simply one
//      more addend of the reduction, so split tiles need no local fix-up);
//   2. the last CTA of the rank to finish its tiles raises the `ready` counter of every rank (one
//      multimem.red through the NVSwitch, or one red per peer);
//   3. token rows are dealt to the ranks in contiguous blocks; CTA i of the owning rank waits for
//      `ready`, pulls row i summed over all ranks (multimem.ld_reduce: the switch adds the ranks'
//      copies in fp32; without a multicast mapping: one peer load per rank), adds bias and the
//      rank-local residual row, applies RMSNorm and optionally quantises to e4m3 with 1x128 scales,
//      and stores the results into EVERY rank's output buffers (multimem.st or one store per peer);
//   4. the rank's last row raises `done` everywhere; CTA 0 leaves only after `done` shows that all
//      rows of all ranks have landed locally, so the next kernel in the stream may read them.
// The residual stream stays sharded by token row (each rank keeps the rows it owns up to date),
// the normalised activations come out replicated. Counters are cumulative over calls (no host
// resets: the kernel is capturable in CUDA graphs); every wait is bounded and reports through
// the status word.
struct AllReduceParams {
  int rank, world;
  int part_splits;                   // K splits the `part` buffer has room for
  int use_mc;                        // 1: entries [0] of the arrays below are multicast aliases
  __nv_bfloat16* part;               // local: [splits][tokens][features] bf16 partial products
  const __nv_bfloat16* part_src[8];  // where to read the partials of all ranks from
  __nv_bfloat16* res;                // local residual stream [tokens][features], updated in place (may be null)
  const __nv_bfloat16* norm_w;       // RMSNorm weight [features] (null: no normalisation)
  const __nv_bfloat16* bias;         // [features], may be null
  float eps;
  int weight_plus_one;
  __nv_bfloat16* out_bf16[8];        // [tokens][features] bf16 (may be null)
  uint8_t* out_q[8];                 // [tokens][features] e4m3 (may be null)
  uint32_t* out_sf[8];               // its scales: fp32 [tokens][features / 128] or blocked UE8M0 words
  int sf_tile_rows;                  // > 0: blocked UE8M0 layout with this many rows per block
  uint32_t* flags[8];                // per rank two counters: [0] ready, [1] done
  uint32_t* flags_local;
  uint32_t* ctr;                     // local: [0] calls completed, [1] CTAs past the GEMM, [2] row CTAs done, [3] CTAs finished
  long long wait_budget;             // cycles
  int debug_skip_ready;              // test aid: this rank never raises `ready`, so the waits on it run out
  // More than 128 tokens (prefill, DiT sequences): the GEMM runs in its large-token orientation
  // without K splits, `part` is [tokens][features], and the reduce phase is elementwise:
  //   out = res + gate * (sum over ranks + bias)      (res, gate optional; no norm, no fp8 emit)
  // `res` is then the replicated residual stream and is only read (the new stream is `out`).
  int large;
  const __nv_bfloat16* gate;         // [features], may be null
  // Reduce-scatter form of the large-token case (sequence-parallel regions): the result rows this
  // rank owns go to `out_local` ([owned rows][features], local memory) and nowhere else; `res` is
  // then the rank's block of the residual stream, indexed from the first owned row.
  __nv_bfloat16* out_local;
};

// All-gather -> GEMM for the column-parallel linears of a sequence-parallel region (more than 128
// tokens): every rank holds a contiguous block of ceil(m / world) token rows (activations, and for
// fp8 their scales). One kernel per linear:
//   1. the epilogue warps of all CTAs copy the rank's block into the same rows of EVERY rank's
//      gather buffer (multimem.st through the NVSwitch, or one store per peer), then the rank's last
//      CTA raises the rank's arrival counter on every rank;
//   2. the TMA producer waits for the arrival counters of the ranks whose rows a token tile covers
//      before it loads that tile from the LOCAL gather buffer; tiles are walked starting with the
//      rank's own rows, so the tensor core works on local data while the peers' rows arrive;
//   3. when the rank's last CTA is through, it raises `done` on every rank; the copy phase of the
//      next call waits for the `done` of all ranks before it overwrites the gather buffers.
// Counters are cumulative (capturable in CUDA graphs); every wait is bounded.
struct GatherParams {
  int rank, world;
  int use_mc;                         // 1: entries [0] of the destination arrays are multicast aliases
  int rows_total, rows_per_rank;      // rank r owns rows [r * rows_per_rank, ...) of rows_total
  const uint8_t* src;                 // local block [rows][row_bytes]
  long long row_bytes;                // bytes of one activation row (a multiple of 16)
  uint8_t* dst[8];                    // every rank's gather buffer [rows_total][row_bytes]
  // scales of an fp8 operand: fp32 [rows][k / 128] (sf_words = 0) or the blocked UE8M0 layout, one
  // 32-bit word per (row, group of four 128-wide K blocks) (sf_words = words per row = k groups)
  const uint32_t* src_scale;
  uint32_t* dst_scale[8];
  int scale_words;                    // fp32 scales per row (fp32 mode)
  int sf_words;                       // > 0: blocked UE8M0 layout
  uint32_t* flags[8];                 // per rank: [0, 8) arrival of source rank s, [8] done
  uint32_t* flags_local;
  uint32_t* ctr;                      // local: [0] calls completed, [1] CTAs past the copy, [2] CTAs finished
  long long wait_budget;
};
constexpr int kAgFlagDone = 8;

struct GemmParams {
  int rows_a;          // rows of the A operand (tiled by 128)
  int rows_b;          // rows of the B operand (tiled by BN)
  int k;               // reduction length in elements
  int stages;
  int swap_out;        // 0: C[a_row][b_row]; 1: C[b_row][a_row]
  // Grouped mode (MoE experts): A stacks `rows_a / group_n` weight matrices of group_n rows, B
  // stacks one BN-row token block per group; A tile t pairs with B block (t * 128) / group_n and
  // the output column is a_row % group_n. 0 = ordinary GEMM.
  int group_n;
  // Grouped mode: number of used slots per group (device memory, may be null). Groups with a zero
  // count are skipped by every role of every CTA, so idle experts cost no weight traffic.
  const int* group_counts;
  // Grouped "column-batched" variant (per-head projections): every group reads the SAME token rows
  // of B at column offset g * group_b_koff (elements) and writes output columns starting at
  // g * group_out_stride. 0 = stacked token blocks as described above.
  int group_b_koff;
  int group_out_stride;
  // Stacked grouped mode with several token blocks per weight group (`group_chunks` > 1): B block
  // e * chunks + c pairs with weight group e. Tiles are ordered (group, A tile, chunk) so that the
  // chunks of one weight tile run next to each other and the second read of the weights hits L2.
  int group_chunks;
  // Stacked grouped mode with a DEVICE-SIDE block list (variable tokens per group): B block b
  // belongs to weight group block_group[b] and *dyn_blocks blocks are in use; tile t is
  // (block t / tpg, A tile t % tpg). Null = the static layouts above.
  const int* block_group;
  const int* dyn_blocks;
  // MX mode (hardware block scaling): UE8M0 scale factors in the blocked layout
  // [row tile][k group of 512][128 x uint32], see quant_mx.cuh; sf_tile_b = B rows per SF block.
  const uint32_t* sf_a;
  const uint32_t* sf_b;
  int sf_kgroups;
  int sf_tile_b;
  // Shifted-row accumulation (convolutions as one GEMM): K is a sequence of taps of tap_kblocks
  // k-blocks each; tap t reads A rows shifted down by tap_shift[t] and A columns
  // [0, tap_kblocks * 64). 0 = ordinary GEMM.
  int tap_kblocks;
  int tap_shift[28];
  // 1: every tile is split over the CTAs of a thread-block cluster (cluster size = splits, one work
  // item per CTA); the partials stay in shared memory and are summed through distributed shared
  // memory, each CTA reducing its share of the tile. No scratch traffic, no second kernel.
  int cluster_reduce;
  // 1: every tile is split and a second kernel (splitk_reduce_kernel) sums the partials with the
  // whole machine; 0: the last CTA to arrive at a split tile sums them inside this kernel.
  int external_reduce;
  // K-split of the trailing tiles: tiles [0, first_split_tile) are whole, every later tile is
  // cut into `splits` ranges of `kblocks_per_split` k-blocks
  int first_split_tile;
  int num_tiles;
  int splits;
  int kblocks_per_split;
  float* split_ws;          // [split tiles][splits][BN][128] fp32 partials
  uint32_t* split_counter;  // [split tiles], zero between launches
  long long ldc;            // leading dimension of C in elements
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;      // per output feature (column of C), may be null
  const __nv_bfloat16* gate;      // per output feature multiplicative gate, may be null
  const __nv_bfloat16* residual;  // same layout as C, may be null
  int act;                        // 0 none, 1 gelu-tanh, 2 silu
  // fp8 block scales, K-contiguous: scale(row, kb) = s[(row / gran) * ld + kb], ld = K / 128.
  // A thread walks one row's scales along K, so consecutive k-blocks hit the same cache line.
  const float* scale_a;
  const float* scale_b;
  int sa_gran, sa_ld, sb_gran, sb_ld;
  DeviceStatus* status;
  AllReduceParams ar;   // ar.world == 0: plain GEMM
  GatherParams ag;      // ag.world == 0: the A operand is complete when the kernel starts
  int ta_rotate;        // plain GEMM: A tiles are walked starting with this one
};

constexpr int kTileA = 128;
constexpr int kStageBytesA = kTileA * 128;
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps

struct alignas(16) GemmBarriers {
  uint64_t full[12];
  uint64_t empty[12];
  uint64_t tmem_full[8];
  uint64_t tmem_empty[8];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t flag;      // broadcast slot of the epilogue warps
  uint32_t pad;
  // per epilogue warp: the 32 (x2 chunks) column scales of the current k-block, double-buffered
  // by k-block parity, so that every lane can read all of them as broadcast vector loads
  alignas(16) float cs_bcast[8][2][64];
};

// One unit of work of a CTA: an output tile and a range of k-blocks.
struct WorkItem {
  int ta, tb;        // tile coordinates
  int kb0, kb1;      // k-block range
  int slot;          // index among the split tiles, -1 for a whole tile
  int split;         // which range of the split tile
  bool skip;         // grouped mode: the group has no tokens
  int bk;            // element offset of the group's columns in B (column-batched mode)
};

__device__ __forceinline__ long long num_work_items(const GemmParams& p) {
  if (p.block_group != nullptr) return static_cast<long long>(*p.dyn_blocks) * (p.group_n / kTileA);
  return p.first_split_tile + static_cast<long long>(p.num_tiles - p.first_split_tile) * p.splits;
}

__device__ __forceinline__ WorkItem decode_item(const GemmParams& p, long long w, int tiles_a,
                                                int total_kblocks) {
  WorkItem it;
  long long tile;
  if (w < p.first_split_tile) {
    tile = w;
    it.slot = -1;
    it.split = 0;
    it.kb0 = 0;
    it.kb1 = total_kblocks;
  } else {
    const long long r = w - p.first_split_tile;
    it.slot = static_cast<int>(r / p.splits);
    it.split = static_cast<int>(r % p.splits);
    tile = p.first_split_tile + it.slot;
    it.kb0 = it.split * p.kblocks_per_split;
    it.kb1 = min(total_kblocks, it.kb0 + p.kblocks_per_split);
  }
  it.ta = static_cast<int>(tile % tiles_a);
  it.bk = 0;
  if (p.group_n > 0) {
    if (p.group_b_koff > 0) {
      const int g = (it.ta * kTileA) / p.group_n;
      it.tb = 0;
      it.bk = g * p.group_b_koff;
      it.skip = false;
    } else if (p.block_group != nullptr) {
      const int tpg = p.group_n / kTileA;
      const int t = static_cast<int>(tile);
      const int blk = t / tpg;
      it.ta = p.block_group[blk] * tpg + (t - blk * tpg);
      it.tb = blk;
      it.skip = false;
    } else {
      const int chunks = p.group_chunks > 1 ? p.group_chunks : 1;
      const int tpg = p.group_n / kTileA;                 // A tiles per weight group
      const int t = static_cast<int>(tile);
      const int chunk = t % chunks, within = (t / chunks) % tpg, e = t / (chunks * tpg);
      it.ta = e * tpg + within;
      it.tb = e * chunks + chunk;
      it.skip = p.group_counts != nullptr && p.group_counts[it.tb] == 0;
    }
  } else {
    it.tb = static_cast<int>(tile / tiles_a);
    it.skip = false;
    if (p.ta_rotate > 0) {
      it.ta += p.ta_rotate;
      if (it.ta >= tiles_a) it.ta -= tiles_a;
    }
  }
  return it;
}

// Output column of weight row `a_row` in the small-token orientation.
__device__ __forceinline__ long long swap_col(const GemmParams& p, int a_row) {
  if (p.group_n <= 0) return a_row;
  const int g = a_row / p.group_n, c = a_row - g * p.group_n;
  return p.group_b_koff > 0 ? static_cast<long long>(g) * p.group_out_stride + c : c;
}

__device__ __forceinline__ float apply_epilogue(const GemmParams& p, float v, long long row,
                                                long long col) {
  // row = token index, col = output feature, both already bounds-checked
  if (p.bias) v += __bfloat162float(p.bias[col]);
  if (p.act == 1) v = gelu_tanh(v);
  else if (p.act == 2) v = silu(v);
  if (p.gate) v *= __bfloat162float(p.gate[col]);
  if (p.residual) v += __bfloat162float(p.residual[row * p.ldc + col]);
  return v;
}

__device__ __forceinline__ void epilogue_barrier() {   // the 8 epilogue warps only
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Stores 32 consecutive accumulator columns (B rows b0..b0+31) of A row `a_row` of a whole tile
// to its destination: C, or (fused all-reduce) the staging buffer of the owning rank.
// `b_end` is the end of the tile's B rows (a 16-row tile fills only half of a 32-column chunk; the
// rest of the chunk is not this tile's data).
__device__ __forceinline__ void store_chunk(const GemmParams& p, const float (&v)[32], int a_row,
                                            int b0, int b_end, int split = 0) {
  if (a_row >= p.rows_a) return;
  if (p.ar.world > 0) {
    // fused all-reduce: raw bf16 partial of this K split into the rank's own [split][token][feature]
    // buffer (always the small-token orientation: a_row is the feature, the chunk walks tokens)
    if (!p.swap_out) {
      // large-token orientation: a_row is the token, the chunk walks 32 features (whole chunks:
      // the feature count is a multiple of 128)
      if (b0 >= b_end) return;
      __nv_bfloat16* dst = p.ar.part + static_cast<long long>(a_row) * p.rows_b + b0;
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(dst + j) =
            make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]), pack_bf16x2(v[j + 4], v[j + 5]),
                       pack_bf16x2(v[j + 6], v[j + 7]));
      return;
    }
    __nv_bfloat16* dst = p.ar.part + (static_cast<long long>(split) * p.rows_b + b0) * p.rows_a + a_row;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (b0 + j < b_end) dst[static_cast<long long>(j) * p.rows_a] = __float2bfloat16(v[j]);
    return;
  }
  if (!p.swap_out) {
    __nv_bfloat16* dst = p.out + static_cast<long long>(a_row) * p.ldc + b0;
    if (b0 + 32 <= b_end && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2)
        w[j >> 1] = pack_bf16x2(apply_epilogue(p, v[j], a_row, b0 + j),
                                apply_epilogue(p, v[j + 1], a_row, b0 + j + 1));
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (b0 + j < b_end)
          dst[j] = __float2bfloat16(apply_epilogue(p, v[j], a_row, b0 + j));
    }
  } else {
    const long long col = swap_col(p, a_row);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (b0 + j < b_end)
        p.out[static_cast<long long>(b0 + j) * p.ldc + col] =
            __float2bfloat16(apply_epilogue(p, v[j], b0 + j, col));
  }
}

// fp32 partial of a split tile: slot layout [BN columns][128 rows], so that the 32 lanes of a warp
// (consecutive rows) write and later read consecutive addresses.
template <int BN>
__device__ __forceinline__ void store_partial(const GemmParams& p, const float (&v)[32], int row_local,
                                              int col0_local, const WorkItem& it) {
  float* ws = p.split_ws + (static_cast<long long>(it.slot) * p.splits + it.split) * (BN * 128);
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (col0_local + j < BN) ws[(col0_local + j) * 128 + row_local] = v[j];
}

// Routes one 32-column chunk of accumulator values of work item `it`.
template <int BN>
__device__ __forceinline__ void emit_chunk(const GemmParams& p, const float (&v)[32], const WorkItem& it,
                                           int row_local, int chunk) {
  if (it.slot >= 0 && p.ar.world == 0) store_partial<BN>(p, v, row_local, chunk * 32, it);
  else store_chunk(p, v, it.ta * kTileA + row_local, it.tb * BN + chunk * 32, min(p.rows_b, (it.tb + 1) * BN),
                   it.split);
}

// Sums the partials of four consecutive weight rows (one 16-byte load per partial) of split tile
// `it`, applies the epilogue and writes C. kBatch loads are issued together so that their L2
// latencies overlap.
template <int kBatch>
__device__ __forceinline__ void reduce_partials(const GemmParams& p, const WorkItem& it, int bn, int e4) {
  const float* ws = p.split_ws + static_cast<long long>(it.slot) * p.splits * (bn * 128);
  const int e = e4 * 4;
  const int a_local = e & 127, b_local = e >> 7;
  const int a_row = it.ta * kTileA + a_local, b_row = it.tb * bn + b_local;
  if (a_row >= p.rows_a || b_row >= p.rows_b) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int sp = 0;
  for (; sp + kBatch <= p.splits; sp += kBatch) {
    float4 t[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      t[u] = __ldcg(reinterpret_cast<const float4*>(ws + static_cast<long long>(sp + u) * (bn * 128) + e));
#pragma unroll
    for (int u = 0; u < kBatch; ++u) { acc.x += t[u].x; acc.y += t[u].y; acc.z += t[u].z; acc.w += t[u].w; }
  }
  for (; sp < p.splits; ++sp) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(ws + static_cast<long long>(sp) * (bn * 128) + e));
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    if (a_row + u >= p.rows_a) break;
    if (p.swap_out) {
      const long long col = swap_col(p, a_row + u);
      p.out[static_cast<long long>(b_row) * p.ldc + col] = __float2bfloat16(apply_epilogue(p, v[u], b_row, col));
    } else {
      p.out[static_cast<long long>(a_row + u) * p.ldc + b_row] =
          __float2bfloat16(apply_epilogue(p, v[u], a_row + u, b_row));
    }
  }
}

// Called by all 256 epilogue threads once the item's values are stored. Whole tile: nothing to do
// (or, fused all-reduce: tell the owner rank). Split tile: count the arrival; the last CTA to
// arrive sums the partials in split order, applies the epilogue and writes C.
// The barriers are executed even after a failed wait (`ok` false) so that the eight warps never
// disagree on the number of barrier calls; only signals and stores are suppressed then.
template <int BN>
__device__ __forceinline__ void finish_item(const GemmParams& p, const WorkItem& it, bool ok,
                                            uint32_t* smem_flag) {
  const int et = threadIdx.x - 64;
  if (p.ar.world > 0) return;   // the partials are complete as stored; see ar_finish
  if (it.slot < 0 || p.external_reduce || p.cluster_reduce) return;
  __threadfence();
  epilogue_barrier();
  if (et == 0) {
    uint32_t last = 0;
    if (ok) {
      const uint32_t old = atomicAdd(p.split_counter + it.slot, 1u);
      last = old == static_cast<uint32_t>(p.splits) - 1 ? 1u : 0u;
      if (last) p.split_counter[it.slot] = 0;   // ready for the next launch
    }
    *smem_flag = last;
  }
  epilogue_barrier();
  const bool last = *smem_flag != 0;
  epilogue_barrier();
  if (!last) return;
  __threadfence();
  for (int e4 = et; e4 < BN * 32; e4 += 256) reduce_partials<4>(p, it, BN, e4);
}

// ---- fused all-reduce: everything after the rank's own tiles are stored (see AllReduceParams) ----
constexpr float kArFp8Max = 448.f;

__device__ __forceinline__ float epilogue_block_sum(float v, float* red) {   // the 8 epilogue warps
  v = warp_sum(v);
  const int w = (threadIdx.x >> 5) - 2, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  epilogue_barrier();
  float t = l < 8 ? red[l] : 0.f;
  t = warp_sum(t);
  epilogue_barrier();
  return t;
}

// One value of `bytes` (16, 8 or 4) to the same offset of every rank's buffer.
template <typename T>
__device__ __forceinline__ void ar_store_all(const AllReduceParams& a, T* const (&dst)[8], long long elem_off,
                                             const uint4& v, int bytes) {
  if (a.use_mc) {
    T* d = dst[0] + elem_off;
    if (bytes == 16) multimem_st_v4(d, v);
    else if (bytes == 8) multimem_st_v2(d, make_uint2(v.x, v.y));
    else multimem_st_b32(d, v.x);
    return;
  }
  for (int r = 0; r < a.world; ++r) {
    // start with the neighbour so that the ranks do not all write to rank 0 first
    T* d = dst[(a.rank + r) % a.world] + elem_off;
    if (bytes == 16) *reinterpret_cast<uint4*>(d) = v;
    else if (bytes == 8) *reinterpret_cast<uint2*>(d) = make_uint2(v.x, v.y);
    else *reinterpret_cast<uint32_t*>(d) = v.x;
  }
}

__device__ __forceinline__ void ar_signal(const AllReduceParams& a, int which) {
  if (a.use_mc) {
    multimem_red_release_add(a.flags[0] + which, 1u);
  } else {
    // one release fence at system scope, then a relaxed add per peer (a release on every add
    // would pay the fence once per peer)
    fence_acq_rel_sys();
    for (int r = 0; r < a.world; ++r) red_relaxed_sys_add(a.flags[(a.rank + r) % a.world] + which, 1u);
  }
}

// Layout of the rank-local counter block `ctr` (u32 words, zero-initialised once):
//   [0] calls completed   [1] CTAs past the GEMM   [2] CTAs done with their reduce units   [3] CTAs finished
//   [64, 192)    per owned row: segments of the row whose sum of squares has been posted
//   [256, 2304)  per owned row 16 floats: the segments' sums of squares
constexpr int kArRowCounters = 64, kArRowPartials = 256, kArCtrWords = 2304, kArMaxSegs = 16;

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Called by the 256 epilogue threads of every CTA once all its work items are stored.
__device__ __forceinline__ void ar_finish(const GemmParams& p, GemmBarriers* bars) {
  const AllReduceParams& a = p.ar;
  const int et = threadIdx.x - 64;
  const int m = p.swap_out ? p.rows_b : p.rows_a, n = p.swap_out ? p.rows_a : p.rows_b;          // tokens, features
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(a.ctr) + 1u;   // 1-based index of this call
  // ---- 2. this CTA's partial tiles are written; the rank's last CTA tells every rank. Peers read
  // the tiles through this GPU's L2, so a device-scope fence per CTA orders them; the one release
  // at system scope by the last CTA then covers all of them (fences are cumulative).
  epilogue_barrier();
  if (et == 0) {
    __threadfence();
    if (atomicAdd(a.ctr + 1, 1u) == gridDim.x - 1 && !a.debug_skip_ready) {
      __threadfence();
      ar_signal(a, 0);
    }
  }
  // ---- 3. rows owned by this rank: a contiguous block of ceil(m / world). A row is cut into
  // segments of 256 vectors of eight features (one vector per thread) and the (row, segment) units
  // are dealt to the CTAs, so that even a few rows keep many SMs' worth of loads in flight; the
  // segments of a row meet through a sum-of-squares slot per segment and a counter per row.
  const int per = (m + a.world - 1) / a.world;
  const int row0 = a.rank * per;
  const int owned = max(0, min(per, m - row0));
  const int nvec = n >> 3;
  const int nseg = (nvec + 255) >> 8;
  const int units = owned * nseg;
  const int unit_ctas = min(units, static_cast<int>(gridDim.x));
  if (static_cast<int>(blockIdx.x) < unit_ctas) {
    if (et == 0) {
      const bool ok = wait_flag_geq(a.flags_local, call * static_cast<uint32_t>(a.world), a.wait_budget);
      if (!ok) report_status(p.status, kWaitTimeout, kKernelGemmAllReduce, 1, blockIdx.x);
      bars->flag = ok ? 1u : 0u;
    }
    epilogue_barrier();
    bool ok = bars->flag != 0;
    epilogue_barrier();
    float* red = &bars->cs_bcast[0][0][0];
    uint8_t* sfb = reinterpret_cast<uint8_t*>(&bars->cs_bcast[1][0][0]);   // exponent bytes of this unit
    uint32_t* rowcnt = a.ctr + kArRowCounters;
    float* rowpart = reinterpret_cast<float*>(a.ctr + kArRowPartials);
    const int kb_n = n >> 7, kgroups = (n + 511) >> 9;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int ri = u / nseg, seg = u - ri * nseg;
      const int row = row0 + ri;
      const int v = seg * 256 + et;
      const bool active = v < nvec;
      // -- sum over ranks (and K splits) of this thread's eight features, + bias, + residual
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      if (active) {
        if (a.use_mc) {
          uint4 x[4];
#pragma unroll
          for (int sp = 0; sp < 4; ++sp)
            if (sp < p.splits)
              x[sp] = multimem_ld_reduce_bf16x8(a.part_src[0] + (static_cast<long long>(sp) * m + row) * n + v * 8);
#pragma unroll
          for (int sp = 0; sp < 4; ++sp)
            if (sp < p.splits) add_bf16x8(acc, x[sp]);
        } else {
          for (int sp = 0; sp < p.splits; ++sp) {
            const long long off = (static_cast<long long>(sp) * m + row) * n + v * 8;
            uint4 x[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < a.world) x[r] = ld_relaxed_sys_v4(a.part_src[r] + off);
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < a.world) add_bf16x8(acc, x[r]);     // fixed rank order: deterministic
          }
        }
        if (a.bias) add_bf16x8(acc, *reinterpret_cast<const uint4*>(a.bias + v * 8));
        if (a.gate) {
          float g[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) g[i] = 0.f;
          add_bf16x8(g, *reinterpret_cast<const uint4*>(a.gate + v * 8));
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] *= g[i];
        }
      }
      // what the unfused path would have stored as the all-reduce result is bf16: round here too
      uint4 packed;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
      for (int i = 0; i < 4; ++i) pw[i] = pack_bf16x2(acc[2 * i], acc[2 * i + 1]);
      if (active && a.res) {
        __nv_bfloat16* rr = a.res + static_cast<long long>(a.out_local ? ri : row) * n + v * 8;
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = 0.f;
        add_bf16x8(t, packed);
        add_bf16x8(t, *reinterpret_cast<const uint4*>(rr));
#pragma unroll
        for (int i = 0; i < 4; ++i) pw[i] = pack_bf16x2(t[2 * i], t[2 * i + 1]);
        if (!a.large) *reinterpret_cast<uint4*>(rr) = packed;          // new residual row (this rank only)
      }
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = 0.f;
      add_bf16x8(y, packed);
      float rstd = 1.f;
      if (a.norm_w) {
        float sumsq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sumsq += y[i] * y[i];
        const float part = epilogue_block_sum(sumsq, red);
        if (et == 0) {
          float total = part;
          if (nseg > 1) {
            // post this segment's share, then wait for the row's other segments (all resident: every
            // CTA of the grid is; units are taken in ascending order, so the lowest unfinished row
            // never waits on a CTA that is itself blocked)
            rowpart[ri * kArMaxSegs + seg] = part;
            __threadfence();
            atomicAdd(rowcnt + ri, 1u);
            long long t0 = 0;
            uint32_t spins = 0;
            while (ld_acquire_gpu(rowcnt + ri) < static_cast<uint32_t>(nseg)) {
              if ((++spins & 0x3f) == 0) {
                const long long now = clock64();
                if (t0 == 0) t0 = now;
                else if (now - t0 > a.wait_budget) { ok = false; break; }
              }
            }
            total = 0.f;
            for (int sg = 0; sg < nseg; ++sg) total += __ldcg(rowpart + ri * kArMaxSegs + sg);   // fixed order
            if (!ok) report_status(p.status, kWaitTimeout, kKernelGemmAllReduce, 3, blockIdx.x);
          }
          red[8] = rsqrtf(total / n + a.eps);
          bars->flag = ok ? 1u : 0u;
        }
        epilogue_barrier();
        rstd = red[8];
        ok = bars->flag != 0;
        epilogue_barrier();
        if (!ok) break;
      }
      const long long rbase = static_cast<long long>(row) * n;
      if (active) {
        if (a.norm_w) {
          float w[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = 0.f;
          add_bf16x8(w, *reinterpret_cast<const uint4*>(a.norm_w + v * 8));
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = y[i] * rstd * (a.weight_plus_one ? 1.f + w[i] : w[i]);
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) ow[i] = pack_bf16x2(y[2 * i], y[2 * i + 1]);
        if (a.out_local) *reinterpret_cast<uint4*>(a.out_local + static_cast<long long>(ri) * n + v * 8) = o;
        else if (a.out_bf16[0]) ar_store_all(a, a.out_bf16, rbase + v * 8, o, 16);
        // fp8 consumers see the bf16-rounded activations, like the unfused path
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = 0.f;
        add_bf16x8(y, o);
      }
      if (a.out_q[0]) {
        // n % 128 == 0: a 16-lane group is all-active or all-inactive
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (active) {
          float sc = fmaxf(amax, 1e-12f) / kArFp8Max;
          float inv = 1.f / sc;
          uint32_t eb = 127;
          if (a.sf_tile_rows > 0) {
            // UE8M0: the smallest power of two >= amax / 448
            const uint32_t bits = __float_as_uint(amax / kArFp8Max);
            int e = static_cast<int>(bits >> 23) - 127 + ((bits & 0x7fffffu) != 0 ? 1 : 0);
            e = max(-126, min(126, e));
            eb = static_cast<uint32_t>(e + 127);
            inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
          }
          uint4 q = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            q.x |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(y[i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            q.y |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(y[4 + i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
          ar_store_all(a, a.out_q, rbase + v * 8, q, 8);
          if ((et & 15) == 0) {
            if (a.sf_tile_rows > 0) sfb[et >> 4] = static_cast<uint8_t>(eb);
            else ar_store_all(a, a.out_sf, static_cast<long long>(row) * kb_n + (v >> 4),
                              make_uint4(__float_as_uint(sc), 0, 0, 0), 4);
          }
        }
        if (a.sf_tile_rows > 0) {
          // blocked UE8M0 layout: one 32-bit word per (row, group of four 128-wide K blocks); a
          // segment of 2048 features owns four whole words
          epilogue_barrier();
          const int kg = seg * 4 + et;
          if (et < 4 && kg < kgroups) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              word |= static_cast<uint32_t>(kg * 4 + i < kb_n ? sfb[et * 4 + i] : 127) << (8 * i);
            const int tile = row / a.sf_tile_rows, r = row - tile * a.sf_tile_rows;
            const long long widx = (static_cast<long long>(tile) * kgroups + kg) * 128 + (r & 31) * 4 + (r >> 5);
            ar_store_all(a, a.out_sf, widx, make_uint4(word, 0, 0, 0), 4);
          }
          epilogue_barrier();
        }
      }
    }
  }
  // ---- 4. this rank's rows are out: the last CTA with units raises `done` everywhere (a rank
  // without rows does so right away), and CTA 0 holds the kernel until every rank's rows have
  // landed here
  epilogue_barrier();
  if (et == 0) {
    bool signal = false;
    if (unit_ctas == 0) {
      signal = blockIdx.x == 0;
    } else if (static_cast<int>(blockIdx.x) < unit_ctas) {
      // this CTA's stores went to other GPUs: they must have been performed system-wide before the
      // count below lets another CTA announce them
      __threadfence_system();
      signal = atomicAdd(a.ctr + 2, 1u) == static_cast<uint32_t>(unit_ctas) - 1;
    }
    if (signal) {
      __threadfence();
      ar_signal(a, 1);
    }
    if (blockIdx.x == 0 &&
        !wait_flag_geq(a.flags_local + 1, call * static_cast<uint32_t>(a.world), a.wait_budget))
      report_status(p.status, kWaitTimeout, kKernelGemmAllReduce, 2, blockIdx.x);
  }
}

// ---- all-gather -> GEMM (see GatherParams) --------------------------------------------------------
// Copy phase, run by the 256 epilogue threads of every CTA before their first tile.
__device__ __forceinline__ void ag_copy(const GemmParams& p, GemmBarriers* bars) {
  const GatherParams& g = p.ag;
  const int et = threadIdx.x - 64;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(g.ctr) + 1u;
  // the gather buffers still hold the previous call's rows until every rank is done with them
  if (et == 0) {
    bool ok = true;
    if (call > 1) ok = wait_flag_geq(g.flags_local + kAgFlagDone, (call - 1u) * static_cast<uint32_t>(g.world), g.wait_budget);
    if (!ok) report_status(p.status, kWaitTimeout, kKernelAllToAll, 11, blockIdx.x);
    bars->flag = ok ? 1u : 0u;
  }
  epilogue_barrier();
  const bool ok = bars->flag != 0;
  epilogue_barrier();
  const int row0 = g.rank * g.rows_per_rank;
  const int rows = max(0, min(g.rows_per_rank, g.rows_total - row0));
  if (ok) {
    const long long vec_per_row = g.row_bytes >> 4;
    const long long nvec = static_cast<long long>(rows) * vec_per_row;
    const long long base = static_cast<long long>(row0) * g.row_bytes;
    for (long long v = static_cast<long long>(blockIdx.x) * 256 + et; v < nvec; v += static_cast<long long>(gridDim.x) * 256) {
      const uint4 x = *reinterpret_cast<const uint4*>(g.src + v * 16);
      if (g.use_mc) {
        multimem_st_v4(g.dst[0] + base + v * 16, x);
      } else {
        for (int r = 0; r < g.world; ++r) *reinterpret_cast<uint4*>(g.dst[(g.rank + r) % g.world] + base + v * 16) = x;
      }
    }
    if (g.src_scale != nullptr) {
      const int wpr = g.sf_words > 0 ? g.sf_words : g.scale_words;
      const long long nw = static_cast<long long>(rows) * wpr;
      for (long long i = static_cast<long long>(blockIdx.x) * 256 + et; i < nw; i += static_cast<long long>(gridDim.x) * 256) {
        const int r = static_cast<int>(i / wpr), c = static_cast<int>(i - static_cast<long long>(r) * wpr);
        long long si, di;
        if (g.sf_words > 0) {
          // blocked layout: [row tile of 128][k group][(row % 32) * 4 + (row % 128) / 32]
          const int gr = row0 + r;
          si = (static_cast<long long>(r >> 7) * wpr + c) * 128 + (r & 31) * 4 + ((r & 127) >> 5);
          di = (static_cast<long long>(gr >> 7) * wpr + c) * 128 + (gr & 31) * 4 + ((gr & 127) >> 5);
        } else {
          si = i;
          di = static_cast<long long>(row0) * wpr + i;
        }
        const uint32_t w = g.src_scale[si];
        if (g.use_mc) {
          multimem_st_b32(g.dst_scale[0] + di, w);
        } else {
          for (int q = 0; q < g.world; ++q) g.dst_scale[(g.rank + q) % g.world][di] = w;
        }
      }
    }
  }
  // the stores went to other GPUs: system-wide before the count lets another CTA announce them
  __threadfence_system();
  epilogue_barrier();
  if (et == 0) {
    __threadfence();
    if (atomicAdd(g.ctr + 1, 1u) == gridDim.x - 1) {
      __threadfence();
      if (g.use_mc) {
        multimem_red_release_add(g.flags[0] + g.rank, 1u);
      } else {
        fence_acq_rel_sys();
        for (int r = 0; r < g.world; ++r) red_relaxed_sys_add(g.flags[(g.rank + r) % g.world] + g.rank, 1u);
      }
    }
  }
}

// Producer side: the rows of A tile `ta` have arrived from the ranks that own them. `seen` caches the
// sources already found complete in this call.
__device__ __forceinline__ bool ag_wait_tile(const GemmParams& p, int ta, uint32_t call, uint32_t& seen) {
  const GatherParams& g = p.ag;
  const int first = (ta * kTileA) / g.rows_per_rank;
  const int last = min(g.world - 1, (min(g.rows_total, (ta + 1) * kTileA) - 1) / g.rows_per_rank);
  bool waited = false;
  for (int s = first; s <= last; ++s) {
    if (seen & (1u << s)) continue;
    if (!wait_flag_geq(g.flags_local + s, call, g.wait_budget)) return false;
    seen |= 1u << s;
    waited = true;
  }
  // the rows arrived as ordinary (or multimem) stores; the loads that follow are issued by the TMA unit
  if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// Second kernel of a fully split GEMM: one thread per four output values, grid.y = tile. Sums the
// partials in split order (deterministic), so a small GEMM whose few tiles were split to fill
// the machine is also reduced by the whole machine instead of by one CTA per tile.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmParams p, int bn, int tiles_a,
                                                            int total_kblocks) {
  pdl_wait();
  pdl_trigger();
  const int e4 = blockIdx.x * blockDim.x + threadIdx.x;
  if (e4 >= bn * 32) return;
  const WorkItem it = decode_item(p, p.first_split_tile + static_cast<long long>(blockIdx.y) * p.splits,
                                  tiles_a, total_kblocks);
  if (it.skip) return;
  reduce_partials<8>(p, it, bn, e4);
}

template <int kMode, int BN, int kAtoms>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b) {
  // A stage holds kAtoms swizzle atoms (128 bytes of K each) per operand: [A atoms][B atoms].
  // kMode: 0 = bf16, 1 = e4m3 with fp32 block scales promoted by the epilogue warps per k-block,
  // 2 = e4m3 with UE8M0 block scales applied by the tensor core (kind::mxf8f6f4.block_scale).
  // 3 = int8 operands (W8A8): s32 accumulation over the whole K in TMEM, one scale per token row and
  // one per output channel applied by the epilogue.
  constexpr bool kFp8Data = kMode != 0;            // one-byte operands
  constexpr bool kFp8 = kMode == 1;                // software promotion
  constexpr bool kMx = kMode == 2;
  constexpr bool kI8 = kMode == 3;
  constexpr int kAtomBytesB = BN * 128;
  constexpr int kSfBytes = kMx ? 1536 : 0;         // per stage: SF block of A + up to two of B
  constexpr int kStageBytes = kAtoms * (kStageBytesA + kAtomBytesB) + (kMx ? 2048 : 0);
  constexpr int kSfOffset = kAtoms * (kStageBytesA + kAtomBytesB);
  constexpr int kElemsPerAtom = kFp8Data ? 128 : 64;   // K elements in one 128-byte atom
  // Accumulator ring in TMEM: as many buffers as fit in the 512 columns (at most 8). The
  // block-scaled path hands one buffer per 128-deep K block to the epilogue warps, so a deep ring
  // lets the tensor core run ahead of the promotion; the bf16 path uses one buffer per work item.
  constexpr int kBufStride = BN < 32 ? 32 : BN;   // loads are 32 columns wide
  constexpr int kAccCols = kMx ? 480 : 512;        // MX keeps 32 columns for the scale factors
  constexpr int kAccBufsRaw = (kAccCols / kBufStride) < 8 ? (kAccCols / kBufStride) : 8;
  constexpr int kAccBufs = kMx && kAccBufsRaw > 4 ? 4 : kAccBufsRaw;
  constexpr uint32_t kSfCol = kAccBufs * kBufStride;                  // first SF column
  constexpr uint32_t kTmemNeed = kAccBufs * kBufStride + (kMx ? 32 : 0);
  constexpr uint32_t kTmemCols = kTmemNeed <= 32 ? 32 : kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128
                               : kTmemNeed <= 256 ? 256 : 512;
  constexpr uint32_t kIdesc = kMx ? make_idesc_mx(128, BN)
                            : kI8 ? make_idesc(128, BN, kFmtS8, kFmtS8, 2)
                            : kFp8Data ? make_idesc(128, BN, kFmtE4m3, kFmtE4m3)
                                       : make_idesc(128, BN, kFmtBf16, kFmtBf16);
  static_assert(BN == 16 || BN == 32 || BN == 64 || BN == 128 || BN == 256,
                "tcgen05.mma M=128 needs N % 16 == 0; TMEM allocations are powers of two");
  static_assert(!kFp8 || BN <= 128, "fp8 path keeps BN / 2 fp32 accumulators per thread");

  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte aligned bases.
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int stages = p.stages;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + stages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_a = (p.rows_a + kTileA - 1) / kTileA;
  const int total_kblocks = (p.k + kElemsPerAtom - 1) / kElemsPerAtom;
  const long long work_items = num_work_items(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 8; ++b) {
      mbar_init(&bars->tmem_full[b], 1);
      mbar_init(&bars->tmem_empty[b], 8);   // one arrival per epilogue warp
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    bars->flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  pdl_trigger();   // the next kernel may be scheduled; it waits for this grid to finish before it reads

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      long long issued = 0;
      bool ok = true;
      // One stage of loads, in two parts: 1 = A operand (+ its scale factors) and the transaction
      // count of the whole stage, 2 = B operand (+ its scale factors).
      auto issue_stage = [&](const WorkItem& it, int kb, int st, int parts) {
        const int na = min(kAtoms, it.kb1 - kb);
        uint8_t* sa = smem + st * kStageBytes;
        uint8_t* sb = sa + kAtoms * kStageBytesA;
        // MX: the stage that starts a group of four k-blocks also carries the group's scale factors
        const bool with_sf = kMx && ((kb & 3) == 0 || kb == it.kb0);
        constexpr int kSfBlocksB = BN > 128 ? 2 : 1;
        if (parts & 1) {
          mbar_arrive_expect_tx(&bars->full[st], na * (kStageBytesA + kAtomBytesB) +
                                                     (with_sf ? 512 * (1 + kSfBlocksB) : 0));
          if (with_sf) {
            const long long ga = (static_cast<long long>(it.ta) * p.sf_kgroups + (kb >> 2)) * 128;
            bulk_load(sa + kSfOffset, p.sf_a + ga, 512, &bars->full[st]);
          }
          for (int a = 0; a < na; ++a) {
            int ax = (kb + a) * kElemsPerAtom, ay = it.ta * kTileA;
            if (p.tap_kblocks > 0) {
              const int tap = (kb + a) / p.tap_kblocks;
              ax = ((kb + a) - tap * p.tap_kblocks) * kElemsPerAtom;
              ay += p.tap_shift[tap];
            }
            tma_load_2d(sa + a * kStageBytesA, &tm_a, &bars->full[st], ax, ay);
          }
        }
        if (parts & 2) {
          if (with_sf) {
            const long long tile_b = (static_cast<long long>(it.tb) * BN) / p.sf_tile_b;
#pragma unroll
            for (int j = 0; j < kSfBlocksB; ++j) {
              const long long gb = ((tile_b + j) * p.sf_kgroups + (kb >> 2)) * 128;
              bulk_load(sa + kSfOffset + 512 * (1 + j), p.sf_b + gb, 512, &bars->full[st]);
            }
          }
          for (int a = 0; a < na; ++a)
            tma_load_2d(sb + a * kAtomBytesB, &tm_b, &bars->full[st], (kb + a) * kElemsPerAtom + it.bk,
                        it.tb * BN);
        }
      };
      // Programmatic dependent launch: this grid may start while the kernel before it is still
      // running. In the small-token orientation the A operand is a weight matrix, which no earlier
      // kernel of the step writes, so the first stages of weights are requested BEFORE waiting for
      // the predecessor; the activation tiles follow after the wait.
      int pre = 0;                 // stage iterations of the first item already half-issued
      long long w_first = blockIdx.x;
      if (p.swap_out && p.group_n == 0 && w_first < work_items) {
        const WorkItem it = decode_item(p, w_first, tiles_a, total_kblocks);
        for (int kb = it.kb0; kb < it.kb1 && pre < stages; kb += kAtoms, ++pre) issue_stage(it, kb, pre, 1);
        pdl_wait();
        for (int i = 0; i < pre; ++i) issue_stage(it, it.kb0 + i * kAtoms, i, 2);
        issued = pre;
        s = pre;
        if (s == stages) { s = 0; ph ^= 1; }
      } else {
        pdl_wait();
      }
      const uint32_t ag_call = p.ag.world > 0 ? *reinterpret_cast<volatile uint32_t*>(p.ag.ctr) + 1u : 0u;
      uint32_t ag_seen = 0;
      for (long long w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
        const WorkItem it = decode_item(p, w, tiles_a, total_kblocks);
        if (it.skip) continue;
        if (p.ag.world > 0 && !ag_wait_tile(p, it.ta, ag_call, ag_seen)) {
          report_status(p.status, kWaitTimeout, kKernelAllToAll, 12, blockIdx.x);
          *abort_flag = 1;
          ok = false;
          break;
        }
        int kb = it.kb0;
        if (w == w_first && pre > 0) kb += pre * kAtoms;      // already issued above
        for (; kb < it.kb1; kb += kAtoms) {
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag)) {
            report_status(p.status, kWaitTimeout, kKernelGemm, 1, blockIdx.x);
            ok = false;
            break;
          }
          issue_stage(it, kb, s, 3);
          ++issued;
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // Let copies that are still in flight land before the CTA exits.
        for (int i = 0; i < stages && i < issued; ++i) {
          int ss = s - 1 - i;
          uint32_t pp = ph;
          if (ss < 0) { ss += stages; pp ^= 1; }
          uint32_t dummy = 0;
          mbar_wait(&bars->full[ss], pp, &dummy, 4000000ll);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      pdl_wait();
      int s = 0;
      uint32_t ph = 0;
      int abuf = 0;
      uint32_t aph = 0;
      bool ok = true;
      bool issued_any = false;
      for (long long w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
        const WorkItem it = decode_item(p, w, tiles_a, total_kblocks);
        if (it.skip) continue;
        if (!kFp8) {
          if (!mbar_wait(&bars->tmem_empty[abuf], aph ^ 1, abort_flag)) {
            report_status(p.status, kWaitTimeout, kKernelGemm, 2, blockIdx.x);
            ok = false;
            break;
          }
          tc_fence_after_sync();
        }
        for (int kb = it.kb0; kb < it.kb1 && ok; kb += kAtoms) {
          const int na = min(kAtoms, it.kb1 - kb);
          if (!mbar_wait(&bars->full[s], ph, abort_flag)) {
            report_status(p.status, kWaitTimeout, kKernelGemm, 3, blockIdx.x);
            ok = false;
            break;
          }
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kAtoms * kStageBytesA;
          if (kMx && ((kb & 3) == 0 || kb == it.kb0)) {
            // scale factors of this group of four k-blocks: shared memory -> TMEM (4 columns per
            // 128 rows), two TMEM slots used alternately
            tc_fence_after_sync();
            const uint32_t slot = tmem_base + kSfCol + ((kb >> 2) & 1) * 16;
            tmem_cp_sf(slot, make_desc_sf(sa + kSfOffset));
            tmem_cp_sf(slot + 4, make_desc_sf(sa + kSfOffset + 512));
            if (BN > 128) tmem_cp_sf(slot + 8, make_desc_sf(sa + kSfOffset + 1024));
          }
          for (int a = 0; a < na; ++a) {
            if (kFp8) {
              if (!mbar_wait(&bars->tmem_empty[abuf], aph ^ 1, abort_flag)) {
                report_status(p.status, kWaitTimeout, kKernelGemm, 4, blockIdx.x);
                ok = false;
                break;
              }
            }
            tc_fence_after_sync();
            const uint64_t adesc = make_desc_sw128(sa + a * kStageBytesA);
            const uint64_t bdesc = make_desc_sw128(sb + a * kAtomBytesB);
            const uint32_t d_tmem = tmem_base + abuf * kBufStride;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // advancing 32 bytes along K inside the 128-byte swizzle atom = +2 in the
              // (address >> 4) field of the descriptor
              const uint32_t acc = kFp8 ? (k > 0) : (kb + a > it.kb0 || k > 0);
              if (kMx) {
                const uint32_t sf_id = static_cast<uint32_t>(kb + a) & 3u;
                const uint32_t slot = tmem_base + kSfCol + (((kb + a) >> 2) & 1) * 16;
                mma_mxf8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc | (sf_id << 29) | (sf_id << 4), acc,
                            slot, slot + 4);
              } else if (kI8) {
                mma_i8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
              } else if (kFp8Data) {
                mma_fp8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
              } else {
                mma_bf16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
              }
            }
            issued_any = true;
            if (kFp8) {
              tc_commit(&bars->tmem_full[abuf]);
              if (++abuf == kAccBufs) { abuf = 0; aph ^= 1; }
            }
          }
          tc_commit(&bars->empty[s]);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        if (!kFp8 && ok) {
          tc_commit(&bars->tmem_full[abuf]);
          if (++abuf == kAccBufs) { abuf = 0; aph ^= 1; }
        }
      }
      if (!ok && issued_any) {
        // make sure no MMA still reads shared memory / writes TMEM when the CTA tears down
        tc_commit(&bars->drain);
        uint32_t dummy = 0;
        mbar_wait(&bars->drain, 0, &dummy, 4000000ll);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..9
    // Two warps share each TMEM lane quarter; they split the accumulator columns in 32-column
    // chunks (even chunks -> first warp, odd chunks -> second warp).
    pdl_wait();
    if (p.ag.world > 0) ag_copy(p, bars);
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int hsel = (warp - 2) >> 2;  // which half of the chunks
    constexpr int kChunks = (BN + 31) / 32;
    constexpr int kMine = (kChunks + 1) / 2;
    const int row_local = q * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    int abuf = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (long long w = blockIdx.x; w < work_items; w += gridDim.x) {
      const WorkItem it = decode_item(p, w, tiles_a, total_kblocks);
      if (it.skip) continue;
      if (ok) {
        if constexpr (!kFp8) {
          if (!__all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[abuf], aph, abort_flag))) {
            if (lane == 0) report_status(p.status, kWaitTimeout, kKernelGemm, 5, blockIdx.x);
            ok = false;
          } else {
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = hsel; c < kChunks; c += 2) {
              uint32_t r[32];
              tmem_ld_32x32(lane_base + abuf * kBufStride + c * 32, r);
              tmem_ld_wait();
              float v[32];
              if constexpr (kI8) {
                // s32 accumulators -> fp32 with the row scale of the A operand and the row scales of
                // the 32 B rows of this chunk (whichever of the two is the token side)
                const float sa = p.scale_a[min(it.ta * kTileA + row_local, p.rows_a - 1)];
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  v[j] = static_cast<float>(static_cast<int>(r[j])) * sa *
                         __ldg(p.scale_b + min(it.tb * BN + c * 32 + j, p.rows_b - 1));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
              }
              if (p.cluster_reduce) {
                // partial of this CTA's K range, kept in its own shared memory: [BN columns][128 rows]
                // fp32 over the (now idle) pipeline stages
                float* part = reinterpret_cast<float*>(smem);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (c * 32 + j < BN) part[(c * 32 + j) * 128 + row_local] = v[j];
              } else {
                emit_chunk<BN>(p, v, it, row_local, c);
              }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[abuf]);
            if (++abuf == kAccBufs) { abuf = 0; aph ^= 1; }
          }
        } else {
          float acc[kMine * 32];
#pragma unroll
          for (int j = 0; j < kMine * 32; ++j) acc[j] = 0.f;
          const int a_row_c = min(it.ta * kTileA + row_local, p.rows_a - 1);
          const bool col_vector = p.sb_gran == 1;
          // Scales are fetched one k-block ahead so that their latency never sits between the
          // accumulator becoming ready and the FMAs. Row scale: one value per thread. Column
          // scale: one value per tile (128-wide weight blocks) or one per column, in which case
          // lane l holds the scale of column (chunk * 32 + l) and it is broadcast with shuffles.
          // (index arithmetic hoisted out of the k loop: the granularities are run-time values
          // and an integer division per k-block kept the conversion pipe busy)
          const float* sa_ptr = p.scale_a + static_cast<long long>(a_row_c / p.sa_gran) * p.sa_ld;
          const float* cs_ptr[kMine];
#pragma unroll
          for (int i = 0; i < kMine; ++i) {
            if (!col_vector) {
              cs_ptr[i] = p.scale_b + static_cast<long long>((it.tb * BN) / p.sb_gran) * p.sb_ld;
            } else {
              const int col = min(it.tb * BN + (hsel + 2 * i) * 32 + lane, p.rows_b - 1);
              cs_ptr[i] = p.scale_b + static_cast<long long>(col) * p.sb_ld;
            }
          }
          auto load_row_scale = [&](int kb) { return __ldg(sa_ptr + kb); };
          auto load_col_scale = [&](int kb, int i) { return __ldg(cs_ptr[i] + kb); };
          float sa_next = load_row_scale(it.kb0);
          float cs_next[kMine];
#pragma unroll
          for (int i = 0; i < kMine; ++i) cs_next[i] = load_col_scale(it.kb0, i);
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            const float sa = sa_next;
            float cs[kMine];
#pragma unroll
            for (int i = 0; i < kMine; ++i) cs[i] = cs_next[i];
            if (kb + 1 < it.kb1) {
              sa_next = load_row_scale(kb + 1);
#pragma unroll
              for (int i = 0; i < kMine; ++i) cs_next[i] = load_col_scale(kb + 1, i);
            }
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[abuf], aph, abort_flag))) {
              if (lane == 0) report_status(p.status, kWaitTimeout, kKernelGemm, 6, blockIdx.x);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            float* bc = bars->cs_bcast[warp - 2][kb & 1];
            if (col_vector) {
#pragma unroll
              for (int i = 0; i < kMine; ++i) bc[i * 32 + lane] = cs[i];
              __syncwarp();
            }
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
              const int c = hsel + 2 * i;
              const bool last_chunk = (i == kMine - 1) || (hsel + 2 * (i + 1) >= kChunks);
              if (c < kChunks) {
                uint32_t r[32];
                tmem_ld_32x32(lane_base + abuf * kBufStride + c * 32, r);
                tmem_ld_wait();
                if (last_chunk) {
                  // the values are in registers: hand the TMEM buffer back before the FMAs
                  tc_fence_before_sync();
                  __syncwarp();
                  if (lane == 0) mbar_arrive(&bars->tmem_empty[abuf]);
                }
                if (!col_vector) {
                  const float sc = sa * cs[i];
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    acc[i * 32 + j] = fmaf(__uint_as_float(r[j]), sc, acc[i * 32 + j]);
                } else {
                  const float4* b4 = reinterpret_cast<const float4*>(bc + i * 32);
#pragma unroll
                  for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 sv = b4[j4];
                    acc[i * 32 + 4 * j4 + 0] = fmaf(__uint_as_float(r[4 * j4 + 0]), sa * sv.x, acc[i * 32 + 4 * j4 + 0]);
                    acc[i * 32 + 4 * j4 + 1] = fmaf(__uint_as_float(r[4 * j4 + 1]), sa * sv.y, acc[i * 32 + 4 * j4 + 1]);
                    acc[i * 32 + 4 * j4 + 2] = fmaf(__uint_as_float(r[4 * j4 + 2]), sa * sv.z, acc[i * 32 + 4 * j4 + 2]);
                    acc[i * 32 + 4 * j4 + 3] = fmaf(__uint_as_float(r[4 * j4 + 3]), sa * sv.w, acc[i * 32 + 4 * j4 + 3]);
                  }
                }
              }
            }
            if (hsel >= kChunks) {
              // a warp without a chunk of its own still takes part in the buffer hand-back
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->tmem_empty[abuf]);
            }
            if (++abuf == kAccBufs) { abuf = 0; aph ^= 1; }
          }
          if (ok) {
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
              const int c = hsel + 2 * i;
              if (c < kChunks) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = acc[i * 32 + j];
                emit_chunk<BN>(p, v, it, row_local, c);
              }
            }
          }
        }
      }
      finish_item<BN>(p, it, ok, &bars->flag);
    }
    if (p.ar.world > 0) ar_finish(p, bars);
  }

  // the single-lane roles rejoin their warps before the CTA-wide barrier
  __syncwarp();
  if (p.cluster_reduce) {
    // every CTA of the cluster has its partial in shared memory -> each sums its share of the tile
    // over all CTAs (fixed order: deterministic), applies the epilogue and stores C
    cluster_sync_all();
    if (warp >= 2) {
      const WorkItem it = decode_item(p, blockIdx.x, tiles_a, total_kblocks);
      const int et = threadIdx.x - 64;
      const uint32_t rank = cluster_ctarank();
      const int total4 = BN * 32;                                  // float4 groups of the tile
      const int per = (total4 + p.splits - 1) / p.splits;
      const int lo = static_cast<int>(rank) * per, hi = min(total4, lo + per);
      const uint32_t part = smem_u32(smem);
      for (int e4 = lo + et; e4 < hi; e4 += 256) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.splits; ++r) {
          const float4 t = ld_dsmem_f4(part + e4 * 16, static_cast<uint32_t>(r));
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        const int e = e4 * 4;
        const int a_row = it.ta * kTileA + (e & 127), b_row = it.tb * BN + (e >> 7);
        if (a_row >= p.rows_a || b_row >= p.rows_b) continue;
        const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (a_row + u >= p.rows_a) break;
          if (p.swap_out) {
            const long long col = swap_col(p, a_row + u);
            p.out[static_cast<long long>(b_row) * p.ldc + col] = __float2bfloat16(apply_epilogue(p, v[u], b_row, col));
          } else {
            p.out[static_cast<long long>(a_row + u) * p.ldc + b_row] =
                __float2bfloat16(apply_epilogue(p, v[u], a_row + u, b_row));
          }
        }
      }
    }
    cluster_sync_all();   // nobody leaves while a peer may still read its shared memory
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (p.ag.world > 0 && threadIdx.x == 0) {
    // the last CTA to finish tells every rank that this rank no longer reads its gather buffer and
    // closes the call (every CTA has read the call counter by now)
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.ag.ctr);
    __threadfence();
    if (atomicAdd(p.ag.ctr + 2, 1u) == gridDim.x - 1) {
      p.ag.ctr[1] = 0;
      p.ag.ctr[2] = 0;
      *reinterpret_cast<volatile uint32_t*>(p.ag.ctr) = e + 1u;
      __threadfence();
      if (p.ag.use_mc) {
        multimem_red_release_add(p.ag.flags[0] + kAgFlagDone, 1u);
      } else {
        fence_acq_rel_sys();
        for (int r = 0; r < p.ag.world; ++r) red_relaxed_sys_add(p.ag.flags[(p.ag.rank + r) % p.ag.world] + kAgFlagDone, 1u);
      }
    }
  }
  if (p.ar.world > 0 && threadIdx.x == 0) {
    // the last CTA to finish closes the call: every CTA has read the call counter by now
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.ar.ctr);
    __threadfence();
    if (atomicAdd(p.ar.ctr + 3, 1u) == gridDim.x - 1) {
      p.ar.ctr[1] = 0;
      p.ar.ctr[2] = 0;
      p.ar.ctr[3] = 0;
      for (int i = 0; i < 128; ++i) p.ar.ctr[kArRowCounters + i] = 0;
      *reinterpret_cast<volatile uint32_t*>(p.ar.ctr) = e + 1u;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D K-major matrix [rows][k] with row pitch ld elements; box = 128 bytes x box_rows, 128B swizzle.
int make_kmajor_map(CUtensorMap* out, const void* base, int elem_bytes, long long rows,
                    long long k, long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld * elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes),
                       static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 100;
}

// Programmatic dependent launch of the GEMM (see the producer warp); switchable for A/B timing.
}  // namespace b200
bool b200::g_b200_pdl = true;
namespace b200 {
static bool g_cluster_reduce = false;   // measured slower than the other two ways; opt-in
static bool g_external_reduce = true;    // fully split GEMMs: second kernel (true) or last-arriving CTA (false)

template <int kMode, int BN, int kAtoms>
int launch_gemm(const GemmParams& p, const CUtensorMap& ta, const CUtensorMap& tb, int grid,
                cudaStream_t stream) {
  const int stage_bytes = kAtoms * (kStageBytesA + BN * 128) + (kMode == 2 ? 2048 : 0);
  const int smem = p.stages * stage_bytes + static_cast<int>(sizeof(GemmBarriers)) + 1024;
  static PerDeviceOnce configured;
  if (configured.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<kMode, BN, kAtoms>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return -static_cast<int>(e) - 200;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_b200_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.cluster_reduce) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = static_cast<unsigned>(p.splits);
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<kMode, BN, kAtoms>, p, ta, tb) != cudaSuccess) return -300;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 300;
}

static int g_num_sms[64] = {};
int num_sms() {   // of the current device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_num_sms[dev] == 0) {
    cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms[dev] <= 0) g_num_sms[dev] = 148;
  }
  return g_num_sms[dev];
}

constexpr long long kSplitCounterBytes = 16384;   // head of the scratch buffer: 4096 tile counters

// Host description of a grouped launch (see GemmParams::group_n and ::group_b_koff).
struct GroupSpec {
  int groups;
  const int* counts;     // device, optional: one per token block (groups * chunks)
  int b_koff;            // > 0: column-batched variant
  int out_stride;
  int chunks = 1;        // token blocks per weight group (stacked mode)
  const int* block_group = nullptr;   // device block list (see GemmParams::block_group) ...
  const int* dyn_blocks = nullptr;    // ... and its length; `chunks` is then the CAPACITY of the list
};

// Host description of a shifted-row (convolution) launch: x is [x_rows][cin] (cin a multiple of
// 64), w is [n][taps * cin], output row r = sum over taps of x[r + shift[t]] . w[:, t * cin ...].
struct ConvSpec {
  int taps;
  int cin;
  long long x_rows;
  int shift[28];
};

int gemm_impl(const void* x, const void* w, void* out, int m, int n, int k, long long ldx,
                     long long ldw, long long ldc, int dtype, const float* x_scale,
                     const float* w_scale, const void* bias, const void* gate, const void* residual,
                     int act, int splits, void* workspace, long long workspace_bytes, void* status,
                     cudaStream_t stream, const AllReduceParams* ar, const GroupSpec* gs = nullptr,
                     const ConvSpec* cs = nullptr, int* defer_info = nullptr, const GatherParams* ag = nullptr) {
  const int groups = gs ? gs->groups : 0;
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  // grouped: x is [groups * m][k], w is [groups * n][k], out is [groups * m][n]; m = tokens per group
  const bool i8 = dtype == 3;           // int8 operands, one fp32 scale per x row and per w row
  const bool fp8 = dtype != 0;          // one-byte operands. 1: fp32 block scales, 2: UE8M0 scale factors (blocked layout)
  const bool mx = dtype == 2;
  const int esz = fp8 ? 1 : 2;
  const int kelems = fp8 ? 128 : 64;
  if ((ldx * esz) % 16 != 0 || (ldw * esz) % 16 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -3;
  if (fp8 && ((!mx && !i8 && k % 128 != 0) || k % 16 != 0 || !x_scale || !w_scale)) return -4;
  if (i8 && (groups > 0 || cs != nullptr || ar != nullptr)) return -4;
  if (groups > 0) {
    if (m < 1 || m > 128 || n % 128 != 0) return -9;
    if (gs->b_koff > 0) {
      if (fp8 || k % kelems != 0 || (gs->b_koff * esz) % 16 != 0) return -9;
    } else if (m != 16 && m != 32 && m != 64 && m != 128) {
      return -9;
    }
  }

  // Small token counts: weights take the 128-row MMA dimension, tokens the N dimension.
  const bool swap = m <= 128 && cs == nullptr;
  GemmParams p{};
  p.k = k;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.act = act;
  p.status = static_cast<DeviceStatus*>(status);
  p.swap_out = swap ? 1 : 0;
  if (ar != nullptr) {
    if ((m > 128) != (ar->large != 0)) return -6;
    if (n % 128 != 0 || groups > 0 || cs != nullptr || ar->part_splits > 4) return -6;   // whole feature tiles
    if (bias != nullptr || gate != nullptr || residual != nullptr || act != 0) return -6;   // see AllReduceParams
    p.ar = *ar;
    // K splits fill the machine when there are fewer tiles than SMs; every split is one more
    // addend of the cross-rank reduction, so the limit is what the partial buffer holds
    int s_ar = num_sms() / (n / 128);
    if (s_ar > ar->part_splits) s_ar = ar->part_splits;
    if (s_ar > 4) s_ar = 4;
    const int kb_all = (k + kelems - 1) / kelems;
    if (s_ar > kb_all / 4) s_ar = kb_all / 4;
    splits = s_ar < 1 || ar->large ? 1 : s_ar;
  }

  if (ag != nullptr) {
    // the gathered operand is the 128-row MMA operand: the large-token orientation only
    if (swap || groups > 0 || cs != nullptr || ar != nullptr) return -11;
    p.ag = *ag;
    // start with the tiles of this rank's own rows
    p.ta_rotate = (ag->rank * ag->rows_per_rank) / kTileA;
    splits = 1;
  }
  int bn;
  const void *a_ptr, *b_ptr;
  long long lda, ldb;
  if (groups > 0) {
    p.group_n = n;
    p.group_counts = gs->counts;
    p.group_b_koff = gs->b_koff;
    p.group_out_stride = gs->out_stride;
    p.rows_a = groups * n;
    p.group_chunks = gs->chunks < 1 ? 1 : gs->chunks;
    p.block_group = gs->block_group;
    p.dyn_blocks = gs->dyn_blocks;
    // with a device block list `chunks` is the total number of blocks the buffers can hold
    p.rows_b = gs->b_koff > 0 ? m : (gs->block_group ? p.group_chunks * m : groups * p.group_chunks * m);
    a_ptr = w; lda = ldw; b_ptr = x; ldb = ldx;
    bn = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    p.scale_a = w_scale; p.sa_gran = 128; p.sa_ld = k / 128;
    p.scale_b = x_scale; p.sb_gran = 1;   p.sb_ld = k / 128;
  } else if (swap) {
    p.rows_a = n; p.rows_b = m;
    a_ptr = w; lda = ldw; b_ptr = x; ldb = ldx;
    bn = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    p.scale_a = w_scale; p.sa_gran = 128; p.sa_ld = k / 128;
    p.scale_b = x_scale; p.sb_gran = 1;   p.sb_ld = k / 128;
  } else {
    p.rows_a = m; p.rows_b = n;
    a_ptr = x; lda = ldx; b_ptr = w; ldb = ldw;
    bn = fp8 && !i8 ? 128 : 256;
    if ((!fp8 || i8) && n <= 128) bn = 128;
    p.scale_a = x_scale; p.sa_gran = 1;   p.sa_ld = k / 128;
    p.scale_b = w_scale; p.sb_gran = 128; p.sb_ld = k / 128;
  }
  if (mx) {
    const bool a_is_w = groups > 0 || swap;
    p.sf_a = reinterpret_cast<const uint32_t*>(a_is_w ? w_scale : x_scale);
    p.sf_b = reinterpret_cast<const uint32_t*>(a_is_w ? x_scale : w_scale);
    p.sf_kgroups = (k + 511) / 512;
    // SF blocks of the token operand cover one tile of `m` slots per group in the stacked grouped
    // mode (each padded to 128 rows), otherwise 128 consecutive rows
    p.sf_tile_b = (groups > 0 && gs->b_koff == 0) ? m : 128;
    if (groups > 0 && gs->b_koff > 0) return -9;
  }
  const int total_kblocks = (k + kelems - 1) / kelems;
  const int tiles = groups > 0 ? (gs->block_group ? p.group_chunks * (n / 128)
                                                  : ((p.rows_a + 127) / 128) * (gs->b_koff > 0 ? 1 : p.group_chunks))
                               : ((p.rows_a + 127) / 128) * ((p.rows_b + bn - 1) / bn);
  const int sms = num_sms();
  p.num_tiles = tiles;

  // ---- K-split policy (see the header comment)
  int first_split = tiles, s_eff = 1;
  const long long slot_bytes = static_cast<long long>(bn) * 128 * 4;
  if (splits > 1) {                                  // caller-forced uniform split
    first_split = 0;
    s_eff = splits;
  } else if (splits <= 0 && !(groups > 0 && gs->block_group)) {   // automatic (never with a device block list)
    const int q = tiles / sms, r = tiles % sms;
    // worthwhile when the partial wave is a visible share of the run: always for the
    // bandwidth-bound orientation, for the other only when there are few waves
    if (r != 0 && (swap || q < 4)) {
      int s = sms / r;
      if (s > total_kblocks / 2) s = total_kblocks / 2;   // at least two k-blocks per range
      // after full waves a modest split already shrinks the tail to 1/s of a tile; without full
      // waves the split is what fills the machine
      const int cap = q >= 1 ? 8 : 16;
      if (s > cap) s = cap;
      if (s > 1) { first_split = q * sms; s_eff = s; }
    }
  }
  if (s_eff > total_kblocks) s_eff = total_kblocks;
  p.kblocks_per_split = (total_kblocks + s_eff - 1) / s_eff;
  if (mx) p.kblocks_per_split = (p.kblocks_per_split + 3) / 4 * 4;   // ranges start on a scale-factor group
  s_eff = (total_kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;
  if (s_eff <= 1) { first_split = tiles; s_eff = 1; p.kblocks_per_split = total_kblocks; }
  const int split_tiles = tiles - first_split;
  if (split_tiles > 0 && ar == nullptr) {
    const long long need = kSplitCounterBytes + static_cast<long long>(split_tiles) * s_eff * slot_bytes;
    if (workspace == nullptr || need > workspace_bytes || split_tiles > 4096) {
      if (splits > 1) return -5;                     // forced split without room: say so
      first_split = tiles; s_eff = 1; p.kblocks_per_split = total_kblocks;
    }
  }
  p.first_split_tile = first_split;
  p.splits = s_eff;
  p.external_reduce = (first_split == 0 && s_eff > 1 && ar == nullptr && (g_external_reduce || g_cluster_reduce)) ? 1 : 0;
  int cluster = 1;
  if (p.external_reduce && g_cluster_reduce && dtype != 1 && splits <= 0 && groups == 0 && cs == nullptr) {
    // power-of-two cluster of at most 8 CTAs (portable size), every CTA exactly one K range
    int c = 1;
    while (c * 2 <= s_eff && c * 2 <= 8) c *= 2;
    int kps = (total_kblocks + c - 1) / c;
    if (mx) kps = (kps + 3) / 4 * 4;
    if (c > 1 && (total_kblocks + kps - 1) / kps == c) {
      cluster = c;
      p.splits = s_eff = c;
      p.kblocks_per_split = kps;
      p.external_reduce = 0;
      p.cluster_reduce = 1;
    }
  }
  p.split_counter = static_cast<uint32_t*>(workspace);
  p.split_ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kSplitCounterBytes);

  // two atoms per stage for the bandwidth-bound small-token orientation
  const int atoms = swap ? 2 : 1;
  const int stage_bytes = atoms * (kStageBytesA + bn * 128) + (mx ? 2048 : 0);
  int stages = (200 * 1024) / stage_bytes;
  if (stages > 12) stages = 12;
  p.stages = stages;

  CUtensorMap ta, tb;
  if (cs != nullptr) {
    if (fp8 || groups > 0 || ar != nullptr || cs->taps < 1 || cs->taps > 28 || cs->cin % 64 != 0) return -10;
    p.tap_kblocks = cs->cin / 64;
    for (int t = 0; t < cs->taps; ++t) p.tap_shift[t] = cs->shift[t];
  }
  int rc = cs != nullptr ? make_kmajor_map(&ta, a_ptr, esz, cs->x_rows, cs->cin, lda, kTileA)
                         : make_kmajor_map(&ta, a_ptr, esz, p.rows_a, k, lda, kTileA);
  if (rc) return rc;
  rc = make_kmajor_map(&tb, b_ptr, esz, p.rows_b, p.group_b_koff > 0 ? ldb : k, ldb, bn);
  if (rc) return rc;

  const long long items = first_split + static_cast<long long>(tiles - first_split) * s_eff;
  // a cluster launch runs one work item per CTA: the grid is the item count, not the SM count
  const int grid = p.cluster_reduce ? static_cast<int>(items) : static_cast<int>(items < sms ? items : sms);
  (void)cluster;

  if (i8) {
    // scales: one per row of either operand
    p.sa_gran = p.sb_gran = 1;
    p.sa_ld = p.sb_ld = 1;
    if (swap) {
      switch (bn) {
        case 16: rc = launch_gemm<3, 16, 2>(p, ta, tb, grid, stream); break;
        case 32: rc = launch_gemm<3, 32, 2>(p, ta, tb, grid, stream); break;
        case 64: rc = launch_gemm<3, 64, 2>(p, ta, tb, grid, stream); break;
        default: rc = launch_gemm<3, 128, 2>(p, ta, tb, grid, stream); break;
      }
    } else if (bn == 128) {
      rc = launch_gemm<3, 128, 1>(p, ta, tb, grid, stream);
    } else {
      rc = launch_gemm<3, 256, 1>(p, ta, tb, grid, stream);
    }
  } else if (mx) {
    if (swap) {
      switch (bn) {
        case 16: rc = launch_gemm<2, 16, 2>(p, ta, tb, grid, stream); break;
        case 32: rc = launch_gemm<2, 32, 2>(p, ta, tb, grid, stream); break;
        case 64: rc = launch_gemm<2, 64, 2>(p, ta, tb, grid, stream); break;
        default: rc = launch_gemm<2, 128, 2>(p, ta, tb, grid, stream); break;
      }
    } else {
      rc = launch_gemm<2, 128, 1>(p, ta, tb, grid, stream);
    }
  } else if (fp8) {
    if (swap) {
      switch (bn) {
        case 16: rc = launch_gemm<1, 16, 2>(p, ta, tb, grid, stream); break;
        case 32: rc = launch_gemm<1, 32, 2>(p, ta, tb, grid, stream); break;
        case 64: rc = launch_gemm<1, 64, 2>(p, ta, tb, grid, stream); break;
        default: rc = launch_gemm<1, 128, 2>(p, ta, tb, grid, stream); break;
      }
    } else {
      rc = launch_gemm<1, 128, 1>(p, ta, tb, grid, stream);
    }
  } else {
    if (swap) {
      switch (bn) {
        case 16: rc = launch_gemm<0, 16, 2>(p, ta, tb, grid, stream); break;
        case 32: rc = launch_gemm<0, 32, 2>(p, ta, tb, grid, stream); break;
        case 64: rc = launch_gemm<0, 64, 2>(p, ta, tb, grid, stream); break;
        default: rc = launch_gemm<0, 128, 2>(p, ta, tb, grid, stream); break;
      }
    } else if (bn == 128) {
      rc = launch_gemm<0, 128, 1>(p, ta, tb, grid, stream);
    } else {
      rc = launch_gemm<0, 256, 1>(p, ta, tb, grid, stream);
    }
  }
  if (defer_info != nullptr) {
    // the caller's consumer kernel sums the K ranges itself: report their layout, launch no reduce
    const bool deferred = rc == 0 && p.external_reduce && swap && groups == 0 && bias == nullptr &&
                          gate == nullptr && residual == nullptr && act == 0 && m <= bn;
    defer_info[0] = deferred ? 1 : 0;
    defer_info[1] = p.splits;
    defer_info[2] = bn;
    if (deferred) return rc;
  }
  if (rc == 0 && p.external_reduce) {
    const dim3 rgrid((bn * 32 + 255) / 256, tiles);
    if (launch_pdl(splitk_reduce_kernel, rgrid, dim3(256), 0, stream, p, bn, (p.rows_a + kTileA - 1) / kTileA,
                   total_kblocks) != cudaSuccess) rc = -300;
  }
  return rc;
}

}  // namespace b200

using namespace b200;

// Scratch that b200_gemm needs to be able to split tiles along K: a zero-initialised buffer of at
// least this many bytes (tile counters followed by fp32 partials). The kernel leaves the counters
// at zero again, so the buffer is zeroed once, at allocation.
B200_API void b200_gemm_set_pdl(int enabled) { g_b200_pdl = enabled != 0; }
B200_API void b200_gemm_set_cluster_reduce(int enabled) { g_cluster_reduce = enabled != 0; }
B200_API void b200_gemm_set_external_reduce(int enabled) { g_external_reduce = enabled != 0; }

B200_API long long b200_gemm_workspace_bytes() {
  return 64ll << 20;   // the automatic policy needs at most 16 KB + 148 slots of 64 KB
}

// out[m][n] (bf16, leading dim ldc) = epilogue(x[m][k] * w[n][k]^T)
//   dtype: 0 = bf16 operands, 1 = fp8 e4m3 operands with block scales
//   x_scale: [m][k/128] fp32 (per token, per 128-wide K group); w_scale: [ceil(n/128)][k/128] fp32
//   splits: 0 = automatic (split only the tiles of a partial last wave), 1 = never, > 1 = split
//           every tile that many ways
//   workspace: zero-initialised scratch (see b200_gemm_workspace_bytes), may be null (no splitting)
// Returns 0 on success, negative on a launch-time error.
B200_API int b200_gemm(const void* x, const void* w, void* out, int m, int n, int k, long long ldx,
                       long long ldw, long long ldc, int dtype, const float* x_scale,
                       const float* w_scale, const void* bias, const void* gate,
                       const void* residual, int act, int splits, void* workspace,
                       long long workspace_bytes, void* status, cudaStream_t stream) {
  return gemm_impl(x, w, out, m, n, k, ldx, ldw, ldc, dtype, x_scale, w_scale, bias, gate, residual,
                   act, splits, workspace, workspace_bytes, status, stream, nullptr);
}

// b200_gemm for a consumer that can add split-K ranges itself (b200_glu, b200_rope_kv): when the
// policy cuts every tile along K (small-token GEMMs with fewer tiles than SMs) and no epilogue term
// is asked for, the reduce kernel is NOT launched and `out` is left untouched; info[0] = 1 then and
// the partials sit at workspace + 16384 bytes as [feature tile][info[1] K ranges][info[2] tokens][128]
// fp32. Otherwise info[0] = 0 and `out` holds the result as usual.
B200_API int b200_gemm_deferred(const void* x, const void* w, void* out, int m, int n, int k, long long ldx,
                                long long ldw, long long ldc, int dtype, const float* x_scale,
                                const float* w_scale, void* workspace, long long workspace_bytes, int* info,
                                void* status, cudaStream_t stream) {
  return gemm_impl(x, w, out, m, n, k, ldx, ldw, ldc, dtype, x_scale, w_scale, nullptr, nullptr, nullptr, 0, 0,
                   workspace, workspace_bytes, status, stream, nullptr, nullptr, nullptr, info);
}

// Row-parallel linear of a tensor-parallel group fused with the all-reduce of its output, the
// residual add, the RMSNorm that follows it and the fp8 quantisation of the next linear's input:
//   s      = sum over ranks of x_r[m][k_r] * w_r[n][k_r]^T (+ bias)          (bf16)
//   res    = res + s            (rank-local residual stream; rows this rank owns only, in place)
//   h      = norm_w == null ? res : rmsnorm(res, eps) * norm_w                (res = s when res is null)
//   out_bf16 / out_q + out_sf = h as bf16 / as e4m3 with 1x128 scales, on every rank
// for m <= 128 tokens and n a multiple of 128. For m > 128 (prefill, DiT sequences; norm_w and out_q
// must be null) the reduce phase is  out_bf16 = res + gate * (s + bias)  with `res` the replicated
// residual stream (read only) and `gate` an optional per-feature factor; `part` then holds
// [m][n] bf16. With `out_local` (reduce-scatter form) only the rows this rank owns (a contiguous
// block of ceil(m / world)) are produced, into out_local [owned][n], and `res` is the rank's block
// of the residual stream. See
// AllReduceParams for the protocol. `part_src`, `out_*`, `flags` are arrays of `world` peer
// pointers into the symmetric heap (index = rank), or, with use_mc = 1, arrays whose entry 0 is
// the multicast alias of the buffer. `part` (partials), `flags_local` (two u32) and `ctr`
// (b200_gemm_allreduce_ctr_bytes() bytes) are this rank's own, zero-initialised once. Every wait on a peer is bounded by
// `wait_budget_cycles` and reports through `status`. `debug_skip_ready` = 1 (tests of the timeout
// path) makes this rank withhold its `ready` signal: the waits then give up, report and return, and
// the counters must be cleared on every rank before the next call.
B200_API long long b200_gemm_allreduce_ctr_bytes() { return kArCtrWords * 4; }

B200_API int b200_gemm_allreduce(const void* x, const void* w, int m, int n, int k, long long ldx,
                                 long long ldw, int dtype, const float* x_scale, const float* w_scale,
                                 const void* bias, void* res, const void* norm_w, float eps,
                                 int weight_plus_one, void* part, void* const* part_src,
                                 void* const* out_bf16, void* const* out_q, void* const* out_sf,
                                 int sf_tile_rows, void* const* flags, void* flags_local, void* ctr,
                                 int rank, int world, int use_mc, int part_splits,
                                 long long wait_budget_cycles, int debug_skip_ready, const void* gate,
                                 void* out_local, void* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return -7;
  const bool large = m > 128;
  if (large && (norm_w != nullptr || out_q != nullptr)) return -7;   // the large-token form is elementwise
  if (!large && (gate != nullptr || out_local != nullptr)) return -7;
  if (part == nullptr || part_src == nullptr || flags == nullptr || flags_local == nullptr || ctr == nullptr) return -7;
  if (out_q != nullptr && (out_sf == nullptr || n % 128 != 0)) return -7;
  if (n / 8 > 256 * kArMaxSegs) return -7;   // row segments of the reduce phase
  AllReduceParams ar{};
  const int np = use_mc ? 1 : world;
  for (int r = 0; r < np; ++r) {
    ar.part_src[r] = static_cast<const __nv_bfloat16*>(part_src[r]);
    ar.out_bf16[r] = out_bf16 ? static_cast<__nv_bfloat16*>(out_bf16[r]) : nullptr;
    ar.out_q[r] = out_q ? static_cast<uint8_t*>(out_q[r]) : nullptr;
    ar.out_sf[r] = out_sf ? static_cast<uint32_t*>(out_sf[r]) : nullptr;
    ar.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  ar.part = static_cast<__nv_bfloat16*>(part);
  ar.res = static_cast<__nv_bfloat16*>(res);
  ar.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  ar.bias = static_cast<const __nv_bfloat16*>(bias);
  ar.eps = eps;
  ar.weight_plus_one = weight_plus_one;
  ar.sf_tile_rows = sf_tile_rows;
  ar.flags_local = static_cast<uint32_t*>(flags_local);
  ar.ctr = static_cast<uint32_t*>(ctr);
  ar.rank = rank;
  ar.world = world;
  ar.use_mc = use_mc ? 1 : 0;
  ar.part_splits = part_splits < 1 ? 1 : part_splits;
  ar.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  ar.debug_skip_ready = debug_skip_ready;
  ar.large = large ? 1 : 0;
  ar.gate = static_cast<const __nv_bfloat16*>(gate);
  ar.out_local = static_cast<__nv_bfloat16*>(out_local);
  return gemm_impl(x, w, nullptr, m, n, k, ldx, ldw, n, dtype, x_scale, w_scale, nullptr, nullptr,
                   nullptr, 0, 1, nullptr, 0, status, stream, &ar);
}

// Column-parallel linear of a sequence-parallel region fused with the all-gather of its input (see
// GatherParams): every rank passes its block of token rows (rank r owns rows [r * per, (r + 1) * per)
// of m, per = ceil(m / world)) and gets out[m][n] = X[m][k] * w[n][k]^T (+ bias, activation) for all m
// tokens and its own n output features. x_local: [rows][k] bf16 (dtype 0) or e4m3 (1, 2) with
// x_scale_local fp32 [rows][k / 128] (dtype 1) or blocked UE8M0 words for the local rows (dtype 2).
// gather / gather_scale / flags: arrays of `world` peer pointers into the symmetric heap (index =
// rank), or with use_mc = 1 arrays whose entry 0 is the multicast alias; gather_local,
// gather_scale_local, flags_local (16 u32) and ctr (16 u32) are this rank's own, zeroed once.
B200_API int b200_allgather_gemm(const void* x_local, const void* x_scale_local, const void* w, void* out, int m, int n,
                                 int k, long long ldw, long long ldc, int dtype, const float* w_scale, const void* bias,
                                 int act, void* const* gather, void* gather_local, void* const* gather_scale,
                                 void* gather_scale_local, void* const* flags, void* flags_local, void* ctr, int rank,
                                 int world, int use_mc, long long wait_budget_cycles, void* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || m <= 128) return -7;
  if (gather == nullptr || gather_local == nullptr || flags == nullptr || flags_local == nullptr || ctr == nullptr) return -7;
  const int esz = dtype != 0 ? 1 : 2;
  if ((static_cast<long long>(k) * esz) % 16 != 0) return -2;
  if (dtype != 0 && (gather_scale == nullptr || gather_scale_local == nullptr || x_scale_local == nullptr)) return -7;
  GatherParams g{};
  g.rank = rank;
  g.world = world;
  g.use_mc = use_mc ? 1 : 0;
  g.rows_total = m;
  g.rows_per_rank = (m + world - 1) / world;
  g.src = static_cast<const uint8_t*>(x_local);
  g.row_bytes = static_cast<long long>(k) * esz;
  g.src_scale = static_cast<const uint32_t*>(x_scale_local);
  g.scale_words = dtype == 1 ? k / 128 : 0;
  g.sf_words = dtype == 2 ? (k + 511) / 512 : 0;
  const int np = use_mc ? 1 : world;
  for (int r = 0; r < np; ++r) {
    g.dst[r] = static_cast<uint8_t*>(gather[r]);
    g.dst_scale[r] = gather_scale ? static_cast<uint32_t*>(gather_scale[r]) : nullptr;
    g.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  g.flags_local = static_cast<uint32_t*>(flags_local);
  g.ctr = static_cast<uint32_t*>(ctr);
  g.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  return gemm_impl(gather_local, w, out, m, n, k, k, ldw, ldc, dtype, static_cast<const float*>(gather_scale_local), w_scale,
                   bias, nullptr, nullptr, act, 1, nullptr, 0, status, stream, nullptr, nullptr, nullptr, nullptr, &g);
}

// Convolution as ONE tcgen05 GEMM without an im2col buffer. The input is a zero-padded,
// channels-last volume flattened to rows [x_rows][cin] (cin a multiple of 64, bf16); kernel tap t
// is the same matrix shifted down by shift[t] rows, so the K loop walks taps x cin while the A tile
// coordinate moves by the tap's row offset and the accumulator stays in TMEM for all taps.
// out[r][co] (bf16, row pitch ldc) = bias[co] + sum_t sum_ci x[r + shift[t]][ci] * w[co][t * cin + ci]
// for r < rows. Rows whose window runs past x_rows read zeros.
B200_API int b200_conv_gemm(const void* x, long long x_rows, int cin, const void* w, int cout, int taps,
                            const int* shift, void* out, long long rows, long long ldc, const void* bias,
                            int act, void* workspace, long long workspace_bytes, void* status,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > 0x7fffffffll || taps < 1 || taps > 28) return -10;
  ConvSpec cs{};
  cs.taps = taps;
  cs.cin = cin;
  cs.x_rows = x_rows;
  for (int t = 0; t < taps; ++t) cs.shift[t] = shift[t];
  return gemm_impl(x, w, out, static_cast<int>(rows), cout, taps * cin, cin, static_cast<long long>(taps) * cin, ldc,
                   0, nullptr, nullptr, bias, nullptr, nullptr, act, 0, workspace, workspace_bytes, status, stream,
                   nullptr, nullptr, &cs);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in b200_noalloc.h).
// ------------------------------------------------------------------------------------------
#include "b200_noalloc.h"

// Scratch of the split-K path, resident in the library image: tile counters, then fp32 partials.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200_NOALLOC_SCRATCH_BYTES];

// In host code the symbol above is only a stand-in; the address a kernel can use has to be asked
// for per device. Resolved on the first call on each device and remembered.
static void* g_noalloc_ptr[64] = {nullptr};

B200_API int b200_gemm_noalloc(const void* x, const void* w, void* out, int m, int n, int k,
                               long long ldx, long long ldw, long long ldc, int dtype,
                               const float* x_scale, const float* w_scale, const void* bias,
                               const void* residual, cudaStream_t stream) {
  if (m > B200_NOALLOC_MAX_TOKENS) return B200_NOALLOC_ERR_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200_NOALLOC_ERR_SETUP;
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr)
      return B200_NOALLOC_ERR_SETUP;
    g_noalloc_ptr[dev] = ptr;
  }
  void* scratch = g_noalloc_ptr[dev];
  // m <= 128 keeps every partial slot at 64 KB or less and the automatic policy never uses more
  // than one slot per SM, so counters + partials always fit; gemm_impl re-checks against the size.
  if (cudaMemsetAsync(scratch, 0, b200::kSplitCounterBytes, stream) != cudaSuccess)
    return B200_NOALLOC_ERR_SETUP;
  return b200::gemm_impl(x, w, out, m, n, k, ldx, ldw, ldc, dtype, x_scale, w_scale, bias, nullptr,
                         residual, 0, 0, scratch, B200_NOALLOC_SCRATCH_BYTES, nullptr, stream, nullptr);
}

// Grouped GEMM for expert layers: for every group g, out[g][m][n] = x[g][m][k] * w[g][n][k]^T with
// all groups in ONE launch (weights stacked as [groups * n][k], token blocks as [groups * m][k],
// m in {16, 32, 64, 128} slots per token block, `chunks` token blocks per group (x and out are then
// [groups * chunks * m] rows with block e * chunks + c belonging to group e); blocks whose entry of the optional
// device array group_counts is zero are skipped and their output rows left untouched). Same kernel as b200_gemm: expert
// weights fill the 128-row MMA dimension, each expert's token block is the N operand.
B200_API int b200_gemm_grouped(const void* x, const void* w, void* out, int groups, int m, int n, int k,
                               int dtype, const float* x_scale, const float* w_scale, int act,
                               const int* group_counts, int chunks, void* workspace,
                               long long workspace_bytes, void* status, cudaStream_t stream) {
  if (groups <= 0) return 0;
  GroupSpec gs{groups, group_counts, 0, 0};
  gs.chunks = chunks < 1 ? 1 : chunks;
  return gemm_impl(x, w, out, m, n, k, k, k, n, dtype, x_scale, w_scale, nullptr, nullptr, nullptr, act, 0,
                   workspace, workspace_bytes, status, stream, nullptr, &gs);
}

// Column-batched grouped GEMM (bf16): out[t][g * out_stride + j] = sum_i x[t][g * x_koff + i] *
// w[g * n + j][i] for t < m <= 128 tokens, j < n, i < k. Per-head projections of one token block
// (multi-head latent attention: absorbing W_uk into the query and applying W_uv to the output)
// without transposing activations to head-major order. x_koff * 2 bytes must be a multiple of 16
// and k a multiple of 64.
// Grouped GEMM over a device-side block list: token blocks of `m` slots each, block b uses the
// weights of group block_group[b]; *dyn_blocks (<= max_blocks) blocks are computed. x / out are
// [max_blocks * m] rows. Built by b200_moe_dispatch_dynamic.
B200_API int b200_gemm_grouped_dynamic(const void* x, const void* w, void* out, int groups, int max_blocks, int m,
                                       int n, int k, int dtype, const float* x_scale, const float* w_scale, int act,
                                       const int* block_group, const int* dyn_blocks, void* status,
                                       cudaStream_t stream) {
  if (groups <= 0 || max_blocks <= 0) return 0;
  if (block_group == nullptr || dyn_blocks == nullptr) return -9;
  GroupSpec gs{groups, nullptr, 0, 0};
  gs.chunks = max_blocks;
  gs.block_group = block_group;
  gs.dyn_blocks = dyn_blocks;
  return gemm_impl(x, w, out, m, n, k, k, k, n, dtype, x_scale, w_scale, nullptr, nullptr, nullptr, act, 1,
                   nullptr, 0, status, stream, nullptr, &gs);
}

B200_API int b200_gemm_colbatched(const void* x, const void* w, void* out, int groups, int m, int n, int k,
                                  long long ldx, int x_koff, long long ldc, int out_stride, void* workspace,
                                  long long workspace_bytes, void* status, cudaStream_t stream) {
  if (groups <= 0 || m <= 0) return 0;
  if (x_koff <= 0) return -9;
  GroupSpec gs{groups, nullptr, x_koff, out_stride};
  return gemm_impl(x, w, out, m, n, k, ldx, k, ldc, 0, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0,
                   workspace, workspace_bytes, status, stream, nullptr, &gs);
}
