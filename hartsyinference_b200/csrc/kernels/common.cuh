// Shared device-side building blocks for the sm_100a kernels: PTX wrappers for
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc, MMA, commit, ld),
// bounded waits, and the error-status word every kernel reports into.
//
// Design rules that every kernel in this directory follows:
//  * no wait is unbounded: a spin on an mbarrier or on a flag written by another
//    CTA / GPU gives up after kWaitBudgetNs, records where it gave up in the status
//    word and lets the CTA run to its normal exit (TMEM is released there);
//  * no __trap(), no device assert;
//  * TMA loads are always the plain per-CTA form.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace b200 {

// ---------------------------------------------------------------------------------------------
// Error status. One 4-word record in global memory per library instance; the first failing wait
// wins (atomicCAS on word 0). Host code reads it with b200_last_device_status().
//   word0 = code (0 = ok), word1 = kernel id, word2 = site id, word3 = detail (blockIdx.x etc.)
// ---------------------------------------------------------------------------------------------
enum StatusCode : uint32_t {
  kOk = 0,
  kWaitTimeout = 1,    // an mbarrier / flag wait ran out of budget
  kBadArgument = 2,    // a launch-time check failed on the device side
};

enum KernelId : uint32_t {
  kKernelGemm = 1,
  kKernelGemmSplitKReduce = 2,
  kKernelAttnDecode = 3,
  kKernelAttnPrefill = 4,
  kKernelGemmAllReduce = 5,
  kKernelAllReduce = 6,
  kKernelMoe = 7,
  kKernelSage = 8,
  kKernelCfgStep = 9,
  kKernelAllToAll = 10,
  kKernelWaitProbe = 11,
  kKernelDpExchange = 12,
};

struct DeviceStatus {
  uint32_t code;
  uint32_t kernel;
  uint32_t site;
  uint32_t detail;
};

__device__ __forceinline__ void report_status(DeviceStatus* st, uint32_t code, uint32_t kernel,
                                              uint32_t site, uint32_t detail) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->kernel = kernel;
    st->site = site;
    st->detail = detail;
    __threadfence_system();
  }
}

// Default budget for any single wait, in SM clock cycles (about two seconds at 2 GHz). Waits
// between CTAs of one kernel normally complete in microseconds; a value this long only triggers
// when a peer never arrives. Tests of the timeout path pass a much smaller budget. The budget is
// counted with clock64(), which costs a few cycles; %globaltimer is far too slow to read inside a
// pipeline handshake (it showed up as microseconds per k-block in the block-scaled GEMM).
constexpr long long kWaitBudgetCycles = 4000000000ll;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false when the budget ran out (the caller must then leave its loop).
// `abort_flag` is a CTA-shared word: once any role of the CTA has timed out the others stop
// waiting quickly instead of each burning a full budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile uint32_t* abort_flag,
                                          long long budget_cycles = kWaitBudgetCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag != 0) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Thread-block clusters: rank of this CTA, cluster-wide barrier, loads from a peer CTA's shared
// memory (distributed shared memory).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta_rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// Per-device one-time set-up. Function attributes (dynamic shared memory limit) and device
// properties belong to a device, not to the process: one process may drive several GPUs, so the
// "done once" marks are kept per device ordinal.
// ---------------------------------------------------------------------------------------------
struct PerDeviceOnce {
  bool done[64] = {};
  // True exactly once per device (always true for ordinals past the table, which only repeats work).
  bool first_time() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute
// may start before its predecessor in the stream has finished; pdl_wait() blocks until the
// predecessor grid has completed and its writes are visible (a no-op for an ordinary launch).
// pdl_trigger() in the predecessor lets such a dependent start early.
// ---------------------------------------------------------------------------------------------
// Host side: launch with the programmatic-serialization attribute (when enabled). A kernel launched
// this way MUST call pdl_wait() before it touches anything an earlier kernel wrote or still reads.
extern bool g_b200_pdl;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_b200_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, per-CTA form only)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tile load global -> shared; completion is signalled on `bar` as transaction bytes.
// c0 is the innermost (contiguous) coordinate and must keep c0 * elemsize a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05 op issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle that a TMA box of 128 bytes x R rows produces: 8-row groups are 1024 bytes
// apart (stride byte offset), the leading byte offset is unused for swizzled K-major layouts.
// Layout of the 64-bit descriptor (matrix-descriptor format of tcgen05.mma):
//   [0,14)  start address >> 4      [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4 [46,48) version = 1      [61,64) swizzle: 2 = 128 B
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(1) << 16;            // LBO (ignored for SW128 K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // SBO = 1024 B between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}

// Instruction descriptor for tcgen05.mma kind::f16 / kind::f8f6f4 / kind::i8, dense, A and B both
// K-major, accumulator fp32 (or s32 for kind::i8).
//   [4,6) D format (1 = f32, 2 = s32)  [7,10) A format  [10,13) B format
//   [15] A major (0 = K)  [16] B major (0 = K)  [17,23) N >> 3  [24,29) M >> 4
constexpr uint32_t kFmtBf16 = 1;   // kind::f16: 0 = f16, 1 = bf16
constexpr uint32_t kFmtF16 = 0;
constexpr uint32_t kFmtE4m3 = 0;   // kind::f8f6f4: 0 = e4m3, 1 = e5m2
constexpr uint32_t kFmtS8 = 1;     // kind::i8: 0 = u8, 1 = s8
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t afmt,
                                                  uint32_t bfmt, uint32_t dfmt = 1) {
  return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_fp8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- hardware block scaling (kind::mxf8f6f4.block_scale, one UE8M0 scale per 32 K elements) ----
// Instruction descriptor of the block-scaled form: no D format field (always fp32);
//   [4,6) B scale-factor id  [7,10) A format  [10,13) B format  [17,23) N >> 3
//   [23] scale format (1 = UE8M0)  [24,29) M >> 4  [29,31) A scale-factor id.
// The scale-factor id picks one of the four bytes of a 32-bit TMEM scale column, so a column holds
// the scales of four consecutive K groups and is refreshed once per four.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t m, uint32_t n) {
  return (kFmtE4m3 << 7) | (kFmtE4m3 << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
__device__ __forceinline__ void mma_mxf8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate, uint32_t sfa_tmem,
                                            uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Shared-memory descriptor of one 512-byte scale-factor block: 32 rows of 16 bytes, no swizzle
// (8-row core matrices of 128 bytes, so the stride between them is 128 bytes).
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // SBO
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version for sm_100
  return d;
}
// Copies a 32 x 128-bit block from shared memory into 4 TMEM columns of all four lane quarters.
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_addr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16), completion
// counted as transaction bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns. A warp may only touch
// the TMEM lane quarter (warp_id % 4) * 32 .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// registers -> TMEM: the mirror image of tmem_ld_32x32 (same lane-quarter rule)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D (TMEM) += A (TMEM: lane = row, two bf16 per 32-bit column along K) * B (shared memory, K-major)
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// Deferred split-K sums. A small-token GEMM whose tiles were all cut along K leaves fp32 partials
// in scratch: per 128-feature tile `ta` and K range `s` one slot [bn tokens][128 features]. Instead
// of a reduce kernel of its own, the kernel that consumes the GEMM's output can add the ranges
// while it reads: value(token, feature) = sum over s of ws[((ta * splits + s) * bn + token) * 128 +
// feature % 128], ta = feature / 128, rounded to bf16 as the stored output would have been.
// ---------------------------------------------------------------------------------------------
struct SplitPartials {
  const float* ws;     // nullptr: the consumer reads its ordinary bf16 input
  int splits, bn;
};
__device__ __forceinline__ float split_sum(const SplitPartials& sp, int token, int feature) {
  const float* base = sp.ws + (static_cast<long long>(feature >> 7) * sp.splits * sp.bn + token) * 128 + (feature & 127);
  float acc = 0.f;
  for (int s = 0; s < sp.splits; ++s) acc += __ldcg(base + static_cast<long long>(s) * sp.bn * 128);
  return __bfloat162float(__float2bfloat16(acc));
}
// eight consecutive features (feature0 a multiple of 8)
__device__ __forceinline__ void split_sum8(const SplitPartials& sp, int token, int feature0, float (&out)[8]) {
  const float* base = sp.ws + (static_cast<long long>(feature0 >> 7) * sp.splits * sp.bn + token) * 128 + (feature0 & 127);
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  for (int s = 0; s < sp.splits; ++s) {
    const float4 x = __ldcg(reinterpret_cast<const float4*>(base + static_cast<long long>(s) * sp.bn * 128));
    const float4 y = __ldcg(reinterpret_cast<const float4*>(base + static_cast<long long>(s) * sp.bn * 128 + 4));
    a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
  }
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = __bfloat162float(__float2bfloat16(v[i]));
}

// ---------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

}  // namespace b200
