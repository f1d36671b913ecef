// Latency-oriented all-reduce (sum, bf16) over NVLink peer memory for the decode regime: at most
// a few MB per call, where a ring / tree collective is bound by its launch and hop latencies.
//
// Two-shot inside ONE kernel, every rank running the same grid:
//   1. barrier "inputs ready": block b of rank r raises flag_a[q][b][r] on every peer q and waits
//      for its own row flag_a[r][b][*] (the kernel runs after the producer GEMM in stream order,
//      so a started kernel means a finished producer on that rank);
//   2. rank r owns the r-th 1/W slice: 16-byte vectors of the slice are loaded from all W input
//      buffers (peer loads, many in flight), summed in fp32 (fixed rank order: deterministic and
//      identical on every rank), optionally + residual, and stored as bf16 into all W output
//      buffers (peer stores);
//   3. barrier "outputs written": fence, flag_b, wait.
// Inputs, outputs and flags live in the CUDA-IPC symmetric heap. Flags carry a device-resident
// call counter (no host writes between calls, so the kernel can be captured in CUDA graphs).
// Every wait is bounded and reports into the status word.
//
// Reuse rules that make single buffers safe: a rank leaves barrier 3 only after every peer has
// finished READING its input (peers signal after their stores), and a peer can start WRITING a
// rank's output for the next call only after that rank has entered the next call (barrier 1).
//
// Reference counterpart: NcclComm.AllReduceSum (src/HartsyInference.Cuda/NcclComm.cs:53-85) called
// after the o- and down-projections (TensorParallelTransformer.cs:298,307).
#include "common.cuh"

namespace b200 {

constexpr int kArMaxBlocks = 64;

struct AllReduceArgs {
  const uint4* in[8];
  uint4* out[8];
  uint32_t* flag_a[8];      // [kArMaxBlocks][8] per rank
  uint32_t* flag_b[8];
  uint32_t* epoch;          // local: calls completed
  uint32_t* fin;            // local: blocks finished in the current call
  const uint4* residual;    // optional local bf16 tensor added to the sum
  int rank, world;
  long long vecs;           // 16-byte vectors in the whole tensor
  long long wait_budget;
  DeviceStatus* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const uint4* addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ bool wait_geq(const uint32_t* addr, uint32_t target, long long budget) {
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(addr) - target) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget) return false;
    }
  }
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__global__ void __launch_bounds__(512) allreduce_kernel(const AllReduceArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t s_ok;
  const int tid = threadIdx.x, b = blockIdx.x;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
  if (tid == 0) s_ok = 1u;
  __syncthreads();
  // ---- 1. inputs ready everywhere
  if (tid < a.world) {
    st_release_sys(a.flag_a[tid] + b * 8 + a.rank, e);
    if (!wait_geq(a.flag_a[a.rank] + b * 8 + tid, e, a.wait_budget)) {
      report_status(a.status, kWaitTimeout, kKernelAllReduce, 1, b);
      s_ok = 0u;
    }
  }
  __syncthreads();
  if (s_ok) {
    // ---- 2. reduce this rank's slice, write it everywhere
    const long long slice = a.vecs / a.world, base = static_cast<long long>(a.rank) * slice;
    for (long long v = static_cast<long long>(b) * blockDim.x + tid; v < slice;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      uint4 x[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < a.world) x[r] = ld_relaxed_sys_v4(a.in[r] + base + v);
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      if (a.residual) add_bf16x8(acc, a.residual[base + v]);
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < a.world) add_bf16x8(acc, x[r]);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) ow[i] = pack_bf16x2(acc[2 * i], acc[2 * i + 1]);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        // start with the neighbour so that the ranks do not all write to rank 0 first
        const int dst = (a.rank + r) % a.world;
        if (r < a.world) a.out[dst][base + v] = o;
      }
    }
  }
  // ---- 3. outputs written everywhere
  __threadfence_system();
  __syncthreads();
  if (tid < a.world && s_ok) {
    st_release_sys(a.flag_b[tid] + b * 8 + a.rank, e);
    if (!wait_geq(a.flag_b[a.rank] + b * 8 + tid, e, a.wait_budget))
      report_status(a.status, kWaitTimeout, kKernelAllReduce, 2, b);
  }
  __syncthreads();
  if (tid == 0) {
    // the last block to finish closes the call: every block has read the old counter by now
    __threadfence();
    if (atomicAdd(a.fin, 1u) == gridDim.x - 1) {
      *a.fin = 0;
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = e;
      __threadfence();
    }
  }
}

}  // namespace b200

using namespace b200;

// Flags per rank: two arrays of [64 blocks][8 ranks] u32 (4 KB), zero-initialised once.
B200_API long long b200_allreduce_flag_bytes() { return 2ll * kArMaxBlocks * 8 * 4; }

// in / out / flags: arrays of `world` device pointers (index = rank) into the symmetric heap; epoch
// and fin: two zero-initialised local u32. `elems` bf16 values (a multiple of 8 * world).
B200_API int b200_allreduce(void* const* in, void* const* out, void* const* flags, void* epoch, void* fin,
                            const void* residual, long long elems, int rank, int world,
                            long long wait_budget_cycles, void* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || elems <= 0) return -2;
  if (elems % (8ll * world) != 0) return -3;
  AllReduceArgs a{};
  for (int r = 0; r < world; ++r) {
    a.in[r] = static_cast<const uint4*>(in[r]);
    a.out[r] = static_cast<uint4*>(out[r]);
    a.flag_a[r] = static_cast<uint32_t*>(flags[r]);
    a.flag_b[r] = static_cast<uint32_t*>(flags[r]) + kArMaxBlocks * 8;
  }
  a.epoch = static_cast<uint32_t*>(epoch);
  a.fin = static_cast<uint32_t*>(fin);
  a.residual = static_cast<const uint4*>(residual);
  a.rank = rank;
  a.world = world;
  a.vecs = elems / 8;
  a.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  a.status = static_cast<DeviceStatus*>(status);
  const long long slice = a.vecs / world;
  int blocks = static_cast<int>((slice + 511) / 512);
  if (blocks < 1) blocks = 1;
  if (blocks > kArMaxBlocks) blocks = kArMaxBlocks;
  launch_pdl(allreduce_kernel, dim3(blocks), dim3(512), 0, stream, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
