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

// ------------------------------------------------------------------------------------------
// CFG-parallel combine fused with the scheduler step.
//
// Two ranks denoise the conditional (rank 0) and unconditional (rank 1) branch of the same latents.
// Each writes its velocity prediction into its own slot of the symmetric heap; this kernel then
//   1. tells the peer "my prediction of step e is written" and waits for the peer's flag,
//   2. reads the PEER's prediction straight over NVLink (no gather into a local copy),
//   3. applies v = u + g (c - u) and the Euler update z += v dt to the local fp32 latents.
// Both ranks hold identical latents afterwards. One launch replaces all_gather + combine + step
// (the reference copies the branch result peer to peer and runs a separate CFG/Euler kernel:
// src/HartsyInference.Diffusion/Pipelines/FluxPipeline.cs PredictDrainFree:750-807, CopyFromPeer:780,
// CfgEulerStep:821). A second flag pair keeps a fast rank from overwriting its slot for step e + 1
// while the peer still reads step e.
// ------------------------------------------------------------------------------------------
namespace b200 {

struct CfgCombineArgs {
  const __nv_bfloat16* pred[2];   // [rank] prediction slots (peer-mapped)
  uint32_t* ready[2];             // [rank] -> flag array of that rank: ready[q][r] = step written by r
  uint32_t* consumed[2];          // [rank] -> consumed[q][r] = step that r has finished reading from q
  float* z;                       // local latents
  uint32_t* epoch;                // local call counter
  uint32_t* fin;
  long long n;
  int rank;                       // 0 = conditional branch, 1 = unconditional
  float guidance, dt;
  long long wait_budget;
  DeviceStatus* status;
};

__global__ void __launch_bounds__(256) cfg_combine_kernel(const CfgCombineArgs a) {
  __shared__ uint32_t s_ok;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
  const int peer = a.rank ^ 1;
  if (threadIdx.x == 0) {
    // my prediction (written by the kernels before this one) is complete: publish, then wait
    __threadfence_system();
    if (blockIdx.x == 0) st_release_sys(a.ready[peer] + a.rank, e);
    s_ok = wait_geq(a.ready[a.rank] + peer, e, a.wait_budget) ? 1u : 0u;
    if (!s_ok) report_status(a.status, kWaitTimeout, kKernelCfgStep, 1, blockIdx.x);
  }
  __syncthreads();
  if (s_ok) {
    const __nv_bfloat16* mine = a.pred[a.rank];
    const __nv_bfloat16* theirs = a.pred[peer];
    const long long nvec = a.n >> 3;
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      const uint4 m4 = *reinterpret_cast<const uint4*>(mine + v * 8);
      const uint4 t4 = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(theirs + v * 8));
      const __nv_bfloat162* mh = reinterpret_cast<const __nv_bfloat162*>(&m4);
      const __nv_bfloat162* th = reinterpret_cast<const __nv_bfloat162*>(&t4);
      float4 z0 = *reinterpret_cast<float4*>(a.z + v * 8), z1 = *reinterpret_cast<float4*>(a.z + v * 8 + 4);
      float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fm = __bfloat1622float2(mh[i]), ft = __bfloat1622float2(th[i]);
        const float2 c = a.rank == 0 ? fm : ft, u = a.rank == 0 ? ft : fm;
        zz[2 * i] += (a.guidance * c.x + (1.f - a.guidance) * u.x) * a.dt;
        zz[2 * i + 1] += (a.guidance * c.y + (1.f - a.guidance) * u.y) * a.dt;
      }
      *reinterpret_cast<float4*>(a.z + v * 8) = make_float4(zz[0], zz[1], zz[2], zz[3]);
      *reinterpret_cast<float4*>(a.z + v * 8 + 4) = make_float4(zz[4], zz[5], zz[6], zz[7]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.fin, 1u) == gridDim.x - 1) {
      // every block of this rank is done with the peer's slot: let the peer reuse it, and do not
      // return before the peer is done with ours (the next step overwrites it)
      *a.fin = 0;
      st_release_sys(a.consumed[peer] + a.rank, e);
      if (!wait_geq(a.consumed[a.rank] + peer, e, a.wait_budget))
        report_status(a.status, kWaitTimeout, kKernelCfgStep, 2, blockIdx.x);
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = e;
      __threadfence();
    }
  }
}

}  // namespace b200

// pred / flags: arrays of 2 device pointers (index = rank) into the symmetric heap; flags per rank:
// 4 x u32 (ready[2], consumed[2]), zero-initialised; epoch / fin: local zero-initialised u32.
// n bf16 values (a multiple of 8); z: local fp32 latents [n].
B200_API int b200_cfg_combine(void* const* pred, void* const* flags, void* epoch, void* fin, float* z, long long n,
                              int rank, float guidance, float dt, long long wait_budget_cycles, void* status,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || rank < 0 || rank > 1) return -2;
  CfgCombineArgs a{};
  for (int r = 0; r < 2; ++r) {
    a.pred[r] = static_cast<const __nv_bfloat16*>(pred[r]);
    a.ready[r] = static_cast<uint32_t*>(flags[r]);
    a.consumed[r] = static_cast<uint32_t*>(flags[r]) + 2;
  }
  a.z = z;
  a.epoch = static_cast<uint32_t*>(epoch);
  a.fin = static_cast<uint32_t*>(fin);
  a.n = n;
  a.rank = rank;
  a.guidance = guidance;
  a.dt = dt;
  a.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  a.status = static_cast<DeviceStatus*>(status);
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148) blocks = 148;
  cfg_combine_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
