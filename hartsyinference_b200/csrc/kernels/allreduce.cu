// Latency-oriented all-reduce (sum, bf16) over NVLink for the decode regime: at most a few MB per
// call, where a ring / tree collective is bound by its launch and hop latencies.
//
// One kernel, every rank running the same grid, two counters per rank (cumulative over calls):
//   1. "ready": the kernel runs after the producer of its input in stream order, so a started
//      kernel means a finished producer on that rank; block 0 adds 1 to `ready` on every rank (one
//      multimem.red through the NVSwitch, or one red per peer) and every block waits until its own
//      `ready` shows all ranks of this call;
//   2. rank r owns the r-th 1/W slice: each 16-byte vector of the slice is fetched summed over all
//      ranks (multimem.ld_reduce: the switch adds the ranks' copies in fp32; without a multicast
//      mapping: one peer load per rank, many in flight, summed in fixed rank order), optionally
//      + residual, and stored as bf16 into every rank's output (multimem.st or one store per peer);
//   3. "done": the rank's last block adds 1 to `done` everywhere; block 0 leaves only after its own
//      `done` shows all ranks, i.e. the whole output has landed locally.
// Inputs, outputs and counters live in the symmetric heap. No host writes between calls, so the
// kernel can be captured in CUDA graphs. Every wait is bounded and reports into the status word.
//
// Reuse rules that make single buffers safe: a rank passes "done" of call c only after every peer
// has finished READING its input for call c (peers signal after their stores), and a peer can
// start WRITING a rank's output for call c + 1 only after that rank has entered call c + 1.
//
// Reference counterpart: NcclComm.AllReduceSum (src/HartsyInference.Cuda/NcclComm.cs:53-85) called
// after the o- and down-projections (TensorParallelTransformer.cs:298,307).
#include "comm.cuh"

namespace b200 {

constexpr int kArMaxBlocks = 64;

struct AllReduceArgs {
  const uint4* in[8];       // use_mc: [0] is the multicast alias
  uint4* out[8];
  uint32_t* flags[8];       // per rank: [0] ready, [1] done
  uint32_t* flags_local;
  uint32_t* ctr;            // local: [0] calls completed, [1] blocks done with their slice, [2] blocks finished
  const uint4* residual;    // optional local bf16 tensor added to the sum
  int rank, world, use_mc;
  long long vecs;           // 16-byte vectors in the whole tensor
  long long wait_budget;
  DeviceStatus* status;
};

__device__ __forceinline__ void ar_signal_all(const AllReduceArgs& a, int which) {
  if (a.use_mc) {
    multimem_red_release_add(a.flags[0] + which, 1u);
  } else {
    for (int r = 0; r < a.world; ++r) red_release_sys_add(a.flags[(a.rank + r) % a.world] + which, 1u);
  }
}

__global__ void __launch_bounds__(512) allreduce_kernel(const AllReduceArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t s_ok;
  const int tid = threadIdx.x, b = blockIdx.x;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(a.ctr) + 1u;
  // ---- 1. inputs ready everywhere
  if (tid == 0) {
    if (b == 0) {
      __threadfence_system();
      ar_signal_all(a, 0);
    }
    s_ok = wait_flag_geq(a.flags_local, call * static_cast<uint32_t>(a.world), a.wait_budget) ? 1u : 0u;
    if (!s_ok) report_status(a.status, kWaitTimeout, kKernelAllReduce, 1, b);
  }
  __syncthreads();
  if (s_ok) {
    // ---- 2. reduce this rank's slice, write it everywhere
    const long long slice = a.vecs / a.world, base = static_cast<long long>(a.rank) * slice;
    for (long long v = static_cast<long long>(b) * blockDim.x + tid; v < slice;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      if (a.use_mc) {
        add_bf16x8(acc, multimem_ld_reduce_bf16x8(a.in[0] + base + v));
      } else {
        uint4 x[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < a.world) x[r] = ld_relaxed_sys_v4(a.in[r] + base + v);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < a.world) add_bf16x8(acc, x[r]);
      }
      if (a.residual) add_bf16x8(acc, a.residual[base + v]);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) ow[i] = pack_bf16x2(acc[2 * i], acc[2 * i + 1]);
      if (a.use_mc) {
        multimem_st_v4(a.out[0] + base + v, o);
      } else {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          // start with the neighbour so that the ranks do not all write to rank 0 first
          const int dst = (a.rank + r) % a.world;
          if (r < a.world) a.out[dst][base + v] = o;
        }
      }
    }
  }
  // ---- 3. outputs written everywhere
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    if (atomicAdd(a.ctr + 1, 1u) == gridDim.x - 1) {
      __threadfence_system();
      ar_signal_all(a, 1);
    }
    if (b == 0 && !wait_flag_geq(a.flags_local + 1, call * static_cast<uint32_t>(a.world), a.wait_budget))
      report_status(a.status, kWaitTimeout, kKernelAllReduce, 2, b);
    // the last block to finish closes the call: every block has read the call counter by now
    __threadfence();
    if (atomicAdd(a.ctr + 2, 1u) == gridDim.x - 1) {
      a.ctr[1] = 0;
      a.ctr[2] = 0;
      *reinterpret_cast<volatile uint32_t*>(a.ctr) = call;
      __threadfence();
    }
  }
}

}  // namespace b200

using namespace b200;

// in / out / flags: arrays of `world` device pointers (index = rank) into the symmetric heap, or,
// with use_mc = 1, arrays whose entry 0 is the multicast alias. flags: two u32 per rank;
// flags_local: this rank's own two; ctr: three local u32; all zero-initialised once.
// `elems` bf16 values (a multiple of 8 * world).
B200_API int b200_allreduce(void* const* in, void* const* out, void* const* flags, void* flags_local, void* ctr,
                            const void* residual, long long elems, int rank, int world, int use_mc,
                            long long wait_budget_cycles, void* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || elems <= 0) return -2;
  if (elems % (8ll * world) != 0) return -3;
  AllReduceArgs a{};
  const int np = use_mc ? 1 : world;
  for (int r = 0; r < np; ++r) {
    a.in[r] = static_cast<const uint4*>(in[r]);
    a.out[r] = static_cast<uint4*>(out[r]);
    a.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  a.flags_local = static_cast<uint32_t*>(flags_local);
  a.ctr = static_cast<uint32_t*>(ctr);
  a.residual = static_cast<const uint4*>(residual);
  a.rank = rank;
  a.world = world;
  a.use_mc = use_mc ? 1 : 0;
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
  int mode;                       // 0: z += v dt (Euler step); 1: z = v (the combined prediction, for any other scheduler)
  int pred_f32;                   // the prediction slots hold fp32 instead of bf16
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
    s_ok = wait_flag_geq(a.ready[a.rank] + peer, e, a.wait_budget) ? 1u : 0u;
    if (!s_ok) report_status(a.status, kWaitTimeout, kKernelCfgStep, 1, blockIdx.x);
  }
  __syncthreads();
  if (s_ok) {
    const __nv_bfloat16* mine = a.pred[a.rank];
    const __nv_bfloat16* theirs = a.pred[peer];
    const long long nvec = a.n >> 3;
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      float fm[8], ft[8];
      if (a.pred_f32) {
        const float* mf = reinterpret_cast<const float*>(mine) + v * 8;
        const float* tf = reinterpret_cast<const float*>(theirs) + v * 8;
        const uint4 m0 = *reinterpret_cast<const uint4*>(mf), m1 = *reinterpret_cast<const uint4*>(mf + 4);
        const uint4 t0 = ld_relaxed_sys_v4(tf), t1 = ld_relaxed_sys_v4(tf + 4);
        const uint32_t mw[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        const uint32_t tw[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          fm[i] = __uint_as_float(mw[i]);
          ft[i] = __uint_as_float(tw[i]);
        }
      } else {
        const uint4 m4 = *reinterpret_cast<const uint4*>(mine + v * 8);
        const uint4 t4 = ld_relaxed_sys_v4(theirs + v * 8);
        const __nv_bfloat162* mh = reinterpret_cast<const __nv_bfloat162*>(&m4);
        const __nv_bfloat162* th = reinterpret_cast<const __nv_bfloat162*>(&t4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a2 = __bfloat1622float2(mh[i]), b2 = __bfloat1622float2(th[i]);
          fm[2 * i] = a2.x; fm[2 * i + 1] = a2.y;
          ft[2 * i] = b2.x; ft[2 * i + 1] = b2.y;
        }
      }
      float zz[8];
      if (a.mode == 0) {
        const float4 z0 = *reinterpret_cast<float4*>(a.z + v * 8), z1 = *reinterpret_cast<float4*>(a.z + v * 8 + 4);
        zz[0] = z0.x; zz[1] = z0.y; zz[2] = z0.z; zz[3] = z0.w;
        zz[4] = z1.x; zz[5] = z1.y; zz[6] = z1.z; zz[7] = z1.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = a.rank == 0 ? fm[i] : ft[i], u = a.rank == 0 ? ft[i] : fm[i];
        const float comb = a.guidance * c + (1.f - a.guidance) * u;
        zz[i] = a.mode == 0 ? zz[i] + comb * a.dt : comb;
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
      if (!wait_flag_geq(a.consumed[a.rank] + peer, e, a.wait_budget))
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
// mode 0: z += (u + g (c - u)) dt; mode 1: z = u + g (c - u). pred_f32: the slots hold fp32.
B200_API int b200_cfg_combine(void* const* pred, void* const* flags, void* epoch, void* fin, float* z, long long n,
                              int rank, float guidance, float dt, int mode, int pred_f32, long long wait_budget_cycles,
                              void* status, cudaStream_t stream) {
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
  a.mode = mode;
  a.pred_f32 = pred_f32;
  a.wait_budget = wait_budget_cycles > 0 ? wait_budget_cycles : kWaitBudgetCycles;
  a.status = static_cast<DeviceStatus*>(status);
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148) blocks = 148;
  cfg_combine_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
