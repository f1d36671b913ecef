// Batched token sampling on the device: temperature -> top-k -> top-p -> min-p -> seeded draw, one
// thread block per request row, the vocabulary never sorted and never copied to the host.
//
// With w_i = exp((l_i - max l) / T) every filter of the chain keeps a set of the form {w_i >= tau}:
//   top-k   tau = the k-th largest w (ties at that value are all kept, like a mask "below the k-th");
//   top-p   over the survivors, in descending order, keep an element while the mass in front of it
//           is <= p of the survivors' mass: tau = the smallest w still kept;
//   min-p   tau = min_p * max w = min_p.
// The two order statistics are found by a radix search on the bit pattern of w (positive floats
// order like their bits): three passes of 11 + 11 + 10 bits, each one histogram of counts and of
// (fixed-point) masses in shared memory. The draw walks the vocabulary in index order with a block-wide prefix
// sum of the kept masses. Eight passes over a row that stays in L2.
//
// The reference applies the same chain on the host, one request at a time, after copying the logits
// back (src/HartsyInference.LLM/Sampling/SamplerChain.cs:26-85, TopKSampler.cs, TopPSampler.cs,
// MinPSampler.cs); a row with temperature <= 0 is an argmax (ties -> lowest id) like
// lm_argmax_lastdim_f32 (Kernels/lm/lm_f32.cu:214).
#include "common.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;
constexpr int kSampleBins = 2048;

struct SampleParams {
  const void* logits;          // [rows][ld] fp32 or bf16
  int is_f32;
  long long ld;
  int vocab;
  const float* temperature;    // [rows]; <= 0: argmax
  const int* top_k;            // [rows]; <= 0 or >= vocab: off
  const float* top_p;          // [rows]; <= 0 or >= 1: off
  const float* min_p;          // [rows]; <= 0: off
  const unsigned long long* seed;     // [rows]
  const unsigned long long* counter;  // [rows]: position of the draw in the request's stream
  int* out;                    // [rows]
};

__device__ __forceinline__ float sample_logit(const SampleParams& p, long long row_off, int i) {
  return p.is_f32 ? static_cast<const float*>(p.logits)[row_off + i]
                  : __bfloat162float(static_cast<const __nv_bfloat16*>(p.logits)[row_off + i]);
}

// splitmix64 of (seed, counter) -> uniform in [0, 1)
__device__ __forceinline__ float sample_uniform(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.f / 16777216.f);
}

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
    t = warp_max(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// One level of the radix search. Elements whose bits above `shift + bits` equal `prefix` (all
// elements at the first level) and whose w >= floor are binned by `bits` bits at `shift`. Walking
// the bins from the top, with `count_before` / `mass_before` already in front:
//   by_count: stop in the bin where the count reaches `k`
//   else:     stop in the bin that holds the first element whose mass in front exceeds `limit`
// Leaves the chosen bin in sh->bin (-1: the walk ran off the end, everything is kept) and adds what lies
// in front of that bin to the running totals in `sh`.
// Masses are accumulated in 2^-40 fixed point: integer shared-memory atomics are native and the sums do
// not depend on the order of arrival, so a (seed, counter) pair always draws the same token.
constexpr float kMassScale = 1099511627776.f;        // 2^40

struct RadixState {
  unsigned prefix;                      // bits above the current level (every thread keeps a copy)
};

// Block-wide state of the search (shared memory): what lies in front of the current prefix, the
// chosen bin, and the scratch of the scans.
struct RadixShared {
  unsigned count_before;
  unsigned long long mass_before;       // 2^-40 fixed point
  int bin;
  unsigned warp_cnt[kSampleThreads / 32];
  unsigned long long warp_mass[kSampleThreads / 32];
};

__device__ void radix_level(const SampleParams& p, long long row_off, float mx, float inv_t, float floor_w, int shift, int bits,
                            unsigned hi_mask, const RadixState& st, bool by_count, unsigned long long target, unsigned* hist_cnt,
                            unsigned long long* hist_mass, RadixShared* sh) {
  const int nb = 1 << bits;
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    hist_cnt[b] = 0u;
    hist_mass[b] = 0ull;
  }
  if (threadIdx.x == 0) sh->bin = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
    const float w = __expf((sample_logit(p, row_off, i) - mx) * inv_t);
    if (!(w >= floor_w)) continue;
    const unsigned u = __float_as_uint(w);
    if ((u & hi_mask) != st.prefix) continue;
    const int b = (u >> shift) & (nb - 1);
    atomicAdd(hist_cnt + b, 1u);
    atomicAdd(hist_mass + b, static_cast<unsigned long long>(w * kMassScale));
  }
  __syncthreads();
  // Walk from the top bin down, all bins at once: thread t owns bins 2t and 2t + 1; an inclusive scan
  // over the threads gives every bin what lies at and above it. By count the wanted bin is the
  // highest non-empty one at which the count from the top reaches the target; by mass the highest
  // non-empty one at which the mass from the top exceeds it.
  const int t = threadIdx.x, lane = t & 31, wid = t >> 5;
  const unsigned c0 = 2 * t < nb ? hist_cnt[2 * t] : 0u, c1 = 2 * t + 1 < nb ? hist_cnt[2 * t + 1] : 0u;
  const unsigned long long m0 = 2 * t < nb ? hist_mass[2 * t] : 0ull, m1 = 2 * t + 1 < nb ? hist_mass[2 * t + 1] : 0ull;
  unsigned pc = c0 + c1;
  unsigned long long pm = m0 + m1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned vc = __shfl_up_sync(0xffffffffu, pc, o);
    const unsigned long long vm = __shfl_up_sync(0xffffffffu, pm, o);
    if (lane >= o) { pc += vc; pm += vm; }
  }
  if (lane == 31) { sh->warp_cnt[wid] = pc; sh->warp_mass[wid] = pm; }
  __syncthreads();
  unsigned base_c = 0, total_c = 0;
  unsigned long long base_m = 0, total_m = 0;
#pragma unroll 4
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    const unsigned wc = sh->warp_cnt[w];
    const unsigned long long wm = sh->warp_mass[w];
    if (w < wid) { base_c += wc; base_m += wm; }
    total_c += wc;
    total_m += wm;
  }
  // inclusive prefix (ascending bins) up to and including this thread's pair -> what lies at and above
  const unsigned incl_c = base_c + pc;
  const unsigned long long incl_m = base_m + pm;
  const unsigned above_c = total_c - incl_c;                  // bins above 2t + 1
  const unsigned long long above_m = total_m - incl_m;
  const unsigned before_c = sh->count_before;
  const unsigned long long before_m = sh->mass_before;
  // bin 2t + 1, then bin 2t
  auto hit = [&](unsigned cnt, unsigned front_c, unsigned long long mass, unsigned long long front_m) {
    if (cnt == 0u) return false;
    return by_count ? (static_cast<unsigned long long>(before_c) + front_c + cnt >= target) : (before_m + front_m + mass > target);
  };
  int mine = -1;
  if (hit(c1, above_c, m1, above_m)) mine = 2 * t + 1;
  else if (hit(c0, above_c + c1, m0, above_m + m1)) mine = 2 * t;
  if (mine >= 0) atomicMax(&sh->bin, mine);
  __syncthreads();
  const int chosen = sh->bin;
  __syncthreads();
  if (chosen >= 0 && (chosen >> 1) == t) {
    // what lies in front of the chosen bin joins the running totals
    const bool upper = (chosen & 1) != 0;
    sh->count_before = before_c + above_c + (upper ? 0u : c1);
    sh->mass_before = before_m + above_m + (upper ? 0ull : m1);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const SampleParams p) {
  __shared__ float red[32];
  __shared__ unsigned hist_cnt[kSampleBins];
  __shared__ unsigned long long hist_mass[kSampleBins];
  __shared__ RadixShared rsh;
  __shared__ float s_scan[kSampleThreads / 32];
  __shared__ int s_pick;
  const int row = blockIdx.x;
  const long long row_off = static_cast<long long>(row) * p.ld;
  const float temp = p.temperature[row];

  // ---- maximum (and its first index: the answer of a greedy row)
  float mx = -INFINITY;
  int arg = 0x7fffffff;
  for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
    const float v = sample_logit(p, row_off, i);
    if (v > mx) { mx = v; arg = i; }
  }
  const float bmx = block_reduce_max(mx, red);
  if (temp <= 0.f || !(bmx > -INFINITY)) {
    // ties -> lowest index
    int cand = mx == bmx ? arg : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int s_arg[32];
    if ((threadIdx.x & 31) == 0) s_arg[threadIdx.x >> 5] = cand;
    __syncthreads();
    if (threadIdx.x == 0) {
      int best = 0x7fffffff;
      for (int w = 0; w < kSampleThreads / 32; ++w) best = min(best, s_arg[w]);
      p.out[row] = best == 0x7fffffff ? 0 : best;
    }
    return;
  }
  const float inv_t = 1.f / fmaxf(temp, 1e-6f);
  float tau = 0.f;     // keep w >= tau

  // ---- top-k: the k-th largest w
  const int k = p.top_k[row];
  float kept_mass = -1.f;
  if (k > 0 && k < p.vocab) {
    RadixState st{0u};
    if (threadIdx.x == 0) { rsh.count_before = 0u; rsh.mass_before = 0ull; }
    __syncthreads();
    unsigned hi_mask = 0u;
    int shift = 21;
    const int level_bits[3] = {11, 11, 10};
    bool open_end = false;
    for (int lv = 0; lv < 3; ++lv) {
      shift = lv == 0 ? 21 : lv == 1 ? 10 : 0;
      radix_level(p, row_off, bmx, inv_t, 0.f, shift, level_bits[lv], hi_mask, st, true, static_cast<unsigned long long>(k),
                  hist_cnt, hist_mass, &rsh);
      const int b = rsh.bin;
      if (b < 0) { open_end = true; break; }
      st.prefix |= static_cast<unsigned>(b) << shift;
      hi_mask |= static_cast<unsigned>((1 << level_bits[lv]) - 1) << shift;
    }
    if (!open_end) tau = __uint_as_float(st.prefix);
  }

  // ---- mass of the survivors so far
  {
    float local = 0.f;
    for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
      const float w = __expf((sample_logit(p, row_off, i) - bmx) * inv_t);
      if (w >= tau) local += w;
    }
    local = warp_sum(local);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < kSampleThreads / 32; ++w) t += red[w];
      red[0] = t;
    }
    __syncthreads();
    kept_mass = red[0];
    __syncthreads();
  }

  // ---- top-p over the survivors: the smallest w whose mass in front is <= p * kept_mass
  const float tp = p.top_p[row];
  if (tp > 0.f && tp < 1.f) {
    const unsigned long long limit = static_cast<unsigned long long>(static_cast<double>(tp) * static_cast<double>(kept_mass) *
                                                                   static_cast<double>(kMassScale));
    RadixState st{0u};
    __syncthreads();
    if (threadIdx.x == 0) { rsh.count_before = 0u; rsh.mass_before = 0ull; }
    __syncthreads();
    unsigned hi_mask = 0u;
    const int level_bits[3] = {11, 11, 10};
    bool open_end = false;
    for (int lv = 0; lv < 3; ++lv) {
      const int shift = lv == 0 ? 21 : lv == 1 ? 10 : 0;
      radix_level(p, row_off, bmx, inv_t, tau, shift, level_bits[lv], hi_mask, st, false, limit, hist_cnt, hist_mass, &rsh);
      const int b = rsh.bin;
      if (b < 0) { open_end = true; break; }
      st.prefix |= static_cast<unsigned>(b) << shift;
      hi_mask |= static_cast<unsigned>((1 << level_bits[lv]) - 1) << shift;
    }
    // the chosen value is the first one with MORE than the limit in front of its last copy: it is
    // still kept when the mass in front of its first copy is within the limit (the usual case of a
    // value that occurs once), so the threshold is that value itself
    if (!open_end) tau = fmaxf(tau, __uint_as_float(st.prefix));
  }

  // ---- min-p relative to the largest probability (w = 1)
  const float mp = p.min_p[row];
  if (mp > 0.f) tau = fmaxf(tau, fminf(mp, 1.f));

  // ---- draw: index-ordered prefix sums of the kept masses
  const int per = (p.vocab + kSampleThreads - 1) / kSampleThreads;
  const int i0 = threadIdx.x * per, i1 = min(p.vocab, i0 + per);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float w = __expf((sample_logit(p, row_off, i) - bmx) * inv_t);
    if (w >= tau) local += w;
  }
  // block-wide exclusive scan of `local`
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if ((threadIdx.x & 31) >= o) incl += t;
  }
  if ((threadIdx.x & 31) == 31) s_scan[threadIdx.x >> 5] = incl;
  if (threadIdx.x == 0) s_pick = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) {
      const float t = s_scan[w];
      s_scan[w] = run;
      run += t;
    }
    red[0] = run;
  }
  __syncthreads();
  const float total = red[0];
  const float excl = s_scan[threadIdx.x >> 5] + incl - local;
  const float u = sample_uniform(p.seed[row], p.counter[row]) * total;
  if (local > 0.f && u >= excl && u < excl + local) {
    // walk this thread's chunk
    float acc = excl;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float w = __expf((sample_logit(p, row_off, i) - bmx) * inv_t);
      if (w >= tau) {
        pick = i;
        acc += w;
        if (u < acc) break;
      }
    }
    if (pick >= 0) atomicMax(&s_pick, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pick = s_pick;
    if (pick < 0) {
      // rounding at the very end of the range: fall back to the most probable token
      pick = 0;
      float best = -INFINITY;
      for (int i = 0; i < p.vocab; ++i) {
        const float v = sample_logit(p, row_off, i);
        if (v > best) { best = v; pick = i; }
      }
    }
    p.out[row] = pick;
  }
}

}  // namespace b200

using namespace b200;

// logits [rows][ld] (fp32 when is_f32, else bf16); per-row device arrays as in SampleParams; out int32 [rows].
B200_API int b200_sample(const void* logits, int is_f32, long long ld, int rows, int vocab, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const unsigned long long* seed,
                         const unsigned long long* counter, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || vocab > (1 << 24)) return -2;
  SampleParams p{};
  p.logits = logits; p.is_f32 = is_f32; p.ld = ld; p.vocab = vocab;
  p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
  p.seed = seed; p.counter = counter; p.out = out;
  sample_kernel<<<rows, kSampleThreads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -300;
}
