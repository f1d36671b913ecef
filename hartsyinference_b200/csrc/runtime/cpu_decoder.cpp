// Host-side decoder for batch-1 generation with fp32 weights: the CPU counterpart of the GPU decode
// step for llama-family decoders (pre-norm RMSNorm, grouped-query attention with split-half rotary
// embedding, SwiGLU feed-forward, optional q/k/v bias, tied or separate output embedding).
//
// At batch 1 every linear is a matrix-vector product that streams its weights once, so the step is
// bound by host memory bandwidth; what this file adds over running the same ops one by one through
// a tensor library is (a) AVX-512 row kernels with four independent accumulators per row,
// (b) a persistent thread team (spin-then-yield hand-off, contiguous row ranges per thread so that
// a thread always streams the same slice of every matrix and its pages stay on the memory node it
// first touched), and (c) one call per token instead of a few hundred op dispatches.
//
// Reference counterpart: src/HartsyInference.Cpu/Kernels/MatMulKernels.cs:106 (LinearTransB),
// src/HartsyInference.Cpu/Threading/ComputeThreadPool.cs, CpuBackend.cs (the fp32 CPU backend).
// Weights stay owned by the caller (row-major fp32 [out][in]); nothing is copied.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

// ------------------------------------------------------------------------------------------
// thread team
// ------------------------------------------------------------------------------------------
class Team {
 public:
  explicit Team(int n) : n_(std::max(1, n)) {
    for (int t = 1; t < n_; ++t) workers_.emplace_back([this, t] { loop(t); });
  }
  ~Team() {
    stop_.store(true);
    gen_.fetch_add(1);
    for (auto& w : workers_) w.join();
  }
  int size() const { return n_; }
  // fn(thread index, thread count) runs on every member; returns when all are done
  void run(const std::function<void(int, int)>& fn) {
    fn_ = &fn;
    done_.store(0);
    gen_.fetch_add(1);
    fn(0, n_);
    int spins = 0;
    while (done_.load(std::memory_order_acquire) != n_ - 1) relax(spins);
  }

 private:
  static void relax(int& spins) {
    if (++spins < 2000) {
#if defined(__x86_64__)
      _mm_pause();
#endif
    } else {
      std::this_thread::yield();
    }
  }
  void loop(int t) {
    uint64_t seen = 0;
    while (true) {
      int spins = 0;
      while (gen_.load(std::memory_order_acquire) == seen) relax(spins);
      seen = gen_.load(std::memory_order_acquire);
      if (stop_.load()) return;
      (*fn_)(t, n_);
      done_.fetch_add(1, std::memory_order_release);
    }
  }
  int n_;
  std::vector<std::thread> workers_;
  std::atomic<uint64_t> gen_{0};
  std::atomic<int> done_{0};
  std::atomic<bool> stop_{false};
  const std::function<void(int, int)>* fn_ = nullptr;
};

// ------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------
float dot_scalar(const float* a, const float* b, int k) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int i = 0;
  for (; i + 4 <= k; i += 4) { s0 += a[i] * b[i]; s1 += a[i + 1] * b[i + 1]; s2 += a[i + 2] * b[i + 2]; s3 += a[i + 3] * b[i + 3]; }
  for (; i < k; ++i) s0 += a[i] * b[i];
  return (s0 + s1) + (s2 + s3);
}

#if defined(__x86_64__)
__attribute__((target("avx512f,fma"))) float dot_avx512(const float* a, const float* b, int k) {
  __m512 s0 = _mm512_setzero_ps(), s1 = s0, s2 = s0, s3 = s0;
  int i = 0;
  for (; i + 64 <= k; i += 64) {
    s0 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), s0);
    s1 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 16), _mm512_loadu_ps(b + i + 16), s1);
    s2 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 32), _mm512_loadu_ps(b + i + 32), s2);
    s3 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 48), _mm512_loadu_ps(b + i + 48), s3);
  }
  for (; i + 16 <= k; i += 16) s0 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), s0);
  float s = _mm512_reduce_add_ps(_mm512_add_ps(_mm512_add_ps(s0, s1), _mm512_add_ps(s2, s3)));
  for (; i < k; ++i) s += a[i] * b[i];
  return s;
}
// y[i] += w * x[i]
__attribute__((target("avx512f,fma"))) void axpy_avx512(float* y, const float* x, float w, int n) {
  const __m512 ww = _mm512_set1_ps(w);
  int i = 0;
  for (; i + 16 <= n; i += 16) _mm512_storeu_ps(y + i, _mm512_fmadd_ps(ww, _mm512_loadu_ps(x + i), _mm512_loadu_ps(y + i)));
  for (; i < n; ++i) y[i] += w * x[i];
}
#endif

bool have_avx512() {
#if defined(__x86_64__)
  static const bool ok = __builtin_cpu_supports("avx512f");
  return ok;
#else
  return false;
#endif
}

inline float dot(const float* a, const float* b, int k) {
#if defined(__x86_64__)
  if (have_avx512()) return dot_avx512(a, b, k);
#endif
  return dot_scalar(a, b, k);
}
inline void axpy(float* y, const float* x, float w, int n) {
#if defined(__x86_64__)
  if (have_avx512()) { axpy_avx512(y, x, w, n); return; }
#endif
  for (int i = 0; i < n; ++i) y[i] += w * x[i];
}

struct Layer {
  const float *in_norm = nullptr, *qkv_w = nullptr, *qkv_b = nullptr, *o_w = nullptr, *post_norm = nullptr,
              *gate_up_w = nullptr, *down_w = nullptr;
};

struct Decoder {
  int layers, hidden, heads, kv_heads, d, ffn, vocab, max_pos;
  float eps, theta;
  const float *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr;
  std::vector<Layer> L;
  std::vector<float> kcache, vcache;      // [layers][max_pos][kv_heads * d]
  std::vector<float> x, h, qkv, att, gu, act, logits, inv_freq, scores;
  Team team;
  Decoder(int layers_, int hidden_, int heads_, int kv_, int d_, int ffn_, int vocab_, int max_pos_, float eps_, float theta_,
          int threads)
      : layers(layers_), hidden(hidden_), heads(heads_), kv_heads(kv_), d(d_), ffn(ffn_), vocab(vocab_), max_pos(max_pos_),
        eps(eps_), theta(theta_), L(layers_), team(threads) {
    const size_t kv = static_cast<size_t>(layers) * max_pos * kv_heads * d;
    kcache.assign(kv, 0.f);
    vcache.assign(kv, 0.f);
    x.resize(hidden); h.resize(hidden);
    qkv.resize(static_cast<size_t>(heads + 2 * kv_heads) * d);
    att.resize(static_cast<size_t>(heads) * d);
    gu.resize(2 * static_cast<size_t>(ffn)); act.resize(ffn);
    logits.resize(vocab);
    inv_freq.resize(d / 2);
    for (int i = 0; i < d / 2; ++i) inv_freq[i] = std::pow(theta, -2.0f * i / d);
    scores.resize(static_cast<size_t>(heads) * max_pos);
  }

  void rmsnorm(const float* in, const float* w, float* out) const {
    float ss = dot(in, in, hidden);
    const float r = 1.0f / std::sqrt(ss / hidden + eps);
    for (int i = 0; i < hidden; ++i) out[i] = in[i] * r * w[i];
  }
  // y[rows] = W[rows][k] x (+ bias), rows split over the team in contiguous ranges
  void gemv(const float* W, const float* bias, const float* xin, float* y, int rows, int k) {
    team.run([&](int t, int n) {
      const int per = (rows + n - 1) / n, r0 = std::min(rows, t * per), r1 = std::min(rows, r0 + per);
      for (int r = r0; r < r1; ++r) y[r] = dot(W + static_cast<size_t>(r) * k, xin, k) + (bias ? bias[r] : 0.f);
    });
  }
  void rope(float* v, int pos) const {           // split-half pairs (i, i + d / 2)
    const int half = d / 2;
    for (int i = 0; i < half; ++i) {
      const float a = pos * inv_freq[i], c = std::cos(a), s = std::sin(a);
      const float x0 = v[i], x1 = v[i + half];
      v[i] = x0 * c - x1 * s;
      v[i + half] = x1 * c + x0 * s;
    }
  }

  int forward(int token, int pos, float* logits_out) {
    if (pos < 0 || pos >= max_pos || token < 0 || token >= vocab) return -1;
    std::memcpy(x.data(), embed + static_cast<size_t>(token) * hidden, sizeof(float) * hidden);
    const int qn = heads * d, kn = kv_heads * d, group = heads / kv_heads;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    for (int li = 0; li < layers; ++li) {
      const Layer& w = L[li];
      rmsnorm(x.data(), w.in_norm, h.data());
      gemv(w.qkv_w, w.qkv_b, h.data(), qkv.data(), qn + 2 * kn, hidden);
      float* kc = kcache.data() + (static_cast<size_t>(li) * max_pos + pos) * kn;
      float* vc = vcache.data() + (static_cast<size_t>(li) * max_pos + pos) * kn;
      for (int hh = 0; hh < heads; ++hh) rope(qkv.data() + hh * d, pos);
      for (int hh = 0; hh < kv_heads; ++hh) rope(qkv.data() + qn + hh * d, pos);
      std::memcpy(kc, qkv.data() + qn, sizeof(float) * kn);
      std::memcpy(vc, qkv.data() + qn + kn, sizeof(float) * kn);
      const float* kbase = kcache.data() + static_cast<size_t>(li) * max_pos * kn;
      const float* vbase = vcache.data() + static_cast<size_t>(li) * max_pos * kn;
      team.run([&](int t, int n) {
        for (int hh = t; hh < heads; hh += n) {
          const float* q = qkv.data() + hh * d;
          const int kvh = hh / group;
          float* sc = scores.data() + static_cast<size_t>(hh) * max_pos;
          float mx = -INFINITY;
          for (int p = 0; p <= pos; ++p) {
            sc[p] = dot(q, kbase + static_cast<size_t>(p) * kn + kvh * d, d) * scale;
            mx = std::max(mx, sc[p]);
          }
          float sum = 0.f;
          for (int p = 0; p <= pos; ++p) { sc[p] = std::exp(sc[p] - mx); sum += sc[p]; }
          float* o = att.data() + hh * d;
          std::fill(o, o + d, 0.f);
          const float inv = 1.0f / sum;
          for (int p = 0; p <= pos; ++p) axpy(o, vbase + static_cast<size_t>(p) * kn + kvh * d, sc[p] * inv, d);
        }
      });
      gemv(w.o_w, nullptr, att.data(), h.data(), hidden, qn);
      for (int i = 0; i < hidden; ++i) x[i] += h[i];
      rmsnorm(x.data(), w.post_norm, h.data());
      gemv(w.gate_up_w, nullptr, h.data(), gu.data(), 2 * ffn, hidden);
      for (int i = 0; i < ffn; ++i) {
        const float g = gu[i];
        act[i] = g / (1.0f + std::exp(-g)) * gu[ffn + i];
      }
      gemv(w.down_w, nullptr, act.data(), h.data(), hidden, ffn);
      for (int i = 0; i < hidden; ++i) x[i] += h[i];
    }
    rmsnorm(x.data(), final_norm, h.data());
    gemv(lm_head, nullptr, h.data(), logits.data(), vocab, hidden);
    if (logits_out) std::memcpy(logits_out, logits.data(), sizeof(float) * vocab);
    int best = 0;
    for (int i = 1; i < vocab; ++i)
      if (logits[i] > logits[best]) best = i;
    return best;
  }
};

}  // namespace

B200_API void* b200_cpu_decoder_create(int layers, int hidden, int heads, int kv_heads, int head_dim, int ffn, int vocab,
                                       int max_pos, float eps, float theta, int threads) {
  if (layers <= 0 || hidden <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim <= 0 || (head_dim & 1) ||
      ffn <= 0 || vocab <= 0 || max_pos <= 0)
    return nullptr;
  if (threads <= 0) threads = static_cast<int>(std::max(1u, std::thread::hardware_concurrency()));
  return new Decoder(layers, hidden, heads, kv_heads, head_dim, ffn, vocab, max_pos, eps, theta, threads);
}
B200_API void b200_cpu_decoder_free(void* h) { delete static_cast<Decoder*>(h); }
B200_API int b200_cpu_decoder_threads(void* h) { return static_cast<Decoder*>(h)->team.size(); }
B200_API int b200_cpu_decoder_simd(void) { return have_avx512() ? 512 : 0; }
B200_API void b200_cpu_decoder_set_globals(void* h, const float* embed, const float* lm_head, const float* final_norm) {
  auto* dcd = static_cast<Decoder*>(h);
  dcd->embed = embed; dcd->lm_head = lm_head; dcd->final_norm = final_norm;
}
B200_API int b200_cpu_decoder_set_layer(void* h, int i, const float* in_norm, const float* qkv_w, const float* qkv_b,
                                        const float* o_w, const float* post_norm, const float* gate_up_w,
                                        const float* down_w) {
  auto* dcd = static_cast<Decoder*>(h);
  if (i < 0 || i >= dcd->layers) return -1;
  dcd->L[static_cast<size_t>(i)] = Layer{in_norm, qkv_w, qkv_b, o_w, post_norm, gate_up_w, down_w};
  return 0;
}
// One token at position `pos` (positions must be fed in order from 0; the K/V of earlier positions
// are kept inside). Returns the argmax token, or -1 on a bad argument; `logits_out` (vocab floats)
// may be null.
B200_API int b200_cpu_decoder_forward(void* h, int token, int pos, float* logits_out) {
  return static_cast<Decoder*>(h)->forward(token, pos, logits_out);
}
