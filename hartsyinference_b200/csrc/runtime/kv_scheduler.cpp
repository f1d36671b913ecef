// Paged-KV block allocator and continuous-batching scheduler core (host side, no CUDA).
//
// The allocator hands out fixed-size KV pages from a free list, keeps one block table per
// sequence and reference-counts pages so that a prompt prefix can be shared between sequences.
// The scheduler decides, once per engine step, which waiting requests are admitted (prefill, in
// chunks bounded by a token budget), which running sequences decode, and which running sequence is
// pre-empted (pages released, request re-queued for recompute) when the pool runs dry.
//
// Behavioural model: the reference's PagedKvPool / PagedKvCache (free-list stack of pages,
// KvPoolExhaustedException; src/HartsyInference.LLM/Transformer/PagedKvPool.cs, PagedKvCache.cs:53,
// 193) and DynamicBatchScheduler (SubmitAsync:153, RunLoopAsync:162-268, AdmitAndPrefill:311-383,
// RunDecodeRound:460-483; src/HartsyInference.LLM/Generation/DynamicBatchScheduler.cs). Differences:
// exhaustion queues or pre-empts instead of failing the request, prefill is chunked and batched,
// and the block tables are consumed directly by the attention kernels (no page gather).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

struct Seq {
  std::vector<int32_t> blocks;
  int64_t tokens = 0;   // tokens whose KV is stored
};

struct KvAllocator {
  int32_t num_blocks;
  int32_t block_size;
  std::vector<int32_t> free_list;     // stack: back() is handed out next
  std::vector<int32_t> refcount;
  std::unordered_map<int64_t, Seq> seqs;
  int32_t fail_after = -1;            // fault injection: the N-th next allocation fails
  std::mutex mu;

  KvAllocator(int32_t n, int32_t bs) : num_blocks(n), block_size(bs), refcount(n, 0) {
    free_list.reserve(n);
    for (int32_t i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
  int32_t blocks_needed(const Seq& s, int64_t new_tokens) const {
    const int64_t total = s.tokens + new_tokens;
    const int64_t need = (total + block_size - 1) / block_size;
    return static_cast<int32_t>(std::max<int64_t>(0, need - static_cast<int64_t>(s.blocks.size())));
  }
  bool take(Seq& s, int32_t n) {
    if (fail_after >= 0) {
      if (fail_after < n) { fail_after = -1; return false; }
      fail_after -= n;
    }
    if (static_cast<int32_t>(free_list.size()) < n) return false;
    for (int32_t i = 0; i < n; ++i) {
      const int32_t b = free_list.back();
      free_list.pop_back();
      refcount[b] = 1;
      s.blocks.push_back(b);
    }
    return true;
  }
  void release(Seq& s) {
    for (int32_t b : s.blocks)
      if (--refcount[b] == 0) free_list.push_back(b);
    s.blocks.clear();
    s.tokens = 0;
  }
};

enum ReqState : int32_t { kWaiting = 0, kPrefill = 1, kDecode = 2, kFinished = 3 };

struct Request {
  int64_t id;
  int32_t prompt_len;
  int32_t max_new_tokens;
  int32_t computed = 0;      // prompt tokens whose KV exists
  int32_t generated = 0;
  int32_t state = kWaiting;
  int32_t preemptions = 0;
  int64_t arrival;
};

struct Scheduler {
  KvAllocator* alloc;
  int32_t max_batch;
  int32_t prefill_token_budget;
  int32_t max_prefill_seqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;     // admission order
  std::unordered_map<int64_t, Request> reqs;
  int64_t clock = 0;
  int64_t total_preemptions = 0;
  std::mutex mu;
};

}  // namespace

// ---------------------------------------------------------------------------------- allocator
B200_API void* b200_kv_create(int32_t num_blocks, int32_t block_size) {
  if (num_blocks <= 0 || block_size <= 0) return nullptr;
  return new KvAllocator(num_blocks, block_size);
}
B200_API void b200_kv_destroy(void* h) { delete static_cast<KvAllocator*>(h); }
B200_API int32_t b200_kv_num_free(void* h) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  return static_cast<int32_t>(a->free_list.size());
}
B200_API int32_t b200_kv_num_blocks(void* h) { return static_cast<KvAllocator*>(h)->num_blocks; }
B200_API int32_t b200_kv_block_size(void* h) { return static_cast<KvAllocator*>(h)->block_size; }

// Reserve room for `new_tokens` more tokens of sequence `seq` (created on first use).
// Returns the number of tokens now stored, or -1 when the pool cannot satisfy the request
// (nothing is changed in that case).
B200_API int64_t b200_kv_append(void* h, int64_t seq, int32_t new_tokens) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  Seq& s = a->seqs[seq];
  const int32_t need = a->blocks_needed(s, new_tokens);
  if (need > 0 && !a->take(s, need)) return -1;
  s.tokens += new_tokens;
  return s.tokens;
}
B200_API int32_t b200_kv_can_append(void* h, int64_t seq, int32_t new_tokens) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(seq);
  Seq empty;
  const Seq& s = it == a->seqs.end() ? empty : it->second;
  return a->blocks_needed(s, new_tokens) <= static_cast<int32_t>(a->free_list.size()) ? 1 : 0;
}
// Drop the last tokens of a sequence (speculative-decode rollback); frees whole pages that empty.
B200_API int64_t b200_kv_truncate(void* h, int64_t seq, int64_t new_len) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end()) return -1;
  Seq& s = it->second;
  if (new_len < 0 || new_len > s.tokens) return -1;
  const size_t keep = static_cast<size_t>((new_len + a->block_size - 1) / a->block_size);
  while (s.blocks.size() > keep) {
    const int32_t b = s.blocks.back();
    s.blocks.pop_back();
    if (--a->refcount[b] == 0) a->free_list.push_back(b);
  }
  s.tokens = new_len;
  return new_len;
}
B200_API void b200_kv_free_seq(void* h, int64_t seq) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end()) return;
  a->release(it->second);
  a->seqs.erase(it);
}
// Share the first `tokens` (rounded down to whole pages) of `src` with a new sequence `dst`.
B200_API int64_t b200_kv_fork_prefix(void* h, int64_t src, int64_t dst, int64_t tokens) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(src);
  if (it == a->seqs.end() || a->seqs.count(dst)) return -1;
  const int64_t pages = std::min<int64_t>(tokens, it->second.tokens) / a->block_size;
  Seq d;
  for (int64_t i = 0; i < pages; ++i) {
    const int32_t b = it->second.blocks[static_cast<size_t>(i)];
    ++a->refcount[b];
    d.blocks.push_back(b);
  }
  d.tokens = pages * a->block_size;
  a->seqs[dst] = d;
  return d.tokens;
}
B200_API int64_t b200_kv_seq_len(void* h, int64_t seq) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(seq);
  return it == a->seqs.end() ? -1 : it->second.tokens;
}
// Copies the block table of `seq` into out[0..cap) (padded with -1). Returns the block count.
B200_API int32_t b200_kv_block_table(void* h, int64_t seq, int32_t* out, int32_t cap) {
  auto* a = static_cast<KvAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end()) return -1;
  const auto& b = it->second.blocks;
  const int32_t n = static_cast<int32_t>(b.size());
  for (int32_t i = 0; i < cap; ++i) out[i] = i < n ? b[static_cast<size_t>(i)] : -1;
  return n;
}
// Fault injection for tests: make the allocation that crosses `after_blocks` more blocks fail once.
B200_API void b200_kv_inject_failure(void* h, int32_t after_blocks) {
  static_cast<KvAllocator*>(h)->fail_after = after_blocks;
}

// ---------------------------------------------------------------------------------- scheduler
B200_API void* b200_sched_create(void* kv, int32_t max_batch, int32_t prefill_token_budget,
                                 int32_t max_prefill_seqs) {
  if (!kv) return nullptr;
  auto* s = new Scheduler();
  s->alloc = static_cast<KvAllocator*>(kv);
  s->max_batch = max_batch;
  s->prefill_token_budget = prefill_token_budget;
  s->max_prefill_seqs = max_prefill_seqs > 0 ? max_prefill_seqs : max_batch;
  return s;
}
B200_API void b200_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

B200_API int32_t b200_sched_submit(void* h, int64_t id, int32_t prompt_len, int32_t max_new_tokens) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (s->reqs.count(id) || prompt_len <= 0) return -1;
  // a request that can never fit is rejected up front
  const int64_t pages = (static_cast<int64_t>(prompt_len) + max_new_tokens + s->alloc->block_size - 1) /
                        s->alloc->block_size;
  if (pages > s->alloc->num_blocks) return -2;
  Request r{};
  r.id = id;
  r.prompt_len = prompt_len;
  r.max_new_tokens = max_new_tokens;
  r.arrival = s->clock++;
  s->reqs[id] = r;
  s->waiting.push_back(id);
  return 0;
}

// One scheduling decision. Outputs (caller-allocated, capacity `cap` entries each):
//   prefill_ids / prefill_start / prefill_count : requests that run a prompt chunk this step
//   decode_ids                                  : requests that decode one token this step
//   preempted_ids                               : requests whose pages were taken away
// Pages for every scheduled token are already reserved when this returns.
// counts[0..3) receives the three list lengths.
B200_API int32_t b200_sched_step(void* h, int64_t* prefill_ids, int32_t* prefill_start,
                                 int32_t* prefill_count, int64_t* decode_ids,
                                 int64_t* preempted_ids, int32_t cap, int32_t* counts) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  int32_t np = 0, nd = 0, nx = 0;
  KvAllocator* a = s->alloc;

  // 1. decode: every running request in decode state needs one more slot. When the pool is dry,
  //    pre-empt the most recently admitted running request (its pages go back, it re-queues at
  //    the front and recomputes its prompt + generated tokens later).
  std::vector<int64_t> decoders;
  for (int64_t id : s->running)
    if (s->reqs[id].state == kDecode) decoders.push_back(id);
  size_t i = 0;
  while (i < decoders.size()) {
    const int64_t id = decoders[i];
    if (b200_kv_append(a, id, 1) >= 0) { ++i; continue; }
    // victim = last running request that is not `id` if possible
    int64_t victim = -1;
    for (auto it = s->running.rbegin(); it != s->running.rend(); ++it)
      if (*it != id) { victim = *it; break; }
    if (victim < 0) victim = id;
    Request& v = s->reqs[victim];
    b200_kv_free_seq(a, victim);
    v.state = kWaiting;
    v.computed = 0;
    ++v.preemptions;
    ++s->total_preemptions;
    s->running.erase(std::find(s->running.begin(), s->running.end(), victim));
    s->waiting.push_front(victim);
    if (nx < cap) preempted_ids[nx++] = victim;
    auto dit = std::find(decoders.begin(), decoders.end(), victim);
    if (dit != decoders.end()) {
      const size_t pos = static_cast<size_t>(dit - decoders.begin());
      if (pos < i) {
        // it already reserved its slot this step; freeing the sequence returned it
        --i;
      }
      decoders.erase(dit);
    }
    if (victim == id) continue;
  }
  for (int64_t id : decoders)
    if (nd < cap) decode_ids[nd++] = id;

  // 2. prefill: continue partially prefilled requests first, then admit from the queue, within the
  //    token budget and the batch limit.
  int32_t budget = s->prefill_token_budget;
  auto schedule_chunk = [&](Request& r) -> bool {
    // after a pre-emption the tokens generated so far are part of what must be recomputed
    const int32_t target = r.prompt_len + r.generated - (r.generated > 0 ? 1 : 0);
    const int32_t remaining = target - r.computed;
    if (remaining <= 0) return false;
    int32_t chunk = std::min(remaining, budget);
    if (chunk <= 0) return false;
    if (b200_kv_append(a, r.id, chunk) < 0) return false;
    if (np < cap) {
      prefill_ids[np] = r.id;
      prefill_start[np] = r.computed;
      prefill_count[np] = chunk;
      ++np;
    }
    r.computed += chunk;
    budget -= chunk;
    return true;
  };
  for (int64_t id : s->running) {
    Request& r = s->reqs[id];
    if (r.state == kPrefill && budget > 0 && np < s->max_prefill_seqs) schedule_chunk(r);
  }
  while (!s->waiting.empty() && budget > 0 && np < s->max_prefill_seqs &&
         static_cast<int32_t>(s->running.size()) < s->max_batch) {
    const int64_t id = s->waiting.front();
    Request& r = s->reqs[id];
    // admission needs room for at least the first chunk; keep one page per running decoder in
    // reserve so that an admission does not immediately force a pre-emption
    const int32_t target = r.prompt_len + r.generated - (r.generated > 0 ? 1 : 0);
    const int32_t chunk = std::min(target, budget);
    const int32_t need = (chunk + a->block_size - 1) / a->block_size;
    const int32_t reserve = static_cast<int32_t>(decoders.size());
    if (static_cast<int32_t>(a->free_list.size()) < need + reserve) break;
    r.state = kPrefill;
    if (!schedule_chunk(r)) { r.state = kWaiting; break; }
    s->waiting.pop_front();
    s->running.push_back(id);
  }
  counts[0] = np;
  counts[1] = nd;
  counts[2] = nx;
  return np + nd;
}

// Report the outcome of the step for one request: `prefill_done` (its prompt is now fully
// computed and the first token was sampled) and/or `finished` (EOS / length / cancelled / error).
B200_API int32_t b200_sched_update(void* h, int64_t id, int32_t new_tokens, int32_t finished) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  Request& r = it->second;
  r.generated += new_tokens;
  if (r.state == kPrefill) {
    const int32_t target = r.prompt_len + (r.generated - new_tokens) - ((r.generated - new_tokens) > 0 ? 1 : 0);
    if (r.computed >= target) r.state = kDecode;
  }
  if (finished || r.generated >= r.max_new_tokens) {
    r.state = kFinished;
    b200_kv_free_seq(s->alloc, id);
    auto rit = std::find(s->running.begin(), s->running.end(), id);
    if (rit != s->running.end()) s->running.erase(rit);
    auto wit = std::find(s->waiting.begin(), s->waiting.end(), id);
    if (wit != s->waiting.end()) s->waiting.erase(wit);
    s->reqs.erase(it);
    return 1;
  }
  return 0;
}

B200_API int32_t b200_sched_abort(void* h, int64_t id) { return b200_sched_update(h, id, 0, 1); }

// stats[0] waiting, [1] running, [2] free blocks, [3] total pre-emptions
B200_API void b200_sched_stats(void* h, int64_t* stats) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  stats[0] = static_cast<int64_t>(s->waiting.size());
  stats[1] = static_cast<int64_t>(s->running.size());
  stats[2] = b200_kv_num_free(s->alloc);
  stats[3] = s->total_preemptions;
}
B200_API int32_t b200_sched_request_state(void* h, int64_t id, int32_t* computed, int32_t* generated,
                                          int32_t* preemptions) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  if (computed) *computed = it->second.computed;
  if (generated) *generated = it->second.generated;
  if (preemptions) *preemptions = it->second.preemptions;
  return it->second.state;
}
