// Paged-KV block manager and iteration-level (continuous-batching) scheduler.
//
// The reference specifies this subsystem only in prose
// (docs/new/RONN-Continuous-Batching-Branch-Prompt.md:84-302 request states,
// iteration loop, FCFS / priority / preemption policies;
// docs/new/RONN-KV-Cache-Compression-Branch-Prompt.md:125-195 16-token blocks,
// page table, ref-counted copy-on-write blocks).  This file is the native
// implementation: one object owns the block pool, the page tables, the
// request queues and the token history of every live sequence, and emits a
// flat "step plan" that the device kernels consume directly
// (token ids, positions, KV slot of every new token, block tables, lengths).
//
// Everything is exported as extern "C" for ctypes.  No device code here.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <list>
#include <unordered_map>
#include <vector>

namespace {

enum State : int32_t { WAITING = 0, PREFILL = 1, DECODING = 2, FINISHED = 3, PREEMPTED = 4, CANCELLED = 5 };
enum Policy : int32_t { FCFS = 0, PRIORITY = 1 };
// What happens to the KV blocks of a preempted sequence: dropped and recomputed on resume, copied to a host block pool
// and copied back on resume, or (AUTO) swapped when the sequence has at least `auto_min_tokens` tokens in the cache.
enum PreemptMode : int32_t { RECOMPUTE = 0, SWAP = 1, AUTO = 2 };

struct Config {
  int32_t block_size = 16;
  int32_t num_blocks = 0;
  int32_t max_num_seqs = 256;
  int32_t max_batch_tokens = 8192;
  int32_t prefill_chunk = 0;      // 0 = whole prompts only
  int32_t policy = FCFS;
  int32_t enable_prefix_cache = 0;
  int32_t max_blocks_per_seq = 64;
  int32_t preempt_mode = RECOMPUTE;
  int32_t num_cpu_blocks = 0;
  int32_t auto_min_tokens = 64;
};

struct Request {
  int64_t id = 0;
  int32_t priority = 2;           // 0 critical .. 3 low
  int64_t arrival = 0;
  int32_t state = WAITING;
  int32_t max_new_tokens = 0;
  int32_t prompt_len = 0;         // original prompt length
  int32_t num_computed = 0;       // tokens whose KV is in the cache
  int32_t num_generated = 0;
  int32_t preemptions = 0;
  std::vector<int32_t> tokens;    // prompt + generated
  std::vector<int32_t> blocks;    // logical block -> physical block
  std::vector<uint64_t> block_hashes;  // prefix hash of each full block (prefix cache)
  std::vector<int32_t> cpu_blocks;     // host copies of the first blocks while the request is swapped out
};

struct BlockMeta {
  int32_t ref = 0;
  uint64_t hash = 0;      // 0 = not in the prefix cache
  bool cached_free = false;
};

struct Stats {
  int64_t steps = 0, prefill_steps = 0, decode_steps = 0;
  int64_t preemptions = 0, prefix_hits_blocks = 0, finished = 0, cancelled = 0;
  int64_t scheduled_tokens = 0;
  int64_t swap_preemptions = 0, swapped_out_blocks = 0, swapped_in_blocks = 0;
};

struct SwapOp {
  int32_t src, dst;
};

struct PlanItem {
  int64_t req;
  int32_t start;     // first position computed this step
  int32_t count;     // number of tokens computed this step
  int32_t samples;   // 1 if the step yields a sampled token for this request
};

struct Scheduler {
  Config cfg;
  std::vector<BlockMeta> meta;
  std::vector<int32_t> free_list;                      // plain free blocks (LIFO)
  std::list<int32_t> cached_free;                      // LRU list of free blocks still holding a cached prefix
  std::unordered_map<int32_t, std::list<int32_t>::iterator> cached_pos;
  std::unordered_map<uint64_t, int32_t> hash_to_block;
  std::unordered_map<int64_t, Request> reqs;
  std::deque<int64_t> waiting;                          // WAITING and PREEMPTED, admission order
  std::vector<int64_t> running;                         // PREFILL and DECODING
  std::vector<PlanItem> plan;
  int32_t plan_kind = 0;                                // 0 none, 1 prefill, 2 decode
  int64_t arrival_counter = 0;
  Stats stats;
  // Block copies the engine has to run before this step's forward pass: first every swap_out (device block src ->
  // host block dst), then every swap_in (host block src -> device block dst).  Host blocks released by a swap-in
  // become reusable only at the next schedule() so that no swap-out of the same step overwrites them.
  std::vector<int32_t> cpu_free, cpu_pending_free;
  std::vector<SwapOp> swap_out, swap_in;

  explicit Scheduler(const Config& c) : cfg(c), meta(size_t(c.num_blocks)) {
    free_list.reserve(size_t(c.num_blocks));
    for (int32_t b = c.num_blocks - 1; b >= 0; --b) free_list.push_back(b);
  }

  int32_t num_free() const { return int32_t(free_list.size() + cached_free.size()); }

  void drop_cache_entry(int32_t b) {
    BlockMeta& m = meta[size_t(b)];
    if (m.hash) {
      auto it = hash_to_block.find(m.hash);
      if (it != hash_to_block.end() && it->second == b) hash_to_block.erase(it);
      m.hash = 0;
    }
  }

  int32_t alloc_block() {
    int32_t b;
    if (!free_list.empty()) {
      b = free_list.back();
      free_list.pop_back();
    } else if (!cached_free.empty()) {
      b = cached_free.front();                         // least recently freed cached block
      cached_free.pop_front();
      cached_pos.erase(b);
      meta[size_t(b)].cached_free = false;
      drop_cache_entry(b);
    } else {
      return -1;
    }
    meta[size_t(b)].ref = 1;
    return b;
  }

  void release_block(int32_t b) {
    BlockMeta& m = meta[size_t(b)];
    if (--m.ref > 0) return;
    m.ref = 0;
    if (m.hash && cfg.enable_prefix_cache) {
      m.cached_free = true;
      cached_free.push_back(b);
      cached_pos[b] = std::prev(cached_free.end());
    } else {
      drop_cache_entry(b);
      free_list.push_back(b);
    }
  }

  void free_request_blocks(Request& r) {
    for (int32_t b : r.blocks) release_block(b);
    r.blocks.clear();
    r.block_hashes.clear();
  }

  static uint64_t mix(uint64_t h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
    return h ? h : 1;
  }

  uint64_t hash_block(const Request& r, int32_t logical, uint64_t parent) const {
    uint64_t h = mix(0x243f6a8885a308d3ull, parent);
    const int32_t* t = r.tokens.data() + size_t(logical) * cfg.block_size;
    for (int32_t i = 0; i < cfg.block_size; ++i) h = mix(h, uint64_t(uint32_t(t[i])));
    return h;
  }

  // Reuse cached full blocks that match the request's token prefix.
  void match_prefix(Request& r) {
    if (!cfg.enable_prefix_cache || !r.blocks.empty()) return;
    int32_t total = int32_t(r.tokens.size());
    // at least one token must still be computed so the step yields logits
    int32_t max_full = (total - 1) / cfg.block_size;
    uint64_t parent = 0;
    for (int32_t lb = 0; lb < max_full; ++lb) {
      uint64_t h = hash_block(r, lb, parent);
      auto it = hash_to_block.find(h);
      if (it == hash_to_block.end()) break;
      int32_t b = it->second;
      BlockMeta& m = meta[size_t(b)];
      if (m.cached_free) {
        cached_free.erase(cached_pos[b]);
        cached_pos.erase(b);
        m.cached_free = false;
        m.ref = 1;
      } else {
        m.ref += 1;
      }
      r.blocks.push_back(b);
      r.block_hashes.push_back(h);
      parent = h;
      stats.prefix_hits_blocks += 1;
    }
    r.num_computed = int32_t(r.blocks.size()) * cfg.block_size;
  }

  // Publish the request's newly completed full blocks into the prefix cache.
  void publish_blocks(Request& r) {
    if (!cfg.enable_prefix_cache) return;
    int32_t full = r.num_computed / cfg.block_size;
    while (int32_t(r.block_hashes.size()) < full) {
      int32_t lb = int32_t(r.block_hashes.size());
      uint64_t parent = lb ? r.block_hashes[size_t(lb - 1)] : 0;
      uint64_t h = hash_block(r, lb, parent);
      r.block_hashes.push_back(h);
      int32_t b = r.blocks[size_t(lb)];
      if (hash_to_block.find(h) == hash_to_block.end() && meta[size_t(b)].hash == 0) {
        hash_to_block[h] = b;
        meta[size_t(b)].hash = h;
      }
    }
  }

  // Make sure the request owns blocks covering positions [0, upto).
  bool ensure_blocks(Request& r, int32_t upto) {
    int32_t need = (upto + cfg.block_size - 1) / cfg.block_size;
    if (need > cfg.max_blocks_per_seq) return false;
    int32_t have = int32_t(r.blocks.size());
    if (need - have > num_free()) return false;
    for (int32_t i = have; i < need; ++i) r.blocks.push_back(alloc_block());
    return true;
  }

  bool before(const Request& a, const Request& b) const {
    if (cfg.policy == PRIORITY && a.priority != b.priority) return a.priority < b.priority;
    return a.arrival < b.arrival;
  }

  void set_swap(int32_t mode, int32_t num_cpu_blocks, int32_t auto_min_tokens) {
    cfg.preempt_mode = mode;
    cfg.num_cpu_blocks = num_cpu_blocks;
    cfg.auto_min_tokens = auto_min_tokens;
    cpu_free.clear();
    cpu_pending_free.clear();
    for (int32_t b = num_cpu_blocks - 1; b >= 0; --b) cpu_free.push_back(b);
  }

  void release_cpu_blocks(Request& r, bool deferred) {
    for (int32_t c : r.cpu_blocks) (deferred ? cpu_pending_free : cpu_free).push_back(c);
    r.cpu_blocks.clear();
  }

  // Bring a swapped-out request's blocks back: device blocks for the tokens it has in its host copy.
  bool swap_in_request(Request& r) {
    const int32_t nb = int32_t(r.cpu_blocks.size());
    if (nb > num_free() - int32_t(running.size())) return false;     // same reserve as admission
    for (int32_t i = 0; i < nb; ++i) {
      const int32_t b = alloc_block();
      r.blocks.push_back(b);
      swap_in.push_back({r.cpu_blocks[size_t(i)], b});
    }
    stats.swapped_in_blocks += nb;
    release_cpu_blocks(r, true);
    return true;
  }

  void preempt(int64_t id, bool allow_swap = true) {
    Request& r = reqs[id];
    const int32_t nb = (r.num_computed + cfg.block_size - 1) / cfg.block_size;
    bool swap = allow_swap && nb > 0 && nb <= int32_t(r.blocks.size()) && nb <= int32_t(cpu_free.size()) &&
                (cfg.preempt_mode == SWAP || (cfg.preempt_mode == AUTO && r.num_computed >= cfg.auto_min_tokens));
    if (swap) {
      for (int32_t i = 0; i < nb; ++i) {
        const int32_t c = cpu_free.back();
        cpu_free.pop_back();
        r.cpu_blocks.push_back(c);
        swap_out.push_back({r.blocks[size_t(i)], c});
      }
      stats.swap_preemptions += 1;
      stats.swapped_out_blocks += nb;
    }
    free_request_blocks(r);
    if (!swap) r.num_computed = 0;
    r.state = PREEMPTED;
    r.preemptions += 1;
    stats.preemptions += 1;
    running.erase(std::find(running.begin(), running.end(), id));
    waiting.push_front(id);   // resumes before anything newly admitted
  }

  int64_t pick_victim(int64_t protect) {
    int64_t victim = -1;
    for (int64_t id : running) {
      if (id == protect) continue;
      if (victim < 0 || before(reqs[victim], reqs[id])) victim = id;   // the one scheduled last loses
    }
    return victim;
  }

  int32_t schedule() {
    plan.clear();
    plan_kind = 0;
    swap_out.clear();
    swap_in.clear();
    cpu_free.insert(cpu_free.end(), cpu_pending_free.begin(), cpu_pending_free.end());
    cpu_pending_free.clear();
    // ---- admission + prefill -------------------------------------------------
    if (cfg.policy == PRIORITY && waiting.size() > 1) {
      std::stable_sort(waiting.begin(), waiting.end(), [this](int64_t a, int64_t b) {
        const Request& ra = reqs[a];
        const Request& rb = reqs[b];
        if ((ra.state == PREEMPTED) != (rb.state == PREEMPTED) && ra.priority == rb.priority)
          return ra.state == PREEMPTED;
        return before(ra, rb);
      });
    }
    int32_t budget = cfg.max_batch_tokens;
    // requests already mid-prefill (chunked) continue first
    for (int64_t id : running) {
      Request& r = reqs[id];
      if (r.state != PREFILL) continue;
      int32_t total = int32_t(r.tokens.size());
      int32_t remaining = total - r.num_computed;
      int32_t take = std::min(remaining, budget);
      if (cfg.prefill_chunk > 0) take = std::min(take, cfg.prefill_chunk);
      if (take <= 0) continue;
      if (!ensure_blocks(r, r.num_computed + take)) continue;
      plan.push_back({id, r.num_computed, take, (r.num_computed + take == total) ? 1 : 0});
      budget -= take;
    }
    while (!waiting.empty() && int32_t(running.size()) < cfg.max_num_seqs && budget > 0) {
      int64_t id = waiting.front();
      Request& r = reqs[id];
      if (r.cpu_blocks.empty()) match_prefix(r);        // a swapped-out request keeps its own cache, not a shared prefix
      int32_t total = int32_t(r.tokens.size());
      int32_t remaining = total - r.num_computed;
      int32_t take = remaining;
      if (cfg.prefill_chunk > 0) take = std::min(take, cfg.prefill_chunk);
      if (take > budget) {
        if (cfg.prefill_chunk > 0) take = budget;       // chunking allowed: fill the budget
        else break;                                     // whole prompts only
      }
      // keep one block per running sequence in reserve so decode can make progress
      int32_t need = (r.num_computed + take + cfg.block_size - 1) / cfg.block_size - int32_t(r.blocks.size());
      if (need > num_free() - int32_t(running.size())) {
        if (r.blocks.size() && plan.empty()) { /* keep matched prefix blocks; retry next step */ }
        break;
      }
      if (!r.cpu_blocks.empty() && !swap_in_request(r)) break;      // a swapped-out request resumes with its cache
      if (!ensure_blocks(r, r.num_computed + take)) break;
      waiting.pop_front();
      r.state = PREFILL;
      running.push_back(id);
      plan.push_back({id, r.num_computed, take, (r.num_computed + take == total) ? 1 : 0});
      budget -= take;
    }
    if (!plan.empty()) {
      plan_kind = 1;
      stats.steps += 1;
      stats.prefill_steps += 1;
      for (auto& it : plan) stats.scheduled_tokens += it.count;
      return plan_kind;
    }
    // ---- decode ----------------------------------------------------------------
    std::vector<int64_t> order(running.begin(), running.end());
    std::stable_sort(order.begin(), order.end(), [this](int64_t a, int64_t b) { return before(reqs[a], reqs[b]); });
    for (int64_t id : order) {
      auto itr = reqs.find(id);
      if (itr == reqs.end() || itr->second.state != DECODING) continue;   // may have been preempted below
      Request& r = itr->second;
      int32_t total = int32_t(r.tokens.size());
      bool ok = ensure_blocks(r, total);
      while (!ok) {
        int64_t victim = pick_victim(id);
        if (victim < 0) break;
        // drop the victim from this step's plan if it was already placed
        for (size_t k = 0; k < plan.size(); ++k)
          if (plan[k].req == victim) { plan.erase(plan.begin() + long(k)); break; }
        preempt(victim);
        ok = ensure_blocks(r, total);
      }
      if (!ok) {   // cannot make progress even alone: give the blocks back and wait
        preempt(id);
        continue;
      }
      plan.push_back({id, total - 1, 1, 1});
    }
    if (!plan.empty()) {
      plan_kind = 2;
      stats.steps += 1;
      stats.decode_steps += 1;
      stats.scheduled_tokens += int64_t(plan.size());
    }
    return plan_kind;
  }
};

}  // namespace

extern "C" {

void* ronn_sched_new(int32_t block_size, int32_t num_blocks, int32_t max_num_seqs, int32_t max_batch_tokens,
                     int32_t prefill_chunk, int32_t policy, int32_t enable_prefix_cache,
                     int32_t max_blocks_per_seq) {
  if (block_size <= 0 || num_blocks <= 0 || max_num_seqs <= 0 || max_batch_tokens <= 0) return nullptr;
  Config c;
  c.block_size = block_size;
  c.num_blocks = num_blocks;
  c.max_num_seqs = max_num_seqs;
  c.max_batch_tokens = max_batch_tokens;
  c.prefill_chunk = prefill_chunk;
  c.policy = policy;
  c.enable_prefix_cache = enable_prefix_cache;
  c.max_blocks_per_seq = max_blocks_per_seq;
  return new Scheduler(c);
}
void ronn_sched_free(void* h) { delete static_cast<Scheduler*>(h); }

// returns 0 on success, -1 duplicate id, -2 prompt cannot ever fit
int32_t ronn_sched_add(void* h, int64_t id, const int32_t* prompt, int32_t prompt_len, int32_t max_new_tokens,
                       int32_t priority) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (s->reqs.count(id)) return -1;
  int64_t worst = int64_t(prompt_len) + max_new_tokens;
  int64_t cap = int64_t(s->cfg.max_blocks_per_seq) * s->cfg.block_size;
  if (prompt_len <= 0 || worst > cap || (worst + s->cfg.block_size - 1) / s->cfg.block_size > s->cfg.num_blocks)
    return -2;
  if (s->cfg.prefill_chunk == 0 && prompt_len + max_new_tokens > s->cfg.max_batch_tokens) return -2;
  Request r;
  r.id = id;
  r.priority = priority;
  r.arrival = s->arrival_counter++;
  r.max_new_tokens = max_new_tokens;
  r.prompt_len = prompt_len;
  r.tokens.assign(prompt, prompt + prompt_len);
  s->reqs.emplace(id, std::move(r));
  s->waiting.push_back(id);
  return 0;
}

int32_t ronn_sched_cancel(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  Request& r = it->second;
  if (r.state == FINISHED || r.state == CANCELLED) return 0;
  s->free_request_blocks(r);
  s->release_cpu_blocks(r, true);
  auto w = std::find(s->waiting.begin(), s->waiting.end(), id);
  if (w != s->waiting.end()) s->waiting.erase(w);
  auto ru = std::find(s->running.begin(), s->running.end(), id);
  if (ru != s->running.end()) s->running.erase(ru);
  r.state = CANCELLED;
  s->stats.cancelled += 1;
  return 0;
}

// mode: 0 recompute, 1 swap, 2 auto (swap when at least auto_min_tokens tokens are cached).  Call before any request
// is added; the host pool has num_cpu_blocks blocks of the same size as the device blocks.
int32_t ronn_sched_set_swap(void* h, int32_t mode, int32_t num_cpu_blocks, int32_t auto_min_tokens) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (mode < 0 || mode > 2 || num_cpu_blocks < 0 || !s->reqs.empty()) return -1;
  s->set_swap(mode, num_cpu_blocks, auto_min_tokens);
  return 0;
}
// Block copies of the current plan: counts[0] swap-outs, counts[1] swap-ins.
void ronn_sched_swap_counts(void* h, int32_t* counts) {
  Scheduler* s = static_cast<Scheduler*>(h);
  counts[0] = int32_t(s->swap_out.size());
  counts[1] = int32_t(s->swap_in.size());
}
// out_src/out_dst: device block -> host block; in_src/in_dst: host block -> device block.
void ronn_sched_get_swaps(void* h, int32_t* out_src, int32_t* out_dst, int32_t* in_src, int32_t* in_dst) {
  Scheduler* s = static_cast<Scheduler*>(h);
  for (size_t i = 0; i < s->swap_out.size(); ++i) { out_src[i] = s->swap_out[i].src; out_dst[i] = s->swap_out[i].dst; }
  for (size_t i = 0; i < s->swap_in.size(); ++i) { in_src[i] = s->swap_in[i].src; in_dst[i] = s->swap_in[i].dst; }
}
// out[0..3] = preemptions that swapped, blocks swapped out, blocks swapped in, free host blocks
void ronn_sched_swap_stats(void* h, int64_t* out) {
  Scheduler* s = static_cast<Scheduler*>(h);
  out[0] = s->stats.swap_preemptions;
  out[1] = s->stats.swapped_out_blocks;
  out[2] = s->stats.swapped_in_blocks;
  out[3] = int64_t(s->cpu_free.size() + s->cpu_pending_free.size());
}

int32_t ronn_sched_schedule(void* h) { return static_cast<Scheduler*>(h)->schedule(); }
int32_t ronn_sched_plan_size(void* h) { return int32_t(static_cast<Scheduler*>(h)->plan.size()); }
int32_t ronn_sched_plan_tokens(void* h) {
  int32_t n = 0;
  for (auto& it : static_cast<Scheduler*>(h)->plan) n += it.count;
  return n;
}

// Flatten the current plan into kernel-ready arrays.
//   req_ids[n_items], q_start[n_items+1] (token offsets), seq_lens[n_items] (context length after this step),
//   sample_index[n_items] (flat token index whose logits are sampled, or -1),
//   token_ids/positions/slot_mapping/token_item[n_tokens] (token_item = plan item of the token), block_tables[n_items * max_blocks] (-1 padded)
// Returns the number of tokens, or -1 when the block-table stride is too small.
int32_t ronn_sched_fill(void* h, int64_t* req_ids, int32_t* q_start, int32_t* seq_lens, int32_t* sample_index,
                        int32_t* token_ids, int32_t* positions, int32_t* slot_mapping, int32_t* token_item,
                        int32_t* block_tables, int32_t max_blocks) {
  Scheduler* s = static_cast<Scheduler*>(h);
  int32_t tok = 0;
  int32_t bs = s->cfg.block_size;
  for (size_t i = 0; i < s->plan.size(); ++i) {
    const PlanItem& it = s->plan[i];
    Request& r = s->reqs[it.req];
    if (int32_t(r.blocks.size()) > max_blocks) return -1;
    req_ids[i] = it.req;
    q_start[i] = tok;
    seq_lens[i] = it.start + it.count;
    sample_index[i] = it.samples ? tok + it.count - 1 : -1;
    for (int32_t k = 0; k < it.count; ++k) {
      int32_t pos = it.start + k;
      token_ids[tok] = r.tokens[size_t(pos)];
      positions[tok] = pos;
      slot_mapping[tok] = r.blocks[size_t(pos / bs)] * bs + pos % bs;
      token_item[tok] = int32_t(i);
      ++tok;
    }
    int32_t* bt = block_tables + size_t(i) * max_blocks;
    size_t nb = r.blocks.size();
    for (size_t b = 0; b < nb; ++b) bt[b] = r.blocks[b];
    for (int32_t b = int32_t(nb); b < max_blocks; ++b) bt[b] = -1;
  }
  q_start[s->plan.size()] = tok;
  return tok;
}

// Commit the step: sampled[i] is the token sampled for plan item i (ignored when that item yields none).
// finished_out[i] = 0 running, 1 eos, 2 max_tokens.  Returns number of requests that finished.
int32_t ronn_sched_commit(void* h, const int32_t* sampled, int32_t eos_token, int32_t* finished_out) {
  Scheduler* s = static_cast<Scheduler*>(h);
  int32_t nfin = 0;
  for (size_t i = 0; i < s->plan.size(); ++i) {
    const PlanItem& it = s->plan[i];
    Request& r = s->reqs[it.req];
    r.num_computed = it.start + it.count;
    s->publish_blocks(r);
    int32_t fin = 0;
    if (it.samples) {
      int32_t t = sampled[i];
      r.tokens.push_back(t);
      r.num_generated += 1;
      r.state = DECODING;
      if (eos_token >= 0 && t == eos_token) fin = 1;
      else if (r.num_generated >= r.max_new_tokens) fin = 2;
    }
    if (fin) {
      s->free_request_blocks(r);
      r.state = FINISHED;
      s->running.erase(std::find(s->running.begin(), s->running.end(), it.req));
      s->stats.finished += 1;
      ++nfin;
    }
    if (finished_out) finished_out[i] = fin;
  }
  s->plan.clear();
  s->plan_kind = 0;
  return nfin;
}

// Abort the current plan without committing (failed step): scheduled requests are re-queued for recompute.
void ronn_sched_abort_step(void* h) {
  Scheduler* s = static_cast<Scheduler*>(h);
  std::vector<int64_t> ids;
  for (auto& it : s->plan) ids.push_back(it.req);
  s->plan.clear();
  s->plan_kind = 0;
  for (int64_t id : ids) s->preempt(id, false);    // the failed step may have left their cache half written
}

int32_t ronn_sched_state(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : it->second.state;
}
int32_t ronn_sched_num_tokens(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : int32_t(it->second.tokens.size());
}
int32_t ronn_sched_get_tokens(void* h, int64_t id, int32_t* out, int32_t cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  int32_t n = std::min<int32_t>(cap, int32_t(it->second.tokens.size()));
  memcpy(out, it->second.tokens.data(), size_t(n) * 4);
  return n;
}
int32_t ronn_sched_prompt_len(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : it->second.prompt_len;
}
int32_t ronn_sched_get_blocks(void* h, int64_t id, int32_t* out, int32_t cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  int32_t n = std::min<int32_t>(cap, int32_t(it->second.blocks.size()));
  memcpy(out, it->second.blocks.data(), size_t(n) * 4);
  return n;
}
// Host-pool blocks holding the request's cache while it is swapped out (empty otherwise).
int32_t ronn_sched_get_cpu_blocks(void* h, int64_t id, int32_t* out, int32_t cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  int32_t n = std::min<int32_t>(cap, int32_t(it->second.cpu_blocks.size()));
  memcpy(out, it->second.cpu_blocks.data(), size_t(n) * 4);
  return n;
}
// Tokens of the request whose keys and values are in the cache (device or host copy).
int32_t ronn_sched_num_computed(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : it->second.num_computed;
}
int32_t ronn_sched_preemptions(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : it->second.preemptions;
}
void ronn_sched_forget(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it != s->reqs.end() && (it->second.state == FINISHED || it->second.state == CANCELLED)) s->reqs.erase(it);
}
int32_t ronn_sched_num_waiting(void* h) { return int32_t(static_cast<Scheduler*>(h)->waiting.size()); }
int32_t ronn_sched_num_running(void* h) { return int32_t(static_cast<Scheduler*>(h)->running.size()); }
int32_t ronn_sched_num_free_blocks(void* h) { return static_cast<Scheduler*>(h)->num_free(); }
int32_t ronn_sched_block_ref(void* h, int32_t b) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (b < 0 || b >= s->cfg.num_blocks) return -1;
  return s->meta[size_t(b)].ref;
}
// out[0..7] = steps, prefill_steps, decode_steps, preemptions, prefix_hit_blocks, finished, cancelled, scheduled_tokens
void ronn_sched_stats(void* h, int64_t* out) {
  const Stats& st = static_cast<Scheduler*>(h)->stats;
  out[0] = st.steps; out[1] = st.prefill_steps; out[2] = st.decode_steps; out[3] = st.preemptions;
  out[4] = st.prefix_hits_blocks; out[5] = st.finished; out[6] = st.cancelled; out[7] = st.scheduled_tokens;
}

}  // extern "C"
