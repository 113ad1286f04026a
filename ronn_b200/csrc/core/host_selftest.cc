// Self-test of the host runtime for sanitizer builds (g++ -fsanitize=address,undefined): drives the block manager /
// scheduler, the pooled allocator and the graph algorithms through their C entry points with a deterministic
// pseudo-random workload, so that out-of-bounds accesses, leaks and undefined behaviour in the C++ code show up on a
// CPU box.  The reference only offers `-Z sanitizer=address` for its (disabled) multi-GPU test runner
// (crates/ronn-providers/scripts/run_multi_gpu_tests.sh:141-145).  Exit code 0 = all checks passed.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" {
void* ronn_sched_new(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t);
void ronn_sched_free(void*);
int32_t ronn_sched_add(void*, int64_t, const int32_t*, int32_t, int32_t, int32_t);
int32_t ronn_sched_cancel(void*, int64_t);
int32_t ronn_sched_schedule(void*);
int32_t ronn_sched_plan_size(void*);
int32_t ronn_sched_plan_tokens(void*);
int32_t ronn_sched_fill(void*, int64_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*, int32_t*,
                        int32_t);
int32_t ronn_sched_commit(void*, const int32_t*, int32_t, int32_t*);
int32_t ronn_sched_num_waiting(void*);
int32_t ronn_sched_num_running(void*);
int32_t ronn_sched_num_free_blocks(void*);
int32_t ronn_sched_set_swap(void*, int32_t, int32_t, int32_t);
void ronn_sched_swap_counts(void*, int32_t*);
void ronn_sched_get_swaps(void*, int32_t*, int32_t*, int32_t*, int32_t*);
void ronn_sched_swap_stats(void*, int64_t*);
void* ronn_pool_new(uint64_t, uint64_t, uint64_t, uint64_t);
void ronn_pool_free(void*);
void* ronn_pool_alloc(void*, uint64_t);
int32_t ronn_pool_release(void*, void*);
void* ronn_graph_new();
void ronn_graph_free(void*);
int32_t ronn_graph_add_node(void*, const int32_t*, int32_t, const int32_t*, int32_t);
int32_t ronn_graph_toposort(void*, int32_t*);
int32_t ronn_graph_depth(void*);
}

static uint32_t rng_state = 12345u;
static uint32_t rnd(uint32_t n) {
  rng_state = rng_state * 1664525u + 1013904223u;
  return (rng_state >> 8) % n;
}

#define CHECK(c)                                                         \
  do {                                                                   \
    if (!(c)) {                                                          \
      std::fprintf(stderr, "host_selftest: %s failed (line %d)\n", #c, __LINE__); \
      return 1;                                                          \
    }                                                                    \
  } while (0)

static int64_t total_swapped_blocks = 0;

static int test_scheduler(int policy, int prefix_cache, int chunk, int swap_mode) {
  // few blocks when swapping is exercised, so that decode steps preempt
  const int blocks = swap_mode ? 14 : 40, max_seqs = 6, max_tokens = 96, max_blocks = 10, cpu_blocks = 12;
  void* s = ronn_sched_new(16, blocks, max_seqs, max_tokens, chunk, policy, prefix_cache, max_blocks);
  CHECK(s != nullptr);
  if (swap_mode) CHECK(ronn_sched_set_swap(s, swap_mode, cpu_blocks, 24) == 0);
  std::vector<int32_t> so_src(size_t(blocks), 0), so_dst(size_t(blocks), 0), si_src(size_t(blocks), 0), si_dst(size_t(blocks), 0);
  std::vector<int> cpu_owner(size_t(cpu_blocks), 0);                       // 1 while a host block holds a swapped-out copy
  int added = 0;
  for (int64_t id = 0; id < 25; ++id) {
    const int plen = 1 + int(rnd(70)), newt = 1 + int(rnd(20));
    std::vector<int32_t> prompt(static_cast<size_t>(plen), 0);
    for (int i = 0; i < plen; ++i) prompt[size_t(i)] = int32_t(rnd(4));     // few distinct tokens: prefix hits happen
    if (ronn_sched_add(s, id, prompt.data(), plen, newt, int32_t(rnd(4))) == 0) ++added;
  }
  CHECK(ronn_sched_add(s, 3, nullptr, 0, 1, 0) != 0);                      // duplicate / empty rejected
  const size_t ns = size_t(max_seqs), nt = size_t(max_tokens);
  std::vector<int64_t> ids(ns, 0);
  std::vector<int32_t> q_start(ns + 1, 0), seq_lens(ns, 0), sample(ns, 0), fin(ns, 0);      // q_start: one past the last item
  std::vector<int32_t> tok(nt, 0), pos(nt, 0), slot(nt, 0), item(nt, 0);
  std::vector<int32_t> bt(ns * size_t(max_blocks), 0), sampled(ns, 1);
  int finished = 0, cancelled = 0;
  if (ronn_sched_cancel(s, 1) == 0) cancelled = 1;                        // still waiting: leaves the queue for good
  for (int step = 0; step < 5000; ++step) {
    const int kind = ronn_sched_schedule(s);
    int32_t swaps[2] = {0, 0};
    ronn_sched_swap_counts(s, swaps);
    CHECK(swaps[0] >= 0 && swaps[0] <= blocks && swaps[1] >= 0 && swaps[1] <= blocks);
    CHECK(swap_mode || (swaps[0] == 0 && swaps[1] == 0));
    ronn_sched_get_swaps(s, so_src.data(), so_dst.data(), si_src.data(), si_dst.data());
    for (int i = 0; i < swaps[0]; ++i) {                                     // device -> host: into a host block nobody holds
      CHECK(so_src[size_t(i)] >= 0 && so_src[size_t(i)] < blocks && so_dst[size_t(i)] >= 0 && so_dst[size_t(i)] < cpu_blocks);
      CHECK(cpu_owner[size_t(so_dst[size_t(i)])] == 0);
      cpu_owner[size_t(so_dst[size_t(i)])] = 1;
    }
    for (int i = 0; i < swaps[1]; ++i) {                                     // host -> device: from a block that was filled
      CHECK(si_dst[size_t(i)] >= 0 && si_dst[size_t(i)] < blocks && si_src[size_t(i)] >= 0 && si_src[size_t(i)] < cpu_blocks);
      CHECK(cpu_owner[size_t(si_src[size_t(i)])] == 1);
      cpu_owner[size_t(si_src[size_t(i)])] = 0;
    }
    if (kind == 0) {
      if (ronn_sched_num_waiting(s) == 0 && ronn_sched_num_running(s) == 0) break;
      CHECK(swap_mode != 0);                                               // an all-preempted step: the next one resumes
      continue;
    }
    const int n_items = ronn_sched_plan_size(s);
    CHECK(n_items > 0 && n_items <= max_seqs);
    CHECK(ronn_sched_plan_tokens(s) <= max_tokens);
    const int n_tok = ronn_sched_fill(s, ids.data(), q_start.data(), seq_lens.data(), sample.data(), tok.data(), pos.data(),
                                      slot.data(), item.data(), bt.data(), max_blocks);
    CHECK(n_tok > 0 && n_tok <= max_tokens);
    for (int i = 0; i < n_tok; ++i) CHECK(slot[size_t(i)] >= -1 && slot[size_t(i)] < blocks * 16);
    finished += ronn_sched_commit(s, sampled.data(), -1, fin.data());
    CHECK(ronn_sched_num_free_blocks(s) >= 0 && ronn_sched_num_free_blocks(s) <= blocks);
  }
  CHECK(finished + cancelled == added);
  CHECK(ronn_sched_num_waiting(s) == 0 && ronn_sched_num_running(s) == 0);
  if (!prefix_cache) CHECK(ronn_sched_num_free_blocks(s) == blocks);
  int64_t sw[4] = {0, 0, 0, 0};
  ronn_sched_swap_stats(s, sw);
  CHECK(sw[1] == sw[2] && sw[3] == (swap_mode ? cpu_blocks : 0));          // everything swapped out came back
  total_swapped_blocks += sw[1];
  ronn_sched_free(s);
  return 0;
}

static int test_pool() {
  void* p = ronn_pool_new(256, 64, 8, 1u << 20);
  CHECK(p != nullptr);
  std::vector<void*> live;
  for (int i = 0; i < 2000; ++i) {
    if (live.empty() || rnd(3) != 0) {
      const uint64_t n = 1 + rnd(5000);
      void* q = ronn_pool_alloc(p, n);
      CHECK(q != nullptr && (reinterpret_cast<uintptr_t>(q) & 63) == 0);
      std::memset(q, 0xab, size_t(n));
      live.push_back(q);
    } else {
      const size_t k = rnd(uint32_t(live.size()));
      CHECK(ronn_pool_release(p, live[k]) == 0);
      live[k] = live.back();
      live.pop_back();
    }
  }
  for (void* q : live) CHECK(ronn_pool_release(p, q) == 0);
  int dummy = 0;
  CHECK(ronn_pool_release(p, &dummy) != 0);                                // foreign pointer refused
  ronn_pool_free(p);
  return 0;
}

static int test_graph() {
  void* g = ronn_graph_new();
  const int n = 200;
  for (int i = 0; i < n; ++i) {                                            // node i consumes value i (and an older one), produces i + 1
    int32_t ins[2] = {i, i > 3 ? int32_t(rnd(uint32_t(i))) : 0};
    int32_t outs[1] = {i + 1};
    CHECK(ronn_graph_add_node(g, ins, 2, outs, 1) == i);
  }
  std::vector<int32_t> order(static_cast<size_t>(n), 0);
  CHECK(ronn_graph_toposort(g, order.data()) == n);
  for (int i = 0; i < n; ++i) CHECK(order[size_t(i)] == i);
  CHECK(ronn_graph_depth(g) == n);
  ronn_graph_free(g);
  return 0;
}

int main() {
  for (int policy = 0; policy < 2; ++policy)
    for (int prefix = 0; prefix < 2; ++prefix)
      for (int chunk = 0; chunk <= 32; chunk += 32)
        for (int swap = 0; swap < 3; ++swap)
          if (test_scheduler(policy, prefix, chunk, swap)) return 1;
  CHECK(total_swapped_blocks > 0);                                          // the tight configurations did swap
  if (test_pool()) return 1;
  if (test_graph()) return 1;
  std::printf("host_selftest: ok\n");
  return 0;
}
