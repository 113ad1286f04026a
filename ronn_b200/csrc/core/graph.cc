// Graph algorithms of the IR on interned integer ids.
//
// Covers what the reference implements in crates/ronn-core/src/graph.rs
// (validate :117-151, Kahn topological sort :222-260, depth/statistics
// :347-389) plus the backward reachability that its dead-code pass intends
// (crates/ronn-graph/src/passes/dead_code.rs:15-35).  The Python IR interns
// tensor names to ints and keeps the strings/attributes; this file only sees
// node -> (input value ids, output value ids).
#include <cstdint>
#include <cstring>
#include <queue>
#include <unordered_map>
#include <vector>

namespace {

struct Graph {
  std::vector<std::vector<int32_t>> ins, outs;
};

// producer[value] = node index, or -1
void build_producer(const Graph& g, std::unordered_map<int32_t, int32_t>& producer, int32_t* dup_value) {
  *dup_value = -1;
  for (size_t n = 0; n < g.outs.size(); ++n)
    for (int32_t v : g.outs[n]) {
      if (producer.count(v) && *dup_value < 0) *dup_value = v;
      producer[v] = int32_t(n);
    }
}

}  // namespace

extern "C" {

void* ronn_graph_new() { return new Graph(); }
void ronn_graph_free(void* h) { delete static_cast<Graph*>(h); }

int32_t ronn_graph_add_node(void* h, const int32_t* ins, int32_t n_in, const int32_t* outs, int32_t n_out) {
  Graph* g = static_cast<Graph*>(h);
  g->ins.emplace_back(ins, ins + n_in);
  g->outs.emplace_back(outs, outs + n_out);
  return int32_t(g->ins.size()) - 1;
}

// Kahn topological order (stable: ready nodes are taken in index order).
// Returns the number of nodes placed; fewer than the node count means a cycle.
int32_t ronn_graph_toposort(void* h, int32_t* order) {
  Graph* g = static_cast<Graph*>(h);
  size_t n = g->ins.size();
  std::unordered_map<int32_t, int32_t> producer;
  int32_t dup;
  build_producer(*g, producer, &dup);
  std::vector<int32_t> indeg(n, 0);
  std::vector<std::vector<int32_t>> succ(n);
  for (size_t i = 0; i < n; ++i)
    for (int32_t v : g->ins[i]) {
      auto it = producer.find(v);
      if (it != producer.end()) {
        succ[size_t(it->second)].push_back(int32_t(i));
        indeg[i] += 1;
      }
    }
  std::priority_queue<int32_t, std::vector<int32_t>, std::greater<int32_t>> ready;
  for (size_t i = 0; i < n; ++i)
    if (indeg[i] == 0) ready.push(int32_t(i));
  int32_t placed = 0;
  while (!ready.empty()) {
    int32_t u = ready.top();
    ready.pop();
    order[placed++] = u;
    for (int32_t w : succ[size_t(u)])
      if (--indeg[size_t(w)] == 0) ready.push(w);
  }
  return placed;
}

// Validation.  Returns 0 ok, 1 duplicate producer of a value (detail = value id),
// 2 cycle (detail = a node on it), 3 graph output without producer/source (detail = value id),
// 4 node input with no producer that is neither a graph input nor an initializer (detail = value id).
int32_t ronn_graph_validate(void* h, const int32_t* sources, int32_t n_sources, const int32_t* outputs,
                            int32_t n_outputs, int32_t* detail) {
  Graph* g = static_cast<Graph*>(h);
  std::unordered_map<int32_t, int32_t> producer;
  int32_t dup;
  build_producer(*g, producer, &dup);
  if (dup >= 0) { *detail = dup; return 1; }
  std::vector<int32_t> order(g->ins.size());
  int32_t placed = ronn_graph_toposort(h, order.data());
  if (placed < int32_t(g->ins.size())) {
    std::vector<char> seen(g->ins.size(), 0);
    for (int32_t i = 0; i < placed; ++i) seen[size_t(order[size_t(i)])] = 1;
    for (size_t i = 0; i < seen.size(); ++i)
      if (!seen[i]) { *detail = int32_t(i); break; }
    return 2;
  }
  std::unordered_map<int32_t, char> src;
  for (int32_t i = 0; i < n_sources; ++i) src[sources[i]] = 1;
  for (int32_t i = 0; i < n_outputs; ++i)
    if (!producer.count(outputs[i]) && !src.count(outputs[i])) { *detail = outputs[i]; return 3; }
  for (auto& ins : g->ins)
    for (int32_t v : ins)
      if (v >= 0 && !producer.count(v) && !src.count(v)) { *detail = v; return 4; }
  return 0;
}

// live[n] = 1 when node n contributes to one of the requested outputs.
void ronn_graph_live(void* h, const int32_t* outputs, int32_t n_outputs, uint8_t* live) {
  Graph* g = static_cast<Graph*>(h);
  size_t n = g->ins.size();
  std::unordered_map<int32_t, int32_t> producer;
  int32_t dup;
  build_producer(*g, producer, &dup);
  memset(live, 0, n);
  std::vector<int32_t> stack;
  for (int32_t i = 0; i < n_outputs; ++i) {
    auto it = producer.find(outputs[i]);
    if (it != producer.end() && !live[it->second]) { live[it->second] = 1; stack.push_back(it->second); }
  }
  while (!stack.empty()) {
    int32_t u = stack.back();
    stack.pop_back();
    for (int32_t v : g->ins[size_t(u)]) {
      auto it = producer.find(v);
      if (it != producer.end() && !live[it->second]) { live[it->second] = 1; stack.push_back(it->second); }
    }
  }
}

// Longest path length (in nodes) through the DAG; -1 when cyclic.
int32_t ronn_graph_depth(void* h) {
  Graph* g = static_cast<Graph*>(h);
  size_t n = g->ins.size();
  std::vector<int32_t> order(n);
  if (ronn_graph_toposort(h, order.data()) < int32_t(n)) return -1;
  std::unordered_map<int32_t, int32_t> producer;
  int32_t dup;
  build_producer(*g, producer, &dup);
  std::vector<int32_t> d(n, 1);
  int32_t best = n ? 1 : 0;
  for (int32_t u : order) {
    for (int32_t v : g->ins[size_t(u)]) {
      auto it = producer.find(v);
      if (it != producer.end()) d[size_t(u)] = std::max(d[size_t(u)], d[size_t(it->second)] + 1);
    }
    best = std::max(best, d[size_t(u)]);
  }
  return best;
}

}  // extern "C"
