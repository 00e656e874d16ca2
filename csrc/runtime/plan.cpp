// Planner for dynamically built op graphs.
//
// The reference's DynamicExecutionContext keeps a node cache, an execution order and a "memory plan" that
// only sums output sizes (src/execution/dynamic.rs:190-420), and its JIT graph optimiser is a stub
// (src/serialization/jit.rs:560-635).  Here the plan is computed for real: nodes are appended in
// definition order (inputs must already exist, so the graph is acyclic by construction), levels give the
// waves that may run concurrently on separate CUDA streams, lifetimes (definition .. last use in
// topological order) drive a greedy-by-size offset assignment so that buffers with disjoint lifetimes share
// arena space, and chains of single-consumer elementwise ops are reported for fusion.
#include "plan.h"

#include <algorithm>
#include <set>
#include <stdexcept>

namespace rt {

namespace {
const std::set<std::string>& elementwise_ops() {
  static const std::set<std::string> s = {"add", "sub", "mul", "div", "relu", "sigmoid", "tanh", "gelu", "silu", "exp",
                                         "log", "neg", "abs", "sqrt", "dropout", "scale", "leaky_relu", "elu"};
  return s;
}
}  // namespace

int ExecutionPlan::add_node(const std::string& op, const std::vector<int>& inputs, uint64_t out_bytes) {
  const int id = (int)nodes_.size();
  for (int i : inputs)
    if (i < 0 || i >= id) throw std::invalid_argument("plan: input " + std::to_string(i) + " does not exist yet");
  nodes_.push_back(PlanNode{id, op, inputs, out_bytes});
  return id;
}

void ExecutionPlan::mark_output(int id) {
  if (id < 0 || id >= (int)nodes_.size()) throw std::out_of_range("plan: no such node");
  outputs_.push_back(id);
}

const PlanNode& ExecutionPlan::node(int id) const {
  if (id < 0 || id >= (int)nodes_.size()) throw std::out_of_range("plan: no such node");
  return nodes_[id];
}

std::vector<int> ExecutionPlan::topo_order() const {
  // Kahn's algorithm with the smallest ready id first (deterministic, keeps definition order when legal).
  const int n = (int)nodes_.size();
  std::vector<int> indeg(n, 0);
  std::vector<std::vector<int>> users(n);
  for (const auto& nd : nodes_)
    for (int i : nd.inputs) {
      ++indeg[nd.id];
      users[i].push_back(nd.id);
    }
  std::set<int> ready;
  for (int i = 0; i < n; ++i)
    if (!indeg[i]) ready.insert(i);
  std::vector<int> order;
  order.reserve(n);
  while (!ready.empty()) {
    const int v = *ready.begin();
    ready.erase(ready.begin());
    order.push_back(v);
    for (int u : users[v])
      if (--indeg[u] == 0) ready.insert(u);
  }
  return order;
}

std::vector<std::vector<int>> ExecutionPlan::levels() const {
  const int n = (int)nodes_.size();
  std::vector<int> depth(n, 0);
  int maxd = -1;
  for (const auto& nd : nodes_) {
    int d = 0;
    for (int i : nd.inputs) d = std::max(d, depth[i] + 1);
    depth[nd.id] = d;
    maxd = std::max(maxd, d);
  }
  std::vector<std::vector<int>> out(maxd + 1);
  for (int i = 0; i < n; ++i) out[depth[i]].push_back(i);
  return out;
}

std::vector<int> ExecutionPlan::eliminate_dead() const {
  const int n = (int)nodes_.size();
  std::vector<char> live(n, 0);
  std::vector<int> stack(outputs_.begin(), outputs_.end());
  if (outputs_.empty() && n) stack.push_back(n - 1);  // no explicit outputs: the last node is the result
  while (!stack.empty()) {
    const int v = stack.back();
    stack.pop_back();
    if (live[v]) continue;
    live[v] = 1;
    for (int i : nodes_[v].inputs) stack.push_back(i);
  }
  std::vector<int> dead;
  for (int i = 0; i < n; ++i)
    if (!live[i]) dead.push_back(i);
  return dead;
}

std::pair<std::vector<int64_t>, std::pair<uint64_t, uint64_t>> ExecutionPlan::memory_plan(uint64_t alignment) const {
  if (alignment == 0) alignment = 1;
  const int n = (int)nodes_.size();
  const std::vector<int> order = topo_order();
  std::vector<int> pos(n, 0);
  for (int i = 0; i < (int)order.size(); ++i) pos[order[i]] = i;
  std::vector<int> last(n);
  for (int i = 0; i < n; ++i) last[i] = pos[i];
  for (const auto& nd : nodes_)
    for (int i : nd.inputs) last[i] = std::max(last[i], pos[nd.id]);
  for (int o : outputs_) last[o] = n;  // outputs outlive the plan
  if (outputs_.empty() && n) last[n - 1] = n;

  struct Buf { int id; uint64_t size; int begin, end; };
  std::vector<Buf> bufs;
  uint64_t naive = 0;
  for (int i = 0; i < n; ++i) {
    if (!nodes_[i].out_bytes) continue;
    const uint64_t sz = (nodes_[i].out_bytes + alignment - 1) / alignment * alignment;
    bufs.push_back({i, sz, pos[i], last[i]});
    naive += sz;
  }
  std::sort(bufs.begin(), bufs.end(), [](const Buf& a, const Buf& b) { return a.size != b.size ? a.size > b.size : a.id < b.id; });
  std::vector<int64_t> offsets(n, -1);
  struct Placed { uint64_t off, size; int begin, end; };
  std::vector<Placed> placed;
  uint64_t total = 0;
  for (const Buf& b : bufs) {
    // gaps between already placed buffers whose lifetime overlaps this one, lowest offset first
    std::vector<std::pair<uint64_t, uint64_t>> busy;
    for (const Placed& p : placed)
      if (!(p.end < b.begin || b.end < p.begin)) busy.push_back({p.off, p.off + p.size});
    std::sort(busy.begin(), busy.end());
    uint64_t off = 0;
    for (const auto& iv : busy) {
      if (off + b.size <= iv.first) break;
      off = std::max(off, iv.second);
    }
    offsets[b.id] = (int64_t)off;
    placed.push_back({off, b.size, b.begin, b.end});
    total = std::max(total, off + b.size);
  }
  return {offsets, {total, naive}};
}

std::vector<std::vector<int>> ExecutionPlan::fusible_chains() const {
  const int n = (int)nodes_.size();
  std::vector<int> n_users(n, 0), only_user(n, -1);
  for (const auto& nd : nodes_)
    for (int i : nd.inputs) {
      ++n_users[i];
      only_user[i] = nd.id;
    }
  auto is_ew = [&](int i) { return elementwise_ops().count(nodes_[i].op) > 0; };
  std::vector<char> used(n, 0);
  std::vector<std::vector<int>> chains;
  for (int i = 0; i < n; ++i) {
    if (used[i] || !is_ew(i)) continue;
    // start of a chain: no elementwise single-consumer producer feeding it as first input
    bool has_pred = false;
    for (int p : nodes_[i].inputs)
      if (is_ew(p) && n_users[p] == 1 && !used[p]) has_pred = true;
    if (has_pred) continue;
    std::vector<int> chain{i};
    int cur = i;
    while (n_users[cur] == 1 && is_ew(only_user[cur]) && !used[only_user[cur]]) {
      cur = only_user[cur];
      chain.push_back(cur);
    }
    if (chain.size() >= 2) {
      for (int c : chain) used[c] = 1;
      chains.push_back(chain);
    }
  }
  return chains;
}

}  // namespace rt
