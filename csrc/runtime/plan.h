// Execution plan of a dynamic op graph: ordering, parallel levels, dead-node elimination, liveness-based
// memory planning and elementwise-chain discovery; see plan.cpp.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace rt {

struct PlanNode {
  int id;
  std::string op;
  std::vector<int> inputs;
  uint64_t out_bytes;
};

struct MemoryPlan {
  std::vector<int64_t> offsets;  // per node, -1 for nodes without an output buffer
  uint64_t total_bytes;          // arena size that satisfies every lifetime
  uint64_t naive_bytes;          // sum of all outputs (no reuse)
};

class ExecutionPlan {
 public:
  int add_node(const std::string& op, const std::vector<int>& inputs, uint64_t out_bytes);
  void mark_output(int id);
  int num_nodes() const { return (int)nodes_.size(); }
  const PlanNode& node(int id) const;
  std::vector<int> topo_order() const;
  std::vector<std::vector<int>> levels() const;
  std::vector<int> eliminate_dead() const;  // ids that no output depends on
  // (offsets, total, naive): buffers whose lifetimes do not overlap share arena space.
  std::pair<std::vector<int64_t>, std::pair<uint64_t, uint64_t>> memory_plan(uint64_t alignment) const;
  // Maximal chains (length >= 2) of elementwise ops where each link is the only consumer of its producer.
  std::vector<std::vector<int>> fusible_chains() const;

 private:
  std::vector<PlanNode> nodes_;
  std::vector<int> outputs_;
};

}  // namespace rt
