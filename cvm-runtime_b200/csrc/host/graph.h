// The logical model: graph JSON + params blob, validated exactly as the reference's executor
// validates them (src/runtime/graph_runtime.{h,cc}, infer_attr.cc, param_dict.cc), plus the
// host-only queries (storage size, gas).  No device code here.
#pragma once
#include <map>
#include <string>
#include <vector>
#include "base.h"
#include "ops.h"

namespace cvm {

struct NodeEntry {
  uint32_t node_id = 0, index = 0, version = 0;
};

struct Node {
  std::string op_type;     // "null" or "cvm_op"
  std::string func_name;   // operator name, trailing _<digits> stripped
  std::vector<NodeEntry> inputs;
  const OpDef* op = nullptr;
  Attrs attrs;
  uint32_t num_inputs = 1, num_outputs = 1;
  bool is_variable() const { return op_type == "null"; }
  bool is_data() const { return is_variable() && attrs.name == "data"; }
  const std::string& name() const { return attrs.name; }
};

struct HostTensor {          // one parameter, widened to int32 like the reference does on load
  Shape shape;
  std::vector<int32_t> data;
};

class Graph {
 public:
  // CvmRuntime::Init (graph_runtime.cc:106-112): Load + PrepareGraphWithVersion + CheckAttr.
  void Init(const std::string& json);
  void RaiseRefusal() const;
  void CheckStoragePlan();
  // CvmRuntime::LoadParams (graph_runtime.cc:476-501).
  void LoadParams(const std::string& blob);

  int64_t GetStorageSize() const;   // graph_runtime.cc:503-531, :565-574
  int64_t GetOps() const;           // infer_attr.cc:93-159
  int GetInputIndex(const std::string& name) const;  // graph_runtime.cc:288-298
  int GetOutputPrecision() const;
  int GetInputPrecision() const;

  uint32_t entry_id(uint32_t nid, uint32_t index) const { return node_row_ptr[nid] + index; }
  uint32_t entry_id(const NodeEntry& e) const { return entry_id(e.node_id, e.index); }

  std::vector<Node> nodes;
  std::vector<uint32_t> input_nodes;
  std::vector<uint32_t> node_row_ptr;
  std::vector<NodeEntry> outputs;
  uint32_t num_entries = 0;
  // graph attributes, one per entry except op_attrs (one per node)
  std::vector<int> storage_id, device_index, precision;
  std::vector<std::string> dltype, op_attrs;
  std::vector<Shape> shape;
  std::string version = "cvm_1.0.0";
  std::string refusal;  // see deferred_refusal(); raised by RaiseRefusal() once the reference's checks passed
  std::string postprocess;
  std::map<uint32_t, HostTensor> params;  // by entry id
  bool params_loaded = false;

 private:
  void Load(const std::string& json);
  void Prepare();
  void SetupShape();
  void SetupPrecision();
};

}  // namespace cvm
