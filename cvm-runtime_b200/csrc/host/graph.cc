// Graph loading and validation.  Follows the order of checks of the reference executor so that a
// malformed model fails with the same status class (logic vs runtime error).
#include "graph.h"
#include <algorithm>
#include <map>
#include <cstring>
#include <unordered_set>
#include "json.h"

namespace cvm {

namespace {

// Node::GetOpName, src/runtime/graph_runtime.h:262-270
std::string strip_suffix(const std::string& name) {
  std::string ret = name;
  for (int i = (int)name.size() - 1; i >= 0; --i) {
    if (name[i] >= '0' && name[i] <= '9') continue;
    else if (name[i] == '_') ret = name.substr(0, i);
    break;
  }
  return ret;
}

template <typename T>
std::vector<T> read_int_list(const JValue& v) {
  std::vector<T> out;
  for (const auto& x : v.as_array()) out.push_back((T)x.as_int());
  return out;
}

// NodeEntry::Load, src/runtime/graph_runtime.h:189-205
NodeEntry read_entry(const JValue& v) {
  const auto& a = v.as_array();
  VERIFY(a.size() >= 2) << "invalid json format";
  VERIFY(a.size() <= 3) << "invalid json format";
  NodeEntry e;
  e.node_id = (uint32_t)a[0].as_int();
  e.index = (uint32_t)a[1].as_int();
  e.version = a.size() == 3 ? (uint32_t)a[2].as_int() : 0;
  return e;
}

// GraphAttr::Load helper: ["type_tag", payload]
const JValue& typed_attr(const JValue& v, const char* want) {
  const auto& a = v.as_array();
  VERIFY(a.size() >= 1);
  VERIFY_EQ(a[0].as_string(), want);
  VERIFY(a.size() >= 2);
  VERIFY(a.size() == 2);
  return a[1];
}

}  // namespace

// CvmRuntime::Load + Node::Load + GraphAttr::Load, src/runtime/graph_runtime.h:208-436
void Graph::Load(const std::string& json) {
  JValue root = parse_json(json);
  CHECK(root.is_object()) << "invalid json format: graph must be an object";
  int bitmask = 0;
  for (const auto& kv : root.obj) {
    const std::string& key = kv.first;
    const JValue& val = kv.second;
    if (key == "nodes") {
      for (const auto& jn : val.as_array()) {
        CHECK(jn.is_object()) << "invalid json format: node must be an object";
        Node n;
        int nmask = 0;
        for (const auto& nk : jn.obj) {
          if (nk.first == "op") {
            n.op_type = nk.second.as_string();
            VERIFY((n.op_type == "cvm_op") || (n.op_type == "null"))
                << "CVM executor only supported cvm_op or parameter vs. " << n.op_type;
            nmask |= 1;
          } else if (nk.first == "name") {
            n.attrs.name = nk.second.as_string();
            nmask |= 2;
          } else if (nk.first == "inputs") {
            for (const auto& e : nk.second.as_array()) n.inputs.push_back(read_entry(e));
            nmask |= 4;
          } else if (nk.first == "attrs") {
            CHECK(nk.second.is_object()) << "invalid json format: node attrs must be an object";
            int amask = 0;
            for (const auto& ak : nk.second.obj) {
              const std::string& value = ak.second.as_string();
              if (ak.first == "func_name") { n.func_name = value; amask |= 1; }
              else if (ak.first == "num_inputs" || ak.first == "num_outputs" ||
                       ak.first == "op_attrs" || ak.first == "flatten_data") {}
              else FATAL() << "node attributes do not support key " << ak.first;
            }
            VERIFY_EQ(amask, 1) << "invalid format";
          } else if (nk.first == "precision") {
            (void)nk.second.as_int();
          } else {
            FATAL() << "node do not support key " << nk.first;
          }
        }
        VERIFY_EQ(nmask, 1 | 2 | 4) << "invalid format";
        nodes.push_back(std::move(n));
      }
      bitmask |= 1;
    } else if (key == "arg_nodes") {
      input_nodes = read_int_list<uint32_t>(val);
    } else if (key == "node_row_ptr") {
      node_row_ptr = read_int_list<uint32_t>(val);
    } else if (key == "heads") {
      for (const auto& e : val.as_array()) outputs.push_back(read_entry(e));
      bitmask |= 8;
    } else if (key == "attrs") {
      CHECK(val.is_object()) << "invalid json format: attrs must be an object";
      int amask = 0;
      for (const auto& ak : val.obj) {
        const std::string& k = ak.first;
        if (k == "dltype") {
          for (const auto& s : typed_attr(ak.second, "list_str").as_array()) dltype.push_back(s.as_string());
        } else if (k == "storage_id") {
          storage_id = read_int_list<int>(typed_attr(ak.second, "list_int"));
          amask |= 2;
        } else if (k == "shape") {
          for (const auto& s : typed_attr(ak.second, "list_shape").as_array()) shape.push_back(read_int_list<int64_t>(s));
          amask |= 4;
        } else if (k == "device_index") {
          device_index = read_int_list<int>(typed_attr(ak.second, "list_int"));
        } else if (k == "precision") {
          precision = read_int_list<int>(typed_attr(ak.second, "list_int"));
        } else if (k == "op_attrs") {
          for (const auto& s : typed_attr(ak.second, "list_str").as_array()) op_attrs.push_back(s.as_string());
          amask |= 8;
        } else if (k == "dtype") {
          const auto& a = ak.second.as_array();
          VERIFY(a.size() >= 1);
          const std::string& type = a[0].as_string();
          if (type != "list_int" && type != "list_str") FATAL() << "cannot skip graph attr " << k;
          VERIFY(a.size() == 2);
        } else {
          FATAL() << "graph attribute " << k << " not supported";
        }
      }
      VERIFY_EQ(amask, 2 | 4 | 8) << "invalid format";
      bitmask |= 16;
    } else if (key == "version") {
      version = val.as_string();
    } else if (key == "postprocess") {
      postprocess = val.as_string();
    } else {
      FATAL() << "key " << key << " in json is not supported";
    }
  }
  VERIFY_EQ(bitmask, 1 | 8 | 16) << "invalid format";
}

// CvmRuntime::PrepareGraphWithVersion, src/runtime/graph_runtime.cc:114-261
void Graph::Prepare() {
  std::unordered_set<std::string> name_set;
  for (auto nid : input_nodes) {
    VERIFY_LT(nid, nodes.size()) << "arg_nodes entry " << nid << " out of range";
    if (!name_set.emplace(nodes[nid].name()).second)
      FATAL() << "node name " << nodes[nid].name() << " duplicated in graph";
  }
  VERIFY_EQ(nodes.size(), op_attrs.size())
      << "graph attribute op_attrs size: " << op_attrs.size() << ", Expected " << nodes.size();
  // Node::LoadOpAndAttrs, src/runtime/graph_runtime.h:293-318
  for (size_t i = 0; i < nodes.size(); ++i) {
    Node& n = nodes[i];
    if (n.is_variable()) continue;
    n.func_name = strip_suffix(n.func_name);
    n.op = find_op(n.func_name);
    n.attrs.op = n.func_name;
    JValue d = parse_json(op_attrs[i]);
    CHECK(d.is_object()) << "invalid json format: op_attrs entry must be an object";
    for (const auto& kv : d.obj) n.attrs.dict[kv.first] = kv.second.as_string();
    if (n.op->has_parser) {
      parse_attrs(n.op, &n.attrs);
    } else {
      VERIFY_EQ(n.attrs.dict.size(), 0U) << "operator " << n.op->name << " name=" << n.name()
                                         << " should not have attributes, but " << op_attrs[i];
    }
    if (n.op->num_inputs == kVarg) n.num_inputs = (uint32_t)n.inputs.size();
    else if (n.op->num_inputs == kUseBias) n.num_inputs = n.attrs.b("use_bias") ? 3 : 2;
    else n.num_inputs = (uint32_t)n.op->num_inputs;
    n.num_outputs = (uint32_t)n.op->num_outputs;
    VERIFY_EQ(n.num_inputs, n.inputs.size())
        << "operator " << n.func_name << " name=" << n.name() << "'s inputs length invaild "
        << n.inputs.size() << " vs. " << n.num_inputs;
  }

  num_entries = 0;
  std::vector<uint32_t> row_ptr, in_nodes;
  for (uint32_t i = 0; i < nodes.size(); ++i) {
    if (nodes[i].is_variable()) in_nodes.push_back(i);
    row_ptr.push_back(num_entries);
    num_entries += nodes[i].num_outputs;
  }
  row_ptr.push_back(num_entries);
  const std::vector<uint32_t> json_row_ptr = node_row_ptr;
  node_row_ptr = row_ptr;  // entry ids below always use the recomputed table

  // The reference resolves (node, output) pairs by entry arithmetic alone (graph_runtime.h:466-472):
  // an output index past the node's own outputs names the entry of a later node.  Such pairs are
  // rewritten to the node that owns the entry; pairs that run off the entry table (an
  // out-of-bounds read in the reference) are refused.
  auto resolve = [&](NodeEntry& e, const char* what) {
    VERIFY_LT(e.node_id, nodes.size()) << what << " refers to node " << e.node_id << " out of range";
    if (e.index < nodes[e.node_id].num_outputs) return;
    const uint64_t eid = (uint64_t)row_ptr[e.node_id] + e.index;
    VERIFY_LT(eid, (uint64_t)num_entries) << what << " refers to output " << e.index << " out of range";
    const uint32_t owner = (uint32_t)(std::upper_bound(row_ptr.begin(), row_ptr.end(), (uint32_t)eid) - row_ptr.begin()) - 1;
    e.node_id = owner;
    e.index = (uint32_t)eid - row_ptr[owner];
  };
  for (auto& n : nodes)
    for (auto& e : n.inputs) resolve(e, "input");
  for (auto& e : outputs) resolve(e, "head");

  VERIFY_EQ(num_entries, storage_id.size())
      << "graph attribute storage_id size: " << storage_id.size() << ", Expected " << num_entries;
  for (auto sid : storage_id) VERIFY_GE(sid, 0) << "storage id should not less than 0, but " << sid;
  static const std::unordered_set<std::string> reused_ops{
      "flatten", "relu", "expand_dims", "reshape", "squeeze", "abs", "cvm_precision", "elemwise_add",
      "elemwise_sub", "nagetive", "clip", "cvm_clip", "cvm_right_shift", "cvm_left_shift"};
  for (size_t nid = 0; nid < nodes.size(); ++nid) {
    const Node& n = nodes[nid];
    if (n.is_variable()) continue;
    if (reused_ops.count(n.op->name)) continue;
    for (uint32_t oi = 0; oi < n.num_outputs; ++oi) {
      const int node_sid = storage_id[entry_id(nid, oi)];
      for (const auto& e : n.inputs) {
        const int in_sid = storage_id[entry_id(e)];
        VERIFY_NE(node_sid, in_sid) << "operator " << n.op->name << " input: (" << e.node_id << ", "
                                    << e.index << ") output: (" << nid << ", " << oi
                                    << ") used same storage_id " << in_sid << " vs. " << node_sid;
      }
    }
  }

  VERIFY_EQ(num_entries, shape.size())
      << "graph attribute shape size: " << shape.size() << ", Expected " << num_entries;
  for (const auto& s : shape) {
    uint64_t sx = 1;
    VERIFY((0 < s.size()) && (s.size() <= 6)) << "shape ndim should between (0, 6], but " << s.size();
    for (auto x : s) {
      sx *= (uint64_t)x;
      VERIFY((0 < x) && (x <= (1 << 24))) << "single dimension should between (0, " << (1 << 24) << "], but " << x;
      VERIFY_LE(sx, (uint64_t)(1 << 30)) << "shape size shoule not greater than" << (1 << 30) << ", but " << sx;
    }
  }

  VERIFY_EQ(num_entries, precision.size())
      << "graph attribute precision size: " << precision.size() << ", Expected " << num_entries;
  for (auto p : precision)
    VERIFY((p == -1) || (0 < p && p <= 32)) << "precision should be -1 or between (0, 32], but " << p;
  VERIFY(device_index.empty()) << "attribute device_index must be set empty";

  if (version == "cvm_1.0.0") {
    VERIFY_EQ(num_entries, dltype.size())
        << "graph attribute dltype size: " << dltype.size() << ", Expected " << num_entries;
    for (const auto& t : dltype) VERIFY_EQ(t, "int32") << "type " << t << " are not supported";
    VERIFY_EQ(json_row_ptr.size(), row_ptr.size())
        << "node_row_ptr's size: " << json_row_ptr.size() << ", Expected " << row_ptr.size();
    for (size_t i = 0; i < row_ptr.size(); ++i)
      VERIFY_EQ(row_ptr[i], json_row_ptr[i]) << "node_row_ptr is invalid at index " << i;
    VERIFY_EQ(input_nodes.size(), in_nodes.size())
        << "arg_nodes' size: " << input_nodes.size() << ", Expected " << in_nodes.size();
    for (size_t i = 0; i < in_nodes.size(); ++i)
      VERIFY_EQ(in_nodes[i], input_nodes[i]) << "arg_nodes is invalid at index " << i;
  } else if (version == "cvm_1.1.0") {
    input_nodes = in_nodes;
  } else {
    FATAL() << "graph version " << version << " not supported";
  }

  for (size_t i = 0; i < nodes.size(); ++i) {
    const uint32_t eid = entry_id(i, 0);
    for (const auto& e : nodes[i].inputs)
      VERIFY_LT(entry_id(e), eid) << "the graph does not follow the topological order.";
  }
}

// CvmRuntime::SetupShape, src/runtime/infer_attr.cc:161-217
void Graph::SetupShape() {
  std::vector<Shape> ishape, oshape;
  for (uint32_t nid = 0; nid < nodes.size(); ++nid) {
    const Node& n = nodes[nid];
    if (n.is_variable()) continue;
    ishape.assign(n.num_inputs, Shape());
    for (uint32_t i = 0; i < n.num_inputs; ++i) ishape[i] = shape[entry_id(n.inputs[i])];
    oshape.assign(n.num_outputs, Shape());
    if (!n.op->infer_shape) FATAL() << "operator " << n.op->name << " has not registered FInferShape";
    if (!n.op->infer_shape(n.attrs, &ishape, &oshape))
      FATAL() << "operator " << n.op->name << " name=" << n.name() << ": infer shape failed";
    for (uint32_t i = 0; i < n.num_inputs; ++i)
      VERIFY(ishape[i] == shape[entry_id(n.inputs[i])])
          << "Check input shape failed, expected to be " << shape_str(ishape[i]) << " but "
          << shape_str(shape[entry_id(n.inputs[i])]);
    for (uint32_t i = 0; i < n.num_outputs; ++i)
      VERIFY(oshape[i] == shape[entry_id(nid, i)])
          << "Check output shape failed, expected to be " << shape_str(oshape[i]) << " but "
          << shape_str(shape[entry_id(nid, i)]) << n.op->name;
  }
}

// CvmRuntime::SetupPrecision, src/runtime/infer_attr.cc:31-91
void Graph::SetupPrecision() {
  std::vector<int> iprec, oprec;
  std::vector<Shape> shapes;
  for (uint32_t nid = 0; nid < nodes.size(); ++nid) {
    const Node& n = nodes[nid];
    if (n.is_variable()) {
      VERIFY_NE(precision[entry_id(nid, 0)], -1) << "variable node " << n.name() << "'s precision has not been set";
      continue;
    }
    shapes.assign(n.num_inputs + n.num_outputs, Shape());
    iprec.assign(n.num_inputs, -1);
    oprec.assign(n.num_outputs, -1);
    for (uint32_t i = 0; i < n.num_inputs; ++i) {
      const uint32_t eid = entry_id(n.inputs[i]);
      iprec[i] = precision[eid];
      shapes[i] = shape[eid];
    }
    for (uint32_t i = 0; i < n.num_outputs; ++i) {
      const uint32_t eid = entry_id(nid, i);
      oprec[i] = precision[eid];
      shapes[n.num_inputs + i] = shape[eid];
    }
    if (!n.op->infer_prec) FATAL() << "operator " << n.op->name << " has not registered FInferPrecision";
    if (!n.op->infer_prec(n.attrs, shapes, &iprec, &oprec))
      FATAL() << "operator " << n.op->name << " name=" << n.name() << ": infer precision failed";
    for (uint32_t i = 0; i < n.num_outputs; ++i) {
      precision[entry_id(nid, i)] = oprec[i];
      VERIFY((0 < oprec[i]) && (oprec[i] <= 32))
          << " nid = " << nid << "i = " << i << " precison = " << oprec[i] << " name= " << n.name()
          << " inode.attrs = " << op_attrs[nid];
    }
  }
}

void Graph::Init(const std::string& json) {
  deferred_refusal().clear();
  Load(json);
  Prepare();
  SetupShape();
  // SetupType: every entry is int32 in the reference and every registered FInferType keeps it so.
  SetupPrecision();
  CheckStoragePlan();
  refusal = deferred_refusal();
}

// The reference executes in the buffers the storage plan names (graph_runtime.cc:576-606): two
// entries with one storage id are one piece of memory.  A plan produced by its compiler only
// shares a buffer between entries that are never live together; any other plan makes operators
// read values a later operator has already overwritten.  This library keeps one allocation per
// materialised entry, so it can only honour plans of the first kind and refuses the rest.
void Graph::CheckStoragePlan() {
  if (!deferred_refusal().empty()) return;
  const int64_t kForever = (int64_t)1 << 40;
  std::vector<int64_t> def(num_entries, 0), last(num_entries, 0);
  for (uint32_t nid = 0; nid < nodes.size(); ++nid) {
    const Node& n = nodes[nid];
    for (uint32_t i = 0; i < n.num_outputs; ++i) {
      const uint32_t e = entry_id(nid, i);
      def[e] = n.is_variable() ? -1 : (int64_t)nid;
      last[e] = n.is_variable() && !n.is_data() ? kForever : def[e];   // parameters persist across calls
    }
  }
  for (uint32_t nid = 0; nid < nodes.size(); ++nid)
    for (const auto& e : nodes[nid].inputs) last[entry_id(e)] = std::max<int64_t>(last[entry_id(e)], nid);
  for (const auto& e : outputs) last[entry_id(e)] = kForever;
  std::map<int, std::vector<uint32_t>> groups;
  for (uint32_t e = 0; e < num_entries; ++e) groups[storage_id[e]].push_back(e);
  for (auto& kv : groups) {
    auto& g = kv.second;
    if (g.size() < 2) continue;
    std::stable_sort(g.begin(), g.end(), [&](uint32_t a, uint32_t b) { return def[a] < def[b]; });
    for (size_t i = 0; i + 1 < g.size(); ++i) {
      const uint32_t a = g[i], b = g[i + 1];
      // b may take over a's buffer at the node that consumes a for the last time (in place), not before
      if (def[a] == def[b] || last[a] > def[b]) {
        std::ostringstream os;
        os << "storage plan: entries " << a << " and " << b << " share storage id " << kv.first
           << " while both are live";
        deferred_refusal() = os.str();
        return;
      }
    }
  }
}

void Graph::RaiseRefusal() const {
  VERIFY(refusal.empty()) << refusal;
}

// CvmRuntime::PlanStorage + GetStorageSize, src/runtime/graph_runtime.cc:503-531, :565-574
int64_t Graph::GetStorageSize() const {
  std::vector<size_t> pool;
  for (size_t i = 0; i < shape.size(); ++i) {
    const size_t bytes = (size_t)shape_size(shape[i]) * 4;
    const uint32_t sid = (uint32_t)storage_id[i];
    if (sid >= pool.size()) pool.resize(sid + 1, 0);
    pool[sid] = std::max(pool[sid], bytes);
  }
  int64_t ret = 0;
  const int64_t kMax = (int64_t)1 << 32;
  for (size_t s : pool) {
    ret += ((int64_t)(s + 3) / 4) * 4;
    VERIFY_LE(ret, kMax) << "storage size exceed MAX_STORAGE " << kMax;
  }
  return ret;
}

// CvmRuntime::GetOps, src/runtime/infer_attr.cc:93-159.  The reference tests the operator name
// "get_valid_count" (singular), which no operator has, so get_valid_counts is charged on its
// first output like any other operator; that is kept.
int64_t Graph::GetOps() const {
  int64_t ops = 0, mem_cost = 0;
  const int64_t kMaxBase = (int64_t)1 << 30, kMaxOps = (int64_t)1 << 40, kMaxMem = (int64_t)1 << 40;
  for (uint32_t nid = 0; nid < nodes.size(); ++nid) {
    const Node& n = nodes[nid];
    if (n.is_variable()) {
      mem_cost += shape_size(shape[entry_id(nid, 0)]) * 5;
    } else {
      const uint32_t out_eid = entry_id(nid, 0);
      int64_t base = 1;
      const std::string& op = n.op->name;
      if (op == "dense") {
        base = shape[entry_id(n.inputs[1])][1] * 3;
        if (n.attrs.b("use_bias")) base += 1;
      } else if (op == "non_max_suppression") {
        base = shape[entry_id(n.inputs[0])][0] * 20;
      } else if (op == "conv2d") {
        const Shape& w = shape[entry_id(n.inputs[1])];
        VERIFY(!w.empty() && w[0] != 0) << "conv2d weight of " << n.name() << " has no shape";
        base = shape_size(w) / w[0] * 3;
        if (n.attrs.b("use_bias")) base += 1;
      } else if (op == "max_pool2d") {
        base = shape_size(n.attrs.t("pool_size"));
      } else if (op == "sum") {
        base = shape_size(shape[entry_id(n.inputs[0])]) / shape_size(shape[out_eid]);
      }
      VERIFY_LE(base, kMaxBase) << "single ops foreach output should not greater than 1G, but " << base;
      base *= shape_size(shape[out_eid]);
      ops += base;
      VERIFY_LE(ops, kMaxOps) << "graph ops exceed MAX_OPS " << kMaxOps;
      int64_t mem = 0;
      for (uint32_t i = 0; i < n.num_outputs; ++i) mem += shape_size(shape[entry_id(nid, i)]);
      mem_cost += mem * 5;
    }
    VERIFY_LE(mem_cost, kMaxMem) << "graph memory cost exceed MAX_MEMORY " << kMaxMem;
  }
  return mem_cost + ops;
}

int Graph::GetInputIndex(const std::string& name) const {
  for (size_t i = 0; i < input_nodes.size(); ++i)
    if (nodes[input_nodes[i]].name() == name) return (int)i;
  FATAL() << "cannot find `" << name << "` among input";
  return -1;
}

int Graph::GetOutputPrecision() const {
  int ret = 0;
  for (const auto& e : outputs) ret = std::max(ret, precision[entry_id(e)]);
  return ret;
}

int Graph::GetInputPrecision() const {
  for (size_t i = 0; i < nodes.size(); ++i)
    if (nodes[i].is_data()) return precision[entry_id(i, 0)];
  FATAL() << "can not find input `data`";
  return -1;
}

// ------------------------------------------------------------------------------------------
// Params blob: load_param_dict (src/runtime/param_dict.cc:14-38), NDArray::Load
// (include/cvm/runtime/ndarray.h:485-556), then CvmRuntime::SetInput's checks per parameter
// (src/runtime/graph_runtime.cc:317-397).
// ------------------------------------------------------------------------------------------
namespace {
struct Reader {
  const std::string& s;
  size_t p = 0;
  explicit Reader(const std::string& str) : s(str) {}
  bool read(void* dst, size_t n) {
    if (n > s.size() - p) return false;
    memcpy(dst, s.data() + p, n);
    p += n;
    return true;
  }
  template <typename T>
  bool get(T* v) { return read(v, sizeof(T)); }
};
}  // namespace

void Graph::LoadParams(const std::string& blob) {
  Reader r(blob);
  uint64_t header = 0, reserved = 0;
  VERIFY(r.get(&header)) << "Invalid parameters file format";
  VERIFY(header == 0xF7E58D4F05049CB7ull) << "Invalid parameters file format";
  VERIFY(r.get(&reserved)) << "Invalid parameters file format";
  uint64_t n_names = 0;
  VERIFY(r.get(&n_names)) << "Invalid parameters file format";
  VERIFY(n_names <= blob.size()) << "Invalid parameters file format";
  std::vector<std::string> names(n_names);
  for (auto& nm : names) {
    uint64_t len = 0;
    VERIFY(r.get(&len)) << "Invalid parameters file format";
    VERIFY(len <= blob.size() - r.p) << "Invalid parameters file format";
    nm.resize(len);
    if (len) VERIFY(r.read(&nm[0], len)) << "Invalid parameters file format";
  }
  uint64_t sz = 0;
  r.get(&sz);
  VERIFY(sz == names.size()) << "Invalid parameters file format";

  struct Raw { Shape shape; int code, bits, lanes; int dev_type; std::string bytes; };
  std::vector<Raw> values(sz);
  for (auto& v : values) {
    uint64_t magic = 0, rsv = 0;
    CHECK(r.get(&magic)) << "Invalid DLTensor file format";
    CHECK(r.get(&rsv)) << "Invalid DLTensor file format";
    CHECK(magic == 0xDD5E40F096B4A13Full) << "Invalid DLTensor file format";
    int32_t dev_type = 0, dev_id = 0, ndim = 0;
    uint8_t code = 0, bits = 0;
    uint16_t lanes = 0;
    CHECK(r.get(&dev_type) && r.get(&dev_id)) << "Invalid DLTensor file format";
    CHECK(r.get(&ndim)) << "Invalid DLTensor file format";
    CHECK(r.get(&code) && r.get(&bits) && r.get(&lanes)) << "Invalid DLTensor file format";
    CHECK(ndim >= 0 && ndim <= 64) << "Invalid DLTensor file format";
    v.shape.resize(ndim);
    for (int i = 0; i < ndim; ++i) CHECK(r.get(&v.shape[i])) << "Invalid DLTensor file format";
    int64_t num = 1;
    for (auto d : v.shape) {
      CHECK(d >= 0 && d <= ((int64_t)1 << 32)) << "Invalid DLTensor file format";
      num *= d;
      CHECK(num <= ((int64_t)1 << 40)) << "Invalid DLTensor file format";
    }
    const int elem_bytes = (bits + 7) / 8;
    int64_t nbytes = 0;
    CHECK(r.get(&nbytes)) << "Invalid DLTensor file format";
    CHECK(nbytes == num * elem_bytes) << "Invalid DLTensor file format";
    CHECK(nbytes >= 0 && (uint64_t)nbytes <= blob.size() - r.p) << "Invalid DLTensor file format";
    v.bytes.assign(blob.data() + r.p, (size_t)nbytes);
    r.p += (size_t)nbytes;
    v.code = code; v.bits = bits; v.lanes = lanes; v.dev_type = dev_type;
  }

  std::vector<bool> set_flag(input_nodes.size(), false);
  for (size_t i = 0; i < names.size(); ++i) {
    const int in_idx = GetInputIndex(names[i]);
    set_flag[in_idx] = true;
    const uint32_t nid = input_nodes[in_idx];
    const uint32_t eid = entry_id(nid, 0);
    const Raw& v = values[i];
    VERIFY(v.code == 0) << "cvm runtime only supported INT NDArray, but (" << v.code << ")";
    VERIFY_EQ(v.dev_type, 1) << "cvm runtime only supported input with `cpu` device, but " << v.dev_type;
    const Shape& expected = shape[eid];
    VERIFY_EQ(v.shape.size(), expected.size())
        << "Loaded data shape ndim " << v.shape.size() << " not matched " << expected.size();
    uint64_t size = 1;
    for (size_t d = 0; d < expected.size(); ++d) {
      VERIFY_EQ(v.shape[d], expected[d]) << "Loaded data shape at index " << d << " with value "
                                         << v.shape[d] << ", Expected " << expected[d];
      size *= (uint64_t)v.shape[d];
    }
    VERIFY((v.code == 0) && ((v.bits == 32) || (v.bits == 8)) && (v.lanes == 1))
        << "cvm runtime only supported INT8 or INT32 NDArray, but (" << v.code << ", " << v.bits
        << ", " << v.lanes << ")";
    HostTensor t;
    t.shape = expected;
    t.data.resize(size);
    if (v.bits == 8) {
      const int8_t* p = reinterpret_cast<const int8_t*>(v.bytes.data());
      for (uint64_t k = 0; k < size; ++k) t.data[k] = p[k];
    } else {
      memcpy(t.data.data(), v.bytes.data(), size * 4);
    }
    const int prec = precision[eid];
    const int32_t range = (int32_t)((1u << (prec - 1)) - 1);
    if (nodes[nid].is_data()) {
      for (auto& x : t.data) x = x > range ? range : (x < -range ? -range : x);
    } else {
      for (uint64_t k = 0; k < size; ++k)
        VERIFY((-range <= t.data[k]) && (t.data[k] <= range))
            << "parameter " << nodes[nid].name() << " at index " << k << " value:" << t.data[k]
            << " exceed of precision " << prec;
    }
    params[eid] = std::move(t);
  }
  for (size_t i = 0; i < set_flag.size(); ++i) {
    const uint32_t nid = input_nodes[i];
    VERIFY((set_flag[i] || nodes[nid].is_data()))
        << "parameter nid=" << nid << " name=" << nodes[nid].name() << " has not been loaded";
  }
  params_loaded = true;
}

}  // namespace cvm
