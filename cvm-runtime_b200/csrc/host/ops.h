// Operator registry of the host runtime: attribute parsing, arity, shape and precision inference.
//
// Mirrors the reference's op registry for the operators on the hot path
// (CVM_REGISTER_OP in src/top/**, param structs in include/cvm/top/{nn,tensor}.h, attribute
// parsing rules of include/utils/parameter.h and include/cvm/tuple.h:221-280).
#pragma once
#include <functional>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>
#include "base.h"

namespace cvm {

// Parsed attributes of one node: typed views of the string dictionary.
struct Attrs {
  std::string op;
  std::string name;
  std::unordered_map<std::string, std::string> dict;
  std::map<std::string, int64_t> ints;
  std::map<std::string, bool> bools;
  std::map<std::string, Shape> tuples;
  std::map<std::string, std::string> strs;
  std::map<std::string, bool> has;  // for optional fields

  int64_t i(const char* k) const { return ints.at(k); }
  bool b(const char* k) const { return bools.at(k); }
  const Shape& t(const char* k) const { return tuples.at(k); }
  const std::string& s(const char* k) const { return strs.at(k); }
};

enum FieldKind { F_INT, F_BOOL, F_TUPLE, F_STR, F_OPT_INT, F_DTYPE };

struct FieldSpec {
  const char* name;
  FieldKind kind;
  bool required;
  const char* def;      // textual default when not required
  bool has_lower;
  int64_t lower;
};

typedef std::function<bool(const Attrs&, std::vector<Shape>*, std::vector<Shape>*)> InferShapeFn;
typedef std::function<bool(const Attrs&, const std::vector<Shape>&, std::vector<int>*, std::vector<int>*)>
    InferPrecFn;

enum { kVarg = -1, kUseBias = -2 };

struct OpDef {
  std::string name;
  int num_inputs;   // >= 0, kVarg, or kUseBias (2 + use_bias)
  int num_outputs;
  bool has_parser;
  std::vector<FieldSpec> fields;
  InferShapeFn infer_shape;
  InferPrecFn infer_prec;
  bool sort_axis;   // reduce ops sort their axis tuple when parsed
};

// Throws std::runtime_error for an unknown operator (src/top/op.cc:53-58).
const OpDef* find_op(const std::string& name);

// Parse `dict` according to the op's field table into `out` (ParamError on unknown keys, missing
// required fields, malformed values or violated bounds).
void parse_attrs(const OpDef* op, Attrs* out);

void verify_attr_range(int64_t v, const char* name, int64_t lo = 0, int64_t hi = 4096);

}  // namespace cvm
