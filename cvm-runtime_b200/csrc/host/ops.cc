// Operator table: attribute specs, arity, FInferShape and FInferPrecision equivalents.
// Every function cites the reference definition it reproduces.
#include "ops.h"
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <set>

namespace cvm {

void verify_attr_range(int64_t v, const char* name, int64_t lo, int64_t hi) {
  // src/top/op_common.h:23-39
  VERIFY(lo <= v && v <= hi) << "attribute " << name << " value: " << v << " out of range [" << lo
                             << ", " << hi << "]";
}

// ------------------------------------------------------------------------------------------
// Attribute value parsing (include/utils/parameter.h field entries, include/cvm/tuple.h:221-280)
// ------------------------------------------------------------------------------------------
namespace {

std::string trim(const std::string& s) {
  size_t b = 0, e = s.size();
  while (b < e && isspace((unsigned char)s[b])) ++b;
  while (e > b && isspace((unsigned char)s[e - 1])) --e;
  return s.substr(b, e - b);
}

int64_t parse_int(const std::string& key, const std::string& text) {
  const std::string t = trim(text);
  char* end = nullptr;
  errno = 0;
  long long v = strtoll(t.c_str(), &end, 10);
  if (t.empty() || end == t.c_str() || *end != 0 || errno != 0 || v < INT32_MIN || v > INT32_MAX)
    throw ParamError("Invalid Parameter format for " + key + " expect int but value='" + text + "'");
  return v;
}

bool parse_bool(const std::string& key, const std::string& text) {
  std::string t = trim(text);
  std::transform(t.begin(), t.end(), t.begin(), ::tolower);
  if (t == "true" || t == "1") return true;
  if (t == "false" || t == "0") return false;
  throw ParamError("Invalid Parameter format for " + key + " expect boolean but value='" + text + "'");
}

// Tuple grammar of include/cvm/tuple.h:221-280: "(1, 2)", "[1,2]", "()", or a bare integer.
Shape parse_tuple(const std::string& key, const std::string& text) {
  Shape out;
  size_t p = 0;
  const size_t n = text.size();
  auto fail = [&]() -> Shape {
    throw ParamError("Invalid Parameter format for " + key + " expect tuple but value='" + text + "'");
  };
  auto read_int = [&](int64_t* v) -> bool {
    while (p < n && isspace((unsigned char)text[p])) ++p;
    size_t b = p;
    if (p < n && (text[p] == '-' || text[p] == '+')) ++p;
    size_t d = p;
    while (p < n && isdigit((unsigned char)text[p])) ++p;
    if (p == d) { p = b; return false; }
    *v = strtoll(text.substr(b, p - b).c_str(), nullptr, 10);
    return true;
  };
  while (true) {
    if (p >= n) return fail();
    char ch = text[p];
    if (isdigit((unsigned char)ch) || ch == '-') {
      int64_t v;
      if (!read_int(&v)) return fail();
      out.push_back(v);
      while (p < n && isspace((unsigned char)text[p])) ++p;
      if (p != n) return fail();
      return out;
    }
    ++p;
    if (ch == '(' || ch == '[') break;
    if (!isspace((unsigned char)ch)) return fail();
  }
  while (p < n && isspace((unsigned char)text[p])) ++p;
  if (p < n && (text[p] == ')' || text[p] == ']')) {
    ++p;
  } else {
    int64_t v;
    bool closed = false;
    while (read_int(&v)) {
      out.push_back(v);
      while (p < n && isspace((unsigned char)text[p])) ++p;
      if (p >= n) return fail();
      char ch = text[p++];
      if (ch == 'L') {
        if (p >= n) return fail();
        ch = text[p++];
      }
      if (ch == ',') {
        while (p < n && isspace((unsigned char)text[p])) ++p;
        if (p < n && (text[p] == ')' || text[p] == ']')) { ++p; closed = true; break; }
      } else if (ch == ')' || ch == ']') {
        closed = true;
        break;
      } else {
        return fail();
      }
    }
    if (!closed) return fail();
  }
  while (p < n && isspace((unsigned char)text[p])) ++p;
  if (p != n) return fail();
  return out;
}

int64_t parse_dtype(const std::string& key, const std::string& text) {
  static const std::map<std::string, int> names = {
      {"float32", 0}, {"float64", 1}, {"float16", 2}, {"uint8", 3},  {"int32", 4},  {"int8", 5},
      {"int64", 6},   {"int16", 7},   {"uint16", 8},  {"uint32", 9}, {"uint64", 10}, {"same", -1}};
  auto it = names.find(trim(text));
  if (it == names.end())
    throw ParamError("Invalid Input: '" + text + "', valid values for " + key + " are type names");
  return it->second;
}

void set_field(const FieldSpec& f, const std::string& text, Attrs* a) {
  switch (f.kind) {
    case F_INT: {
      int64_t v = parse_int(f.name, text);
      if (f.has_lower && v < f.lower)
        throw ParamError(std::string("value ") + std::to_string(v) + " for Parameter " + f.name +
                         " should be greater equal to " + std::to_string(f.lower));
      a->ints[f.name] = v;
    } break;
    case F_OPT_INT: {
      std::string t = trim(text);
      if (t == "None") { a->has[f.name] = false; a->ints[f.name] = 0; }
      else { a->ints[f.name] = parse_int(f.name, text); a->has[f.name] = true; }
    } break;
    case F_BOOL: a->bools[f.name] = parse_bool(f.name, text); break;
    case F_TUPLE: a->tuples[f.name] = parse_tuple(f.name, text); break;
    case F_STR: a->strs[f.name] = text; break;
    case F_DTYPE: a->ints[f.name] = parse_dtype(f.name, text); break;
  }
}

}  // namespace

void parse_attrs(const OpDef* op, Attrs* a) {
  try {
    std::set<std::string> seen;
    for (const auto& kv : a->dict) {
      const FieldSpec* spec = nullptr;
      for (const auto& f : op->fields)
        if (kv.first == f.name) { spec = &f; break; }
      if (!spec) {
        const std::string& k = kv.first;
        if (k.size() > 4 && k.compare(0, 2, "__") == 0 && k.compare(k.size() - 2, 2, "__") == 0) continue;
        throw ParamError("Cannot find argument '" + k + "'");
      }
      set_field(*spec, kv.second, a);
      seen.insert(kv.first);
    }
    for (const auto& f : op->fields) {
      if (seen.count(f.name)) continue;
      if (f.required) throw ParamError(std::string("Required parameter ") + f.name + " is not presented");
      if (f.kind == F_OPT_INT) { a->has[f.name] = false; a->ints[f.name] = 0; continue; }
      set_field(f, f.def, a);
    }
  } catch (const ParamError& e) {
    // src/top/op_common.h:46-63 appends the operator context to the message.
    std::ostringstream os;
    os << e.what() << ", in operator " << op->name << "(name=\"" << a->name << "\"";
    for (const auto& kv : a->dict) os << ", " << kv.first << "=\"" << kv.second << "\"";
    os << ")";
    throw ParamError(os.str());
  }
  if (op->sort_axis) {
    Shape& ax = a->tuples["axis"];
    std::sort(ax.begin(), ax.end());  // src/top/tensor/reduce.cc:100-106
  }
}

// ------------------------------------------------------------------------------------------
// Shape / precision inference
// ------------------------------------------------------------------------------------------
namespace {

void in_prec_check(const Attrs& a, const std::vector<int>& ip) {
  // IN_PREC_CHECK, src/top/op_common.h:262-268
  for (size_t i = 0; i < ip.size(); ++i)
    VERIFY_NE(ip[i], -1) << "operator " << a.name << "'s inputs(" << i << ") has not been infered precision";
}

bool same_precision(const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  (*op)[0] = ip->at(0);
  return true;
}
bool binary_plus_precision(const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  VERIFY_EQ(ip->size(), 2U);
  (*op)[0] = std::max(ip->at(0), ip->at(1)) + 1;
  return true;
}
bool binary_mul_precision(const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  VERIFY_EQ(ip->size(), 2U);
  (*op)[0] = ip->at(0) + ip->at(1);
  return true;
}
bool max_in_precision(const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  VERIFY_GT(ip->size(), 0U);
  int m = ip->at(0);
  for (int p : *ip) m = std::max(m, p);
  for (int& v : *op) v = m;
  return true;
}

// ElemwiseShape<n_in, n_out>, src/top/elemwise_op_common.h:26-76: every input and output shares
// one shape; incompatible inputs are a CHECK failure.
bool elemwise_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out, int n_in, int n_out) {
  if (n_in != -1) VERIFY_EQ(in->size(), (size_t)n_in) << " in operator " << a.name;
  if (n_out != -1) VERIFY_EQ(out->size(), (size_t)n_out) << " in operator " << a.name;
  Shape d;
  for (const auto& s : *in) {
    if (d.empty()) d = s;
    else CHECK(d == s) << "Incompatible attr in node " << a.name << ": expected " << shape_str(d) << ", got " << shape_str(s);
  }
  if (d.empty()) return false;
  for (auto& s : *out) s = d;
  return true;
}

// Conv2DInferShape, src/top/nn/convolution.cc:20-120
bool conv2d_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(a.s("layout"), "NCHW") << "Conv2D only supported layout: NCHW vs. " << a.s("layout");
  VERIFY_EQ(a.s("kernel_layout"), "OIHW") << "Conv2D only supported kernel layout: OIHW vs. " << a.s("kernel_layout");
  const std::string& ol = a.s("out_layout");
  VERIFY(ol == "__undef__" || ol == "NCHW") << "Conv2D only supported out layout: NCHW vs. " << ol;
  const bool use_bias = a.b("use_bias");
  if (use_bias) VERIFY_EQ(in->size(), 3U) << "Input:[data, weight, bias]";
  else VERIFY_EQ(in->size(), 2U) << "Input:[data, weight]";
  VERIFY_EQ(out->size(), 1U);
  Shape d = in->at(0);
  if (d.empty()) return false;
  VERIFY_EQ(d.size(), 4U) << "Input data should be 4D";
  const Shape &ks = a.t("kernel_size"), &pad = a.t("padding"), &st = a.t("strides"), &dil = a.t("dilation");
  VERIFY_EQ(ks.size(), 2U);
  VERIFY_EQ(pad.size(), 2U);
  verify_attr_range(pad[0], "Conv2D.padding[0]");
  verify_attr_range(pad[1], "Conv2D.padding[1]");
  VERIFY_EQ(st.size(), 2U) << "incorrect stride size: " << shape_str(st);
  verify_attr_range(st[0], "Conv2D.strides[0]", 1);
  verify_attr_range(st[1], "Conv2D.strides[1]", 1);
  VERIFY_EQ(dil.size(), 2U) << "incorrect dilate size: " << shape_str(dil);
  verify_attr_range(dil[0], "Conv2D.dilation[0]", 1);
  verify_attr_range(dil[1], "Conv2D.dilation[1]", 1);
  const int64_t groups = a.i("groups"), channels = a.i("channels");
  VERIFY(groups > 0 && d[1] % groups == 0 && channels % groups == 0)
      << "Conv2D only supported groups (1 or in_channels " << channels << ") vs. " << groups;
  Shape w = {channels, d[1] / groups, ks[0], ks[1]};
  // The reference only fills an unknown weight shape; a weight whose shape disagrees with the
  // attributes makes its kernels index out of bounds.  Here it is refused.
  if (!(in->at(1) == w) && deferred_refusal().empty())
    deferred_refusal() = "Conv2D weight shape " + shape_str(in->at(1)) + " does not match attributes " + shape_str(w);
  if (use_bias) {
    Shape bs = {channels};
    CHECK(in->at(2) == bs) << "Operator conv2d(name=" << a.name << ") expects bias's shape to be "
                           << shape_str(bs) << ", but got " << shape_str(in->at(2)) << ".";
  }
  const int64_t dky = 1 + (ks[0] - 1) * dil[0], dkx = 1 + (ks[1] - 1) * dil[1];
  Shape o = {d[0], channels, 0, 0};
  o[2] = (d[2] + pad[0] * 2 - dky) / st[0] + 1;
  o[3] = (d[3] + pad[1] * 2 - dkx) / st[1] + 1;
  (*out)[0] = o;
  if (o[2] && st[0] == 1) d[2] = o[2] + dky - 1 - 2 * pad[0];
  if (o[3] && st[1] == 1) d[3] = o[3] + dkx - 1 - 2 * pad[1];
  CHECK(in->at(0) == d) << "Operator conv2d(name=" << a.name << ") expects data's shape to be " << shape_str(d);
  VERIFY_LE(dky, d[2] + 2 * pad[0]) << "kernel size exceed input";
  VERIFY_LE(dkx, d[3] + 2 * pad[1]) << "kernel size exceed input";
  return true;
}

// Conv2DInferPrecision, src/top/nn/convolution.cc:147-175
bool conv2d_prec(const Attrs& a, const std::vector<Shape>& shapes, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  VERIFY_LE(ip->at(0), 8) << "Conv2D " << a.name << " input must be INT8 vs. INT" << ip->at(0);
  VERIFY_LE(ip->at(1), 8) << "Conv2D " << a.name << " weight must be INT8 vs. INT" << ip->at(1);
  const Shape& w = shapes.at(1);
  VERIFY_EQ(w.size(), 4U);
  const int64_t max_size = shape_size(w) / w[0];
  int oprec = ip->at(0) + ip->at(1) + reduce_sum_bits(max_size);
  if (a.b("use_bias")) oprec = std::max(oprec, ip->at(2)) + 1;
  (*op)[0] = oprec;
  return true;
}

// DenseInferShape, src/top/nn/nn.cc:46-77
bool dense_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  const bool use_bias = a.b("use_bias");
  if (use_bias) VERIFY_EQ(in->size(), 3U) << "Input:[data, weight, bias]";
  else VERIFY_EQ(in->size(), 2U) << "Input:[data, weight]";
  VERIFY_EQ((*in)[0].size(), 2U) << "dense require 2-D data";
  VERIFY_EQ((*in)[1].size(), 2U) << "dense require 2-D weight";
  VERIFY_EQ(out->size(), 1U);
  const int64_t units = a.i("units");
  Shape o = (*in)[0];
  const int64_t num_inputs = o.back();
  o.back() = units;
  (*out)[0] = o;
  Shape w = {units, num_inputs};
  CHECK((*in)[1] == w) << "Operator dense(name=" << a.name << ") expects weight's shape to be "
                       << shape_str(w) << ", but got " << shape_str((*in)[1]) << ".";
  if (use_bias) {
    Shape bs = {units};
    CHECK((*in)[2] == bs) << "Operator dense(name=" << a.name << ") expects bias's shape to be "
                          << shape_str(bs) << ", but got " << shape_str((*in)[2]) << ".";
  }
  return true;
}

// DenseInferPrecision, src/top/nn/nn.cc:21-44
bool dense_prec(const Attrs& a, const std::vector<Shape>& shapes, std::vector<int>* ip, std::vector<int>* op) {
  VERIFY_LE(ip->at(0), 8) << "Dense " << a.name << " input must be INT8 vs. INT" << ip->at(0);
  VERIFY_LE(ip->at(1), 8) << "Dense " << a.name << " weight must be INT8 vs. INT" << ip->at(1);
  int oprec = ip->at(0) + ip->at(1) + reduce_sum_bits(shapes.at(0)[1]);
  if (a.b("use_bias")) oprec = std::max(oprec, ip->at(2)) + 1;
  (*op)[0] = oprec;
  return true;
}

// Pool2DInferShape, src/top/nn/pooling.cc:20-100
bool max_pool_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& d = (*in)[0];
  if (d.empty()) return false;
  VERIFY_EQ(d.size(), 4U) << "Pool2D only support input = 4-D: NCHW";
  VERIFY_EQ(a.s("layout"), "NCHW") << "Pool2D only supported NCHW layout vs. " << a.s("layout");
  const Shape &pad = a.t("padding"), &ps = a.t("pool_size"), &st = a.t("strides");
  VERIFY(pad.size() == 1U || pad.size() == 2U) << "Pool2D only supported 1-D or 2-D padding vs. " << shape_str(pad);
  verify_attr_range(pad[0], "MaxPool2D.padding[0]");
  int64_t pad_h = pad[0] * 2, pad_w = pad[0] * 2;
  if (pad.size() == 2) {
    pad_w = pad[1] * 2;
    verify_attr_range(pad[1], "MaxPool2D.padding[1]");
  }
  VERIFY(ps.size() == 2);
  VERIFY(st.size() == 2);
  verify_attr_range(st[0], "MaxPool2D.strides[0]", 1);
  verify_attr_range(st[1], "MaxPool2D.strides[1]", 1);
  verify_attr_range(ps[0], "MaxPool2D.pool_size[0]", 0, d[2] + pad_h);
  verify_attr_range(ps[1], "MaxPool2D.pool_size[1]", 0, d[3] + pad_w);
  const int64_t tp0 = pad[0], tp1 = pad.size() == 2 ? pad[1] : pad[0];
  VERIFY(tp0 < ps[0]);
  VERIFY(tp1 < ps[1]);
  Shape o = d;
  if (!a.b("ceil_mode")) {
    o[2] = (d[2] + pad_h - ps[0]) / st[0] + 1;
    o[3] = (d[3] + pad_w - ps[1]) / st[1] + 1;
  } else {
    o[2] = (d[2] + pad_h - ps[0] + st[0] - 1) / st[0] + 1;
    int32_t min_o_h = (int32_t)((o[2] - 1) * st[0] - pad[0]);
    VERIFY(min_o_h < d[2]);
    o[3] = (d[3] + pad_w - ps[1] + st[1] - 1) / st[1] + 1;
    int32_t min_o_w = (int32_t)((o[3] - 1) * st[1] - tp1);
    VERIFY(min_o_w < d[3]);
  }
  (*out)[0] = o;
  return true;
}

// UpSamplingInferShape, src/top/nn/upsampling.cc:20-42
bool upsampling_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& d = (*in)[0];
  if (d.empty()) return false;
  VERIFY_EQ(d.size(), 4U) << "dimension should be 4D, Got: " << shape_str(d);
  VERIFY_EQ(a.s("method"), "NEAREST_NEIGHBOR") << "only accept method = NEAREST_NEIGHBOR ";
  verify_attr_range(a.i("scale"), "UpSampling.scale", 1);
  VERIFY_EQ(a.s("layout"), "NCHW") << "UpSampling only supported NCHW layout vs. " << a.s("layout");
  Shape o = d;
  o[2] *= a.i("scale");
  o[3] *= a.i("scale");
  (*out)[0] = o;
  return true;
}

// FlattenInferShape, src/top/tensor/transform.cc:169-182
bool flatten_shape(const Attrs&, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U) << "Input: [data]";
  VERIFY_EQ(out->size(), 1U);
  const Shape& d = (*in)[0];
  uint32_t target = 1;
  for (size_t i = 1; i < d.size(); ++i) target *= (uint32_t)d[i];
  (*out)[0] = Shape{d[0], (int64_t)target};
  return true;
}

// ConcatenateInferShape, src/top/tensor/transform.cc:217-258
bool concat_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY(!in->empty());
  const int ndim = (int)in->at(0).size();
  verify_attr_range(a.i("axis"), "concatenate.axis", -ndim, ndim - 1);
  const int axis = a.i("axis") >= 0 ? (int)a.i("axis") : ndim + (int)a.i("axis");
  for (const auto& s : *in) VERIFY_EQ((int)s.size(), ndim);
  Shape d;
  int64_t size = 0;
  for (const auto& s : *in) {
    Shape tmp = s;
    size += tmp[axis];
    tmp[axis] = 0;
    if (d.empty()) d = tmp;
    else VERIFY(d == tmp) << "concatenate inputs differ outside the axis";
  }
  d[axis] = size;
  (*out)[0] = d;
  return shape_size(d) != 0;
}

// ExpandDimsInferShape, src/top/tensor/transform.cc:355-378
bool expand_dims_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  const Shape& d = in->at(0);
  const int ndim = (int)d.size();
  verify_attr_range(a.i("axis"), "expand_dims.axis", -ndim - 1, ndim);
  verify_attr_range(a.i("num_newaxis"), "expand_dims.num_newaxis");
  const int axis = a.i("axis") < 0 ? ndim + (int)a.i("axis") + 1 : (int)a.i("axis");
  Shape o;
  for (int i = 0; i < axis; ++i) o.push_back(d[i]);
  for (int i = 0; i < a.i("num_newaxis"); ++i) o.push_back(1);
  for (int i = axis; i < ndim; ++i) o.push_back(d[i]);
  (*out)[0] = o;
  return true;
}

// ReshapeInferShape, src/top/tensor/transform.cc:401-481
bool reshape_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  const Shape& target = a.t("shape");
  VERIFY_GT(target.size(), 0U);
  VERIFY_EQ(in->size(), 1U) << "Input: [data]";
  VERIFY_EQ(out->size(), 1U);
  const Shape& d = (*in)[0];
  Shape o;
  size_t src = 0;
  int infer_idx = -1;
  for (size_t i = 0; i < target.size(); ++i) {
    int64_t sv = target[i];
    if (sv > 0) { o.push_back(sv); ++src; }
    else if (sv == 0) { VERIFY_LT(src, d.size()); o.push_back(d[src++]); }
    else if (sv == -1) {
      VERIFY_LT(infer_idx, 0) << "One and only one dim can be inferred";
      infer_idx = (int)i;
      o.push_back(1);
      ++src;
    } else if (sv == -2) {
      while (src < d.size()) o.push_back(d[src++]);
    } else if (sv == -3) {
      VERIFY_LT(src + 1, d.size());
      int64_t d1 = d[src++], d2 = d[src++];
      o.push_back(d1 * d2);
    } else if (sv == -4) {
      VERIFY_LT(i + 2, target.size());
      VERIFY_LT(src, d.size());
      int64_t d0 = d[src++];
      int d1 = (int)target[++i], d2 = (int)target[++i];
      VERIFY(d1 != -1 || d2 != -1) << "Split dims cannot both be -1.";
      if (d1 == -1) d1 = (int)(d0 / d2);
      if (d2 == -1) d2 = (int)(d0 / d1);
      VERIFY_EQ(d1 * d2, (int)d0) << "Split dims " << d1 << ", " << d2 << " do not divide original dim " << d0;
      o.push_back(d1);
      o.push_back(d2);
    }
  }
  if (infer_idx >= 0) {
    int new_size = 1;
    for (int64_t x : o) new_size *= (int)x;
    o[infer_idx] = shape_size(d) / new_size;
  }
  VERIFY_EQ(shape_size(o), shape_size(d)) << "Target shape size is different to source. Target: "
                                          << shape_str(o) << "\nSource: " << shape_str(d);
  (*out)[0] = o;
  return true;
}

// SqueezeShape, src/top/tensor/transform.cc:553-603
bool squeeze_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& s = (*in)[0];
  const int ndim = (int)s.size();
  const Shape& axis = a.t("axis");
  Shape o;
  if (axis.empty()) {
    for (int i = 0; i < ndim; ++i)
      if (s[i] != 1) o.push_back(s[i]);
  } else {
    std::set<int64_t> chk;
    for (int64_t ax : axis) {
      verify_attr_range(ax, "squeeze.axis", -ndim, ndim - 1);
      chk.insert(ax < 0 ? ax + ndim : ax);
    }
    for (int i = 0; i < ndim; ++i) {
      if (!chk.count(i)) o.push_back(s[i]);
      else VERIFY_EQ(s[i], 1) << "The squeezed axis must have shape 1!Want to squeeze " << i << ", which has shape" << s[i];
    }
  }
  if (o.empty()) o.push_back(1);
  VERIFY_EQ(shape_size(o), shape_size(s));
  (*out)[0] = o;
  return true;
}

// BinaryBroadcastShape, src/top/tensor/broadcast.cc:17-53
bool broadcast_shape(const Attrs&, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 2U);
  VERIFY_EQ(out->size(), 1U);
  const Shape &l = (*in)[0], &r = (*in)[1];
  if (l.empty() || r.empty()) return false;
  if (l == r) { (*out)[0] = l; return true; }
  Shape o(std::max(l.size(), r.size()));
  const size_t bl = o.size() - l.size(), br = o.size() - r.size();
  for (size_t i = 0; i < o.size(); ++i) {
    int64_t lv = 1, rv = 1;
    if (i >= bl) lv = l[i - bl];
    if (i >= br) rv = r[i - br];
    if (lv != rv) {
      VERIFY(lv == 1 || rv == 1) << "operands could not be broadcast together with shapes "
                                 << shape_str(l) << " " << shape_str(r) << ", l=" << lv << ", r=" << rv;
      o[i] = std::max(lv, rv);
    } else {
      o[i] = lv;
    }
  }
  (*out)[0] = o;
  return true;
}

// GetReduceAxes / ReduceShapeImpl, src/top/tensor/reduce.cc:18-84
Shape reduce_axes(int indim, const Shape& axis, bool exclude) {
  if (axis.empty()) {
    Shape r(indim);
    for (int i = 0; i < indim; ++i) r[i] = i;
    return r;
  }
  Shape in_axis = axis;
  for (auto& i : in_axis) {
    i = i < 0 ? i + indim : i;
    verify_attr_range(i, "reduce.axis", 0, indim - 1);
  }
  std::sort(in_axis.begin(), in_axis.end());
  for (size_t i = 0; i + 1 < in_axis.size(); ++i) VERIFY(in_axis[i] != in_axis[i + 1]);
  if (!exclude) return in_axis;
  Shape r;
  for (int i = 0, j = 0; i < indim; ++i) {
    if (j < (int)in_axis.size() && i == in_axis[j]) { ++j; continue; }
    r.push_back(i);
  }
  return r;
}

bool reduce_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& is = (*in)[0];
  if (is.empty()) return false;
  const int indim = (int)is.size();
  const bool keepdims = a.b("keepdims");
  Shape r = reduce_axes(indim, a.t("axis"), a.b("exclude"));
  Shape o;
  if (r.empty()) {
    o = is;
  } else if ((int)r.size() == indim) {
    o = Shape(keepdims ? indim : 1, 1);
  } else {
    if (keepdims) {
      o = is;
      for (int i = 0, j = 0; i < indim; ++i) {
        if (j >= (int)r.size() || i != r[j]) continue;
        o[i] = 1;
        ++j;
      }
    } else {
      for (int i = 0, j = 0; i < indim; ++i) {
        if (j < (int)r.size() && i == r[j]) { ++j; continue; }
        o.push_back(is[i]);
      }
    }
  }
  (*out)[0] = o;
  return true;
}

bool sum_prec(const Attrs& a, const std::vector<Shape>& shapes, std::vector<int>* ip, std::vector<int>* op) {
  // src/top/tensor/reduce.cc:143-156
  in_prec_check(a, *ip);
  const int64_t suml = shape_size(shapes.at(0)) / shape_size(shapes.at(1));
  (*op)[0] = ip->at(0) + reduce_sum_bits(suml);
  return true;
}

// NMSShape, src/top/nn/nms.cc:32-67
bool nms_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 2U) << "Inputs: [data, valid_count]";
  const Shape &d = in->at(0), &v = in->at(1);
  VERIFY_EQ(d.size(), 3U) << "Input data should be 3-D.";
  VERIFY_EQ(v.size(), 1U) << "Input valid count should be 1-D.";
  VERIFY_EQ(d[2], 6) << "Data input should have shape (batch_size, num_anchors, 6).";
  VERIFY_EQ(d[0], v[0]) << "batch_size mismatch.";
  VERIFY(a.i("coord_start") == 2);
  VERIFY(a.i("score_index") == 1);
  VERIFY(a.i("id_index") == 0);
  VERIFY(a.i("iou_threshold") > 0);
  VERIFY_EQ(a.b("return_indices"), false) << "NonMaximumSuppressionParam only supported return_indices false";
  VERIFY_EQ(a.b("invalid_to_bottom"), true) << "NonMaximumSuppressionParam only supported invalid_to_bottom true";
  (*out)[0] = d;
  return true;
}

// GetValidShape / GetValidInferPrecision, src/top/nn/nms.cc:119-172
bool gvc_shape(const Attrs&, std::vector<Shape>* in, std::vector<Shape>* out) {
  const Shape& s = in->at(0);
  CHECK_EQ(in->size(), 1U);
  CHECK_EQ(out->size(), 2U);
  VERIFY(s.size() == 3);
  VERIFY(s[2] < 32 && s[2] >= 2);
  (*out)[0] = Shape{s[0]};
  (*out)[1] = s;
  return true;
}
bool gvc_prec(const Attrs& a, const std::vector<Shape>& shapes, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  const Shape& s = shapes.at(0);
  (*op)[0] = number_precision(shape_size(s) / s[0]);
  (*op)[1] = ip->at(0);
  return true;
}

// RepeatShape, src/top/tensor/transform.cc:22-49
bool repeat_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& s = (*in)[0];
  const int ndim = (int)s.size();
  VERIFY_GT(a.i("repeats"), 0) << "operator " << a.name << " repeats:" << a.i("repeats") << " must greater than 0";
  verify_attr_range(a.i("axis"), "repeat.axis", -ndim, ndim - 1);
  const int pivot = a.i("axis") < 0 ? ndim + (int)a.i("axis") : (int)a.i("axis");
  Shape o = s;
  o[pivot] = s[pivot] * a.i("repeats");
  (*out)[0] = o;
  return true;
}

// TileShape, src/top/tensor/transform.cc:72-99
bool tile_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& s = (*in)[0];
  const Shape& reps = a.t("reps");
  const size_t sdim = s.size(), rdim = reps.size();
  VERIFY(rdim > 0) << "repetition array is not defined. data.ndim = " << sdim;
  for (int64_t r : reps) verify_attr_range(r, "tile.reps", 1);
  const size_t odim = std::max(sdim, rdim);
  Shape o(odim);
  for (size_t i = 0; i < odim; ++i) {
    const int64_t sv = i < sdim ? s[sdim - 1 - i] : 1;
    const int64_t rv = i < rdim ? reps[rdim - 1 - i] : 1;
    o[odim - 1 - i] = sv * rv;
  }
  (*out)[0] = o;
  return true;
}

// TransposeShape, src/top/tensor/transform.cc:635-666
bool transpose_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 1U);
  VERIFY_EQ(out->size(), 1U);
  const Shape& s = (*in)[0];
  const int ndim = (int)s.size();
  Shape axes = a.t("axes");
  Shape o(ndim);
  if (axes.empty()) {
    for (int i = 0; i < ndim; ++i) o[i] = s[ndim - 1 - i];
  } else {
    VERIFY_EQ(s.size(), axes.size());
    for (int i = 0; i < ndim; ++i) {
      int64_t ax = axes[i];
      verify_attr_range(ax, "transpose.axis", -ndim, ndim - 1);
      if (ax < 0) { ax += ndim; axes[i] = ax; }
      for (int j = 0; j < ndim; ++j)
        if (i != j) VERIFY(ax != axes[j]) << "repeated axis in transpose";
      o[i] = s[ax];
    }
  }
  (*out)[0] = o;
  return true;
}

// StridedSliceInferShape, src/top/tensor/transform.cc:755-799
bool strided_slice_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  const Shape& d = (*in)[0];
  const size_t nd = d.size();
  Shape b = a.t("begin"), e = a.t("end"), st = a.t("stride");
  for (size_t i = b.size(); i < nd; ++i) b.push_back(0);
  for (size_t i = e.size(); i < nd; ++i) e.push_back(d[i]);
  for (size_t i = st.size(); i < nd; ++i) st.push_back(1);
  Shape o = d;
  for (size_t i = 0; i < nd; ++i) {
    VERIFY(st[i] != 0);
    const int64_t lo = st[i] < 0 ? -1 : 0, hi = st[i] < 0 ? d[i] - 1 : d[i];
    int64_t bg = b[i] < 0 ? d[i] + b[i] : b[i];
    int64_t en = e[i] < 0 ? d[i] + e[i] : e[i];
    bg = std::min(std::max(bg, lo), hi);
    en = std::min(std::max(en, lo), hi);
    const int interval = (int)std::llabs(en - bg);
    const int size = (int)((interval + std::llabs(st[i]) - 1) / std::llabs(st[i]));
    VERIFY(st[i] < 0 ? (en < bg) : (bg < en))
        << ": Input [Begin=" << b[i] << ", End=" << e[i] << "] is invalid for axis=" << i;
    o[i] = size;
  }
  (*out)[0] = o;
  return true;
}

// TakeInferShape, src/top/tensor/transform.cc:840-875
bool take_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 2U);
  VERIFY_EQ(out->size(), 1U);
  const Shape &d = (*in)[0], &idx = (*in)[1];
  const int ndim = (int)d.size();
  Shape o;
  if (!a.has.at("axis")) {
    o = idx;
  } else {
    int axis = (int)a.i("axis");
    verify_attr_range(axis, "take.axis", -ndim, ndim - 1);
    if (axis < 0) axis += ndim;
    for (int i = 0; i < ndim; ++i) {
      if (i == axis) o.insert(o.end(), idx.begin(), idx.end());
      else o.push_back(d[i]);
    }
  }
  (*out)[0] = o;
  return shape_size(d) != 0;
}

// LUTInferShape / LUTInferPrecision, src/top/tensor/transform.cc:945-996
bool lut_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 2U);
  VERIFY_EQ(out->size(), 1U);
  VERIFY_EQ(shape_size((*in)[1]), a.i("in_dim"));
  (*out)[0] = (*in)[0];
  return true;
}
bool lut_prec(const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
  in_prec_check(a, *ip);
  (*op)[0] = ip->at(1);
  return true;
}

// SliceLikeShape, src/top/tensor/transform.cc:1017-1054
bool slice_like_shape(const Attrs& a, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 2U);
  VERIFY_EQ(out->size(), 1U);
  const Shape &src = (*in)[0], &target = (*in)[1];
  const Shape& axis = a.t("axis");
  VERIFY(src.size() == target.size() || !axis.empty())
      << "input X and shape_like must be of the same shape if no axis is given";
  Shape end = src;
  if (axis.empty()) {
    for (size_t i = 0; i < src.size(); ++i) {
      if (i < target.size()) {
        end[i] = target[i];
        VERIFY_LE(end[i], src[i]) << "End index of axis " << i << " exceeds input shape: " << end[i] << " vs " << src[i];
      }
    }
  } else {
    for (int64_t i : axis) {
      if (i < 0) i += (int64_t)src.size();
      verify_attr_range(i, "slice_like.axis", 0, (int64_t)std::min(target.size(), src.size()) - 1);
      end[i] = target[i];
      VERIFY_LE(end[i], src[i]) << "End index of axis " << i << " exceeds input shape: " << end[i] << " vs " << src[i];
    }
  }
  (*out)[0] = end;
  return true;
}

// WhereShape, src/top/tensor/transform.cc:1059-1079
bool where_shape(const Attrs&, std::vector<Shape>* in, std::vector<Shape>* out) {
  VERIFY_EQ(in->size(), 3U);
  VERIFY_EQ(out->size(), 1U);
  const Shape &c = (*in)[0], &x = (*in)[1], &y = (*in)[2];
  VERIFY(x == y) << "x and y must have the same shape: " << shape_str(x) << " vs " << shape_str(y);
  if (c != x) {
    VERIFY_EQ(c.size(), 1U) << "Shape of condition " << shape_str(c)
                            << " must be either equal to x or has dimension of 1.";
    VERIFY_EQ(c[0], x[0]) << "If dim of condition is 1, " << shape_str(c)
                          << " must be the same as the first dimension of input shape.";
  }
  (*out)[0] = x;
  return true;
}

#define REQ(n, k) {n, k, true, "", false, 0}
#define REQ_LB(n, k, lb) {n, k, true, "", true, lb}
#define OPT(n, k, d) {n, k, false, d, false, 0}
#define OPT_LB(n, k, d, lb) {n, k, false, d, true, lb}

std::vector<OpDef> build_table() {
  std::vector<OpDef> t;
  auto unary = [&](const char* name, InferPrecFn prec) {
    t.push_back({name, 1, 1, false, {}, [](const Attrs& a, std::vector<Shape>* i, std::vector<Shape>* o) {
                   return elemwise_shape(a, i, o, 1, 1); }, prec, false});
  };
  auto binary = [&](const char* name, InferPrecFn prec) {
    t.push_back({name, 2, 1, false, {}, [](const Attrs& a, std::vector<Shape>* i, std::vector<Shape>* o) {
                   return elemwise_shape(a, i, o, 2, 1); }, prec, false});
  };
  auto unary_attr = [&](const char* name, std::vector<FieldSpec> f, InferPrecFn prec) {
    t.push_back({name, 1, 1, true, f, [](const Attrs& a, std::vector<Shape>* i, std::vector<Shape>* o) {
                   return elemwise_shape(a, i, o, 1, 1); }, prec, false});
  };
  auto bcast = [&](const char* name, InferPrecFn prec) {
    t.push_back({name, 2, 1, false, {}, broadcast_shape, prec, false});
  };

  t.push_back({"conv2d", kUseBias, 1, true,
               {REQ("channels", F_INT), REQ("kernel_size", F_TUPLE), OPT("strides", F_TUPLE, "(1, 1)"),
                OPT("padding", F_TUPLE, "(0, 0)"), OPT("dilation", F_TUPLE, "(1, 1)"), OPT("groups", F_INT, "1"),
                OPT("layout", F_STR, "NCHW"), OPT("out_layout", F_STR, "__undef__"),
                OPT("kernel_layout", F_STR, "OIHW"), OPT("out_dtype", F_DTYPE, "same"), OPT("use_bias", F_BOOL, "1")},
               conv2d_shape, conv2d_prec, false});
  t.push_back({"dense", kUseBias, 1, true, {REQ_LB("units", F_INT, 1), OPT("use_bias", F_BOOL, "1")},
               dense_shape, dense_prec, false});
  unary("relu", same_precision);             // src/top/nn/nn.cc:109-118
  unary("abs", same_precision);              // src/top/tensor/elemwise.cc:18-23
  unary("negative", same_precision);         // src/top/tensor/elemwise.cc:73-78
  unary("cvm_precision",                     // src/top/tensor/elemwise.cc:45-55, MaxPrecision<6>
        [](const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
          in_prec_check(a, *ip);
          for (int& v : *op) v = 6;
          return true;
        });
  binary("elemwise_add", binary_plus_precision);  // src/top/tensor/elemwise.cc:58-63
  binary("elemwise_sub", binary_plus_precision);  // src/top/tensor/elemwise.cc:65-70
  unary_attr("clip", {REQ("a_min", F_INT), REQ("a_max", F_INT)},  // src/top/tensor/elemwise.cc:82-115
             [](const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
               in_prec_check(a, *ip);
               const int64_t r = ((int64_t)1 << 31) - 1;
               verify_attr_range(a.i("a_max"), "clip.a_max", -r, r);
               verify_attr_range(a.i("a_min"), "clip.a_min", -r, r);
               VERIFY(a.i("a_min") < a.i("a_max")) << "clip a_min must less than a_max";
               int64_t range = std::max(std::abs(a.i("a_max")), std::abs(a.i("a_min")));
               (*op)[0] = number_precision(range);
               return true;
             });
  unary_attr("cvm_clip", {REQ("precision", F_INT), OPT("is_sign", F_BOOL, "1")},  // :120-160
             [](const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
               in_prec_check(a, *ip);
               verify_attr_range(a.i("precision"), "cvm_clip.precision", 1, 32);
               (*op)[0] = (int)a.i("precision");
               return true;
             });
  unary_attr("cvm_left_shift", {REQ("precision", F_INT), OPT("is_sign", F_BOOL, "1"), REQ("shift_bit", F_INT)},  // :164-196
             [](const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
               in_prec_check(a, *ip);
               verify_attr_range(a.i("precision"), "cvm_left_shift.precision", 1, 32);
               verify_attr_range(a.i("shift_bit"), "cvm_left_shift.shift_bit", 1, 32);
               if (ip->at(0) + a.i("shift_bit") > 32) return false;
               (*op)[0] = (int)a.i("precision");
               return true;
             });
  unary_attr("cvm_right_shift", {REQ("precision", F_INT), OPT("is_sign", F_BOOL, "1"), REQ("shift_bit", F_INT)},  // :199-235
             [](const Attrs& a, const std::vector<Shape>&, std::vector<int>* ip, std::vector<int>* op) {
               in_prec_check(a, *ip);
               verify_attr_range(a.i("precision"), "cvm_right_shift.precision", 1, 32);
               verify_attr_range(a.i("shift_bit"), "cvm_right_shift.shift_bit", 1, 32);
               (*op)[0] = (int)a.i("precision");
               return true;
             });
  t.push_back({"max_pool2d", 1, 1, true,
               {REQ("pool_size", F_TUPLE), OPT("strides", F_TUPLE, "(1, 1)"), OPT("padding", F_TUPLE, "(0, 0)"),
                OPT("layout", F_STR, "NCHW"), OPT("ceil_mode", F_BOOL, "0")},
               max_pool_shape, same_precision, false});
  t.push_back({"upsampling", 1, 1, true,
               {REQ("scale", F_INT), OPT("layout", F_STR, "NCHW"), OPT("method", F_STR, "NEAREST_NEIGHBOR")},
               upsampling_shape, same_precision, false});
  t.push_back({"flatten", 1, 1, false, {}, flatten_shape, same_precision, false});
  t.push_back({"concatenate", kVarg, 1, true, {OPT("axis", F_INT, "1")}, concat_shape, max_in_precision, false});
  t.push_back({"expand_dims", 1, 1, true, {REQ("axis", F_INT), OPT_LB("num_newaxis", F_INT, "1", 1)},
               expand_dims_shape, same_precision, false});
  t.push_back({"reshape", 1, 1, true, {REQ("shape", F_TUPLE)}, reshape_shape, same_precision, false});
  t.push_back({"squeeze", 1, 1, true, {OPT("axis", F_TUPLE, "()")}, squeeze_shape, same_precision, false});
  std::vector<FieldSpec> red = {OPT("axis", F_TUPLE, "()"), OPT("keepdims", F_BOOL, "0"),
                                OPT("exclude", F_BOOL, "0"), OPT("dtype", F_DTYPE, "int32")};
  t.push_back({"sum", 1, 1, true, red, reduce_shape, sum_prec, true});
  t.push_back({"max", 1, 1, true, red, reduce_shape, same_precision, true});
  bcast("broadcast_add", binary_plus_precision);   // src/top/tensor/broadcast.cc:143-160
  bcast("broadcast_sub", binary_plus_precision);   // :162-179
  bcast("broadcast_mul", binary_mul_precision);    // :181-197
  bcast("broadcast_max", max_in_precision);        // :218-234
  bcast("broadcast_div", same_precision);          // :236-252
  bcast("broadcast_greater", same_precision);      // :254-269
  t.push_back({"repeat", 1, 1, true, {REQ("repeats", F_INT), OPT("axis", F_INT, "0")}, repeat_shape, same_precision, false});
  t.push_back({"tile", 1, 1, true, {OPT("reps", F_TUPLE, "(0,)")}, tile_shape, same_precision, false});
  t.push_back({"transpose", 1, 1, true, {OPT("axes", F_TUPLE, "()")}, transpose_shape, same_precision, false});
  t.push_back({"strided_slice", 1, 1, true,
               {OPT("begin", F_TUPLE, "(0,)"), OPT("end", F_TUPLE, "(1,)"), OPT("stride", F_TUPLE, "()")},
               strided_slice_shape, same_precision, false});
  t.push_back({"take", 2, 1, true, {{"axis", F_OPT_INT, false, "None", false, 0}}, take_shape, same_precision, false});
  t.push_back({"cvm_lut", 2, 1, true, {REQ("in_dim", F_INT)}, lut_shape, lut_prec, false});
  t.push_back({"slice_like", 2, 1, true, {OPT("axis", F_TUPLE, "()")}, slice_like_shape, same_precision, false});
  t.push_back({"where", 3, 1, false, {}, where_shape, same_precision, false});  // SamePrecision: follows the condition
  t.push_back({"get_valid_counts", 1, 2, true, {OPT("score_threshold", F_INT, "0")}, gvc_shape, gvc_prec, false});
  t.push_back({"non_max_suppression", 2, 1, true,
               {OPT("max_output_size", F_INT, "-1"), OPT("iou_threshold", F_INT, "50"),
                OPT("force_suppress", F_BOOL, "0"), OPT("top_k", F_INT, "-1"), OPT("coord_start", F_INT, "2"),
                OPT("score_index", F_INT, "1"), OPT("id_index", F_INT, "0"), OPT("return_indices", F_BOOL, "0"),
                OPT("invalid_to_bottom", F_BOOL, "1")},
               nms_shape, same_precision, false});  // registered with SamePrecision, src/top/nn/nms.cc:106
  return t;
}

}  // namespace

const OpDef* find_op(const std::string& name) {
  static const std::vector<OpDef> table = build_table();
  for (const auto& o : table)
    if (o.name == name) return &o;
  FATAL() << "Operator " << name << " is not registered";
  return nullptr;
}

}  // namespace cvm
