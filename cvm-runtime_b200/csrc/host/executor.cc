// Lowering of a Graph into kernel launches, and the per-inference replay.
#include "executor.h"
#include <cuda.h>
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <map>

namespace cvm {

#define CUDA_OK(expr)                                                                      \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    CHECK(e__ == cudaSuccess) << "CUDA: " << #expr << ": " << cudaGetErrorString(e__);     \
  } while (0)

#define KERNEL_OK(expr)                                                                    \
  do {                                                                                     \
    int rc__ = (expr);                                                                     \
    CHECK(rc__ == CVMK_OK) << "kernel launcher failed (" << rc__ << "): " << cvmk_last_error(); \
  } while (0)

namespace {

bool nhwc_equiv(const Shape& s) {  // NCHW and NHWC orders coincide
  return s.size() == 4 && ((s[2] == 1 && s[3] == 1) || s[1] == 1);
}
bool wants_nhwc(const Shape& s) { return s.size() == 4 && !nhwc_equiv(s); }

// Element stride of every logical dimension in the buffer's physical layout.
std::vector<int64_t> phys_strides(const Shape& s, bool nhwc) {
  std::vector<int64_t> st(s.size(), 1);
  if (nhwc) {
    st[1] = 1;
    st[3] = s[1];
    st[2] = s[3] * s[1];
    st[0] = s[2] * s[3] * s[1];
  } else {
    for (int i = (int)s.size() - 2; i >= 0; --i) st[i] = st[i + 1] * s[i + 1];
  }
  return st;
}
// Logical dimensions in physical order, outermost first.
std::vector<int> phys_order(const Shape& s, bool nhwc) {
  std::vector<int> o(s.size());
  for (size_t i = 0; i < s.size(); ++i) o[i] = (int)i;
  if (nhwc) o = {0, 2, 3, 1};
  return o;
}

void plan_deleter(void* p) { free(p); }

}  // namespace

void* Executor::dalloc(size_t bytes) {
  void* p = nullptr;
  const size_t sz = std::max<size_t>((bytes + 255) / 256 * 256, 256);
  CUDA_OK(cudaMalloc(&p, sz));
  allocs_.push_back(p);
  device_bytes_ += sz;
  return p;
}

// ---- CUDA virtual memory management, through the driver entry points -------------------------
namespace {
struct Vmm {
  CUresult (*get_granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
};
const Vmm& vmm() {
  static Vmm v = [] {
    Vmm t;
    auto get = [](const char* name) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fn = nullptr;
      return fn;
    };
    t.get_granularity = reinterpret_cast<decltype(t.get_granularity)>(get("cuMemGetAllocationGranularity"));
    t.reserve = reinterpret_cast<decltype(t.reserve)>(get("cuMemAddressReserve"));
    t.address_free = reinterpret_cast<decltype(t.address_free)>(get("cuMemAddressFree"));
    t.create = reinterpret_cast<decltype(t.create)>(get("cuMemCreate"));
    t.release = reinterpret_cast<decltype(t.release)>(get("cuMemRelease"));
    t.map = reinterpret_cast<decltype(t.map)>(get("cuMemMap"));
    t.unmap = reinterpret_cast<decltype(t.unmap)>(get("cuMemUnmap"));
    t.set_access = reinterpret_cast<decltype(t.set_access)>(get("cuMemSetAccess"));
    t.ok = t.get_granularity && t.reserve && t.address_free && t.create && t.release && t.map && t.unmap && t.set_access;
    cudaGetLastError();
    return t;
  }();
  return v;
}
CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}
}  // namespace

void* Executor::dalloc_activation(size_t bytes, uint32_t root) {
  // small buffers are not worth a mapping of their own (the granularity is 2 MiB)
  if (!vmm_ || bytes < (size_t)1 << 20) return dalloc(bytes);
  ActBuf a;
  a.bytes = std::max<size_t>(bytes, 256);
  a.va_size = (a.bytes + vmm_gran_ - 1) / vmm_gran_ * vmm_gran_;
  a.root = root;
  CUdeviceptr va = 0;
  const CUresult r = vmm().reserve(&va, a.va_size, vmm_gran_, 0, 0);
  CHECK(r == CUDA_SUCCESS) << "cuMemAddressReserve(" << a.va_size << ") failed (" << (int)r << ")";
  a.va = reinterpret_cast<void*>(va);
  act_.push_back(a);
  return a.va;
}

// Backs the activation buffers with physical memory in chunks of the allocation granularity (2 MiB):
// walking the buffers in the order of their first write, a buffer takes any chunks that are free by
// then (most recently freed first: they are the likeliest to be still in L2) and new ones for the
// rest; its chunks are free again after its last read.  Chunks need not be contiguous -- the
// virtual range of a buffer is -- so nothing is lost to fragmentation.
void Executor::PlanForPrefix(size_t prefix) {
  if (!vmm_ || act_.empty()) return;
  if (!phys_.empty()) {
    for (auto& a : act_)
      if (a.block >= 0) { vmm().unmap(reinterpret_cast<CUdeviceptr>(a.va), a.va_size); a.block = -1; }
    for (auto& b : phys_) {
      vmm().release((CUmemGenericAllocationHandle)b.handle);
      device_bytes_ -= b.size;
    }
    phys_.clear();
  }
  const int p = prefix > 0 ? step_pos_[prefix - 1] : -2;
  for (auto& a : act_) {
    a.first = a.first0;
    a.last = a.last0;
    if (a.first <= p) { a.first = -1; a.last = std::max(a.last, p); }
  }
  MapActivations();
}

void Executor::MapActivations() {
  if (!vmm_ || act_.empty()) return;
  const CUmemAllocationProp prop = device_prop(device_);
  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location = prop.location;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  std::vector<size_t> order(act_.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](size_t x, size_t y) { return act_[x].first < act_[y].first; });
  for (size_t i : order) {
    ActBuf& a = act_[i];
    const size_t need = a.va_size / vmm_gran_;
    std::vector<int> cand;
    for (size_t c = 0; c < phys_.size(); ++c)
      if (phys_[c].free_at <= a.first) cand.push_back((int)c);
    std::stable_sort(cand.begin(), cand.end(), [&](int x, int y) { return phys_[x].free_at > phys_[y].free_at; });
    std::vector<int> mine(cand.begin(), cand.begin() + std::min(cand.size(), need));
    while (mine.size() < need) {
      PhysBlock nb;
      CUmemGenericAllocationHandle h = 0;
      const CUresult r = vmm().create(&h, vmm_gran_, &prop, 0);
      CHECK(r == CUDA_SUCCESS) << "cuMemCreate failed (" << (int)r << ") after " << device_bytes_ << " bytes";
      nb.handle = (unsigned long long)h;
      nb.size = vmm_gran_;
      phys_.push_back(nb);
      device_bytes_ += vmm_gran_;
      mine.push_back((int)phys_.size() - 1);
    }
    const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(a.va);
    for (size_t k = 0; k < need; ++k) {
      phys_[mine[k]].free_at = a.last + 1;
      const CUresult r = vmm().map(va + k * vmm_gran_, vmm_gran_, 0, (CUmemGenericAllocationHandle)phys_[mine[k]].handle, 0);
      CHECK(r == CUDA_SUCCESS) << "cuMemMap failed (" << (int)r << ")";
    }
    const CUresult r = vmm().set_access(va, a.va_size, &access, 1);
    CHECK(r == CUDA_SUCCESS) << "cuMemSetAccess failed (" << (int)r << ")";
    a.block = mine.empty() ? -1 : mine[0];
  }
}

struct Lowering {
  Executor& ex;
  const Graph& g;
  std::vector<DevBuf> buf;
  std::vector<int> uses;
  std::vector<char> is_head, safe8, absorbed;
  uint32_t data_eid = 0;
  uint32_t cur_root = UINT32_MAX;   // node being lowered: tags the activation buffers it allocates
  std::vector<uint32_t> root_of;    // node -> root of the fused group it runs in
  // activation memory: planned when a node is being lowered, persistent otherwise (heads, staging)
  void* act_alloc(size_t bytes) { return cur_root == UINT32_MAX ? ex.dalloc(bytes) : ex.dalloc_activation(bytes, cur_root); }
  DevBuf raw_in;          // the input exactly as the C-ABI delivers it (row-major int8 / int32)
  int32_t data_range = 127;

  Lowering(Executor& e, const Graph& gr) : ex(e), g(gr) {}

  void add_step(const std::string& label, std::function<int(cudaStream_t)> fn) {
    ex.steps_.push_back({label, std::move(fn), {}});
  }
  // Batch chunks for upload / compute overlap: four (CVM_B200_UPLOAD_CHUNKS) when the batch
  // divides, else none.
  static int upload_chunks() {
    static const int k = [] {
      const char* e = dev_env("CVM_B200_UPLOAD_CHUNKS");
      const int v = e ? atoi(e) : 4;
      return v >= 2 && v <= 16 ? v : 4;
    }();
    return k;
  }
  static int batch_chunks(int64_t n) {
    const int k = upload_chunks();
    return (n % k == 0 && n >= 2 * k && !dev_env("CVM_B200_NO_UPLOAD_OVERLAP")) ? k : 1;
  }

  // ------------------------------------------------------------------ analysis
  void analyse() {
    const uint32_t ne = g.num_entries;
    buf.assign(ne, DevBuf());
    uses.assign(ne, 0);
    is_head.assign(ne, 0);
    safe8.assign(ne, 0);
    absorbed.assign(g.nodes.size(), 0);
    for (const auto& n : g.nodes)
      for (const auto& e : n.inputs) uses[g.entry_id(e)]++;
    for (const auto& e : g.outputs) is_head[g.entry_id(e)] = 1;
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid) {
      const Node& n = g.nodes[nid];
      const uint32_t e0 = g.entry_id(nid, 0);
      auto in_safe = [&](size_t i) { return (bool)safe8[g.entry_id(n.inputs[i])]; };
      if (n.is_variable()) { safe8[e0] = g.precision[e0] <= 8; continue; }
      const std::string& op = n.op->name;
      bool s = false;
      if (op == "cvm_clip" || op == "cvm_left_shift") s = n.attrs.i("precision") <= 8;
      else if (op == "clip") s = n.attrs.i("a_min") >= -127 && n.attrs.i("a_max") <= 127;
      else if (op == "cvm_right_shift") {
        const int64_t p = n.attrs.i("precision"), b = n.attrs.i("shift_bit");
        s = p == 1 || b >= 31 || (p <= 8 && p + b < 32);
      } else if (op == "relu" || op == "max_pool2d" || op == "upsampling" || op == "flatten" ||
                 op == "reshape" || op == "squeeze" || op == "expand_dims" || op == "abs" ||
                 op == "negative" || op == "max") s = in_safe(0);
      else if (op == "concatenate" || op == "broadcast_max") {
        s = true;
        for (size_t i = 0; i < n.inputs.size(); ++i) s = s && in_safe(i);
      } else if (op == "transpose" || op == "strided_slice" || op == "slice_like" || op == "repeat" ||
                 op == "tile" || op == "take") s = in_safe(0);
      else if (op == "cvm_lut") s = in_safe(1);
      else if (op == "where") s = in_safe(1) && in_safe(2);
      else if (op == "cvm_precision" || op == "broadcast_greater") s = true;
      safe8[e0] = s;
    }
    for (uint32_t e = 0; e < ne; ++e) {
      buf[e].shape = g.shape[e];
      buf[e].dtype = safe8[e] ? CVMK_I8 : CVMK_I32;
      buf[e].nhwc = wants_nhwc(g.shape[e]);
    }
    // transpose(0, 2, 3, 1) of a tensor stored channels-last: the row-major bytes of the result ARE
    // the input's bytes.  The result is therefore kept row-major (not channels-last again, which
    // would shuffle it once here and once more at the reshape that usually follows: the detection
    // heads of SSD do this twelve times per step) and the node becomes an alias.
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid)
      if (transpose_is_identity(nid)) buf[g.entry_id(nid, 0)].nhwc = false;
  }

  // true for transpose nodes with axes (0, 2, 3, 1) over a 4-D input that is stored channels-last
  bool transpose_is_identity(uint32_t nid) {
    const Node& n = g.nodes[nid];
    if (n.is_variable() || n.op->name != "transpose" || n.inputs.size() != 1) return false;
    const uint32_t ei = g.entry_id(n.inputs[0]);
    if (g.shape[ei].size() != 4 || !buf[ei].nhwc || g.params.count(ei)) return false;
    const Shape axes = n.attrs.t("axes");
    if (!(axes.size() == 4 && axes[0] == 0 && axes[1] == 2 && axes[2] == 3 && axes[3] == 1)) return false;
    // only when every reader takes the tensor by its layout flag: the reshape-like operators (and
    // the output copy of a graph head); convolutions and pooling expect channels-last operands
    const uint32_t eo = g.entry_id(nid, 0);
    for (uint32_t m = nid + 1; m < g.nodes.size(); ++m) {
      const Node& c = g.nodes[m];
      if (c.is_variable()) continue;
      for (const auto& e : c.inputs) {
        if (g.entry_id(e) != eo) continue;
        const std::string& op = c.op->name;
        if (op != "flatten" && op != "reshape" && op != "squeeze" && op != "expand_dims") return false;
      }
    }
    return true;
  }

  // ------------------------------------------------------------------ buffers
  DevBuf& materialize(uint32_t eid) {
    DevBuf& b = buf[eid];
    if (b.ptr) return b;
    auto it = g.params.find(eid);
    b.ptr = it != g.params.end() ? ex.dalloc(b.bytes()) : act_alloc(b.bytes());
    if (it != g.params.end()) {
      // parameter: convert on the host into the entry's dtype and layout, upload once
      const HostTensor& t = it->second;
      const int64_t n = shape_size(b.shape);
      std::vector<int32_t> phys(n);
      if (b.nhwc) {
        const int64_t C = b.shape[1], H = b.shape[2], W = b.shape[3];
        for (int64_t i = 0; i < n; ++i) {
          const int64_t w = i % W, h = (i / W) % H, c = (i / (W * H)) % C, nn = i / (W * H * C);
          phys[((nn * H + h) * W + w) * C + c] = t.data[i];
        }
      } else {
        phys = t.data;
      }
      if (b.dtype == CVMK_I8) {
        std::vector<int8_t> p8(n);
        for (int64_t i = 0; i < n; ++i) p8[i] = (int8_t)phys[i];
        CUDA_OK(cudaMemcpy(b.ptr, p8.data(), n, cudaMemcpyHostToDevice));
      } else {
        CUDA_OK(cudaMemcpy(b.ptr, phys.data(), n * 4, cudaMemcpyHostToDevice));
      }
    }
    return b;
  }

  // Same logical tensor copied between two buffers that may differ in layout and dtype.
  void emit_convert(const DevBuf& src, const DevBuf& dst, const std::string& label,
                    const cvmk_epilogue* ep = nullptr) {
    if (src.nhwc == dst.nhwc && src.shape == dst.shape) {
      // same element order on both sides: the vectorised contiguous kernel does it
      cvmk_epilogue e;
      memset(&e, 0, sizeof(e));
      if (ep) e = *ep;
      const DevBuf a = src, b = dst;
      const int64_t cnt = shape_size(dst.shape);
      add_step(label, [a, b, e, cnt](cudaStream_t s_) {
        return cvmk_elemwise(a.ptr, a.dtype, b.ptr, b.dtype, cnt, &e, s_);
      });
      return;
    }
    // NCHW <-> NHWC of one element type: a batched matrix transpose through shared memory
    if (src.nhwc != dst.nhwc && src.shape == dst.shape && src.shape.size() == 4 && src.dtype == dst.dtype &&
        (!ep || ep->n == 0 || (ep->n == 1 && ep->s[0].op == CVMK_EP_CLIP)) && !dev_env("CVM_B200_NO_TILED_TRANSPOSE")) {
      const Shape& sh = src.shape;
      const int64_t batch = sh[0];
      const int64_t c = sh[1], hw = sh[2] * sh[3];
      const int rows = (int)(src.nhwc ? hw : c), cols = (int)(src.nhwc ? c : hw);
      const int clamp = ep && ep->n == 1;
      const int lo = clamp ? ep->s[0].a : 0, hi = clamp ? ep->s[0].b : 0;
      const DevBuf a = src, b = dst;
      add_step(label, [a, b, batch, rows, cols, clamp, lo, hi](cudaStream_t s_) {
        return cvmk_transpose_batched(a.ptr, b.ptr, a.dtype, batch, rows, cols, clamp, lo, hi, s_);
      });
      return;
    }
    cvmk_strided_desc d;
    memset(&d, 0, sizeof(d));
    d.op = CVMK_OP_COPY;
    const Shape& s = dst.shape;
    const auto order = phys_order(s, dst.nhwc);
    const auto ss = phys_strides(src.shape, src.nhwc), ds = phys_strides(s, dst.nhwc);
    d.ndim = (int)s.size();
    for (int k = 0; k < d.ndim; ++k) {
      d.extent[k] = s[order[k]];
      d.a_stride[k] = ss[order[k]];
      d.y_stride[k] = ds[order[k]];
    }
    d.a = src.ptr; d.a_dtype = src.dtype;
    d.y = dst.ptr; d.y_dtype = dst.dtype;
    if (ep) d.ep = *ep;
    add_step(label, [d](cudaStream_t s_) { return cvmk_strided(&d, s_); });
  }

  // A row-major view of an entry; converts into a temporary when the entry is channels-last.
  DevBuf canon_view(uint32_t eid, const std::string& label) {
    DevBuf& b = materialize(eid);
    if (!b.nhwc) return b;
    DevBuf t = b;
    t.nhwc = false;
    t.ptr = act_alloc(t.bytes());
    emit_convert(b, t, label + ":to_rowmajor");
    return t;
  }
  // int32 row-major view (get_valid_counts / nms operands).
  DevBuf canon_i32_view(uint32_t eid, const std::string& label) {
    DevBuf& b = materialize(eid);
    if (!b.nhwc && b.dtype == CVMK_I32) return b;
    DevBuf t = b;
    t.nhwc = false;
    t.dtype = CVMK_I32;
    t.ptr = act_alloc(t.bytes());
    emit_convert(b, t, label + ":to_i32");
    return t;
  }
  // int8 view in the entry's own layout; narrows like static_cast<int8_t> when stored as int32.
  DevBuf i8_view(uint32_t eid, const std::string& label) {
    DevBuf& b = materialize(eid);
    if (b.dtype == CVMK_I8) return b;
    DevBuf t = b;
    t.dtype = CVMK_I8;
    t.ptr = act_alloc(t.bytes());
    const DevBuf src = b;
    const int64_t n = shape_size(b.shape);
    add_step(label + ":narrow", [src, t, n](cudaStream_t s) {
      return cvmk_elemwise(src.ptr, src.dtype, t.ptr, t.dtype, n, nullptr, s);
    });
    return t;
  }

  // ------------------------------------------------------------------ chains
  struct Chain {
    cvmk_epilogue ep;
    uint32_t tail_eid;
    uint32_t tail_nid;
  };

  bool scalar_param(uint32_t eid, int32_t* v) const {
    auto it = g.params.find(eid);
    if (it == g.params.end() || it->second.data.size() != 1) return false;
    *v = it->second.data[0];
    return true;
  }

  // Translate node `nid`, consuming entry `cur`, into one chain step.  False if not expressible.
  bool node_as_step(uint32_t nid, uint32_t cur, cvmk_ep_step* st) {
    const Node& n = g.nodes[nid];
    const std::string& op = n.op->name;
    memset(st, 0, sizeof(*st));
    auto alpha = [&](int64_t p) { return (int32_t)((((int64_t)1) << (p - 1)) - 1); };
    if (op == "relu") st->op = CVMK_EP_RELU;
    else if (op == "abs") st->op = CVMK_EP_ABS;
    else if (op == "negative") st->op = CVMK_EP_NEG;
    else if (op == "cvm_precision") st->op = CVMK_EP_PRECISION;
    else if (op == "clip") { st->op = CVMK_EP_CLIP; st->a = (int32_t)n.attrs.i("a_min"); st->b = (int32_t)n.attrs.i("a_max"); }
    else if (op == "cvm_clip") { st->op = CVMK_EP_CLIP; st->b = alpha(n.attrs.i("precision")); st->a = -st->b; }
    else if (op == "cvm_right_shift") { st->op = CVMK_EP_RSHIFT; st->a = (int32_t)n.attrs.i("shift_bit"); st->b = (int32_t)n.attrs.i("precision"); }
    else if (op == "cvm_left_shift") { st->op = CVMK_EP_LSHIFT; st->a = (int32_t)n.attrs.i("shift_bit"); st->b = (int32_t)n.attrs.i("precision"); }
    else if (op == "elemwise_add" || op == "elemwise_sub") {
      const uint32_t e0 = g.entry_id(n.inputs[0]), e1 = g.entry_id(n.inputs[1]);
      if (e0 == e1) return false;
      const uint32_t other = e0 == cur ? e1 : e0;
      if (op == "elemwise_add") st->op = CVMK_EP_ADD_T;
      else st->op = e0 == cur ? CVMK_EP_SUB_T : CVMK_EP_RSUB_T;
      st->ptr = reinterpret_cast<const void*>((uintptr_t)other + 1);  // resolved in bind_chain()
    } else if (op.compare(0, 10, "broadcast_") == 0) {
      const uint32_t e0 = g.entry_id(n.inputs[0]), e1 = g.entry_id(n.inputs[1]);
      if (e0 == e1) return false;
      const uint32_t other = e0 == cur ? e1 : e0;
      int32_t v;
      if (!scalar_param(other, &v)) return false;
      if (g.shape[g.entry_id(nid, 0)] != g.shape[cur]) return false;
      const bool lhs = e0 == cur;
      if (op == "broadcast_add") { st->op = CVMK_EP_ADD_S; st->a = v; }
      else if (op == "broadcast_sub") {
        if (lhs) { st->op = CVMK_EP_ADD_S; st->a = (int32_t)(0u - (uint32_t)v); }
        else { st->op = CVMK_EP_RSUB_S; st->a = v; }
      } else if (op == "broadcast_mul") { st->op = CVMK_EP_MUL_S; st->a = v; }
      else if (op == "broadcast_max") { st->op = CVMK_EP_MAX_S; st->a = v; }
      else if (op == "broadcast_div") { st->op = lhs ? CVMK_EP_DIV_S : CVMK_EP_RDIV_S; st->a = v; }
      else if (op == "broadcast_greater") { st->op = lhs ? CVMK_EP_GT_S : CVMK_EP_LT_S; st->a = v; }
      else return false;
    } else {
      return false;
    }
    return true;
  }

  // non_max_suppression nodes that overwrite rows of their INPUT entry (the CPU operator's side
  // effect, nms.cc:93-97, reproduced when that entry is read again): (node, entry) pairs.  They are
  // the only in-place writers of the graph, so they are the only thing a deferred read can miss.
  std::vector<std::pair<uint32_t, uint32_t>> input_writers;
  void find_input_writers() {
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid) {
      const Node& n = g.nodes[nid];
      if (n.is_variable() || n.op->name != "non_max_suppression" || n.attrs.i("top_k") <= 0) continue;
      const uint32_t in_eid = g.entry_id(n.inputs[0]);
      bool observed = false;
      for (const auto& h : g.outputs) observed |= g.entry_id(h) == in_eid;
      for (uint32_t m = nid + 1; m < g.nodes.size(); ++m)
        for (const auto& e : g.nodes[m].inputs) observed |= g.entry_id(e) == in_eid;
      if (observed) input_writers.emplace_back(nid, in_eid);
    }
  }

  // Greedily absorb single-consumer element-wise successors of entry `start`.  A fused group runs
  // at the position of its last member, so every read of the group happens there: a member that
  // reads an entry BEFORE a node that overwrites it in place must not be carried past that node.
  void extend_chain(Chain* c) {
    std::vector<std::pair<uint32_t, uint32_t>> reads;   // (entry, reading node)
    for (const auto& e : g.nodes[c->tail_nid].inputs) reads.emplace_back(g.entry_id(e), c->tail_nid);
    while (c->ep.n < CVMK_MAX_EP_STEPS) {
      const uint32_t cur = c->tail_eid;
      if (is_head[cur] || uses[cur] != 1) break;
      uint32_t consumer = UINT32_MAX;
      for (uint32_t nid = c->tail_nid + 1; nid < g.nodes.size() && consumer == UINT32_MAX; ++nid)
        for (const auto& e : g.nodes[nid].inputs)
          if (g.entry_id(e) == cur) { consumer = nid; break; }
      if (consumer == UINT32_MAX || absorbed[consumer]) break;  // e.g. a join taken by its other branch
      bool crosses_writer = false;
      for (const auto& w : input_writers)
        for (const auto& r : reads)
          crosses_writer |= r.first == w.second && r.second < w.first && w.first < consumer;
      if (crosses_writer) break;
      cvmk_ep_step st;
      if (!node_as_step(consumer, cur, &st)) break;
      for (const auto& e : g.nodes[consumer].inputs)
        if (g.entry_id(e) != cur) reads.emplace_back(g.entry_id(e), consumer);
      c->ep.s[c->ep.n++] = st;
      absorbed[consumer] = 1;
      c->tail_nid = consumer;
      c->tail_eid = g.entry_id(consumer, 0);
    }
  }

  // Replace the entry placeholders of *_T steps by device pointers.
  void bind_chain(cvmk_epilogue* ep) {
    for (int i = 0; i < ep->n; ++i) {
      cvmk_ep_step& s = ep->s[i];
      if (s.op == CVMK_EP_ADD_T || s.op == CVMK_EP_SUB_T || s.op == CVMK_EP_RSUB_T) {
        const uint32_t other = (uint32_t)((uintptr_t)s.ptr - 1);
        DevBuf& o = materialize(other);
        s.ptr = o.ptr;
        s.ptr_dtype = o.dtype;
      }
    }
  }

  // ------------------------------------------------------------------ operators
  const int32_t* bias_vector(uint32_t eid) {
    auto it = g.params.find(eid);
    if (it != g.params.end()) {  // the usual case: upload the int32 vector once
      const auto& v = it->second.data;
      // zero padded to a multiple of 32 entries: a convolution whose output channels are padded
      // for the tensor-core kernel reads that far
      const size_t padded = (v.size() + 31) / 32 * 32;
      void* p = ex.dalloc(padded * 4);
      CUDA_OK(cudaMemset(p, 0, padded * 4));
      CUDA_OK(cudaMemcpy(p, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
      return reinterpret_cast<const int32_t*>(p);
    }
    DevBuf b = canon_i32_view(eid, "bias");
    return reinterpret_cast<const int32_t*>(b.ptr);
  }

  void lower_conv_like(uint32_t nid, bool dense) {
    const Node& n = g.nodes[nid];
    const uint32_t ex_ = g.entry_id(n.inputs[0]), ew = g.entry_id(n.inputs[1]);
    const bool use_bias = n.attrs.b("use_bias");
    const Shape& xs = g.shape[ex_];
    const Shape& wsh = g.shape[ew];
    auto wit = g.params.find(ew);
    CHECK(wit != g.params.end()) << n.op->name << " " << n.name() << ": weights must be a parameter";
    const HostTensor& wt = wit->second;

    int N, H, W, C, OC, KH, KW, OH, OW, groups, sh, sw, ph, pw, dh, dw;
    if (dense) {
      N = (int)xs[0]; H = W = 1; C = (int)xs[1]; OC = (int)wsh[0]; KH = KW = 1; OH = OW = 1; groups = 1;
      sh = sw = dh = dw = 1; ph = pw = 0;
    } else {
      const Shape& os = g.shape[g.entry_id(nid, 0)];
      N = (int)xs[0]; C = (int)xs[1]; H = (int)xs[2]; W = (int)xs[3];
      OC = (int)wsh[0]; KH = (int)wsh[2]; KW = (int)wsh[3]; OH = (int)os[2]; OW = (int)os[3];
      groups = (int)n.attrs.i("groups");
      sh = (int)n.attrs.t("strides")[0]; sw = (int)n.attrs.t("strides")[1];
      ph = (int)n.attrs.t("padding")[0]; pw = (int)n.attrs.t("padding")[1];
      dh = (int)n.attrs.t("dilation")[0]; dw = (int)n.attrs.t("dilation")[1];
    }
    const int icg = C / groups;

    Chain ch;
    memset(&ch.ep, 0, sizeof(ch.ep));
    ch.tail_eid = g.entry_id(nid, 0);
    ch.tail_nid = nid;
    if (use_bias) {
      ch.ep.s[0].op = CVMK_EP_ADD_C;
      ch.ep.s[0].ptr = bias_vector(g.entry_id(n.inputs[2]));
      ch.ep.n = 1;
    }
    extend_chain(&ch);
    bind_chain(&ch.ep);
    DevBuf& out = materialize(ch.tail_eid);
    const std::string label = n.op->name + ":" + n.name();

    cvmk_conv_desc probe;
    memset(&probe, 0, sizeof(probe));
    probe.N = N; probe.H = H; probe.W = W; probe.C = C; probe.OC = OC; probe.KH = KH; probe.KW = KW;
    probe.OH = OH; probe.OW = OW; probe.stride_h = sh; probe.stride_w = sw; probe.pad_h = ph; probe.pad_w = pw;
    probe.dil_h = dh; probe.dil_w = dw;
    // |sum + bias| can never exceed this: int8 operands (|x| <= 128 even after a narrowing view)
    // and the bias values themselves when they are parameters.
    {
      int64_t bias_max = 0;
      if (use_bias) {
        const uint32_t eb = g.entry_id(n.inputs[2]);
        auto bit = g.params.find(eb);
        if (bit != g.params.end()) {
          for (int32_t v : bit->second.data) bias_max = std::max<int64_t>(bias_max, std::llabs((long long)v));
        } else {
          bias_max = ((int64_t)1 << (g.precision[eb] - 1)) - 1;
        }
      }
      probe.acc_bound = (int64_t)icg * KH * KW * 128 * 128 + bias_max;
      probe.bias_static = (!use_bias || g.params.count(g.entry_id(n.inputs[2])) > 0) ? 1 : 0;
    }
    const bool depthwise = !dense && groups == C && OC == C && C % 16 == 0 && safe8[ex_];
    // Depthwise 3x3 stride-1 layers over a multiple of 128 channels run on the tensor cores as
    // groups of 32 channels with block-diagonal weights when the kernel's 8 x 16 pixel tiles fit
    // the image: the CUDA-core form is bound by instruction issue at a fraction of the memory
    // rate (measured 15-25 % slower on such layers; faster for 32 and 64 channels, which stay there).
    const int dw_cg = 32;
    bool dw_tc = false;
    if (depthwise && C % 128 == 0 && KH == 3 && KW == 3 && sh == 1 && sw == 1 && dh == 1 && dw == 1 &&
        out.dtype == CVMK_I8 && !dev_env("CVM_B200_NO_DW_TC") && !dev_env("CVM_B200_NO_TC")) {
      const int64_t linear = ((int64_t)N * OH * OW + 127) / 128;
      const int64_t tiles = (int64_t)((OW + 7) / 8) * ((OH + 15) / 16) * N;
      probe.groups = C / dw_cg;
      dw_tc = tiles * 20 <= linear * 27 && cvmk_conv2d_tc_supported(&probe);
      if (!dw_tc) probe.groups = 0;
    }
    // 32 and 64 channels: 4 or 2 neighbouring pixels of a row are 128 contiguous bytes, so the layer
    // is given to the same kernel as a 128-channel one over a quarter / half of the width, whose
    // filter moves in steps of one real pixel (cvmk_conv_desc.group_fold).
    int dw_fold = 1;
    if (depthwise && !dw_tc && (C == 32 || C == 64) && KH == 3 && KW == 3 && sh == 1 && sw == 1 && dh == 1 && dw == 1 &&
        pw == 1 && OW == W && W % (128 / C) == 0 && out.dtype == CVMK_I8 &&
        (!use_bias || g.params.count(g.entry_id(n.inputs[2])) > 0) && !dev_env("CVM_B200_NO_DW_TC") &&
        !dev_env("CVM_B200_NO_DW_FOLD") && !dev_env("CVM_B200_NO_TC")) {
      const int F = 128 / C;
      const int64_t linear = ((int64_t)N * OH * (OW / F) + 127) / 128;
      const int64_t tiles = (int64_t)((OW / F + 7) / 8) * ((OH + 15) / 16) * N;
      cvmk_conv_desc fp = probe;
      fp.W = W / F; fp.OW = OW / F; fp.C = fp.OC = 128;
      fp.groups = 4; fp.group_fold = F;
      if (tiles * 20 <= linear * 27 && cvmk_conv2d_tc_supported(&fp)) {
        probe = fp;
        dw_tc = true;
        dw_fold = F;
      }
    }
    const bool tc = (dw_tc || groups == 1) && cvmk_conv2d_tc_supported(&probe) && !dev_env("CVM_B200_NO_TC");
    const int wcg = dw_tc ? dw_cg : icg;   // input channels per weight row as the kernels take them
    // Few-channel convolutions (image stems): gather patches into a [M, Kp] matrix, then run the
    // tensor-core kernel on it as a 1x1 convolution.
    const int kflat = KH * KW * icg, kp = kflat > 64 ? (kflat + 63) / 64 * 64 : (kflat + 31) / 32 * 32;
    cvmk_conv_desc packed = probe;
    packed.N = N * OH * OW; packed.H = packed.W = 1; packed.C = kp; packed.KH = packed.KW = 1;
    packed.OH = packed.OW = 1; packed.stride_h = packed.stride_w = 1; packed.pad_h = packed.pad_w = 0;
    packed.dil_h = packed.dil_w = 1;
    const bool via_pack = !tc && !dense && groups == 1 && safe8[ex_] && C <= 255 && kflat <= 8192 &&
                          (KW - 1) * dw <= 4095 && (KH - 1) * dh <= 2047 &&
                          cvmk_conv2d_tc_supported(&packed) && !dev_env("CVM_B200_NO_TC");

    // Output channel counts the tensor-core kernel does not take (not a multiple of 8: detection
    // heads with anchors x classes channels) run on it with zero weight rows up to a multiple of
    // 32 and a copy of the real channels afterwards, when nothing in the chain indexes the
    // output tensor (no fused tensor operand) and the bias is a parameter.
    const int OCp = (OC + 31) / 32 * 32;
    bool tc_pad = false;
    if (!tc && !dense && groups == 1 && OC % 8 != 0 && !depthwise && !dev_env("CVM_B200_NO_TC")) {
      cvmk_conv_desc pp = probe;
      pp.OC = OCp;
      bool plain_chain = true;
      for (int i = 0; i < ch.ep.n; ++i)
        plain_chain &= !(ch.ep.s[i].op == CVMK_EP_ADD_T || ch.ep.s[i].op == CVMK_EP_SUB_T || ch.ep.s[i].op == CVMK_EP_RSUB_T);
      const bool bias_param = !use_bias || g.params.count(g.entry_id(n.inputs[2])) > 0;
      tc_pad = cvmk_conv2d_tc_supported(&pp) && plain_chain && bias_param && safe8[ex_] && out.shape.size() == 4;
    }
    // weights: OIHW int32 -> int8, [OC, KH, KW, C/groups] (depthwise: [KH, KW, C])
    std::vector<int8_t> w8((size_t)(tc_pad ? OCp : OC) * dw_fold * KH * KW * wcg, 0);
    if (dw_tc) {   // [OC, KH, KW, 32]: row o holds its filter in column o % 32 of every tap
      for (int o = 0; o < OC * dw_fold; ++o) {   // (folded: the C filters once per sub-pixel)
        const int c = o % OC;
        for (int k = 0; k < KH * KW; ++k)
          w8[((size_t)o * KH * KW + k) * wcg + (c % wcg)] = (int8_t)wt.data[(size_t)c * KH * KW + k];
      }
    } else if (depthwise && !tc) {
      for (int c = 0; c < C; ++c)
        for (int k = 0; k < KH * KW; ++k) w8[(size_t)k * C + c] = (int8_t)wt.data[(size_t)c * KH * KW + k];
    } else {
      for (int o = 0; o < OC; ++o)
        for (int i = 0; i < icg; ++i)
          for (int k = 0; k < KH * KW; ++k)
            w8[((size_t)o * KH * KW + k) * icg + i] = (int8_t)wt.data[((size_t)o * icg + i) * KH * KW + k];
    }
    if (via_pack) {  // rows padded with zeros from K to Kp
      std::vector<int8_t> wp((size_t)OC * kp, 0);
      for (int o = 0; o < OC; ++o) memcpy(&wp[(size_t)o * kp], &w8[(size_t)o * kflat], kflat);
      w8.swap(wp);
    }
    int8_t* wdev = (int8_t*)ex.dalloc(w8.size());
    CUDA_OK(cudaMemcpy(wdev, w8.data(), w8.size(), cudaMemcpyHostToDevice));

    // Stem on the tensor cores without a patch matrix: the network input itself, few channels.
    if (via_pack && ex_ == data_eid && raw_in.dtype == CVMK_I8 && dh == 1 && dw == 1 && out.dtype == CVMK_I8 &&
        !dev_env("CVM_B200_NO_STEM_FUSED")) {
      cvmk_stem_conv_desc sd;
      memset(&sd, 0, sizeof(sd));
      sd.x = (const int8_t*)raw_in.ptr; sd.y = out.ptr;
      sd.N = N; sd.H = H; sd.W = W; sd.C = C; sd.OC = OC; sd.KH = KH; sd.KW = KW; sd.OH = OH; sd.OW = OW;
      sd.stride_h = sh; sd.stride_w = sw; sd.pad_h = ph; sd.pad_w = pw;
      sd.clamp = data_range;
      sd.status = ex.status_dev_;
      sd.acc_bound = probe.acc_bound;
      sd.ep = ch.ep;
      if (cvmk_conv2d_stem_supported(&sd)) {
        std::vector<int8_t> ws((size_t)cvmk_conv2d_stem_weight_bytes(&sd), 0);
        KERNEL_OK(cvmk_conv2d_stem_pack_weights(&sd, wt.data.data(), ws.data()));
        int8_t* wsdev = (int8_t*)ex.dalloc(ws.size());
        CUDA_OK(cudaMemcpy(wsdev, ws.data(), ws.size(), cudaMemcpyHostToDevice));
        sd.w = wsdev;
        // The batch is cut into chunks with a plan each, so that an inference can run the stem on
        // the first images while the later ones are still being uploaded.
        const int chunks = (uses[ex_] == 1 && !is_head[ex_]) ? batch_chunks(N) : 1;
        const int per = N / chunks;
        // plan 0 covers the whole batch (one launch when the input is already on the device);
        // plans 1.. cover one chunk each
        std::vector<cvmk_stem_conv_plan*> plans;
        for (int c = -1; c < (chunks > 1 ? chunks : 0); ++c) {
          cvmk_stem_conv_desc cd = sd;
          if (c >= 0) {
            cd.N = per;
            cd.x = sd.x + (size_t)c * per * C * H * W;
            cd.y = (int8_t*)sd.y + (size_t)c * per * OH * OW * OC;
          }
          void* mem = nullptr;
          CHECK(posix_memalign(&mem, 64, sizeof(cvmk_stem_conv_plan)) == 0);
          ex.stem_plans_.emplace_back((cvmk_stem_conv_plan*)mem, plan_deleter);
          KERNEL_OK(cvmk_conv2d_stem_prepare(&cd, ex.stem_plans_.back().get()));
          plans.push_back(ex.stem_plans_.back().get());
        }
        cvmk_stem_conv_plan* whole = plans[0];
        add_step(label + "[stem]", [whole](cudaStream_t s) { return cvmk_conv2d_stem_launch(whole, s); });
        if (chunks > 1) {
          ex.chunk_bytes_ = (size_t)per * C * H * W;
          for (size_t c = 1; c < plans.size(); ++c) {
            cvmk_stem_conv_plan* pl = plans[c];
            ex.steps_.back().chunk.push_back([pl](cudaStream_t s) { return cvmk_conv2d_stem_launch(pl, s); });
          }
        }
        return;
      }
    }

    if (via_pack) {
      int8_t* amat = (int8_t*)act_alloc((size_t)packed.N * kp);
      cvmk_stem_pack_desc sp;
      memset(&sp, 0, sizeof(sp));
      sp.x = (const int8_t*)raw_in.ptr; sp.a = amat;
      sp.N = N; sp.H = H; sp.W = W; sp.C = C; sp.KH = KH; sp.KW = KW; sp.OH = OH; sp.OW = OW;
      sp.stride_h = sh; sp.stride_w = sw; sp.pad_h = ph; sp.pad_w = pw; sp.dil_h = dh; sp.dil_w = dw;
      sp.Kp = kp; sp.clamp = data_range;
      const bool from_raw = ex_ == data_eid && raw_in.dtype == CVMK_I8 && cvmk_stem_pack_supported(&sp) &&
                            !dev_env("CVM_B200_NO_STEM_PACK");
      if (from_raw) {  // gather straight from the NCHW input: no channels-last copy of it is needed
        add_step(label + "[stem_pack]", [sp](cudaStream_t s) { return cvmk_stem_pack(&sp, s); });
      }
      DevBuf xin_holder;
      if (!from_raw) xin_holder = materialize(ex_);
      const DevBuf& xin = xin_holder;
      cvmk_im2col_desc pk;
      memset(&pk, 0, sizeof(pk));
      pk.x = (const int8_t*)xin.ptr; pk.a = amat;
      pk.N = N; pk.H = H; pk.W = W; pk.C = C; pk.KH = KH; pk.KW = KW; pk.OH = OH; pk.OW = OW;
      pk.stride_h = sh; pk.stride_w = sw; pk.pad_h = ph; pk.pad_w = pw; pk.dil_h = dh; pk.dil_w = dw;
      pk.Kp = kp;
      if (!from_raw) add_step(label + "[pack]", [pk](cudaStream_t s) { return cvmk_im2col_pack(&pk, s); });
      cvmk_conv_desc d = packed;
      d.x = amat; d.w = wdev; d.y = out.ptr; d.y_dtype = out.dtype;
      d.status = ex.status_dev_;
      d.ep = ch.ep;
      void* mem = nullptr;
      CHECK(posix_memalign(&mem, 64, sizeof(cvmk_conv_plan)) == 0);
      ex.plans_.emplace_back((cvmk_conv_plan*)mem, plan_deleter);
      cvmk_conv_plan* plan = ex.plans_.back().get();
      KERNEL_OK(cvmk_conv2d_tc_prepare(&d, plan));
      add_step(label + "[tc]", [plan](cudaStream_t s) { return cvmk_conv2d_tc_launch(plan, s); });
      return;
    }

    if (tc_pad) {
      DevBuf xin = i8_view(ex_, label);
      DevBuf tmp = out;
      tmp.shape = Shape{(int64_t)N, (int64_t)OCp, (int64_t)OH, (int64_t)OW};
      tmp.nhwc = true;
      tmp.ptr = act_alloc(tmp.bytes());
      cvmk_conv_desc d = probe;
      d.OC = OCp;
      d.x = (const int8_t*)xin.ptr; d.w = wdev; d.y = tmp.ptr; d.y_dtype = tmp.dtype;
      d.status = ex.status_dev_;
      d.ep = ch.ep;
      void* mem = nullptr;
      CHECK(posix_memalign(&mem, 64, sizeof(cvmk_conv_plan)) == 0);
      ex.plans_.emplace_back((cvmk_conv_plan*)mem, plan_deleter);
      cvmk_conv_plan* plan = ex.plans_.back().get();
      KERNEL_OK(cvmk_conv2d_tc_prepare(&d, plan));
      add_step(label + "[tc]", [plan](cudaStream_t s) { return cvmk_conv2d_tc_launch(plan, s); });
      const auto ss = phys_strides(tmp.shape, true), ds = phys_strides(out.shape, out.nhwc);
      std::vector<GDim> dims;
      for (int k = 0; k < 4; ++k) dims.push_back({out.shape[k], ss[k], ds[k]});
      emit_gather(tmp, 0, out, dims, label + ":channels");
      return;
    }

    if (tc) {
      DevBuf xin = i8_view(ex_, label);
      cvmk_conv_desc d = probe;
      d.x = (const int8_t*)xin.ptr; d.w = wdev; d.y = out.ptr; d.y_dtype = out.dtype;
      d.status = ex.status_dev_;
      d.ep = ch.ep;
      // Narrow 1x1 layers (few input and output channels) make tiles with one or two tensor-core
      // instructions each, and what a tile costs beside them dominates.  f neighbouring pixels of
      // an NHWC tensor are f * C contiguous bytes, so the same layer is also [M / f, f * C] x
      // block-diagonal weights [f * OC, f * C] -> [M / f, f * OC], byte for byte the same output:
      // f times the multiplies (zeros), 1 / f of the tiles.  32 -> 64 channels at 112 x 112, batch
      // 256: 0.116 -> 0.058 ms with f = 4; 64 -> 64 at 56 x 56: 0.032 -> 0.022 ms with f = 2.
      if (dw_fold > 1 && use_bias) {   // the bias once per sub-pixel
        const auto& bv = g.params.find(g.entry_id(n.inputs[2]))->second.data;
        std::vector<int32_t> bf(128, 0);
        for (int j = 0; j < dw_fold; ++j)
          for (int o = 0; o < OC; ++o) bf[(size_t)j * OC + o] = bv[o];
        int32_t* bfdev = (int32_t*)ex.dalloc(bf.size() * 4);
        CUDA_OK(cudaMemcpy(bfdev, bf.data(), bf.size() * 4, cudaMemcpyHostToDevice));
        d.ep.s[0].ptr = bfdev;
      }
      int fold = 1;
      const int bchunks = batch_chunks(N);
      if (!dense && !dw_tc && groups == 1 && KH == 1 && KW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0 &&
          xin.nhwc && out.nhwc && (!use_bias || g.params.count(g.entry_id(n.inputs[2])) > 0) &&
          !dev_env("CVM_B200_NO_PIXEL_FOLD")) {
        const int64_t per_chunk = (int64_t)(N / bchunks) * OH * OW;
        while (fold < 4 && 2 * fold * C <= 128 && 2 * fold * OC <= 256 && per_chunk % (2 * fold) == 0) fold *= 2;
      }
      if (fold > 1) {
        const int Cf = fold * C, OCf = fold * OC;
        std::vector<int8_t> wf((size_t)OCf * Cf, 0);   // block j: rows j * OC .., columns j * C ..
        for (int j = 0; j < fold; ++j)
          for (int o = 0; o < OC; ++o)
            memcpy(&wf[((size_t)(j * OC + o)) * Cf + (size_t)j * C], &w8[(size_t)o * C], (size_t)C);
        int8_t* wfdev = (int8_t*)ex.dalloc(wf.size());
        CUDA_OK(cudaMemcpy(wfdev, wf.data(), wf.size(), cudaMemcpyHostToDevice));
        d.w = wfdev;
        if (use_bias) {   // the bias once per folded pixel
          const auto& bv = g.params.find(g.entry_id(n.inputs[2]))->second.data;
          std::vector<int32_t> bf((size_t)(OCf + 31) / 32 * 32, 0);
          for (int j = 0; j < fold; ++j)
            for (int o = 0; o < OC; ++o) bf[(size_t)j * OC + o] = bv[o];
          int32_t* bfdev = (int32_t*)ex.dalloc(bf.size() * 4);
          CUDA_OK(cudaMemcpy(bfdev, bf.data(), bf.size() * 4, cudaMemcpyHostToDevice));
          d.ep.s[0].ptr = bfdev;
        }
        d.N = (int32_t)((int64_t)N * OH * OW / fold);
        d.H = d.W = d.OH = d.OW = 1;
        d.C = Cf; d.OC = OCf;
      }
      d.workspace_bytes = cvmk_conv2d_tc_workspace_bytes(&d);   // > 0: few rows over a long K, cut along K
      if (d.workspace_bytes > 0) d.workspace = act_alloc((size_t)d.workspace_bytes);
      void* mem = nullptr;
      CHECK(posix_memalign(&mem, 64, sizeof(cvmk_conv_plan)) == 0);
      ex.plans_.emplace_back((cvmk_conv_plan*)mem, plan_deleter);
      cvmk_conv_plan* plan = ex.plans_.back().get();
      KERNEL_OK(cvmk_conv2d_tc_prepare(&d, plan));
      add_step(label + (dw_tc ? "[dw]" : (plan->k_slices > 1 ? ":k-slices[tc]" : "[tc]")),
               [plan](cudaStream_t s) { return cvmk_conv2d_tc_launch(plan, s); });
      // Quarter-batch plans (every operand is batch-major, so a chunk is a contiguous slice).
      const int chunks = fold > 1 ? bchunks : batch_chunks(d.N);
      if (chunks > 1 && xin.nhwc && out.nhwc) {
        const int per = d.N / chunks;
        const size_t out_elems = (size_t)per * d.OH * d.OW * d.OC;
        for (int c = 0; c < chunks; ++c) {
          cvmk_conv_desc cd = d;
          cd.N = per;
          cd.x = d.x + (size_t)c * per * d.H * d.W * d.C;
          cd.y = (char*)d.y + (size_t)c * out_elems * d.y_dtype;
          for (int i = 0; i < cd.ep.n; ++i) {
            cvmk_ep_step& st = cd.ep.s[i];
            if ((st.op == CVMK_EP_ADD_T || st.op == CVMK_EP_SUB_T || st.op == CVMK_EP_RSUB_T) && st.ptr)
              st.ptr = (const char*)st.ptr + (size_t)c * out_elems * st.ptr_dtype;
          }
          void* cmem = nullptr;
          CHECK(posix_memalign(&cmem, 64, sizeof(cvmk_conv_plan)) == 0);
          ex.plans_.emplace_back((cvmk_conv_plan*)cmem, plan_deleter);
          cvmk_conv_plan* cp = ex.plans_.back().get();
          KERNEL_OK(cvmk_conv2d_tc_prepare(&cd, cp));
          ex.steps_.back().chunk.push_back([cp](cudaStream_t s) { return cvmk_conv2d_tc_launch(cp, s); });
        }
      }
    } else {
      DevBuf& xin = materialize(ex_);
      cvmk_conv_direct_desc d;
      memset(&d, 0, sizeof(d));
      d.x = xin.ptr; d.x_dtype = xin.dtype; d.narrow_x = groups == 1;
      d.w = wdev; d.y = out.ptr; d.y_dtype = out.dtype;
      d.N = N; d.H = H; d.W = W; d.C = C; d.OC = OC; d.KH = KH; d.KW = KW; d.OH = OH; d.OW = OW; d.groups = groups;
      d.stride_h = sh; d.stride_w = sw; d.pad_h = ph; d.pad_w = pw; d.dil_h = dh; d.dil_w = dw;
      d.depthwise = depthwise;
      d.acc_bound = probe.acc_bound;
      d.ep = ch.ep;
      add_step(label + (depthwise ? "[dw]" : "[direct]"), [d](cudaStream_t s) { return cvmk_conv2d_direct(&d, s); });
      // Quarter-batch forms (batch-major operands: a chunk is a contiguous slice), when no step of
      // the chain indexes another tensor.
      const int chunks = batch_chunks(d.N);
      bool sliceable = chunks > 1 && xin.nhwc && out.nhwc;
      for (int i = 0; i < d.ep.n; ++i)
        sliceable &= !(d.ep.s[i].op == CVMK_EP_ADD_T || d.ep.s[i].op == CVMK_EP_SUB_T || d.ep.s[i].op == CVMK_EP_RSUB_T);
      if (sliceable) {
        const int per = d.N / chunks;
        for (int c = 0; c < chunks; ++c) {
          cvmk_conv_direct_desc cd = d;
          cd.N = per;
          cd.x = (const char*)d.x + (size_t)c * per * d.H * d.W * d.C * d.x_dtype;
          cd.y = (char*)d.y + (size_t)c * per * d.OH * d.OW * d.OC * d.y_dtype;
          ex.steps_.back().chunk.push_back([cd](cudaStream_t s) { return cvmk_conv2d_direct(&cd, s); });
        }
      }
    }
  }

  // Element-wise root: unary ops, elemwise_add/sub, broadcast with a scalar parameter.
  bool lower_elemwise_root(uint32_t nid) {
    const Node& n = g.nodes[nid];
    uint32_t src = g.entry_id(n.inputs[0]);
    cvmk_ep_step st;
    if (!node_as_step(nid, src, &st)) {
      if (n.inputs.size() == 2) {
        src = g.entry_id(n.inputs[1]);
        if (!node_as_step(nid, src, &st)) return false;
      } else {
        return false;
      }
    }
    if (g.shape[src] != g.shape[g.entry_id(nid, 0)]) return false;
    Chain ch;
    memset(&ch.ep, 0, sizeof(ch.ep));
    ch.ep.s[0] = st;
    ch.ep.n = 1;
    ch.tail_eid = g.entry_id(nid, 0);
    ch.tail_nid = nid;
    extend_chain(&ch);
    bind_chain(&ch.ep);
    const DevBuf x = materialize(src);
    const DevBuf y = materialize(ch.tail_eid);
    const cvmk_epilogue ep = ch.ep;
    const int64_t cnt = shape_size(x.shape);
    add_step(n.op->name + ":" + n.name(), [x, y, ep, cnt](cudaStream_t s) {
      return cvmk_elemwise(x.ptr, x.dtype, y.ptr, y.dtype, cnt, &ep, s);
    });
    return true;
  }

  void lower_broadcast(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const std::string& op = n.op->name;
    const uint32_t ea = g.entry_id(n.inputs[0]), eb = g.entry_id(n.inputs[1]), eo = g.entry_id(nid, 0);
    const DevBuf a = materialize(ea), b = materialize(eb);
    Chain ch;
    memset(&ch.ep, 0, sizeof(ch.ep));
    ch.tail_eid = eo;
    ch.tail_nid = nid;
    // A fused tail must keep the shape (and with it the layout) of this node's output.
    extend_chain(&ch);
    bind_chain(&ch.ep);
    const DevBuf y = materialize(ch.tail_eid);
    cvmk_strided_desc d;
    memset(&d, 0, sizeof(d));
    d.op = (op == "broadcast_add" || op == "elemwise_add") ? CVMK_OP_ADD
         : (op == "broadcast_sub" || op == "elemwise_sub") ? CVMK_OP_SUB
         : op == "broadcast_mul" ? CVMK_OP_MUL : op == "broadcast_max" ? CVMK_OP_MAX
         : op == "broadcast_div" ? CVMK_OP_DIV : CVMK_OP_GREATER;
    const Shape& os = y.shape;
    const auto order = phys_order(os, y.nhwc);
    const auto ys = phys_strides(os, y.nhwc);
    const auto as = phys_strides(a.shape, a.nhwc), bs = phys_strides(b.shape, b.nhwc);
    d.ndim = (int)os.size();
    const int offa = (int)os.size() - (int)a.shape.size(), offb = (int)os.size() - (int)b.shape.size();
    for (int k = 0; k < d.ndim; ++k) {
      const int j = order[k];
      d.extent[k] = os[j];
      d.y_stride[k] = ys[j];
      d.a_stride[k] = (j - offa >= 0 && a.shape[j - offa] != 1) ? as[j - offa] : 0;
      d.b_stride[k] = (j - offb >= 0 && b.shape[j - offb] != 1) ? bs[j - offb] : 0;
    }
    d.a = a.ptr; d.a_dtype = a.dtype; d.b = b.ptr; d.b_dtype = b.dtype; d.y = y.ptr; d.y_dtype = y.dtype;
    d.ep = ch.ep;
    add_step(op + ":" + n.name(), [d](cudaStream_t s) { return cvmk_strided(&d, s); });
  }

  void lower_pool(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const uint32_t ei = g.entry_id(n.inputs[0]), eo = g.entry_id(nid, 0);
    const DevBuf x = materialize(ei);
    const DevBuf y = materialize(eo);
    CHECK(x.dtype == y.dtype);
    const Shape& pad = n.attrs.t("padding");
    cvmk_pool_desc d;
    memset(&d, 0, sizeof(d));
    d.x = x.ptr; d.y = y.ptr; d.dtype = x.dtype;
    d.N = (int)x.shape[0]; d.C = (int)x.shape[1]; d.H = (int)x.shape[2]; d.W = (int)x.shape[3];
    d.OH = (int)y.shape[2]; d.OW = (int)y.shape[3];
    d.KH = (int)n.attrs.t("pool_size")[0]; d.KW = (int)n.attrs.t("pool_size")[1];
    d.stride_h = (int)n.attrs.t("strides")[0]; d.stride_w = (int)n.attrs.t("strides")[1];
    d.pad_h = (int)pad[0]; d.pad_w = (int)(pad.size() == 2 ? pad[1] : pad[0]);
    add_step("max_pool2d:" + n.name(), [d](cudaStream_t s) { return cvmk_max_pool2d(&d, s); });
    const int chunks = batch_chunks(d.N);
    if (chunks > 1 && x.nhwc && y.nhwc) {
      const int per = d.N / chunks;
      for (int c = 0; c < chunks; ++c) {
        cvmk_pool_desc cd = d;
        cd.N = per;
        cd.x = (const char*)d.x + (size_t)c * per * d.H * d.W * d.C * d.dtype;
        cd.y = (char*)d.y + (size_t)c * per * d.OH * d.OW * d.C * d.dtype;
        ex.steps_.back().chunk.push_back([cd](cudaStream_t s) { return cvmk_max_pool2d(&cd, s); });
      }
    }
  }

  void lower_upsampling(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const DevBuf x = materialize(g.entry_id(n.inputs[0]));
    const DevBuf y = materialize(g.entry_id(nid, 0));
    const int64_t sc = n.attrs.i("scale");
    const int64_t N = x.shape[0], C = x.shape[1], H = x.shape[2], W = x.shape[3];
    const auto xs = phys_strides(x.shape, x.nhwc), ys = phys_strides(y.shape, y.nhwc);
    cvmk_strided_desc d;
    memset(&d, 0, sizeof(d));
    d.op = CVMK_OP_COPY;
    d.ndim = 6;
    // iteration space (N, H, s, W, s, C); the two s extents do not move the source
    const int64_t ext[6] = {N, H, sc, W, sc, C};
    const int64_t as[6] = {xs[0], xs[2], 0, xs[3], 0, xs[1]};
    const int64_t yst[6] = {ys[0], ys[2] * sc, ys[2], ys[3] * sc, ys[3], ys[1]};
    for (int k = 0; k < 6; ++k) { d.extent[k] = ext[k]; d.a_stride[k] = as[k]; d.y_stride[k] = yst[k]; }
    d.a = x.ptr; d.a_dtype = x.dtype; d.y = y.ptr; d.y_dtype = y.dtype;
    add_step("upsampling:" + n.name(), [d](cudaStream_t s) { return cvmk_strided(&d, s); });
  }

  void lower_concat(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const DevBuf y = materialize(g.entry_id(nid, 0));
    const int nd = (int)y.shape.size();
    int axis = (int)n.attrs.i("axis");
    if (axis < 0) axis += nd;
    const auto ys = phys_strides(y.shape, y.nhwc);
    int64_t offset = 0;
    std::vector<cvmk_strided_desc> all;
    for (size_t m = 0; m < n.inputs.size(); ++m) {
      const DevBuf x = materialize(g.entry_id(n.inputs[m]));
      const auto order = phys_order(x.shape, y.nhwc);
      const auto xs = phys_strides(x.shape, x.nhwc);
      cvmk_strided_desc d;
      memset(&d, 0, sizeof(d));
      d.op = CVMK_OP_COPY;
      d.ndim = nd;
      for (int k = 0; k < nd; ++k) {
        d.extent[k] = x.shape[order[k]];
        d.a_stride[k] = xs[order[k]];
        d.y_stride[k] = ys[order[k]];
      }
      d.a = x.ptr; d.a_dtype = x.dtype; d.y = y.ptr; d.y_dtype = y.dtype;
      d.y_off = offset * ys[axis];
      offset += x.shape[axis];
      all.push_back(d);
    }
    // all inputs in one launch when they move whole vectors, else one launch each
    add_step("concatenate:" + n.name(), [all](cudaStream_t s) { return cvmk_strided_batch(all.data(), (int32_t)all.size(), s); });
  }

  // flatten / reshape / squeeze / expand_dims: the row-major element order is preserved.
  void lower_reshape(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const uint32_t ei = g.entry_id(n.inputs[0]), eo = g.entry_id(nid, 0);
    DevBuf src = canon_view(ei, n.op->name + ":" + n.name());
    DevBuf& out = buf[eo];
    CHECK(out.dtype == src.dtype);
    if (!out.nhwc) {
      out.ptr = src.ptr;  // alias
      return;
    }
    materialize(eo);
    DevBuf as_canon = out;
    as_canon.nhwc = false;
    as_canon.ptr = src.ptr;
    emit_convert(as_canon, out, n.op->name + ":" + n.name() + ":to_nhwc");
  }

  // sum / max.  The kept-dimension mapping follows cpu/ops/reduce.cc:66-89 literally, including
  // its pairing of the output's non-unit dimensions with the input's non-reduced ones from the
  // right.
  void lower_reduce(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const uint32_t ei = g.entry_id(n.inputs[0]), eo = g.entry_id(nid, 0);
    DevBuf x = materialize(ei);
    const Shape xs = x.shape;
    const Shape& ysh = g.shape[eo];
    const int xnd = (int)xs.size();
    Shape axis = n.attrs.t("axis");
    const bool exclude = n.attrs.b("exclude");
    for (auto& a : axis) if (a < 0) a += xnd;
    std::vector<int64_t> real;
    if (!exclude) real.assign(axis.begin(), axis.end());
    else {
      for (int i = 0; i < xnd; ++i)
        if (std::find(axis.begin(), axis.end(), i) == axis.end()) real.push_back(i);
    }
    Chain ch;
    memset(&ch.ep, 0, sizeof(ch.ep));
    ch.tail_eid = eo;
    ch.tail_nid = nid;
    const std::string label = n.op->name + ":" + n.name();
    if (exclude && real.empty()) {  // plain copy, reduce.cc:38-39
      extend_chain(&ch);
      bind_chain(&ch.ep);
      DevBuf y = materialize(ch.tail_eid);
      DevBuf srcv = x;
      srcv.shape = y.shape;  // same element order when both are row-major
      if (x.nhwc || y.nhwc) {
        DevBuf c = canon_view(ei, label);
        c.shape = y.shape;
        emit_convert(c, y, label, &ch.ep);
      } else {
        emit_convert(srcv, y, label, &ch.ep);
      }
      return;
    }
    const bool out_needs_convert = wants_nhwc(ysh);
    if (!out_needs_convert) { extend_chain(&ch); bind_chain(&ch.ep); }
    // The reference pairs the output's non-unit dimensions with the input's kept ones from the
    // right and steps by row-major strides (reduce.cc:66-89).  When unit dimensions make the
    // pairing land on a dimension of another extent, the walk leaves that dimension and carries
    // into its neighbours; only the row-major layout reproduces that, so such inputs are read
    // from a row-major copy.
    if (x.nhwc && !real.empty()) {
      std::vector<char> fl(xnd, 0);
      for (auto a : real) fl[a] = 1;
      std::vector<int64_t> nz;
      for (auto v : ysh) if (v != 1) nz.push_back(v);
      bool straight = true;
      int xj = xnd - 1;
      for (int j = (int)nz.size() - 1; j >= 0; --j) {
        while (xj >= 0 && fl[xj--]) {}
        straight &= xj + 1 >= 0 && xj + 1 < xnd && xs[xj + 1] == nz[j];
      }
      if (!straight) x = canon_view(ei, label);
    }
    const auto xst = phys_strides(xs, x.nhwc);
    cvmk_reduce_desc d;
    memset(&d, 0, sizeof(d));
    d.is_max = n.op->name == "max";
    if (real.empty()) {
      d.init_zero = 1;
      d.n_keep = 0;
      d.n_red = xnd;
      for (int k = 0; k < xnd; ++k) { d.red_extent[k] = xs[k]; d.red_stride[k] = xst[k]; }
    } else {
      std::vector<char> flag(xnd, 0);
      for (auto a : real) flag[a] = 1;
      std::sort(real.begin(), real.end());
      d.n_red = (int)real.size();
      for (int k = 0; k < d.n_red; ++k) { d.red_extent[k] = xs[real[k]]; d.red_stride[k] = xst[real[k]]; }
      // every_xdim_size of the reference is the row-major stride; here the physical one is used,
      // which addresses the same logical element.
      std::vector<int64_t> ynz;
      for (auto v : ysh) if (v != 1) ynz.push_back(v);
      d.n_keep = (int)ynz.size();
      int xj = xnd - 1;
      for (int j = d.n_keep - 1; j >= 0; --j) {
        while (xj >= 0 && flag[xj--]) {}
        d.keep_extent[j] = ynz[j];
        d.keep_stride[j] = xj + 1 >= 0 && xj + 1 < xnd ? xst[xj + 1] : 0;
      }
    }
    d.x = x.ptr; d.x_dtype = x.dtype;
    if (out_needs_convert) {
      DevBuf tmp = buf[eo];
      tmp.nhwc = false;
      tmp.ptr = act_alloc(tmp.bytes());
      d.y = tmp.ptr; d.y_dtype = tmp.dtype;
      add_step(label, [d](cudaStream_t s) { return cvmk_reduce(&d, s); });
      emit_convert(tmp, materialize(eo), label + ":to_nhwc");
    } else {
      DevBuf y = materialize(ch.tail_eid);
      d.y = y.ptr; d.y_dtype = y.dtype;
      d.ep = ch.ep;
      add_step(label, [d](cudaStream_t s) { return cvmk_reduce(&d, s); });
    }
  }

  // ------------------------------------------------------------------ index-map transforms
  // One dimension of a gather: `extent` points, each moving the source by a_stride and the
  // destination by y_stride elements.
  struct GDim { int64_t extent, a_stride, y_stride; };

  // dst[y_off + sum c_k ys_k] = src[a_off + sum c_k as_k] as strided copies.  Unit extents are
  // dropped, the destination order decides the iteration order (coalesced writes), neighbours
  // that form one run in both tensors are merged, and spaces of more than six extents are
  // peeled into several launches.
  void emit_gather(const DevBuf& src, int64_t a_off, const DevBuf& dst, std::vector<GDim> dims,
                   const std::string& label) {
    std::vector<GDim> v;
    for (const auto& d : dims) if (d.extent != 1) v.push_back(d);
    std::stable_sort(v.begin(), v.end(), [](const GDim& a, const GDim& b) { return a.y_stride > b.y_stride; });
    std::vector<GDim> m;
    for (const auto& d : v) {
      if (!m.empty() && m.back().a_stride == d.a_stride * d.extent && m.back().y_stride == d.y_stride * d.extent) {
        m.back().extent *= d.extent;
        m.back().a_stride = d.a_stride;
        m.back().y_stride = d.y_stride;
      } else {
        m.push_back(d);
      }
    }
    if (m.empty()) m.push_back({1, 0, 0});
    emit_gather_peeled(src, a_off, dst, 0, m, label);
  }
  void emit_gather_peeled(const DevBuf& src, int64_t a_off, const DevBuf& dst, int64_t y_off,
                          const std::vector<GDim>& m, const std::string& label) {
    if (m.size() > 6) {
      std::vector<GDim> rest(m.begin() + 1, m.end());
      for (int64_t c = 0; c < m[0].extent; ++c)
        emit_gather_peeled(src, a_off + c * m[0].a_stride, dst, y_off + c * m[0].y_stride, rest, label);
      return;
    }
    cvmk_strided_desc d;
    memset(&d, 0, sizeof(d));
    d.op = CVMK_OP_COPY;
    d.ndim = (int)m.size();
    for (int k = 0; k < d.ndim; ++k) {
      d.extent[k] = m[k].extent;
      d.a_stride[k] = m[k].a_stride;
      d.y_stride[k] = m[k].y_stride;
    }
    d.a = src.ptr; d.a_dtype = src.dtype; d.a_off = a_off;
    d.y = dst.ptr; d.y_dtype = dst.dtype; d.y_off = y_off;
    add_step(label, [d](cudaStream_t s) { return cvmk_strided(&d, s); });
  }

  // transpose / strided_slice / slice_like / repeat / tile (cpu/ops/ops.cc:603-683, :743-866):
  // every output element is one input element, at an index that is affine in the output index.
  void lower_index_map(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const std::string& op = n.op->name;
    const DevBuf x = materialize(g.entry_id(n.inputs[0]));
    if (transpose_is_identity(nid) && !dev_env("CVM_B200_NO_TRANSPOSE_ALIAS")) {
      DevBuf& out = buf[g.entry_id(nid, 0)];
      bool written = false;   // an entry that non_max_suppression overwrites in place keeps its own memory
      for (const auto& wv : input_writers) written |= wv.second == g.entry_id(nid, 0) || wv.second == g.entry_id(n.inputs[0]);
      if (!out.ptr && !out.nhwc && out.dtype == x.dtype && !written) {
        out.ptr = x.ptr;  // alias
        return;
      }
    }
    const DevBuf y = materialize(g.entry_id(nid, 0));
    const Shape &xsh = x.shape, &ysh = y.shape;
    const auto xs = phys_strides(xsh, x.nhwc), ys = phys_strides(ysh, y.nhwc);
    const int xnd = (int)xsh.size(), ynd = (int)ysh.size();
    std::vector<GDim> dims;
    int64_t a_off = 0;
    if (op == "transpose") {
      Shape axes = n.attrs.t("axes");
      for (int j = 0; j < ynd; ++j) {
        int64_t ax = axes.empty() ? ynd - 1 - j : axes[j];
        if (ax < 0) ax += xnd;
        dims.push_back({ysh[j], xs[ax], ys[j]});
      }
    } else if (op == "strided_slice") {
      Shape b = n.attrs.t("begin"), st = n.attrs.t("stride");
      for (int i = (int)b.size(); i < xnd; ++i) b.push_back(0);
      for (int i = (int)st.size(); i < xnd; ++i) st.push_back(1);
      for (int j = 0; j < xnd; ++j) {
        const int64_t lo = st[j] < 0 ? -1 : 0, hi = st[j] < 0 ? xsh[j] - 1 : xsh[j];
        int64_t bg = b[j] < 0 ? b[j] + xsh[j] : b[j];
        bg = std::min(std::max(bg, lo), hi);
        a_off += bg * xs[j];
        dims.push_back({ysh[j], xs[j] * st[j], ys[j]});
      }
    } else if (op == "slice_like") {
      for (int j = 0; j < xnd; ++j) dims.push_back({ysh[j], xs[j], ys[j]});
    } else if (op == "repeat") {
      int axis = (int)n.attrs.i("axis");
      if (axis < 0) axis += xnd;
      const int64_t rep = n.attrs.i("repeats");
      for (int j = 0; j < xnd; ++j) {
        if (j == axis) {
          dims.push_back({xsh[j], xs[j], ys[j] * rep});
          dims.push_back({rep, 0, ys[j]});
        } else {
          dims.push_back({ysh[j], xs[j], ys[j]});
        }
      }
    } else {  // tile: right-aligned, output column c reads input column c % extent
      for (int j = 0; j < ynd; ++j) {
        const int xj = j - (ynd - xnd);
        if (xj < 0) {
          dims.push_back({ysh[j], 0, ys[j]});
        } else {
          dims.push_back({ysh[j] / xsh[xj], 0, ys[j] * xsh[xj]});
          dims.push_back({xsh[xj], xs[xj], ys[j]});
        }
      }
    }
    emit_gather(x, a_off, y, dims, op + ":" + n.name());
  }

  // A row-major buffer to produce entry `eid` into; finish_rowmajor() moves it into the entry's
  // own layout when that is channels-last.
  DevBuf rowmajor_target(uint32_t eid) {
    DevBuf& b = materialize(eid);
    if (!b.nhwc) return b;
    DevBuf t = b;
    t.nhwc = false;
    t.ptr = act_alloc(t.bytes());
    return t;
  }
  void finish_rowmajor(const DevBuf& t, uint32_t eid, const std::string& label) {
    if (t.ptr != buf[eid].ptr) emit_convert(t, buf[eid], label + ":to_nhwc");
  }

  // take (cpu/ops/ops.cc:868-945) and cvm_lut (:947-956)
  void lower_take(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const bool lut = n.op->name == "cvm_lut";
    const std::string label = n.op->name + ":" + n.name();
    const uint32_t e_x = g.entry_id(n.inputs[lut ? 1 : 0]), e_i = g.entry_id(n.inputs[lut ? 0 : 1]);
    const uint32_t eo = g.entry_id(nid, 0);
    cvmk_take_desc d;
    memset(&d, 0, sizeof(d));
    const DevBuf x = canon_view(e_x, label);
    d.x = x.ptr; d.x_dtype = x.dtype;
    if (lut || !n.attrs.has.at("axis")) {
      d.outer = 1; d.inner = 1;
      d.extent = shape_size(x.shape);
    } else {
      int axis = (int)n.attrs.i("axis");
      if (axis < 0) axis += (int)x.shape.size();
      d.outer = d.inner = 1;
      for (int j = 0; j < axis; ++j) d.outer *= x.shape[j];
      for (int j = axis + 1; j < (int)x.shape.size(); ++j) d.inner *= x.shape[j];
      d.extent = x.shape[axis];
    }
    d.count = shape_size(g.shape[e_i]);
    if (lut) {
      // flat lookup: the output has the shape, and therefore the layout, of the index tensor
      const DevBuf idx = materialize(e_i);
      const DevBuf y = materialize(eo);
      d.indices = idx.ptr; d.idx_dtype = idx.dtype; d.y = y.ptr; d.y_dtype = y.dtype;
      add_step(label, [d](cudaStream_t s) { return cvmk_take(&d, s); });
      return;
    }
    const DevBuf idx = canon_view(e_i, label + ":indices");
    const DevBuf y = rowmajor_target(eo);
    d.indices = idx.ptr; d.idx_dtype = idx.dtype; d.y = y.ptr; d.y_dtype = y.dtype;
    add_step(label, [d](cudaStream_t s) { return cvmk_take(&d, s); });
    finish_rowmajor(y, eo, label);
  }

  // where (cpu/ops/ops.cc:1049-1075).  x, y and the result share a shape, hence a layout; a
  // condition of that shape does too, and a 1-D condition indexes the outermost dimension, which is
  // outermost in both layouts.
  void lower_where(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const DevBuf c = materialize(g.entry_id(n.inputs[0]));
    const DevBuf x = materialize(g.entry_id(n.inputs[1]));
    const DevBuf y = materialize(g.entry_id(n.inputs[2]));
    const DevBuf o = materialize(g.entry_id(nid, 0));
    cvmk_where_desc d;
    memset(&d, 0, sizeof(d));
    d.cond = c.ptr; d.cond_dtype = c.dtype;
    d.x = x.ptr; d.x_dtype = x.dtype;
    d.y = y.ptr; d.y_dtype = y.dtype;
    d.out = o.ptr; d.out_dtype = o.dtype;
    d.n = shape_size(x.shape);
    d.inner = c.shape.size() == x.shape.size() ? 1 : d.n / x.shape[0];
    add_step("where:" + n.name(), [d](cudaStream_t s) { return cvmk_where(&d, s); });
  }

  void lower_gvc(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const std::string label = "get_valid_counts:" + n.name();
    const uint32_t in_eid = g.entry_id(n.inputs[0]);
    // Rows that are the network input, read by nobody else: the operator reads the uploaded bytes
    // and applies the input clamp itself, instead of a copy of the whole tensor doing it first.
    const bool from_raw = in_eid == data_eid && raw_in.dtype == CVMK_I32 && uses[in_eid] == 1 && !is_head[in_eid] &&
                          !buf[in_eid].ptr && !dev_env("CVM_B200_NO_GVC_FROM_INPUT");
    const DevBuf x = from_raw ? raw_in : canon_i32_view(in_eid, label);
    const int clamp = from_raw ? data_range : 0;
    const DevBuf vc = materialize(g.entry_id(nid, 0));
    const DevBuf y = materialize(g.entry_id(nid, 1));
    CHECK(vc.dtype == CVMK_I32 && y.dtype == CVMK_I32);
    const int B = (int)x.shape[0], N = (int)x.shape[1], K = (int)x.shape[2];
    const int thr = (int)n.attrs.i("score_threshold");
    add_step(label, [x, y, vc, B, N, K, thr, clamp](cudaStream_t s) {
      return cvmk_get_valid_counts_clamped((const int32_t*)x.ptr, (int32_t*)y.ptr, (int32_t*)vc.ptr, B, N, K, thr, clamp, s);
    });
  }

  void lower_nms(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const std::string label = "non_max_suppression:" + n.name();
    const DevBuf x = canon_i32_view(g.entry_id(n.inputs[0]), label);
    const DevBuf vc = canon_i32_view(g.entry_id(n.inputs[1]), label);
    const DevBuf y = materialize(g.entry_id(nid, 0));
    CHECK(y.dtype == CVMK_I32);
    cvmk_nms_desc d;
    memset(&d, 0, sizeof(d));
    d.x = (const int32_t*)x.ptr; d.valid_count = (const int32_t*)vc.ptr; d.y = (int32_t*)y.ptr;
    d.B = (int)x.shape[0]; d.N = (int)x.shape[1];
    d.max_output_size = (int)n.attrs.i("max_output_size");
    d.iou_threshold = (int)n.attrs.i("iou_threshold");
    d.top_k = (int)n.attrs.i("top_k");
    d.force_suppress = n.attrs.b("force_suppress") ? 1 : 0;
    d.scratch_bytes = cvmk_nms_scratch_bytes(d.B, d.N);
    d.scratch = act_alloc((size_t)d.scratch_bytes);
    // The CPU operator writes -1 over the input rows outside the top_k (nms.cc:93-97).  That is
    // visible when the input entry is a head or is read again by a later node.
    const uint32_t in_eid = g.entry_id(n.inputs[0]);
    bool observed = false;
    for (const auto& h : g.outputs) observed |= g.entry_id(h) == in_eid;
    for (uint32_t m = nid + 1; m < g.nodes.size(); ++m)
      for (const auto& e : g.nodes[m].inputs) observed |= g.entry_id(e) == in_eid;
    if (observed) {
      const DevBuf own = materialize(in_eid);
      VERIFY(own.ptr == x.ptr) << label << ": its input is read again after the operator, which needs the input "
                               << "stored as int32 rows";
      d.x_writeback = (int32_t*)own.ptr;
    }
    add_step(label, [d](cudaStream_t s) { return cvmk_non_max_suppression(&d, s); });
  }

  // Lifetimes of the activation buffers in schedule positions (one position per fused group, in
  // the order the groups are launched), then their physical backing.  A buffer is live from the
  // group that first writes it (the group of the producing node, which for a shortcut operand of
  // a fused join can precede the group whose lowering allocated it) to the last group that reads
  // it: the groups of all consumers of every graph entry stored in it (aliases of reshape-like
  // nodes included), the end of the inference for a head.  Reads and writes inside one group all
  // happen at that group's position.  Every kernel launched with programmatic dependent launch
  // waits for the whole preceding kernel before it touches global memory, so a buffer whose last
  // reader sits at position p can be overwritten from position p + 1 on.  The steps that are
  // launched per batch chunk while the input uploads run chunk after chunk, so everything they
  // touch stays live across that whole prefix.
  std::vector<int> step_pos;   // step -> schedule position (-1: before the first group)
  void plan_activations(const std::vector<std::pair<uint32_t, uint32_t>>& order) {
    auto& act = ex.act_;
    if (act.empty()) return;
    const int end = (int)order.size() + 1;
    std::vector<int> pos(g.nodes.size(), -1);
    for (size_t i = 0; i < order.size(); ++i) pos[order[i].second] = (int)i;
    auto group_pos = [&](uint32_t nid) { return root_of[nid] == UINT32_MAX ? -1 : pos[root_of[nid]]; };
    for (auto& a : act) a.first = a.last = pos[a.root];
    auto find = [&](const void* p) -> Executor::ActBuf* {
      for (auto& a : act)
        if ((const char*)p >= (const char*)a.va && (const char*)p < (const char*)a.va + a.va_size) return &a;
      return nullptr;
    };
    std::vector<Executor::ActBuf*> of_entry(g.num_entries, nullptr);
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid)
      for (uint32_t eid = g.node_row_ptr[nid]; eid < g.node_row_ptr[nid + 1]; ++eid) {
        if (!buf[eid].ptr) continue;
        Executor::ActBuf* a = of_entry[eid] = find(buf[eid].ptr);
        if (!a) continue;
        a->first = std::min(a->first, g.nodes[nid].is_variable() ? -1 : group_pos(nid));
        if (is_head[eid]) a->last = end;
      }
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid)
      for (const auto& e : g.nodes[nid].inputs)
        if (Executor::ActBuf* a = of_entry[g.entry_id(e)]) a->last = std::max(a->last, group_pos(nid));
    for (auto& a : act) { a.first0 = a.first; a.last0 = a.last; }
    ex.step_pos_ = step_pos;
    // first with the longest prefix that may be chosen; the constructor plans again once it is known
    ex.PlanForPrefix(ex.prefix_max_);
  }

  void lower_node(uint32_t nid) {
    const Node& n = g.nodes[nid];
    const std::string& op = n.op->name;
    if (op == "conv2d") return lower_conv_like(nid, false);
    if (op == "dense") return lower_conv_like(nid, true);
    if (op == "max_pool2d") return lower_pool(nid);
    if (op == "upsampling") return lower_upsampling(nid);
    if (op == "concatenate") return lower_concat(nid);
    if (op == "flatten" || op == "reshape" || op == "squeeze" || op == "expand_dims") return lower_reshape(nid);
    if (op == "sum" || op == "max") return lower_reduce(nid);
    if (op == "transpose" || op == "strided_slice" || op == "slice_like" || op == "repeat" || op == "tile")
      return lower_index_map(nid);
    if (op == "take" || op == "cvm_lut") return lower_take(nid);
    if (op == "where") return lower_where(nid);
    if (op == "get_valid_counts") return lower_gvc(nid);
    if (op == "non_max_suppression") return lower_nms(nid);
    if (lower_elemwise_root(nid)) return;
    if (op.compare(0, 10, "broadcast_") == 0 || op == "elemwise_add" || op == "elemwise_sub")
      return lower_broadcast(nid);
    FATAL() << "function undefined cvm.runtime.gpu." << op;
  }

  void run() {
    analyse();
    find_input_writers();
    // graph input: raw API bytes -> clamp to the declared precision -> entry buffer
    int data_nid = -1;
    for (uint32_t nid = 0; nid < g.nodes.size(); ++nid)
      if (g.nodes[nid].is_data()) data_nid = (int)nid;
    CHECK(data_nid >= 0) << "can not find input `data`";
    {
      const uint32_t eid = g.entry_id(data_nid, 0);
      const int prec = g.precision[eid];
      data_eid = eid;
      raw_in.shape = g.shape[eid];
      raw_in.dtype = prec > 8 ? CVMK_I32 : CVMK_I8;
      raw_in.nhwc = false;
      ex.in_bytes_ = raw_in.bytes();
      ex.in_dev_ = ex.dalloc(ex.in_bytes_);
      CUDA_OK(cudaMallocHost(&ex.in_host_, ex.in_bytes_));
      memset(ex.in_host_, 0, ex.in_bytes_);
      ex.pinned_.push_back(ex.in_host_);
      raw_in.ptr = ex.in_dev_;
      data_range = (int32_t)((1u << (prec - 1)) - 1);
    }
    // Fused groups are emitted at the position of their last member, so every operand of the
    // chain already exists when the kernel runs.
    std::vector<std::pair<uint32_t, uint32_t>> order;  // (schedule position, root)
    {
      // A dry pass decides the groups; the step lists of the groups are then ordered by tail.
      std::vector<std::vector<Step>> per_root(g.nodes.size());
      std::vector<uint32_t> tail(g.nodes.size(), 0);
      root_of.assign(g.nodes.size(), UINT32_MAX);
      std::vector<Step> prologue = ex.steps_;
      ex.steps_.clear();
      for (uint32_t nid = 0; nid < g.nodes.size(); ++nid) {
        const Node& n = g.nodes[nid];
        if (n.is_variable() || absorbed[nid]) continue;
        const size_t before = ex.steps_.size();
        uint32_t last = nid;
        cur_root = nid;
        root_of[nid] = nid;
        lower_node(nid);
        cur_root = UINT32_MAX;
        for (uint32_t k = nid + 1; k < g.nodes.size(); ++k)
          if (absorbed[k] == 1) { absorbed[k] = 2; root_of[k] = nid; last = std::max(last, k); }
        per_root[nid].assign(ex.steps_.begin() + before, ex.steps_.end());
        ex.steps_.resize(before);
        tail[nid] = last;
        order.emplace_back(last, nid);
      }
      std::stable_sort(order.begin(), order.end());
      ex.steps_ = prologue;
      if (buf[data_eid].ptr || is_head[data_eid]) {
        // some consumer reads the input tensor itself: raw API bytes -> clamp to the declared
        // precision (graph_runtime.cc:379-386) -> the entry's own layout
        cvmk_epilogue ep;
        memset(&ep, 0, sizeof(ep));
        ep.n = 1;
        ep.s[0].op = CVMK_EP_CLIP;
        ep.s[0].a = -data_range;
        ep.s[0].b = data_range;
        emit_convert(raw_in, materialize(data_eid), "input:data", &ep);
      }
      step_pos.assign(ex.steps_.size(), -1);
      for (size_t i = 0; i < order.size(); ++i)
        for (auto& s : per_root[order[i].second]) {
          ex.steps_.push_back(std::move(s));
          step_pos.push_back((int)i);
        }
    }
    // Upload / compute overlap: when the inference starts with the stem, the leading run of steps
    // that can be cut along the batch (about as much work as the upload takes) is launched per
    // chunk, outside the graph.
    {
      const std::string tag = "[stem]";
      const bool first = !ex.steps_.empty() && ex.steps_[0].chunk.size() > 1 && ex.steps_[0].label.size() >= tag.size() &&
                         ex.steps_[0].label.compare(ex.steps_[0].label.size() - tag.size(), tag.size(), tag) == 0;
      // The lengths actually used are chosen after the load-time measurements.  Everything the prefix
      // touches is live for all of it (whole-batch buffers, filled chunk by chunk), so its length is
      // also a memory decision: ten steps of ResNet-50 at batch 256 hold 1.3 GB, twenty 2.1 GB.
      const size_t cap = 10;
      ex.prefix_max_ = 0;
      if (first)
        while (ex.prefix_max_ < ex.steps_.size() && ex.prefix_max_ < cap && ex.steps_[ex.prefix_max_].chunk.size() == ex.steps_[0].chunk.size())
          ++ex.prefix_max_;
    }
    plan_activations(order);
    // heads: row-major staging + pinned host mirrors
    for (const auto& e : g.outputs) {
      const uint32_t eid = g.entry_id(e);
      DevBuf c = canon_view(eid, "head");
      HeadOut h;
      h.shape = c.shape;
      h.dtype = c.dtype;
      h.dev = c.ptr;
      h.bytes = c.bytes();
      CUDA_OK(cudaMallocHost(&h.host, h.bytes));
      ex.pinned_.push_back(h.host);
      ex.heads_.push_back(h);
    }
  }
};

Executor::Executor(const Graph& g, int device_id) : g_(g), device_(device_id) {
  int count = 0;
  CUDA_OK(cudaGetDeviceCount(&count));
  CHECK(device_id >= 0 && device_id < count) << "device_id " << device_id << " out of range (" << count << " GPUs)";
  CUDA_OK(cudaSetDevice(device_));
  CUDA_OK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  status_dev_ = (int32_t*)dalloc(256);
  CUDA_OK(cudaMemset(status_dev_, 0, 256));
  CUDA_OK(cudaMallocHost((void**)&status_host_, 256));
  pinned_.push_back(status_host_);
  *status_host_ = 0;
  use_graph_ = dev_env("CVM_B200_NO_GRAPH") == nullptr;
  if (vmm().ok && !dev_env("CVM_B200_NO_PLANNER")) {
    const CUmemAllocationProp prop = device_prop(device_);
    size_t gran = 0;
    if (vmm().get_granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) == CUDA_SUCCESS && gran > 0) {
      vmm_ = true;
      vmm_gran_ = gran;
    }
  }
  Lowering low(*this, g);
  low.run();
  // One eager pass sets per-kernel attributes and surfaces launch errors before capture.
  Upload(in_host_, stream_);
  Enqueue(stream_);
  CUDA_OK(cudaStreamSynchronize(stream_));
  if (use_graph_) {
    ChoosePrefixes();
    CUDA_OK(cudaStreamSynchronize(stream_));
    PlanForPrefix(std::max(prefix_steps_, prefix_steps_pageable_));   // memory for the prefix actually used
    if (prefix_steps_ > 0 || prefix_steps_pageable_ > 0) {
      CUDA_OK(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
      chunk_events_.resize(steps_[0].chunk.size());
      for (auto& e : chunk_events_) CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    auto capture_from = [&](size_t first, cudaGraphExec_t* exec) {
      cudaGraph_t graph = nullptr;
      CUDA_OK(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
      Enqueue(stream_, first);  // the chunked prefix is launched outside the graph
      CUDA_OK(cudaStreamEndCapture(stream_, &graph));
      CUDA_OK(cudaGraphInstantiate(exec, graph, 0));
      CUDA_OK(cudaGraphDestroy(graph));
    };
    capture_from(prefix_steps_, &graph_exec_);
    if (prefix_steps_pageable_ != prefix_steps_) capture_from(prefix_steps_pageable_, &graph_exec_pageable_);
  }
}

bool Executor::IsDirect(const void* input) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, input) == cudaSuccess)
    return at.type == cudaMemoryTypeHost || at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
  cudaGetLastError();
  return false;
}

// How many leading steps to run chunk by chunk: the fewest whose device time, measured here step
// by step on the whole batch and scaled by 1.3 (a quarter of the batch runs less efficiently than
// the whole), reaches the time the upload takes -- measured here too, once for a page-locked source
// and once through the staging path a pageable source takes.
void Executor::ChoosePrefixes() {
  prefix_steps_ = prefix_steps_pageable_ = 0;
  if (prefix_max_ == 0 || dev_env("CVM_B200_NO_UPLOAD_OVERLAP")) { prefix_max_ = 0; return; }
  if (const char* e = dev_env("CVM_B200_PREFIX_STEPS")) {
    prefix_steps_ = prefix_steps_pageable_ = std::min(prefix_max_, (size_t)atoi(e));
    return;
  }
  std::vector<cudaEvent_t> ev(prefix_max_ + 1);
  for (auto& e : ev) CUDA_OK(cudaEventCreate(&e));
  std::vector<double> step_ms(prefix_max_, 0.0);
  for (int rep = 0; rep < 2; ++rep) {   // the second pass is the warm one
    CUDA_OK(cudaEventRecord(ev[0], stream_));
    for (size_t k = 0; k < prefix_max_; ++k) {
      KERNEL_OK(steps_[k].launch(stream_));
      CUDA_OK(cudaEventRecord(ev[k + 1], stream_));
    }
    CUDA_OK(cudaStreamSynchronize(stream_));
  }
  for (size_t k = 0; k < prefix_max_; ++k) {
    float ms = 0;
    CUDA_OK(cudaEventElapsedTime(&ms, ev[k], ev[k + 1]));
    step_ms[k] = ms;
  }
  auto upload_ms = [&](const void* src) {
    double best = 1e30;
    for (int rep = 0; rep < 2; ++rep) {
      CUDA_OK(cudaEventRecord(ev[0], stream_));
      Upload(src, stream_);
      CUDA_OK(cudaEventRecord(ev[1], stream_));
      const auto t0 = std::chrono::steady_clock::now();
      CUDA_OK(cudaStreamSynchronize(stream_));
      float ms = 0;
      CUDA_OK(cudaEventElapsedTime(&ms, ev[0], ev[1]));
      // a pageable source is staged by host threads while the stream waits: wall time counts
      const double wall = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
      best = std::min(best, std::max((double)ms, wall));
    }
    return best;
  };
  const double t_pinned = upload_ms(in_host_);
  std::vector<char> pageable(in_bytes_, 0);
  const double t_pageable = upload_ms(pageable.data());
  auto pick = [&](double t_upload) {
    double sum = 0;
    size_t n = 0;
    while (n < prefix_max_ && 1.3 * sum < t_upload) sum += step_ms[n++];
    return n;
  };
  prefix_steps_ = pick(t_pinned);
  prefix_steps_pageable_ = std::max(prefix_steps_, pick(t_pageable));
  if (dev_env("CVM_B200_VERBOSE"))
    fprintf(stderr, "upload %.3f ms page-locked, %.3f ms pageable: %zu / %zu of %zu leading steps run per chunk\n", t_pinned,
            t_pageable, prefix_steps_, prefix_steps_pageable_, prefix_max_);
  for (auto& e : ev) cudaEventDestroy(e);
}

Executor::~Executor() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
  if (graph_exec_pageable_) cudaGraphExecDestroy(graph_exec_pageable_);
  if (kernels_exec_) cudaGraphExecDestroy(kernels_exec_);
  for (auto e : chunk_events_) cudaEventDestroy(e);
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
  for (void* p : allocs_) cudaFree(p);
  for (auto& a : act_) {
    if (a.block >= 0) vmm().unmap(reinterpret_cast<CUdeviceptr>(a.va), a.va_size);
    vmm().address_free(reinterpret_cast<CUdeviceptr>(a.va), a.va_size);
  }
  for (auto& b : phys_) vmm().release((CUmemGenericAllocationHandle)b.handle);
  for (void* p : pinned_) cudaFreeHost(p);
  if (stream_) cudaStreamDestroy(stream_);
}

StagePool::StagePool(int threads) {
  for (int i = 0; i < threads; ++i) workers_.emplace_back([this] { Work(); });
}

StagePool::~StagePool() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
}

void StagePool::Start(const char* src, char* dst, size_t bytes, size_t piece) {
  std::lock_guard<std::mutex> lk(mu_);
  src_ = src; dst_ = dst; bytes_ = bytes; piece_ = piece;
  pieces_ = (bytes + piece - 1) / piece;
  if (pieces_ > done_cap_) {
    done_.reset(new std::atomic<int>[pieces_]);
    done_cap_ = pieces_;
  }
  for (size_t k = 0; k < pieces_; ++k) done_[k].store(0, std::memory_order_relaxed);
  next_.store(0, std::memory_order_release);
  ++job_;
  cv_.notify_all();
}

void StagePool::Work() {
  uint64_t seen = 0;
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return stop_ || job_ != seen; });
      if (stop_) return;
      seen = job_;
    }
    for (;;) {
      const size_t k = next_.fetch_add(1, std::memory_order_acq_rel);
      if (k >= pieces_) break;
      const size_t off = k * piece_;
      memcpy(dst_ + off, src_ + off, std::min(piece_, bytes_ - off));
      done_[k].store(1, std::memory_order_release);
    }
  }
}

void StagePool::WaitPiece(size_t k) {
  // the caller helps out instead of idling: pieces are small, so this never waits long
  while (!done_[k].load(std::memory_order_acquire)) {
    const size_t j = next_.fetch_add(1, std::memory_order_acq_rel);
    if (j < pieces_) {
      const size_t off = j * piece_;
      memcpy(dst_ + off, src_ + off, std::min(piece_, bytes_ - off));
      done_[j].store(1, std::memory_order_release);
    } else {
      std::this_thread::yield();
    }
  }
}

// Queues the upload of one input.  Page-locked (or device) memory is read where it lies; pageable
// memory goes through the pinned staging buffer in pieces that a few host threads copy in
// parallel, each piece being sent to the device as soon as it is staged.
void Executor::Upload(const void* input, cudaStream_t s) { UploadRange(input, 0, in_bytes_, s); }

void Executor::UploadRange(const void* input, size_t begin, size_t bytes, cudaStream_t s) {
  if (IsDirect(input)) {
    CUDA_OK(cudaMemcpyAsync((char*)in_dev_ + begin, (const char*)input + begin, bytes, cudaMemcpyDefault, s));
    return;
  }
  const size_t piece = (size_t)1 << 20;
  if (bytes <= 2 * piece) {   // small inputs: not worth waking anyone
    memcpy((char*)in_host_ + begin, (const char*)input + begin, bytes);
    CUDA_OK(cudaMemcpyAsync((char*)in_dev_ + begin, (char*)in_host_ + begin, bytes, cudaMemcpyHostToDevice, s));
    return;
  }
  if (!stage_pool_) {
    unsigned hw = std::thread::hardware_concurrency();
    int gpus = 1;
    cudaGetDeviceCount(&gpus);
    // three helpers beside the calling thread, fewer when the host has few cores per GPU
    int helpers = hw ? std::max(1, std::min(3, (int)hw / std::max(1, gpus) - 1)) : 1;
    stage_pool_.reset(new StagePool(helpers));
  }
  stage_pool_->Start((const char*)input + begin, (char*)in_host_ + begin, bytes, piece);
  // the transfer is issued in groups of four pieces: fewer driver calls, still well pipelined
  const size_t group = 4;
  for (size_t k = 0; k < stage_pool_->pieces(); k += group) {
    const size_t last = std::min(stage_pool_->pieces(), k + group);
    for (size_t j = k; j < last; ++j) stage_pool_->WaitPiece(j);
    const size_t off = begin + k * piece;
    const size_t n = std::min(group * piece, begin + bytes - off);
    CUDA_OK(cudaMemcpyAsync((char*)in_dev_ + off, (char*)in_host_ + off, n, cudaMemcpyHostToDevice, s));
  }
}

void Executor::Enqueue(cudaStream_t s, size_t first) {
  for (size_t k = first; k < steps_.size(); ++k) {
    auto& st = steps_[k];
    int rc = st.launch(s);
    CHECK(rc == CVMK_OK) << "step " << st.label << " failed (" << rc << "): " << cvmk_last_error();
  }
  for (auto& h : heads_) CUDA_OK(cudaMemcpyAsync(h.host, h.dev, h.bytes, cudaMemcpyDeviceToHost, s));
  CUDA_OK(cudaMemcpyAsync(status_host_, status_dev_, 4, cudaMemcpyDeviceToHost, s));
}

void Executor::Run(const void* input, size_t input_bytes) {
  CHECK(input_bytes == in_bytes_) << "input size " << input_bytes << " vs. " << in_bytes_;
  CUDA_OK(cudaSetDevice(device_));
  const bool pageable = graph_exec_pageable_ && !IsDirect(input);
  const size_t prefix = pageable ? prefix_steps_pageable_ : prefix_steps_;
  if (graph_exec_ && prefix > 0) {
    // chunk c of the batch is uploaded on the copy stream while the leading steps run on chunk c - 1
    for (size_t c = 0; c < steps_[0].chunk.size(); ++c) {
      UploadRange(input, c * chunk_bytes_, chunk_bytes_, copy_stream_);
      CUDA_OK(cudaEventRecord(chunk_events_[c], copy_stream_));
      CUDA_OK(cudaStreamWaitEvent(stream_, chunk_events_[c], 0));
      for (size_t k = 0; k < prefix; ++k) {
        const int rc = steps_[k].chunk[c](stream_);
        CHECK(rc == CVMK_OK) << "step " << steps_[k].label << " (chunk) failed (" << rc << "): " << cvmk_last_error();
      }
    }
    CUDA_OK(cudaGraphLaunch(pageable ? graph_exec_pageable_ : graph_exec_, stream_));
  } else {
    Upload(input, stream_);
    if (graph_exec_) CUDA_OK(cudaGraphLaunch(graph_exec_, stream_));
    else Enqueue(stream_);
  }
  CUDA_OK(cudaStreamSynchronize(stream_));
  if (*status_host_ != 0) {
    const int code = *status_host_;
    *status_host_ = 0;
    cudaMemsetAsync(status_dev_, 0, 4, stream_);
    cudaStreamSynchronize(stream_);
    FATAL() << "a device-side wait ran out (status word 0x" << std::hex << code << ")";
  }
}

void Executor::SetStatusWord(int code) {
  CUDA_OK(cudaSetDevice(device_));
  const int32_t v = code;
  CUDA_OK(cudaMemcpyAsync(status_dev_, &v, sizeof(v), cudaMemcpyHostToDevice, stream_));
  CUDA_OK(cudaStreamSynchronize(stream_));
}

float Executor::ReplayDevice(int iters) {
  CHECK(iters > 0);
  CUDA_OK(cudaSetDevice(device_));
  if (use_graph_ && !kernels_exec_) {
    cudaGraph_t graph = nullptr;
    CUDA_OK(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
    for (auto& st : steps_) KERNEL_OK(st.launch(stream_));
    CUDA_OK(cudaStreamEndCapture(stream_, &graph));
    CUDA_OK(cudaGraphInstantiate(&kernels_exec_, graph, 0));
    CUDA_OK(cudaGraphDestroy(graph));
  }
  cudaEvent_t e0, e1;
  CUDA_OK(cudaEventCreate(&e0));
  CUDA_OK(cudaEventCreate(&e1));
  CUDA_OK(cudaEventRecord(e0, stream_));
  for (int i = 0; i < iters; ++i) {
    if (kernels_exec_) CUDA_OK(cudaGraphLaunch(kernels_exec_, stream_));
    else for (auto& st : steps_) KERNEL_OK(st.launch(stream_));
  }
  CUDA_OK(cudaEventRecord(e1, stream_));
  CUDA_OK(cudaEventSynchronize(e1));
  float ms = 0;
  CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return ms;
}

std::vector<std::pair<std::string, float>> Executor::ProfileOnce(const void* input, size_t input_bytes) {
  CHECK(input_bytes == in_bytes_);
  CUDA_OK(cudaSetDevice(device_));
  std::vector<std::pair<std::string, float>> out;
  std::vector<cudaEvent_t> ev(steps_.size() + 1);
  for (auto& e : ev) CUDA_OK(cudaEventCreate(&e));
  Upload(input, stream_);
  CUDA_OK(cudaEventRecord(ev[0], stream_));
  for (size_t i = 0; i < steps_.size(); ++i) {
    KERNEL_OK(steps_[i].launch(stream_));
    CUDA_OK(cudaEventRecord(ev[i + 1], stream_));
  }
  CUDA_OK(cudaStreamSynchronize(stream_));
  for (size_t i = 0; i < steps_.size(); ++i) {
    float ms = 0;
    CUDA_OK(cudaEventElapsedTime(&ms, ev[i], ev[i + 1]));
    out.emplace_back(steps_[i].label, ms);
  }
  for (auto& e : ev) cudaEventDestroy(e);
  return out;
}

}  // namespace cvm
