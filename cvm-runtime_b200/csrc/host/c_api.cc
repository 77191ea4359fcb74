// The model wrapper (CVMModel, src/core/model.cc) and the C entry points (src/core/c_api.cc).
#include "cvm/c_api.h"
#include "cvm/c_api_ext.h"
#include <cstdio>
#include <cstring>
#include <memory>
#include "executor.h"
#include "graph.h"

namespace cvm {

// Host-side pre/post-processing of one loaded model; byte-for-byte the behaviour of
// cvm::runtime::CVMModel.
class Model {
 public:
  Model(const std::string& graph_json, int device_id) : device_id_(device_id) {
    g_.Init(graph_json);
    g_.GetStorageSize();  // the reference constructor evaluates it and fails above 4 GiB (model.cc:39)
    out_num_ = (int)g_.outputs.size();
    if (out_num_ < 1) return;
    postprocess_ = g_.postprocess.substr(0, 32);
    const int input_precision = g_.GetInputPrecision();
    input_bytes_ = input_precision > 8 ? 4 : 1;
    output_bytes_ = g_.GetOutputPrecision() > 8 ? 4 : 1;
    if (postprocess_ == "argmax" || postprocess_ == "detection") output_bytes_ = 4;
    version_ = g_.version.substr(0, 32);
    // get_input_shape("data") indexes the shape table with the position of `data` among the
    // arg nodes, not with its entry id (graph_runtime.cc:722-733 + :269-279); kept as is.
    const int in_idx = g_.GetInputIndex("data");
    VERIFY_LE((size_t)in_idx, g_.shape.size());
    CHECK((size_t)in_idx < g_.shape.size());
    in_shape_ = g_.shape[in_idx];
    in_size_ = shape_size(in_shape_);
    for (const auto& e : g_.outputs) {
      out_shapes_.push_back(g_.shape[g_.entry_id(e)]);
      out_size_.push_back(shape_size(out_shapes_.back()));
    }
    loaded_ = true;
  }

  bool IsReady() const { return loaded_; }

  void LoadParams(const std::string& params) {
    VERIFY_NE(params.size(), 0U);
    g_.LoadParams(params);
    g_.RaiseRefusal();
    exec_.reset(new Executor(g_, device_id_));
  }

  int GetInputLength() const { return (int)in_size_ * input_bytes_; }

  // model.cc:297-327
  int GetOutputLength() const {
    int ret = 0;
    if (postprocess_ == "argmax") {
      for (int k = 0; k < out_num_; ++k) {
        const uint32_t last_dim = (uint32_t)out_shapes_[k].back();
        ret += (int)((uint32_t)out_size_[k] / last_dim);
      }
    } else if (postprocess_ == "detection") {
      const Shape& s0 = out_shapes_[0];
      const int rows = s0.size() >= 2 ? (int)s0[s0.size() - 2] : 0;
      for (int k = 0; k < out_num_; ++k) ret += (int)(uint32_t)out_shapes_[k].back();
      ret *= rows;
    } else {
      for (int k = 0; k < out_num_; ++k) ret += (int)out_size_[k];
    }
    return ret * output_bytes_;
  }

  void Inference(const char* input, int input_len, char* output) {
    VERIFY_EQ(GetInputLength(), input_len);
    CHECK(exec_) << "model parameters have not been loaded";
    // CvmRuntime::SetInput compares the tensor handed in (shaped as above) with the data entry.
    const Shape* expected = nullptr;
    for (size_t i = 0; i < g_.nodes.size(); ++i)
      if (g_.nodes[i].is_data()) expected = &g_.shape[g_.entry_id(i, 0)];
    CHECK(expected);
    VERIFY_EQ(in_shape_.size(), expected->size())
        << "Loaded data shape ndim " << in_shape_.size() << " not matched " << expected->size();
    for (size_t i = 0; i < expected->size(); ++i)
      VERIFY_EQ(in_shape_[i], (*expected)[i]) << "Loaded data shape at index " << i << " with value "
                                              << in_shape_[i] << ", Expected " << (*expected)[i];
    exec_->Run(input, (size_t)input_len);
    SaveTensor(output);
  }

  Executor& executor() {
    CHECK(exec_) << "model parameters have not been loaded";
    return *exec_;
  }
  int64_t GetStorageSize() const { return g_.GetStorageSize(); }
  int64_t GetOps() const { return g_.GetOps(); }
  int input_bytes() const { return input_bytes_; }
  int output_bytes() const { return output_bytes_; }
  const std::string& version() const { return version_; }
  const std::string& postprocess() const { return postprocess_; }

 private:
  Graph g_;
  std::unique_ptr<Executor> exec_;
  int device_id_;
  int out_num_ = 0;
  int input_bytes_ = 1, output_bytes_ = 1;
  std::string postprocess_, version_;
  Shape in_shape_;
  int64_t in_size_ = 0;
  std::vector<Shape> out_shapes_;
  std::vector<int64_t> out_size_;
  bool loaded_ = false;

  inline int32_t at(const HeadOut& h, size_t i) const {
    return h.dtype == CVMK_I8 ? (int32_t) reinterpret_cast<const int8_t*>(h.host)[i]
                              : reinterpret_cast<const int32_t*>(h.host)[i];
  }

  // CVMModel::SaveTensor, model.cc:181-263
  void SaveTensor(char* mem) const {
    const auto& heads = exec_->heads();
    if (postprocess_ == "argmax") {
      int32_t* cp = reinterpret_cast<int32_t*>(mem);
      for (int k = 0; k < out_num_; ++k) {
        const uint32_t last_dim = (uint32_t)out_shapes_[k].back();
        const uint32_t out_size_ap = (uint32_t)out_size_[k] / last_dim;
        // The loop bound is the row count while the index advances by a row length; reproduced.
        for (size_t i = 0; i < out_size_ap; i += last_dim) {
          uint32_t max_id = 0;
          for (size_t j = i; j < i + last_dim; j++)
            if ((int8_t)at(heads[k], j) > (int8_t)at(heads[k], i + max_id)) max_id = (uint32_t)(j - i);
          *cp++ = (int32_t)max_id;
        }
      }
    } else if (postprocess_ == "detection" || heads.size() > 1) {
      bool can_concat = heads.size() != 1;
      std::vector<uint64_t> xs(heads.size()), ys(heads.size());
      if (can_concat) {
        for (size_t k = 0; k < heads.size(); ++k) {
          ys[k] = (uint64_t)out_shapes_[k].back();
          xs[k] = (uint64_t)out_size_[k] / ys[k];
        }
        for (size_t k = 1; k < heads.size(); ++k)
          if (xs[k] != xs[0]) { can_concat = false; break; }
      }
      VERIFY(can_concat) << "detection model output cannot concat";
      if (output_bytes_ == 4) {
        int32_t* cp = reinterpret_cast<int32_t*>(mem);
        const int32_t nx = (int32_t)xs[0];
        for (int x = 0; x < nx; x++)
          for (size_t k = 0; k < heads.size(); ++k)
            for (size_t i = 0; i < ys[k]; ++i) *cp++ = at(heads[k], (size_t)x * ys[k] + i);
      } else {
        char* cp = mem;
        for (size_t x = 0; x < xs[0]; x++)
          for (size_t k = 0; k < heads.size(); ++k)
            for (size_t i = 0; i < ys[k]; ++i) *cp++ = (char)(int8_t)at(heads[k], x * ys[k] + i);
      }
    } else if (output_bytes_ == 4) {
      int32_t* ref = reinterpret_cast<int32_t*>(mem);
      for (size_t k = 0; k < heads.size(); ++k) {
        if (heads[k].dtype == CVMK_I32) memcpy(ref, heads[k].host, sizeof(int32_t) * out_size_[k]);
        else for (int64_t i = 0; i < out_size_[k]; ++i) ref[i] = at(heads[k], i);
        ref += out_size_[k];
      }
    } else {
      for (size_t k = 0; k < heads.size(); ++k) {
        if (heads[k].dtype == CVMK_I8) { memcpy(mem, heads[k].host, out_size_[k]); mem += out_size_[k]; }
        else for (int64_t i = 0; i < out_size_[k]; ++i) *mem++ = (char)(int8_t)at(heads[k], i);
      }
    }
  }
};

}  // namespace cvm

using cvm::Model;

// include/cvm/errors.h:15-36
static std::string& last_error_text() {
  static thread_local std::string text;
  return text;
}
static int report(const std::exception& e, int status) {
  last_error_text() = e.what();
  printf("ERROR: %s\n", e.what());
  return status;
}

#define API_BEGIN() try {
#define API_END()                                                             \
  }                                                                           \
  catch (const std::runtime_error& e) { return report(e, ERROR_RUNTIME); }    \
  catch (const std::logic_error& e) { return report(e, ERROR_LOGIC); }        \
  catch (const std::exception& e) { return report(e, ERROR_RUNTIME); }        \
  return SUCCEED;

extern "C" {

int CVMAPILoadModel(const char* graph_json, int graph_strlen, const char* param_bytes, int param_strlen,
                    void** net, int device_type, int device_id) {
  API_BEGIN();
  CHECK(graph_json != nullptr && param_bytes != nullptr && net != nullptr);
  std::string graph(graph_json, graph_strlen);
  std::string params(param_bytes, param_strlen);
  CHECK(device_type == 0 || device_type == 1 || device_type == 2)
      << "Invalid device type: " << device_type << ", only supported 0(CPU), 1(GPU), 2(FORMAL)\n";
  CHECK(device_type == 1) << "device type " << device_type
                          << " is not available in this library: operators run on the GPU only (use 1)";
  std::unique_ptr<Model> model(new Model(graph, device_id));
  if (!model->IsReady()) return ERROR_LOGIC;
  model->LoadParams(params);
  *net = (void*)model.release();
  API_END();
}

int CVMAPIFreeModel(void* net) {
  API_BEGIN();
  if (net) delete static_cast<Model*>(net);
  API_END();
}

int CVMAPIInference(void* net, char* input_data, int input_len, char* output_data) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(input_data != nullptr); CHECK(output_data != nullptr);
  static_cast<Model*>(net)->Inference(input_data, input_len, output_data);
  API_END();
}

int CVMAPIGetVersion(void* net, char* version) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(version != nullptr);
  strcpy(version, static_cast<Model*>(net)->version().c_str());
  API_END();
}

int CVMAPIGetPreprocessMethod(void* net, char* method) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(method != nullptr);
  strcpy(method, static_cast<Model*>(net)->postprocess().c_str());
  API_END();
}

int CVMAPIGetInputLength(void* net, unsigned long long* size) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(size != nullptr);
  *size = (unsigned long long)static_cast<Model*>(net)->GetInputLength();
  API_END();
}

int CVMAPIGetOutputLength(void* net, unsigned long long* size) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(size != nullptr);
  *size = (unsigned long long)static_cast<Model*>(net)->GetOutputLength();
  API_END();
}

int CVMAPIGetOutputTypeSize(void* net, unsigned long long* size) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(size != nullptr);
  *size = (unsigned long long)static_cast<Model*>(net)->output_bytes();
  API_END();
}

int CVMAPIGetInputTypeSize(void* net, unsigned long long* size) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(size != nullptr);
  *size = (unsigned long long)static_cast<Model*>(net)->input_bytes();
  API_END();
}

int CVMAPIGetStorageSize(void* net, unsigned long long* gas) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(gas != nullptr);
  *gas = (unsigned long long)static_cast<Model*>(net)->GetStorageSize();
  API_END();
}

int CVMAPIGetGasFromModel(void* net, unsigned long long* gas) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(gas != nullptr);
  *gas = (unsigned long long)static_cast<Model*>(net)->GetOps();
  API_END();
}

int CVMAPIGetGasFromGraphFile(const char* graph_json, unsigned long long* gas) {
  API_BEGIN();
  std::string json(graph_json);
  cvm::Graph g;
  g.Init(json);
  const int64_t ops = g.GetOps();
  g.RaiseRefusal();
  *gas = (unsigned long long)ops;
  API_END();
}

// ---- measurement helpers (include/cvm/c_api_ext.h); not part of the reference ABI ----------

const char* CVMXLastError(void) { return last_error_text().c_str(); }

int CVMXStepCount(void* net, unsigned long long* n) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(n != nullptr);
  *n = (unsigned long long)static_cast<Model*>(net)->executor().num_steps();
  API_END();
}

int CVMXDeviceBytes(void* net, unsigned long long* n) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(n != nullptr);
  *n = (unsigned long long)static_cast<Model*>(net)->executor().device_bytes();
  API_END();
}

int CVMXActivationBytes(void* net, unsigned long long* buffers, unsigned long long* physical) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(buffers != nullptr); CHECK(physical != nullptr);
  static_cast<Model*>(net)->executor().activation_bytes(buffers, physical);
  API_END();
}

int CVMXReplayDevice(void* net, int iters, float* total_ms) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(total_ms != nullptr);
  *total_ms = static_cast<Model*>(net)->executor().ReplayDevice(iters);
  API_END();
}

int CVMXProfileSteps(void* net, const char* input_data, int input_len, char* text, int text_len) {
  API_BEGIN();
  CHECK(net != nullptr); CHECK(input_data != nullptr); CHECK(text != nullptr); CHECK(text_len > 0);
  auto rows = static_cast<Model*>(net)->executor().ProfileOnce(input_data, (size_t)input_len);
  std::string out;
  char line[64];
  for (const auto& r : rows) {
    snprintf(line, sizeof(line), "\t%.6f\n", r.second);
    out += r.first;
    out += line;
  }
  CHECK((int)out.size() < text_len) << "profile text needs " << out.size() + 1 << " bytes";
  memcpy(text, out.c_str(), out.size() + 1);
  API_END();
}

int CVMXSetStatusWord(void* net, int code) {
  API_BEGIN();
  CHECK(net != nullptr);
  static_cast<Model*>(net)->executor().SetStatusWord(code);
  API_END();
}

}  // extern "C"
