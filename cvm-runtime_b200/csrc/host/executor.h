// Device executor: lowers a validated Graph into a static list of kernel launches on one GPU and
// replays it per inference.
//
// The reference executor (CvmRuntime::SetupStorage / SetupOpExecs / Run,
// src/runtime/graph_runtime.cc:576-698, :61-68) binds one int32 buffer per entry and runs one
// operator body per node.  This one keeps the node-by-node semantics but chooses, at load time,
//   - a storage type per entry: int8 where every value is provably within [-127, 127], else int32;
//   - a physical layout: 4-D entries are held channels-last (NHWC), everything else row-major;
//   - fusion: chains of element-wise successors with a single consumer are folded into the
//     producing kernel (conv2d / dense / reduce / element-wise), so their int32 intermediates are
//     never written;
//   - pre-packed int8 weights (OIHW -> OHWI) and TMA tensor maps for the tensor-core convolutions;
//   - a CUDA graph of the whole step list and the output download; the input upload is queued
//     in front of it (straight from page-locked caller memory, staged in chunks otherwise).
// There is no CPU fallback: every step is a CUDA kernel from this library.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include "cvmk_kernels.h"
#include "graph.h"

namespace cvm {

struct DevBuf {
  Shape shape;          // logical shape
  int dtype = CVMK_I32; // CVMK_I8 / CVMK_I32
  bool nhwc = false;    // 4-D tensor stored as N,H,W,C
  void* ptr = nullptr;
  size_t bytes() const { return (size_t)shape_size(shape) * dtype; }
};

struct Step {
  std::string label;
  std::function<int(cudaStream_t)> launch;
  // The same operator on one quarter of the batch each (empty when the step cannot be cut along
  // the batch): the leading steps of an inference run chunk by chunk while later chunks upload.
  std::vector<std::function<int(cudaStream_t)>> chunk;
};

struct HeadOut {
  Shape shape;
  int dtype;
  void* dev = nullptr;       // canonical row-major copy on the device
  void* host = nullptr;      // pinned
  size_t bytes = 0;
};

// A few host threads that copy a pageable caller buffer into the page-locked staging buffer piece
// by piece, so that the copy runs at several times one core's memcpy rate and the transfer of a
// piece to the device starts as soon as that piece is staged.
class StagePool {
 public:
  explicit StagePool(int threads);
  ~StagePool();
  // Starts copying [src, src + bytes) to dst in pieces of `piece` bytes; returns at once.
  void Start(const char* src, char* dst, size_t bytes, size_t piece);
  // Blocks until piece k (0-based) of the current job has been copied.
  void WaitPiece(size_t k);
  size_t pieces() const { return pieces_; }

 private:
  void Work();
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  uint64_t job_ = 0;                 // generation counter: a new value wakes the workers
  const char* src_ = nullptr;
  char* dst_ = nullptr;
  size_t bytes_ = 0, piece_ = 0, pieces_ = 0;
  std::atomic<size_t> next_{0};
  std::unique_ptr<std::atomic<int>[]> done_;
  size_t done_cap_ = 0;
};

class Executor {
 public:
  Executor(const Graph& g, int device_id);
  ~Executor();
  // Runs one inference.  `input` holds the `data` tensor in API form (int8 or int32, row-major).
  // On return heads()[k].host holds head k (row-major, heads()[k].dtype).
  void Run(const void* input, size_t input_bytes);
  const std::vector<HeadOut>& heads() const { return heads_; }
  size_t num_steps() const { return steps_.size(); }
  size_t device_bytes() const { return device_bytes_; }
  void activation_bytes(unsigned long long* buffers, unsigned long long* physical) const {
    *buffers = 0;
    for (const auto& a : act_) *buffers += a.va_size;
    *physical = 0;
    for (const auto& b : phys_) *physical += b.size;
  }
  // Per-step device times of one eager pass (label, milliseconds); used by the profiling table.
  std::vector<std::pair<std::string, float>> ProfileOnce(const void* input, size_t input_bytes);
  // Replays only the kernels (input already in device memory, no upload / download) `iters`
  // times and returns the device time in milliseconds measured with CUDA events on the stream.
  float ReplayDevice(int iters);
  // Writes `code` into the device status word the kernels report their expired waits in.
  void SetStatusWord(int code);

 private:
  struct Impl;
  const Graph& g_;
  int device_;
  cudaStream_t stream_ = nullptr;
  std::vector<Step> steps_;
  // Leading steps launched per batch chunk, outside the graph, while later chunks upload: as many
  // as take about as long as the upload, which differs for a page-locked caller buffer (read by the
  // copy engine where it lies) and a pageable one (staged by host threads first).  Both lengths are
  // chosen at load from step times and upload rates measured there; prefix_max_ bounds them (the
  // memory planner keeps everything those steps touch live together).
  size_t prefix_steps_ = 0;            // page-locked input
  size_t prefix_steps_pageable_ = 0;   // pageable input
  size_t prefix_max_ = 0;
  cudaGraphExec_t graph_exec_pageable_ = nullptr;   // the steps from prefix_steps_pageable_ on
  void ChoosePrefixes();
  static bool IsDirect(const void* input);
  size_t chunk_bytes_ = 0;    // input bytes of one batch chunk
  std::vector<HeadOut> heads_;
  std::vector<void*> allocs_;
  std::vector<void*> pinned_;
  std::vector<std::unique_ptr<cvmk_conv_plan, void (*)(void*)>> plans_;
  std::vector<std::unique_ptr<cvmk_stem_conv_plan, void (*)(void*)>> stem_plans_;
  size_t device_bytes_ = 0;
  // input staging
  void* in_host_ = nullptr;
  void* in_dev_ = nullptr;
  size_t in_bytes_ = 0;
  int32_t* status_dev_ = nullptr;
  int32_t* status_host_ = nullptr;
  cudaGraphExec_t graph_exec_ = nullptr;
  cudaGraphExec_t kernels_exec_ = nullptr;
  bool use_graph_ = true;
  // upload / stem overlap: per-chunk stem plans, the copy stream and one event per chunk
  cudaStream_t copy_stream_ = nullptr;
  std::vector<cudaEvent_t> chunk_events_;
  std::unique_ptr<StagePool> stage_pool_;   // created by the first inference from pageable memory

  void* dalloc(size_t bytes);
  // Activation memory.  Every activation buffer gets a virtual address range of its own when the
  // graph is lowered (kernel descriptors and tensor maps are built on those addresses); once the
  // schedule is known, buffers whose lifetimes do not overlap are backed by the SAME physical
  // memory (CUDA virtual memory management: one physical allocation mapped at several addresses),
  // which is what the reference's storage planner does with its shared pool
  // (src/runtime/graph_runtime.cc:503-610).  Falls back to one cudaMalloc per buffer when the
  // driver's virtual memory calls are not available.
  struct ActBuf {
    void* va = nullptr;
    size_t bytes = 0, va_size = 0;
    uint32_t root = UINT32_MAX;   // node whose lowering made the allocation
    int first = 0, last = 0;      // schedule positions of the first write and the last read
    int first0 = 0, last0 = 0;    // the same before the chunked prefix stretched them
    int block = -1;               // physical block backing it
  };
  struct PhysBlock { unsigned long long handle = 0; size_t size = 0; int free_at = 0; };
  void* dalloc_activation(size_t bytes, uint32_t root);
  void MapActivations();
  // Lifetimes for a chunked prefix of `prefix` steps (everything those steps touch lives across
  // all of them), then the physical backing; whatever was mapped before is released first.
  void PlanForPrefix(size_t prefix);
  std::vector<int> step_pos_;   // step -> schedule position
  std::vector<ActBuf> act_;
  std::vector<PhysBlock> phys_;
  bool vmm_ = false;
  size_t vmm_gran_ = 0;
  void Upload(const void* input, cudaStream_t s);
  void UploadRange(const void* input, size_t begin, size_t bytes, cudaStream_t s);
  void Enqueue(cudaStream_t s, size_t first = 0);
  friend struct Lowering;
};

}  // namespace cvm
