// get_valid_counts and non_max_suppression, one CTA per batch image, no host round trips.
//
// get_valid_counts (src/runtime/cpu/ops/nms.cc:42-63): ordered stream compaction of the rows whose
// score exceeds the threshold (block scan per 1024-row chunk, running offset), then a -1 fill.
//
// non_max_suppression (src/runtime/cpu/ops/nms.cc:65-140, iou :4-40):
//   1. stable sort of the first valid_count rows by score, descending: LSD radix sort on the
//      inverted score key carrying the row index (a stable ascending sort of the inverted key
//      keeps equal scores in ascending row order, which is what std::stable_sort gives);
//   2. only the first `keep` sorted rows take part (top_k);
//   3. greedy suppression in blocks of 512 sorted boxes: an integer-IoU bit matrix of the block is
//      built in shared memory by all threads, one warp sweeps it serially, then the survivors of
//      the block strike out later boxes in parallel;
//   4. ordered emission of the survivors (ids >= 0), -1 fill, max_output_size cut.
// The CPU loop's corner rules are kept: a box stops suppressing at the first later row whose id
// is negative; rows with a negative id are never emitted but do suppress; valid_count <= 0 ends
// the whole call (later images are left untouched); max_output_size <= 0 means no limit.
// The IoU test inter*100/union >= thr is evaluated as inter*100 >= thr*union (all positive), so
// no division is executed.
#include <cuda_runtime.h>
#include <string.h>
#include "common.cuh"

namespace cvmk {
namespace {

constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;

// Exclusive scan of one int per thread over the CTA; returns the exclusive prefix, *total gets
// the CTA-wide sum.  `ws` is a shared array of WARPS + 1 ints.
__device__ __forceinline__ int block_exclusive_scan(int v, int* ws, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) ws[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < WARPS ? ws[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += t;
    }
    if (lane < WARPS) ws[lane] = winc - w;
    if (lane == 31) ws[WARPS] = winc;
  }
  __syncthreads();
  const int res = ws[warp] + inc - v;
  *total = ws[WARPS];
  __syncthreads();
  return res;
}

__global__ void __launch_bounds__(THREADS) gvc_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ y,
                                                      int32_t* __restrict__ valid_count, int N, int K,
                                                      int thr) {
  __shared__ int ws[WARPS + 1];
  const int b = blockIdx.x;
  const int32_t* xb = x + (size_t)b * N * K;
  int32_t* yb = y + (size_t)b * N * K;
  int running = 0;
  for (int base = 0; base < N; base += THREADS) {
    const int j = base + threadIdx.x;
    const bool ok = j < N && xb[(size_t)j * K + 1] > thr;
    int total;
    const int pos = running + block_exclusive_scan(ok ? 1 : 0, ws, &total);
    if (ok) {
      const int32_t* src = xb + (size_t)j * K;
      int32_t* dst = yb + (size_t)pos * K;
      for (int k = 0; k < K; ++k) dst[k] = src[k];
    }
    running += total;
  }
  if (threadIdx.x == 0) valid_count[b] = running;
  const size_t begin = (size_t)running * K, end = (size_t)N * K;
  for (size_t i = begin + threadIdx.x; i < end; i += THREADS) yb[i] = -1;
}

// ---------------------------------------------------------------------------------------------
struct NmsParams {
  const int32_t* x; const int32_t* vc; int32_t* y;
  int32_t* xw;            // when set: rows outside the top_k best get -1 in the input as well
  int B, N;
  int mos, thr, topk, force;
  uint32_t* scratch;      // per batch: keyA, keyB, idxA, idxB, removed, stop : 6 * npad words
  int64_t per_batch_words;
  int npad;
};

constexpr int TB = 512;            // sweep block
constexpr int TW = TB / 32;        // words per bit row

struct SweepSmem {
  int32_t box[TB][5];              // id, x1, y1, x2, y2 of the block's sorted boxes
  int32_t stop[TB];
  uint32_t mask[TB][TW];
  uint32_t removed_bits[TW];
  int32_t kept_list[TB];
  int32_t kept_count;
};
struct SortSmem {
  int hist[256];
  int base[256];
  int warp_cnt[WARPS][256];
  int flag;
};
union Smem {
  SweepSmem sweep;
  SortSmem sort;
};

// Suppression test of the CPU iou(): result >= thr, with result = inter*100/union (or
// inter/(union/100) when inter*100 would overflow).  thr > 0 is guaranteed by shape inference.
__device__ __forceinline__ bool iou_ge(const int32_t* a, const int32_t* b, int thr) {
  const int64_t sum_area = (int64_t)(a[2] - a[0]) * (a[3] - a[1]) + (int64_t)(b[2] - b[0]) * (b[3] - b[1]);
  if (sum_area <= 0) return false;
  const int32_t w = max(0, min(a[2], b[2]) - max(a[0], b[0]));
  const int32_t h = max(0, min(a[3], b[3]) - max(a[1], b[1]));
  int64_t inter = (int64_t)h * w;
  int64_t uni = sum_area - inter;
  if (uni <= 0) return false;
  const int64_t max64 = INT64_MAX;
  if (max64 / 100 < inter) uni /= 100;
  else inter *= 100;
  if (uni == 0) return true;  // the CPU would divide by zero here; cannot be reached with int32 boxes
  // inter / uni >= thr  <=>  inter >= thr * uni   (uni > 0, thr > 0), in 128 bits
  const unsigned __int128 rhs = (unsigned __int128)(uint64_t)uni * (uint64_t)(uint32_t)thr;
  return (unsigned __int128)(uint64_t)inter >= rhs;
}

__global__ void __launch_bounds__(THREADS) nms_kernel(const __grid_constant__ NmsParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  __shared__ int ws[WARPS + 1];
  const int b = blockIdx.x;
  const int N = p.N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* xb = p.x + (size_t)b * N * 6;
  int32_t* yb = p.y + (size_t)b * N * 6;

  // A batch whose valid count is <= 0 ends the reference loop: it is filled with -1 and every
  // later batch is left as it is.
  for (int q = 0; q < b; ++q)
    if (min(p.vc[q], N) <= 0) return;
  int vc = max(min(p.vc[b], N), 0);
  if (vc <= 0) {
    for (size_t i = tid; i < (size_t)N * 6; i += THREADS) yb[i] = -1;
    return;
  }

  uint32_t* base_ptr = p.scratch + (size_t)b * p.per_batch_words;
  uint32_t* key_in = base_ptr;
  uint32_t* key_out = base_ptr + p.npad;
  uint32_t* idx_in = base_ptr + 2 * (size_t)p.npad;
  uint32_t* idx_out = base_ptr + 3 * (size_t)p.npad;
  uint32_t* removed = base_ptr + 4 * (size_t)p.npad;
  int32_t* stop = reinterpret_cast<int32_t*>(base_ptr + 5 * (size_t)p.npad);

  // ---- 1. keys
  for (int i = tid; i < vc; i += THREADS) {
    const uint32_t s = (uint32_t)xb[(size_t)i * 6 + 1];
    key_in[i] = ~(s ^ 0x80000000u);
    idx_in[i] = (uint32_t)i;
  }
  __syncthreads();

  // ---- 2. LSD radix sort, 8 bits per pass, stable
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = pass * 8;
    for (int i = tid; i < 256; i += THREADS) sm.sort.hist[i] = 0;
    if (tid == 0) sm.sort.flag = 0;
    __syncthreads();
    for (int i = tid; i < vc; i += THREADS) atomicAdd(&sm.sort.hist[(key_in[i] >> shift) & 255], 1);
    __syncthreads();
    if (tid < 256 && sm.sort.hist[tid] == vc) sm.sort.flag = 1;  // every key has the same digit
    __syncthreads();
    if (sm.sort.flag) { __syncthreads(); continue; }
    if (warp == 0) {
      int run = 0;
      for (int c = 0; c < 8; ++c) {
        const int d = c * 32 + lane;
        const int v = sm.sort.hist[d];
        int inc = v;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, inc, k);
          if (lane >= k) inc += t;
        }
        sm.sort.base[d] = run + inc - v;
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
    }
    __syncthreads();
    for (int cb = 0; cb < vc; cb += THREADS) {
      for (int i = tid; i < WARPS * 256; i += THREADS) (&sm.sort.warp_cnt[0][0])[i] = 0;
      __syncthreads();
      const int i = cb + tid;
      const bool ok = i < vc;
      uint32_t key = 0, idx = 0;
      int d = 256 + lane;  // distinct per lane: never matches another thread
      if (ok) { key = key_in[i]; idx = idx_in[i]; d = (key >> shift) & 255; }
      const uint32_t peers = __match_any_sync(0xffffffffu, d);
      const int rank = __popc(peers & ((1u << lane) - 1));
      if (ok && rank == 0) sm.sort.warp_cnt[warp][d] = __popc(peers);
      __syncthreads();
      if (tid < 256) {
        int run = sm.sort.base[tid];
        for (int w = 0; w < WARPS; ++w) {
          const int c = sm.sort.warp_cnt[w][tid];
          sm.sort.warp_cnt[w][tid] = run;
          run += c;
        }
        sm.sort.base[tid] = run;
      }
      __syncthreads();
      if (ok) {
        const int pos = sm.sort.warp_cnt[warp][d] + rank;
        key_out[pos] = key;
        idx_out[pos] = idx;
      }
      __syncthreads();
    }
    uint32_t* t = key_in; key_in = key_out; key_out = t;
    t = idx_in; idx_in = idx_out; idx_out = t;
  }
  const uint32_t* order = idx_in;  // sorted position -> row

  // ---- 3. keep, stop[], removed[]
  const int keep = (p.topk >= 0 && p.topk < vc) ? p.topk : vc;
  for (int i = tid; i < keep; i += THREADS) removed[i] = 0;
  // stop[i] = first j > i (j < keep) whose id is negative, else keep.  Backward chunked scan.
  {
    int carry = keep;
    for (int hi = keep; hi > 0; hi -= THREADS) {
      const int i = hi - 1 - tid;  // thread 0 owns the highest index of the chunk
      const bool ok = i >= 0;
      const int neg = ok && xb[(size_t)order[i] * 6] < 0 ? i : INT32_MAX;
      // inclusive min-scan over threads 0..tid of `neg` (higher indices first)
      int m = neg;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, m, d);
        if (lane >= d) m = min(m, t);
      }
      if (lane == 31) ws[warp] = m;
      __syncthreads();
      if (warp == 0) {
        int w = lane < WARPS ? ws[lane] : INT32_MAX;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, w, d);
          if (lane >= d) w = min(w, t);
        }
        if (lane < WARPS) ws[lane] = w;
      }
      __syncthreads();
      const int before_warp = warp > 0 ? ws[warp - 1] : INT32_MAX;
      // exclusive: minimum over strictly higher indices
      int excl = __shfl_up_sync(0xffffffffu, m, 1);
      if (lane == 0) excl = INT32_MAX;
      excl = min(excl, before_warp);
      if (ok) stop[i] = min(min(excl, carry), keep);
      const int chunk_min = ws[WARPS - 1];
      __syncthreads();
      carry = min(carry, chunk_min);
    }
  }
  __syncthreads();

  // ---- 4. blocked greedy suppression
  for (int b0 = 0; b0 < keep; b0 += TB) {
    const int nb = min(TB, keep - b0);
    for (int i = tid; i < nb; i += THREADS) {
      const int32_t* row = xb + (size_t)order[b0 + i] * 6;
      sm.sweep.box[i][0] = row[0];
      sm.sweep.box[i][1] = row[2]; sm.sweep.box[i][2] = row[3];
      sm.sweep.box[i][3] = row[4]; sm.sweep.box[i][4] = row[5];
      sm.sweep.stop[i] = stop[b0 + i];
    }
    if (tid < TW) {
      uint32_t bits = 0;
      for (int k = 0; k < 32; ++k) {
        const int i = tid * 32 + k;
        if (i < nb && removed[b0 + i]) bits |= 1u << k;
      }
      sm.sweep.removed_bits[tid] = bits;
    }
    __syncthreads();
    // bit matrix: mask[i][w] bit k set iff box i suppresses box j = 32*w + k (j > i)
    for (int e = tid; e < nb * TW; e += THREADS) {
      const int i = e / TW, w = e % TW;
      uint32_t bits = 0;
      if (w * 32 + 31 > i) {
        const int32_t idi = sm.sweep.box[i][0];
        const int st = sm.sweep.stop[i] - b0;
        for (int k = 0; k < 32; ++k) {
          const int j = w * 32 + k;
          if (j <= i || j >= nb || j >= st) continue;
          if (!(p.force || idi == sm.sweep.box[j][0])) continue;
          if (iou_ge(&sm.sweep.box[i][1], &sm.sweep.box[j][1], p.thr)) bits |= 1u << k;
        }
      }
      sm.sweep.mask[i][w] = bits;
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t mine = lane < TW ? sm.sweep.removed_bits[lane] : 0;
      int kept = 0;
      for (int i = 0; i < nb; ++i) {
        const uint32_t word = __shfl_sync(0xffffffffu, mine, i >> 5);
        if (!((word >> (i & 31)) & 1u)) {
          if (lane < TW) mine |= sm.sweep.mask[i][lane];
          if (lane == 0) sm.sweep.kept_list[kept] = i;
          ++kept;
        }
      }
      if (lane < TW) sm.sweep.removed_bits[lane] = mine;
      if (lane == 0) sm.sweep.kept_count = kept;
    }
    __syncthreads();
    for (int i = tid; i < nb; i += THREADS)
      removed[b0 + i] = (sm.sweep.removed_bits[i >> 5] >> (i & 31)) & 1u;
    // survivors of this block strike out later boxes
    const int kept = sm.sweep.kept_count;
    for (int j = b0 + nb + tid; j < keep; j += THREADS) {
      if (removed[j]) continue;
      const int32_t* row = xb + (size_t)order[j] * 6;
      const int32_t idj = row[0];
      if (idj < 0) continue;  // a suppressing scan never reaches past a negative id
      const int32_t bj[4] = {row[2], row[3], row[4], row[5]};
      for (int q = 0; q < kept; ++q) {
        const int i = sm.sweep.kept_list[q];
        if (j >= sm.sweep.stop[i]) continue;
        if (!(p.force || sm.sweep.box[i][0] == idj)) continue;
        if (iou_ge(&sm.sweep.box[i][1], bj, p.thr)) { removed[j] = 1; break; }
      }
    }
    __syncthreads();
  }

  // ---- 5. ordered emission, -1 fill, max_output_size cut
  int running = 0;
  const int limit = p.mos > 0 ? p.mos : INT32_MAX;
  for (int cb = 0; cb < keep; cb += THREADS) {
    const int i = cb + tid;
    bool emit = false;
    const int32_t* row = nullptr;
    if (i < keep) {
      row = xb + (size_t)order[i] * 6;
      emit = !removed[i] && row[0] >= 0;
    }
    int total;
    const int pos = running + block_exclusive_scan(emit ? 1 : 0, ws, &total);
    if (emit && pos < limit) {
      int32_t* dst = yb + (size_t)pos * 6;
#pragma unroll
      for (int k = 0; k < 6; ++k) dst[k] = row[k];
    }
    running += total;
  }
  const int emitted = min(running, limit);
  for (size_t i = (size_t)emitted * 6 + tid; i < (size_t)N * 6; i += THREADS) yb[i] = -1;
  // The CPU implementation's side effect on its input (nms.cc:93-97); nothing above reads the rows
  // past `keep` after the sort.
  if (p.xw != nullptr && p.topk > 0 && p.topk < vc) {
    __syncthreads();
    int32_t* xwb = p.xw + (size_t)b * N * 6;
    for (int e = p.topk * 6 + tid; e < vc * 6; e += THREADS) xwb[(size_t)order[e / 6] * 6 + e % 6] = -1;
  }
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_get_valid_counts(const int32_t* x, int32_t* y, int32_t* valid_count, int32_t B,
                                     int32_t N, int32_t K, int32_t score_threshold,
                                     cvmk_stream_t stream) {
  if (!x || !y || !valid_count || B < 1 || N < 1 || K < 2) {
    set_error("get_valid_counts: bad argument");
    return CVMK_ERR_ARG;
  }
  gvc_kernel<<<B, THREADS, 0, (cudaStream_t)stream>>>(x, y, valid_count, N, K, score_threshold);
  return check_cuda(cudaGetLastError(), "gvc_kernel launch");
}

static inline int nms_npad(int N) { return (N + 3) / 4 * 4; }

extern "C" int64_t cvmk_nms_scratch_bytes(int32_t B, int32_t N) {
  return (int64_t)B * 6 * nms_npad(N) * 4;
}

extern "C" int cvmk_non_max_suppression(const cvmk_nms_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->valid_count || !d->y || !d->scratch || d->B < 1 || d->N < 1 || d->iou_threshold <= 0) {
    set_error("non_max_suppression: bad argument");
    return CVMK_ERR_ARG;
  }
  if (d->scratch_bytes < cvmk_nms_scratch_bytes(d->B, d->N) || ((uintptr_t)d->scratch & 15)) {
    set_error("non_max_suppression: scratch too small or misaligned");
    return CVMK_ERR_ARG;
  }
  NmsParams p;
  p.x = d->x; p.vc = d->valid_count; p.y = d->y; p.xw = d->x_writeback;
  p.B = d->B; p.N = d->N;
  p.mos = d->max_output_size; p.thr = d->iou_threshold; p.topk = d->top_k; p.force = d->force_suppress;
  p.scratch = reinterpret_cast<uint32_t*>(d->scratch);
  p.npad = nms_npad(d->N);
  p.per_batch_words = 6 * (int64_t)p.npad;
  const int smem = (int)sizeof(Smem);
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    if (check_cuda(cudaFuncSetAttribute(nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                   "cudaFuncSetAttribute(nms_kernel)"))
      return CVMK_ERR_CUDA;
    attr_dev = dev;
  }
  nms_kernel<<<d->B, THREADS, smem, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "nms_kernel launch");
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in the library's device image.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_nms_static_scratch[CVMK_NMS_STATIC_SCRATCH_BYTES];

extern "C" int cvmk_non_max_suppression_static(const int32_t* x, const int32_t* valid_count, int32_t* y,
                                               int32_t B, int32_t N, int32_t max_output_size,
                                               int32_t iou_threshold, int32_t top_k,
                                               int32_t force_suppress, cvmk_stream_t stream) {
  if (!x || !valid_count || !y || B < 1 || N < 1 || iou_threshold <= 0) {
    set_error("non_max_suppression_static: bad argument");
    return CVMK_ERR_ARG;
  }
  const int64_t need = cvmk_nms_scratch_bytes(B, N);
  if (need > (int64_t)CVMK_NMS_STATIC_SCRATCH_BYTES) {
    set_error("non_max_suppression_static: B=%d, N=%d needs %lld bytes of scratch, the built-in array "
              "holds %u; use cvmk_non_max_suppression with a caller-provided buffer",
              B, N, (long long)need, (unsigned)CVMK_NMS_STATIC_SCRATCH_BYTES);
    return CVMK_ERR_ARG;
  }
  // In host code the array's name is only a handle; the kernel needs its device address, which
  // differs per GPU.  Resolved once per device, with that device current.
  static void* scratch_of_device[64] = {nullptr};
  static bool attr_of_device[64] = {false};
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return CVMK_ERR_CUDA;
  if (dev < 0 || dev >= 64) { set_error("non_max_suppression_static: device ordinal %d not supported", dev); return CVMK_ERR_ARG; }
  if (!scratch_of_device[dev]) {
    void* ptr = nullptr;
    if (check_cuda(cudaGetSymbolAddress(&ptr, g_nms_static_scratch), "cudaGetSymbolAddress(nms scratch)"))
      return CVMK_ERR_CUDA;
    if (!ptr) { set_error("non_max_suppression_static: null scratch address"); return CVMK_ERR_CUDA; }
    scratch_of_device[dev] = ptr;
  }
  const int smem = (int)sizeof(Smem);
  if (!attr_of_device[dev]) {
    if (check_cuda(cudaFuncSetAttribute(nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                   "cudaFuncSetAttribute(nms_kernel)"))
      return CVMK_ERR_CUDA;
    attr_of_device[dev] = true;
  }
  NmsParams p;
  p.x = x; p.vc = valid_count; p.y = y; p.xw = nullptr;
  p.B = B; p.N = N;
  p.mos = max_output_size; p.thr = iou_threshold; p.topk = top_k; p.force = force_suppress;
  p.scratch = reinterpret_cast<uint32_t*>(scratch_of_device[dev]);
  p.npad = nms_npad(N);
  p.per_batch_words = 6 * (int64_t)p.npad;
  nms_kernel<<<B, THREADS, smem, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "nms_kernel launch (static scratch)");
}
