// get_valid_counts and non_max_suppression, one CTA per batch image, no host round trips.
//
// get_valid_counts (src/runtime/cpu/ops/nms.cc:42-63): ordered stream compaction of the rows whose
// score exceeds the threshold (block scan per 1024-row chunk, running offset), then a -1 fill.
//
// non_max_suppression (src/runtime/cpu/ops/nms.cc:65-140, iou :4-40):
//   1. stable sort of the first valid_count rows by score, descending, of which only the first
//      `keep` (top_k) take part.  When keep <= 1024 -- the usual detection tail: a few hundred of
//      ten thousand rows survive -- the keep best rows are SELECTED first: an MSB-first radix select
//      over the inverted score keys finds the key of the last row that gets in, an ordered
//      compaction gathers the rows below that key (and the first few equal to it, in row order)
//      into shared memory, and a bitonic sort of (key, arrival position) pairs orders them; the rows
//      never leave the SM and nothing is scattered through global memory.  Otherwise: LSD radix
//      sort on the inverted score key carrying the row index (a stable ascending sort of the
//      inverted key keeps equal scores in ascending row order, which is what std::stable_sort gives);
//   2. (the rows past `keep` are dropped);
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
#include <algorithm>
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

// Development builds (-DCVMK_NMS_TIMING): clocks of CTA 0 at the phase boundaries.
#ifdef CVMK_NMS_TIMING
__device__ long long g_nms_phase[16];
#define PHASE(k) do { __syncthreads(); if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_nms_phase[k] = clock64(); } while (0)
#else
#define PHASE(k) do {} while (0)
#endif

// Fill of y[begin, end) (int32 elements) with -1, 16 bytes per store where the address allows.
__device__ __forceinline__ void fill_minus_one(int32_t* y, size_t begin, size_t end) {
  size_t i = begin;
  const size_t head = min(end, (begin + 3) & ~(size_t)3);   // y + 4k is 16-byte aligned when y is
  if (((uintptr_t)y & 15) != 0) {
    for (size_t k = begin + threadIdx.x; k < end; k += THREADS) y[k] = -1;
    return;
  }
  for (size_t k = i + threadIdx.x; k < head; k += THREADS) y[k] = -1;
  const size_t vec_end = head + ((end - head) & ~(size_t)3);
  const int4 m = make_int4(-1, -1, -1, -1);
  for (size_t k = head + 4 * (size_t)threadIdx.x; k < vec_end; k += 4 * (size_t)THREADS)
    *reinterpret_cast<int4*>(y + k) = m;
  for (size_t k = vec_end + threadIdx.x; k < end; k += THREADS) y[k] = -1;
}

// Rows of six int32 (the detection layout), four consecutive rows per thread and round: one block
// scan per 4096 rows, rows moved as three 8-byte words.
//
// An image is cut into gridDim.x chunks of `chunk_rows` rows, one CTA each, so that a small batch
// still uses many SMs: every CTA first counts the valid rows of the whole image (scores only,
// served by L2) to learn where its chunk lands and where the -1 tail begins, then compacts its own
// chunk and fills its share of the tail.  No CTA waits for another.
// `clamp`: every element is first brought into [-clamp, clamp] (the runtime's clamp of the network
// input to its declared precision, when these rows ARE the network input); INT32_MAX = values as
// they are, except that INT32_MIN becomes -INT32_MAX, which is what that clamp does at 32 bits.
__device__ __forceinline__ int clampv(int v, int clamp) { return max(min(v, clamp), -clamp); }
__device__ __forceinline__ int2 clamp2(int2 v, int clamp) { return make_int2(clampv(v.x, clamp), clampv(v.y, clamp)); }

template <bool CLAMP>
__global__ void __launch_bounds__(THREADS, 1) gvc6_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ y,
                                                          int32_t* __restrict__ valid_count, int N, int thr,
                                                          int chunk_rows, int clamp) {
  __shared__ int ws[WARPS + 1];
  __shared__ int red[2][WARPS];
  const int b = blockIdx.y, c = blockIdx.x;
  const int2* xb = reinterpret_cast<const int2*>(x + (size_t)b * N * 6);
  int32_t* yb32 = y + (size_t)b * N * 6;
  int2* yb = reinterpret_cast<int2*>(yb32);
  const int row0 = c * chunk_rows, row1 = min(N, row0 + chunk_rows);
  PHASE(9);
  // valid rows before this chunk, and in the whole image
  int before = 0, total_valid = 0;
  for (int j = threadIdx.x; j < N; j += THREADS) {
    int score = xb[(size_t)j * 3].y;
    if (CLAMP) score = clampv(score, clamp);
    const int ok = score > thr ? 1 : 0;
    total_valid += ok;
    before += (j < row0) ? ok : 0;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, d);
    total_valid += __shfl_xor_sync(0xffffffffu, total_valid, d);
  }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = before; red[1][threadIdx.x >> 5] = total_valid; }
  __syncthreads();
  before = 0; total_valid = 0;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) { before += red[0][w]; total_valid += red[1][w]; }
  int running = before;
  for (int base = row0; base < row1; base += 4 * THREADS) {
    const int j0 = base + 4 * threadIdx.x;
    int2 r[4][3];
    int ok = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (j0 + q < row1) {
        r[q][0] = xb[(size_t)(j0 + q) * 3];
        r[q][1] = xb[(size_t)(j0 + q) * 3 + 1];
        r[q][2] = xb[(size_t)(j0 + q) * 3 + 2];
        if (CLAMP) { r[q][0] = clamp2(r[q][0], clamp); r[q][1] = clamp2(r[q][1], clamp); r[q][2] = clamp2(r[q][2], clamp); }
        if (r[q][0].y > thr) ok |= 1 << q;
      }
    }
    int total;
    int pos = running + block_exclusive_scan(__popc(ok), ws, &total);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (ok & (1 << q)) {
        yb[(size_t)pos * 3] = r[q][0];
        yb[(size_t)pos * 3 + 1] = r[q][1];
        yb[(size_t)pos * 3 + 2] = r[q][2];
        ++pos;
      }
    }
    running += total;
  }
  if (threadIdx.x == 0 && c == 0) valid_count[b] = total_valid;
  PHASE(10);
  // this CTA's share of the -1 tail (shares are multiples of four elements)
  const size_t tail0 = (size_t)total_valid * 6, tail1 = (size_t)N * 6;
  const size_t share = (((tail1 - tail0) + gridDim.x - 1) / gridDim.x + 3) & ~(size_t)3;
  const size_t f0 = min(tail1, tail0 + (size_t)c * share), f1 = min(tail1, f0 + share);
  fill_minus_one(yb32, f0, f1);
  PHASE(11);
}

__global__ void __launch_bounds__(THREADS) gvc_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ y,
                                                      int32_t* __restrict__ valid_count, int N, int K,
                                                      int thr, int clamp) {
  __shared__ int ws[WARPS + 1];
  const int b = blockIdx.x;
  const int32_t* xb = x + (size_t)b * N * K;
  int32_t* yb = y + (size_t)b * N * K;
  int running = 0;
  for (int base = 0; base < N; base += THREADS) {
    const int j = base + threadIdx.x;
    const bool ok = j < N && clampv(xb[(size_t)j * K + 1], clamp) > thr;
    int total;
    const int pos = running + block_exclusive_scan(ok ? 1 : 0, ws, &total);
    if (ok) {
      const int32_t* src = xb + (size_t)j * K;
      int32_t* dst = yb + (size_t)pos * K;
      for (int k = 0; k < K; ++k) dst[k] = clampv(src[k], clamp);
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
  int key_cap;            // score keys that fit the dynamic shared memory behind the work area
  int fill_bound;         // rows from here on are -1 whatever the data says (top_k / max_output_size)
  int dbg;                // development builds: bit 0 skips the IoU tests, bit 1 the pair gathering
};

constexpr int TB = 512;            // sweep block
constexpr int TW = TB / 32;        // words per bit row

constexpr int PAIR_CAP = 64 * TW + TB + 4;   // 64 bucket rows of TW words + (TB + 1) prefix sums
struct SweepSmem {
  int32_t box[TB][5];              // id, x1, y1, x2, y2 of the block's sorted boxes
  int32_t stop[TB];
  uint32_t mask[TB][TW];
  uint32_t removed_bits[TW];
  int32_t kept_list[TB];
  int32_t kept_count;
  uint32_t pairs[PAIR_CAP];        // work area of the pair enumeration: bucket rows, prefix sums
};
struct SortSmem {
  int hist[256];
  int base[256];
  int warp_cnt[WARPS][256];
  int flag;
};
constexpr int SEL_MAX = 1024;      // rows the select-then-sort path orders in shared memory
struct SelectSmem {
  int hist[256];
  unsigned long long pair[SEL_MAX];   // (inverted score key << 32) | arrival position
  int32_t row[SEL_MAX];               // arrival position -> row index
  int warp_a[WARPS], warp_b[WARPS];   // per-warp partial results
  uint32_t prefix, mask;
  int want;
};
union Smem {
  SweepSmem sweep;
  SortSmem sort;
  SelectSmem sel;
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

// The same test when every coordinate of both boxes lies in [-32768, 32767] and thr <= 2^20: areas
// stay below 2^33 and both sides of the comparison below 2^54, so plain 64-bit arithmetic gives the
// result of the general form above (whose overflow branch cannot be taken).
__device__ __forceinline__ bool iou_ge_small(const int32_t* a, const int32_t* b, int thr) {
  const int64_t sum_area = (int64_t)(a[2] - a[0]) * (a[3] - a[1]) + (int64_t)(b[2] - b[0]) * (b[3] - b[1]);
  if (sum_area <= 0) return false;
  const int32_t w = max(0, min(a[2], b[2]) - max(a[0], b[0]));
  const int32_t h = max(0, min(a[3], b[3]) - max(a[1], b[1]));
  const int64_t inter = (int64_t)h * w;
  const int64_t uni = sum_area - inter;
  if (uni <= 0) return false;
  return inter * 100 >= (int64_t)thr * uni;
}

__global__ void __launch_bounds__(THREADS) nms_kernel(const __grid_constant__ NmsParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  __shared__ int ws[WARPS + 1];
  const int b = blockIdx.y;
  const int N = p.N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* xb = p.x + (size_t)b * N * 6;
  int32_t* yb = p.y + (size_t)b * N * 6;

  // A batch whose valid count is <= 0 ends the reference loop: it is filled with -1 and every
  // later batch is left as it is.
  for (int q = 0; q < b; ++q)
    if (min(p.vc[q], N) <= 0) return;
  int vc = max(min(p.vc[b], N), 0);
  // CTAs 1.. of an image only write the part of the -1 tail that is known before any row is looked
  // at: at most top_k (and max_output_size) rows can be emitted, everything after them is -1.  One
  // SM stores 32 bytes a clock, and an image of 24564 rows has 590 KB of tail.
  const int fillers = (int)gridDim.x - 1;
  const int fill_from = vc <= 0 ? 0 : p.fill_bound;     // an image without valid rows is all -1
  if (blockIdx.x > 0) {
    const size_t t0 = (size_t)fill_from * 6, t1 = (size_t)N * 6;
    const size_t share = (((t1 - t0) + fillers - 1) / fillers + 3) & ~(size_t)3;
    const size_t f0 = min(t1, t0 + (size_t)(blockIdx.x - 1) * share), f1 = min(t1, f0 + share);
    fill_minus_one(yb, f0, f1);
    return;
  }
  const int own_end = fillers > 0 ? fill_from : N;       // rows this CTA has to write itself
  if (vc <= 0) {
    fill_minus_one(yb, 0, (size_t)own_end * 6);
    return;
  }

  uint32_t* base_ptr = p.scratch + (size_t)b * p.per_batch_words;
  uint32_t* key_in = base_ptr;
  uint32_t* key_out = base_ptr + p.npad;
  uint32_t* idx_in = base_ptr + 2 * (size_t)p.npad;
  uint32_t* idx_out = base_ptr + 3 * (size_t)p.npad;
  uint32_t* removed = base_ptr + 4 * (size_t)p.npad;
  int32_t* stop = reinterpret_cast<int32_t*>(base_ptr + 5 * (size_t)p.npad);

  const int keep = (p.topk >= 0 && p.topk < vc) ? p.topk : vc;
  const bool select_path = keep <= SEL_MAX;
  PHASE(0);
  if (select_path) {
    // ---- 1'. the keep best rows, selected and sorted in shared memory.  The inverted score keys
    // are read from global memory once and kept behind the work area when they fit.
    uint32_t* skeys = reinterpret_cast<uint32_t*>(smem_raw + ((sizeof(Smem) + 15) & ~(size_t)15));
    const bool keys_in_smem = vc <= p.key_cap;
    auto key_global = [&](int i) { return ~((uint32_t)xb[(size_t)i * 6 + 1] ^ 0x80000000u); };
    // bits in which the keys differ at all: a byte in which they all agree needs no select pass
    uint32_t k_or = 0, k_and = 0xffffffffu;
    for (int i = tid; i < vc; i += THREADS) {
      const uint32_t k = key_global(i);
      if (keys_in_smem) skeys[i] = k;
      k_or |= k;
      k_and &= k;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      k_or |= __shfl_xor_sync(0xffffffffu, k_or, d);
      k_and &= __shfl_xor_sync(0xffffffffu, k_and, d);
    }
    if (lane == 0) { sm.sel.warp_a[warp] = (int)k_or; sm.sel.warp_b[warp] = (int)k_and; }
    __syncthreads();
    k_or = 0; k_and = 0xffffffffu;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) { k_or |= (uint32_t)sm.sel.warp_a[w]; k_and &= (uint32_t)sm.sel.warp_b[w]; }
    const uint32_t differ = k_or ^ k_and;
    __syncthreads();
    auto key_of = [&](int i) { return keys_in_smem ? skeys[i] : key_global(i); };
    uint32_t T = 0xffffffffu;     // rows with a key below T get in, and the first `need_eq` rows equal to T
    int need_eq = 0;
    if (keep < vc && keep > 0) {
      if (tid == 0) { sm.sel.prefix = 0; sm.sel.mask = 0; sm.sel.want = keep; }
      __syncthreads();
      for (int pass = 3; pass >= 0; --pass) {
        const int shift = pass * 8;
        if (((differ >> shift) & 255u) == 0) {   // every key has this byte: nothing to choose
          if (tid == 0) { sm.sel.prefix |= k_and & (255u << shift); sm.sel.mask |= 255u << shift; }
          __syncthreads();
          continue;
        }
        for (int i = tid; i < 256; i += THREADS) sm.sel.hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sm.sel.prefix, mask = sm.sel.mask;
        for (int i = tid; i < vc; i += THREADS) {
          const uint32_t k = key_of(i);
          if ((k & mask) == prefix) atomicAdd(&sm.sel.hist[(k >> shift) & 255], 1);
        }
        __syncthreads();
        if (warp == 0) {
          // digit d with (rows below d) < want <= (rows up to d): inclusive scan over 256 bins
          int want = sm.sel.want, run = 0, found = -1, below = 0;
          for (int c = 0; c < 8 && found < 0; ++c) {
            const int v = sm.sel.hist[c * 32 + lane];
            int inc = v;
#pragma unroll
            for (int k = 1; k < 32; k <<= 1) {
              int t = __shfl_up_sync(0xffffffffu, inc, k);
              if (lane >= k) inc += t;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, run + inc >= want);
            if (hit) {
              const int l = __ffs(hit) - 1;
              found = c * 32 + l;
              below = run + __shfl_sync(0xffffffffu, inc - v, l);
            }
            run += __shfl_sync(0xffffffffu, inc, 31);
          }
          if (lane == 0) {
            sm.sel.prefix = prefix | ((uint32_t)found << shift);
            sm.sel.mask = mask | (255u << shift);
            sm.sel.want = want - below;
          }
        }
        __syncthreads();
      }
      T = sm.sel.prefix;
      need_eq = sm.sel.want;
    }
    __syncthreads();
    PHASE(1);
    // Ordered compaction.  Position among the selected rows = (rows below T before i) + (rows equal
    // to T before i, capped at need_eq).  Every warp owns a contiguous run of rows: one pass counts
    // per warp, one block-wide exchange gives each warp its offsets, a second pass places the rows
    // with ballots; no block barrier per round.
    int32_t* xwb = p.xw ? p.xw + (size_t)b * N * 6 : nullptr;
    const bool writeback = xwb != nullptr && p.topk > 0 && p.topk < vc;
    if (keep > 0) {
      const bool all = keep == vc;
      const int per_warp = (vc + WARPS - 1) / WARPS;
      const int w0 = min(vc, warp * per_warp), w1 = min(vc, w0 + per_warp);
      int cl = 0, ce = 0;
      for (int base = w0; base < w1; base += 32) {
        const int i = base + lane;
        bool less = false, eq = false;
        if (i < w1) { const uint32_t k = key_of(i); less = all || k < T; eq = !all && k == T; }
        cl += __popc(__ballot_sync(0xffffffffu, less));
        ce += __popc(__ballot_sync(0xffffffffu, eq));
      }
      if (lane == 0) { sm.sel.warp_a[warp] = cl; sm.sel.warp_b[warp] = ce; }
      __syncthreads();
      int run_less = 0, run_eq = 0;
      for (int w = 0; w < warp; ++w) { run_less += sm.sel.warp_a[w]; run_eq += sm.sel.warp_b[w]; }
      const uint32_t lt = (1u << lane) - 1u;
      for (int base = w0; base < w1; base += 32) {
        const int i = base + lane;
        uint32_t k = 0;
        bool less = false, eq = false;
        if (i < w1) { k = key_of(i); less = all || k < T; eq = !all && k == T; }
        const uint32_t ml = __ballot_sync(0xffffffffu, less), me = __ballot_sync(0xffffffffu, eq);
        const int less_before = run_less + __popc(ml & lt), eq_before = run_eq + __popc(me & lt);
        const bool sel = less || (eq && eq_before < need_eq);
        if (sel) {
          const int pos = less_before + min(eq_before, need_eq);
          sm.sel.pair[pos] = ((unsigned long long)k << 32) | (unsigned)pos;
          sm.sel.row[pos] = i;
        } else if (writeback && i < w1) {
          // the CPU implementation's side effect on its input (nms.cc:93-97): rows that miss the top_k
#pragma unroll
          for (int e = 0; e < 6; ++e) xwb[(size_t)i * 6 + e] = -1;
        }
        run_less += __popc(ml);
        run_eq += __popc(me);
      }
    }
    PHASE(2);
    // bitonic sort of the pairs (ascending: best score first, ties in arrival = row order), one
    // pair per thread: partners less than a warp apart are exchanged by shuffle, the others
    // through shared memory.  Only the first n2 threads take part (their own named barrier).
    int n2 = 32;
    while (n2 < keep) n2 <<= 1;      // <= SEL_MAX = THREADS
    __syncthreads();
    if (tid < n2) {
      unsigned long long v = tid < keep ? sm.sel.pair[tid] : ~0ull;
      for (int size = 2; size <= n2; size <<= 1) {
        const bool up = (tid & size) == 0;
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          unsigned long long other;
          if (stride >= 32) {
            asm volatile("bar.sync 1, %0;" ::"r"(n2) : "memory");
            sm.sel.pair[tid] = v;
            asm volatile("bar.sync 1, %0;" ::"r"(n2) : "memory");
            other = sm.sel.pair[tid ^ stride];
          } else {
            other = __shfl_xor_sync(0xffffffffu, v, stride);
          }
          const bool take_min = ((tid & stride) == 0) == up;
          v = take_min ? (v < other ? v : other) : (v > other ? v : other);
        }
      }
      if (tid < keep) idx_in[tid] = (uint32_t)sm.sel.row[(uint32_t)v];
    }
    __syncthreads();
  } else {
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
  }
  const uint32_t* order = idx_in;  // sorted position -> row

  // ---- 3. stop[], removed[]
  PHASE(3);
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
  PHASE(4);
  for (int b0 = 0; b0 < keep; b0 += TB) {
    const int nb = min(TB, keep - b0);
    bool small_here = true;
    for (int i = tid; i < nb; i += THREADS) {
      const int32_t* row = xb + (size_t)order[b0 + i] * 6;
      sm.sweep.box[i][0] = row[0];
      sm.sweep.box[i][1] = row[2]; sm.sweep.box[i][2] = row[3];
      sm.sweep.box[i][3] = row[4]; sm.sweep.box[i][4] = row[5];
      sm.sweep.stop[i] = stop[b0 + i];
#pragma unroll
      for (int e = 2; e < 6; ++e) small_here &= row[e] >= -32768 && row[e] <= 32767;
    }
    // every box of the block has 16-bit coordinates: the cheap form of the IoU test applies
    const bool small = __syncthreads_and(small_here ? 1 : 0) != 0 && p.thr <= (1 << 20);
    if (tid < TW) {
      uint32_t bits = 0;
      for (int k = 0; k < 32; ++k) {
        const int i = tid * 32 + k;
        if (i < nb && removed[b0 + i]) bits |= 1u << k;
      }
      sm.sweep.removed_bits[tid] = bits;
    }
    __syncthreads();
    // bit matrix: mask[i][w] bit k set iff box i suppresses box j = 32*w + k (j > i).  A warp takes
    // a row i and walks its words; lane k tests box j = 32*w + k (consecutive boxes: the rows of
    // box[][5] fall into different banks) and a ballot assembles the word.
    //
    // With class-aware suppression only about one pair in (number of classes) needs an IoU test,
    // and a warp that runs the test for one lane pays for all 32.  So the same-class pairs are
    // enumerated first, without looking at every pair: the boxes are dropped into 64 buckets by a
    // hash of their class id, one 512-bit occupancy row per bucket; box i's candidates are the bits
    // of its bucket's row between i and its stop position.  A prefix sum over the candidate counts
    // numbers all candidate pairs of the block, and the threads then take pairs, not rows: find
    // the row by bisection, the k-th candidate bit with __fns, check the class (a bucket can hold
    // two classes), run the IoU test and set the bit.  Forced suppression, or a block with so
    // many candidates that the dense walk is cheaper (one or two classes), tests every pair in place.
    {
      const int words = (nb + 31) >> 5;
      bool listed = !p.force;
      if (listed) {
        uint32_t (*bucket)[TW] = reinterpret_cast<uint32_t (*)[TW]>(sm.sweep.pairs);          // [64][TW]
        int* prefix = reinterpret_cast<int*>(sm.sweep.pairs + 64 * TW);                        // [nb + 1]
        auto hash = [](int32_t id) { return ((uint32_t)id * 0x9E3779B1u) >> 26; };
        for (int e = tid; e < nb * TW; e += THREADS) (&sm.sweep.mask[0][0])[e] = 0;
        for (int e = tid; e < 64 * TW; e += THREADS) (&bucket[0][0])[e] = 0;
        __syncthreads();
        for (int i = tid; i < nb; i += THREADS) atomicOr(&bucket[hash(sm.sweep.box[i][0])][i >> 5], 1u << (i & 31));
        __syncthreads();
        // candidate bits of row i in word w: same bucket, after i, before the row's stop position
        auto candidates = [&](int i, int w, int last) -> uint32_t {
          uint32_t bits = bucket[hash(sm.sweep.box[i][0])][w];
          if (w == (i >> 5)) bits &= (i & 31) == 31 ? 0u : ~0u << ((i & 31) + 1);
          else if (w < (i >> 5)) bits = 0;
          if (w == (last >> 5)) bits &= (last & 31) == 0 ? 0u : ~0u >> (32 - (last & 31));
          else if (w > (last >> 5)) bits = 0;
          return bits;
        };
        int mine = 0;
        const int row_t = tid;       // THREADS >= TB: one row per thread
        int last_t = 0;
        if (row_t < nb) {
          last_t = min(sm.sweep.stop[row_t] - b0, nb);     // candidates j < last
          for (int w = row_t >> 5; w < words; ++w) mine += __popc(candidates(row_t, w, last_t));
        }
        int total_pairs;
        const int before = block_exclusive_scan(mine, ws, &total_pairs);
        if (row_t < nb) prefix[row_t] = before;
        if (tid == 0) prefix[nb] = total_pairs;
        __syncthreads();
        if (total_pairs > 24 * 1024) {
          listed = false;           // uniform; the dense walk below fills the whole mask itself
        } else {
          for (int e = tid; e < total_pairs && !(p.dbg & 1); e += THREADS) {
            int lo = 0, hi = nb - 1;  // the last row whose prefix is <= e
            while (lo < hi) {
              const int mid = (lo + hi + 1) >> 1;
              if (prefix[mid] <= e) lo = mid; else hi = mid - 1;
            }
            const int i = lo;
            int k = e - prefix[i];
            const int last = min(sm.sweep.stop[i] - b0, nb);
            int j = -1;
            for (int w = i >> 5; w < words; ++w) {
              const uint32_t bits = candidates(i, w, last);
              const int c = __popc(bits);
              if (k < c) { j = w * 32 + (int)__fns(bits, 0, k + 1); break; }
              k -= c;
            }
            if (j < 0 || sm.sweep.box[j][0] != sm.sweep.box[i][0]) continue;
            const bool hit = small ? iou_ge_small(&sm.sweep.box[i][1], &sm.sweep.box[j][1], p.thr)
                                   : iou_ge(&sm.sweep.box[i][1], &sm.sweep.box[j][1], p.thr);
            if (hit) atomicOr(&sm.sweep.mask[i][j >> 5], 1u << (j & 31));
          }
        }
      }
      if (!listed) {
        __syncthreads();
        for (int i = warp; i < nb; i += WARPS) {
          const int32_t idi = sm.sweep.box[i][0];
          const int st = sm.sweep.stop[i] - b0;
          const int32_t bi[4] = {sm.sweep.box[i][1], sm.sweep.box[i][2], sm.sweep.box[i][3], sm.sweep.box[i][4]};
          for (int w = 0; w < words; ++w) {
            uint32_t bits = 0;
            if (w * 32 + 31 > i && w * 32 < st) {
              const int j = w * 32 + lane;
              bool hit = false;
              if (j > i && j < nb && j < st && (p.force || idi == sm.sweep.box[j][0]))
                hit = small ? iou_ge_small(bi, &sm.sweep.box[j][1], p.thr) : iou_ge(bi, &sm.sweep.box[j][1], p.thr);
              bits = __ballot_sync(0xffffffffu, hit);
            }
            if (lane == 0) sm.sweep.mask[i][w] = bits;
          }
        }
      }
    }
    __syncthreads();
    if (b0 == 0) PHASE(5);
    if (warp == 0) {
      // Greedy sweep, 32 sorted boxes (one word) at a time.  Inside a group the decisions are a
      // serial chain over the group's 32 x 32 diagonal block: every lane holds one row of it, the
      // rows are gathered into registers by shuffles (no memory on the chain) and all lanes walk the
      // chain redundantly.  The survivors of the group then OR their whole mask rows into the
      // removed bits of the later words, loads that do not depend on one another.
      const int words = (nb + 31) >> 5;
      uint32_t mine = lane < TW ? sm.sweep.removed_bits[lane] : 0;   // lane w: removed bits of word w
      int kept = 0;
#ifdef CVMK_NMS_TIMING
      if (blockIdx.y == 0 && lane == 0) g_nms_phase[12] = clock64();
#endif
      for (int g = 0; g < words; ++g) {
        const int row = g * 32 + lane;
        const uint32_t diag = row < nb ? sm.sweep.mask[row][g] : 0;
        uint32_t rem = __shfl_sync(0xffffffffu, mine, g);
        if (g * 32 + 32 > nb) rem |= ~0u << (nb - g * 32);            // rows past the block end do not exist
#pragma unroll
        for (int r = 0; r < 32; ++r) {
          const uint32_t d = __shfl_sync(0xffffffffu, diag, r);
          if (!((rem >> r) & 1u)) rem |= d;
        }
        const uint32_t alive = ~rem;
        if (lane == g) mine = rem;
        // survivors strike the later words: lane w ORs word w of every survivor's row (independent loads)
        if (lane > g && lane < words) {
          uint32_t acc = 0;
#pragma unroll
          for (int r = 0; r < 32; ++r)
            if ((alive >> r) & 1u) acc |= sm.sweep.mask[g * 32 + r][lane];
          mine |= acc;
        }
        if ((alive >> lane) & 1u) sm.sweep.kept_list[kept + __popc(alive & ((1u << lane) - 1u))] = g * 32 + lane;
        kept += __popc(alive);
      }
      if (nb & 31) { if (lane == (nb >> 5)) mine &= ~(~0u << (nb & 31)); }  // the padding bits are not boxes
      if (lane < TW) sm.sweep.removed_bits[lane] = lane < words ? mine : 0;
      if (lane == 0) sm.sweep.kept_count = kept;
#ifdef CVMK_NMS_TIMING
      if (blockIdx.y == 0 && lane == 0) g_nms_phase[13] = clock64();
#endif
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
  PHASE(6);
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
  PHASE(7);
  fill_minus_one(yb, (size_t)emitted * 6, (size_t)own_end * 6);
  PHASE(8);
  // The CPU implementation's side effect on its input (nms.cc:93-97); nothing above reads the rows
  // past `keep` after the sort.  (The select path has written it while compacting.)
  if (!select_path && p.xw != nullptr && p.topk > 0 && p.topk < vc) {
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
  return cvmk_get_valid_counts_clamped(x, y, valid_count, B, N, K, score_threshold, 0, stream);
}

extern "C" int cvmk_get_valid_counts_clamped(const int32_t* x, int32_t* y, int32_t* valid_count, int32_t B,
                                             int32_t N, int32_t K, int32_t score_threshold, int32_t clamp,
                                             cvmk_stream_t stream) {
  if (!x || !y || !valid_count || B < 1 || N < 1 || K < 2 || clamp < 0) {
    set_error("get_valid_counts: bad argument");
    return CVMK_ERR_ARG;
  }
  if (K == 6 && ((uintptr_t)x & 7) == 0 && ((uintptr_t)y & 7) == 0 && B <= 65535) {
    // about one CTA per SM over the whole batch (a CTA of 1024 threads fills an SM's registers)
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int chunks = sms / B;
    const int max_chunks = (N + THREADS - 1) / THREADS;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    int chunk_rows = ((N + chunks - 1) / chunks + 3) & ~3;
    chunks = (N + chunk_rows - 1) / chunk_rows;
    if (clamp > 0)
      gvc6_kernel<true><<<dim3((unsigned)chunks, (unsigned)B), THREADS, 0, (cudaStream_t)stream>>>(
          x, y, valid_count, N, score_threshold, chunk_rows, clamp);
    else
      gvc6_kernel<false><<<dim3((unsigned)chunks, (unsigned)B), THREADS, 0, (cudaStream_t)stream>>>(
          x, y, valid_count, N, score_threshold, chunk_rows, INT32_MAX);
  } else
    gvc_kernel<<<B, THREADS, 0, (cudaStream_t)stream>>>(x, y, valid_count, N, K, score_threshold,
                                                        clamp > 0 ? clamp : INT32_MAX);
  return check_cuda(cudaGetLastError(), "gvc_kernel launch");
}

static inline int nms_npad(int N) { return (N + 3) / 4 * 4; }

// Grid, shared memory and the data-independent part of the -1 tail; launches the kernel.
static int nms_launch(NmsParams& p, cudaStream_t stream, const char* what) {
  int dev = 0, sms = 148;
  if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return CVMK_ERR_CUDA;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int smem_max = 200 * 1024;
  static bool attr_of_device[64] = {false};
  if (dev < 0 || dev >= 64) { set_error("non_max_suppression: device ordinal %d not supported", dev); return CVMK_ERR_ARG; }
  if (!attr_of_device[dev]) {
    if (check_cuda(cudaFuncSetAttribute(nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max),
                   "cudaFuncSetAttribute(nms_kernel)"))
      return CVMK_ERR_CUDA;
    attr_of_device[dev] = true;
  }
  const int work = ((int)sizeof(Smem) + 15) & ~15;
  // the select path (at most SEL_MAX rows take part) keeps the score keys in shared memory
  const bool may_select = (p.topk >= 0 && p.topk <= SEL_MAX) || p.N <= SEL_MAX;
  p.key_cap = may_select ? std::min(p.N, (smem_max - work) / 4) : 0;
  const int smem = work + 4 * p.key_cap;
  int bound = p.N;
  if (p.topk >= 0) bound = std::min(bound, p.topk);
  if (p.mos > 0) bound = std::min(bound, p.mos);
  p.fill_bound = bound;
  p.dbg = 0;
#ifdef CVMK_NMS_TIMING
  if (getenv("NMS_DBG")) p.dbg = atoi(getenv("NMS_DBG"));
#endif
  int fillers = 0;
  if (bound < p.N) {
    const long long tail_bytes = (long long)(p.N - bound) * 24;
    fillers = (int)std::min<long long>(8, std::max<long long>(1, tail_bytes / 65536));
    fillers = std::min(fillers, std::max(1, 4 * sms / p.B));
  }
  if (p.B > 65535) { set_error("non_max_suppression: batch %d too large", p.B); return CVMK_ERR_ARG; }
  nms_kernel<<<dim3(1 + fillers, p.B), THREADS, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), what);
}

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
  return nms_launch(p, (cudaStream_t)stream, "nms_kernel launch");
}

#ifdef CVMK_NMS_TIMING
extern "C" int cvmk_nms_phase_read(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_nms_phase, sizeof(long long) * 16);
}
#endif

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
  NmsParams p;
  p.x = x; p.vc = valid_count; p.y = y; p.xw = nullptr;
  p.B = B; p.N = N;
  p.mos = max_output_size; p.thr = iou_threshold; p.topk = top_k; p.force = force_suppress;
  p.scratch = reinterpret_cast<uint32_t*>(scratch_of_device[dev]);
  p.npad = nms_npad(N);
  p.per_batch_words = 6 * (int64_t)p.npad;
  return nms_launch(p, (cudaStream_t)stream, "nms_kernel launch (static scratch)");
}
