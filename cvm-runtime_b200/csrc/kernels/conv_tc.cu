// conv2d (groups = 1) and dense as an implicit GEMM on the sm_100a tensor cores; grouped 3 x 3
// convolutions with 32 channels per group as well (how depthwise layers are given to it).
//
//   D[pixel, oc] = sum_{kh,kw,c} X[n, oh*s-p+kh*d, ow*s-p+kw*d, c] * Wt[oc, kh, kw, c]
//
// One CTA owns a 128-pixel x BLOCK_N-channel tile of the output and walks K = KH*KW*C in slabs of
// BLOCK_K bytes.  TMA brings each slab of activations (im2col-mode tensor map: 128 consecutive
// output pixels of one filter tap, zero-filled outside the image; a plain 2-D map when the conv
// is a 1x1 / dense) and of weights into a swizzled shared-memory ring; one thread issues
// tcgen05.mma kind::i8 (int8 x int8 -> int32) into a TMEM accumulator; four warps drain the
// accumulator with tcgen05.ld, run the fused element chain (bias, relu, round-shift, clip,
// residual add ...) and store int8 / int32 NHWC.  Two accumulators alternate (four, when a tile is
// at most 128 columns wide) so the drain of tile i overlaps the MMAs of the tiles after it.  The
// int32 sum never reaches HBM.  Stride-1 3 x 3 filters over at most 128 channels (and every
// grouped layer) stage the input halo of a spatial patch once and let every filter tap multiply a
// window of it; in those modes the second producer warp issues the instructions of every second
// tile instead of loading.
//
// int8 outputs leave through shared memory: eight epilogue warps write their packed results into
// a swizzled staging panel (128 rows x up to 128 bytes) that one thread hands to a TMA store, and
// the int8 operand of a residual join arrives in the same panel by a TMA load issued one tile
// ahead, so neither direction costs per-thread global accesses.  int32 outputs (logits, heads)
// and odd channel counts keep plain vector stores.
//
// Reproduces src/runtime/cpu/ops/ops.cc:368-456 (conv2d: im2col_cpu :204-246, matrix_mul
// :148-200) and :34-75 (dense): int32 accumulation of int8 products is exact, so the order of
// summation cannot change a bit.
//
// Every wait in the kernel is bounded: when one runs out the CTA raises a flag, every role leaves
// its loop, TMEM is released and the kernel returns with a non-zero word in *status.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include "common.cuh"
#include "tc_common.cuh"

namespace cvmk {
namespace {

using namespace tc;

constexpr int MAX_STAGES = 8;
constexpr int NUM_EPI_WARPS = 8;
// warp 0: TMA loads of the operands, warp 1: MMA + TMEM owner, warps 2..9: epilogue,
// warp 10: TMA traffic of the staged output tiles (stores, residual-operand loads)
// warp 11: second TMA producer (issuing a load costs its thread about a hundred cycles, so two
// threads take alternate K blocks); in the halo modes, where a tile is one load, second MMA issuer
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS + 64;
constexpr int IO_WARP = 2 + NUM_EPI_WARPS;
constexpr int PRODUCER2_WARP = IO_WARP + 1;
constexpr int SMEM_DYNAMIC_MAX = 227 * 1024 - 8704;  // 227 KB per CTA minus the static part (bias, barriers)
constexpr int MAX_BIAS = 2048;          // bias vectors up to this length are staged in shared memory

// Division of a non-negative 31-bit number by a divisor fixed at launch: q = umulhi(n, mul) >> shr
// (mul = ceil(2^(31 + ceil(log2 d)) / d)); d = 1 is flagged by mul = 0.  Every thread that walks
// tiles divides several times per tile, and a hardware-emulated 32-bit division is a dependent
// chain of some twenty instructions.
struct FastDiv { uint32_t mul, shr; };
__device__ __forceinline__ int fdiv(int n, const FastDiv& d) {
  return d.mul ? (int)(__umulhi((uint32_t)n, d.mul) >> d.shr) : n;
}
inline FastDiv make_fastdiv(int d) {
  FastDiv f = {0, 0};
  if (d <= 1) return f;
  int lg = 0;
  while ((1LL << lg) < d) ++lg;
  const int pw = 31 + lg;
  f.mul = (uint32_t)((((uint64_t)1 << pw) + (uint64_t)d - 1) / (uint64_t)d);
  f.shr = (uint32_t)(pw - 32);
  return f;
}

struct ConvParams {
  void* y;
  int y_dtype;
  int m_total;
  int oc;
  int oh, ow;
  int c, kh, kw;
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int block_k, block_n, stages;
  int units;            // (filter tap, channel block) pairs loaded and multiplied per ring stage
  int a_mode;           // activations: 0 plain 2-D tiles (1x1, dense), 1 im2col-mode TMA, 2 spatial patches,
                        // 3 spatial patches whose input halo is staged once per channel block,
                        // 4 the same with the whole weight matrix resident in shared memory
  int b_resident;       // a_mode 0 with this CTA's N tile of the weights resident in shared memory
  int grouped;          // grouped convolution (a_mode 4): `c` is the channels of ONE group, an N tile is block_n / c
                        // groups and block_k = block_n; group j of N tile n0 reads input channels n0 + j * c .. and
                        // fills accumulator columns j * c ..; the grid is a multiple of the N tiles
  int group_fold;       // grouped: 1, or F = 2 / 4: a pixel is F sub-pixels of block_n / F channels and the filter
                        // moves in sub-pixel steps (see cvmk_conv_desc.group_fold)
  int patch_w, patch_h, patch_n;  // a_mode 2, 3: an M tile is patch_w x patch_h output pixels of patch_n images
  int tiles_w, tiles_h;           // a_mode 2, 3: patches per image row / column
  int patch_w_log2, patch_h_log2; // patch sides are powers of two
  int num_m_tiles, num_n_tiles;
  int num_units, num_kb;          // (tap, channel block) pairs per tile; ring stages consumed per tile
  FastDiv fd_n_tiles, fd_tiles_w, fd_tiles_h, fd_ohow, fd_ow;
  int tmem_cols;
  int two_issuers;      // halo modes: one producer warp is enough (a load or ten per tile), the other warp issues the
                        // tensor-core instructions of every second tile, so that one warp's barrier checks and
                        // commits run while the other's instructions keep the pipe busy
  int acc_bufs;         // accumulators in TMEM: 2, or 4 when block_n <= 128 (the MMA warp may then run three tiles ahead
                        // of the epilogue groups, each of which drains its tiles into accumulators g and g + 2 in turn)
  int* status;
  const int32_t* bias;  // per-channel add applied first (nullptr: none)
  int first_step;       // chain steps before this one are already covered by `bias`
  int tma_out;          // 1: int8 output staged in shared memory and written with TMA
  int res_step;         // chain step whose int8 tensor operand is fetched with TMA (-1: none)
  int panels;           // 128-column panels per tile (1 or 2) on the TMA output path
  int panel_bytes;      // row length of a panel in bytes: min(block_n, 128)
  int io_bufs;          // staging buffers per epilogue group: 1 or 2
  int ring_bytes;       // bytes of the operand ring (the staging buffers follow it)
  // Requantisation fast path (see fast_requant below): 0 off, 1 shift+clamp, 2 + tensor add/sub + clamp
  int fast_mode;
  int f_shift;          // rounding shift (<= 16); its addend 2^(shift-1) is folded into the staged bias
  int f_mul;            // 2^(16 - shift)
  int f_add;
  uint32_t f_lo1, f_hi1;  // first clamp, both halves of an s16x2 word
  uint32_t f_lo2, f_hi2;  // clamp after the tensor step
  int f_sub;            // tensor step subtracts its operand
  int dbg;              // development builds: bit 0 skips the weight loads (timing experiments only)
  int fast_wide;        // the biased sum may exceed the multiply-add's range: clamp it first (f_pre_lo / f_pre_hi)
  int f_pre_lo, f_pre_hi;
  int fast_variant;     // (first clamp starts at 0) + 2 * kind; kind: 0 none, 1 add + clamp from 0, 2 add, 3 subtract
  int bias_static;      // the bias vector is a parameter: it may be read before the previous kernel has finished
  const int8_t* w;      // the weight matrix [oc, kh * kw * c] and its size, for the L2 warm-up
  unsigned w_bytes;
  int k_slices;         // > 1: `oc` counts k_slices x oc_real virtual columns; column block s reduces over
  int oc_real;          //      K slice s (c bytes long) of the real columns and writes int32 partial sums
  DevChain chain;
};

template <int V>
__device__ __forceinline__ void store_vals(const ConvParams& p, size_t lin, const int32_t* v) {
  if (p.y_dtype == CVMK_I8) {
    int8_t* dst = reinterpret_cast<int8_t*>(p.y) + lin;
    if (V == 32) {
      uint4 a, b;
      a.x = pack4(v[0], v[1], v[2], v[3]);     a.y = pack4(v[4], v[5], v[6], v[7]);
      a.z = pack4(v[8], v[9], v[10], v[11]);   a.w = pack4(v[12], v[13], v[14], v[15]);
      b.x = pack4(v[16], v[17], v[18], v[19]); b.y = pack4(v[20], v[21], v[22], v[23]);
      b.z = pack4(v[24], v[25], v[26], v[27]); b.w = pack4(v[28], v[29], v[30], v[31]);
      reinterpret_cast<uint4*>(dst)[0] = a;
      reinterpret_cast<uint4*>(dst)[1] = b;
    } else {  // V == 8
      uint2 a;
      a.x = pack4(v[0], v[1], v[2], v[3]);
      a.y = pack4(v[4], v[5], v[6], v[7]);
      *reinterpret_cast<uint2*>(dst) = a;
    }
  } else {
    int32_t* dst = reinterpret_cast<int32_t*>(p.y) + lin;
#pragma unroll
    for (int q = 0; q < V / 4; ++q)
      reinterpret_cast<int4*>(dst)[q] = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
}

// One thread's row of a tile on the fast path: `chunks` groups of 32 columns are read from TMEM,
// biased (the rounding addend is part of the staged bias), requantised and written to the
// swizzled staging panels, in place of the tensor operand when there is one.
template <int RELU1, int KIND, int WIDE>
__device__ __forceinline__ void fast_chunk(const ConvParams& p, const FastQ& fq, int32_t (&v)[32], int ci,
                                           const int32_t* bias_row, uint8_t* io_base, int panel_size,
                                           uint32_t row_off, uint32_t sw) {
  // (acc + bias + rounding addend) << (16 - shift) as one multiply-add per element: bits
  // [16, 32) of the result are bits [shift, shift + 16) of the biased sum, i.e. the low half of
  // its arithmetic right shift, which is all the packed arithmetic below needs.
  const int4* bp = reinterpret_cast<const int4*>(bias_row + ci * 32);
  const int mul = p.f_mul;
  if (WIDE) {
    // Sums too wide for the multiply-add: the staged bias is the plain one; the biased sum is
    // first clamped to the range the chain's own clamp keeps (after which it fits), then scaled.
    const int lo = p.f_pre_lo, hi = p.f_pre_hi, am = p.f_add * mul;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int4 b4 = bp[j];
      v[4 * j] = min(max(v[4 * j] + b4.x, lo), hi) * mul + am;
      v[4 * j + 1] = min(max(v[4 * j + 1] + b4.y, lo), hi) * mul + am;
      v[4 * j + 2] = min(max(v[4 * j + 2] + b4.z, lo), hi) * mul + am;
      v[4 * j + 3] = min(max(v[4 * j + 3] + b4.w, lo), hi) * mul + am;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int4 b4 = bp[j];
      v[4 * j] = v[4 * j] * mul + b4.x;
      v[4 * j + 1] = v[4 * j + 1] * mul + b4.y;
      v[4 * j + 2] = v[4 * j + 2] * mul + b4.z;
      v[4 * j + 3] = v[4 * j + 3] * mul + b4.w;
    }
  }
  const int c0 = ci * 32;
  uint8_t* pb = io_base + (size_t)(c0 >> 7) * panel_size + row_off;
  const uint32_t j0 = (uint32_t)(c0 & 127) >> 4;
  uint4* q0 = reinterpret_cast<uint4*>(pb + ((j0 ^ sw) << 4));
  uint4* q1 = reinterpret_cast<uint4*>(pb + (((j0 + 1) ^ sw) << 4));
  uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0;
  if (KIND != 0) { r0 = *q0; r1 = *q1; }
  uint4 a, b;
  fast_requant<RELU1, KIND>(fq, v, r0, r1, &a, &b);
  *q0 = a;
  *q1 = b;
}

// `acc_free`: the barrier that hands the accumulator back to the MMA warp.  The warp arrives at it
// as soon as its last columns are in registers (the loads have completed: tcgen05.wait::ld), not
// after the arithmetic on them: the MMA warp's way back to a full accumulator (it notices, issues,
// the instructions run, this group notices) then overlaps the last quarter of this tile's work
// instead of following it.  Used when the tile is so wide that TMEM holds only two accumulators
// (nullptr otherwise: with four, the MMA warp is tiles ahead anyway).
template <int RELU1, int KIND, int WIDE>
__device__ __forceinline__ void fast_row(const ConvParams& p, uint32_t tbase, int chunks, const int32_t* bias_row,
                                         uint8_t* io_base, int panel_size, int row_in_tile, int pw, uint64_t* acc_free) {
  const FastQ fq = {p.f_lo1, p.f_hi1, p.f_lo2, p.f_hi2};
  const uint32_t row_off = (uint32_t)row_in_tile * (uint32_t)pw;
  const uint32_t sw = (row_off >> 7) & (((uint32_t)pw - 1u) >> 4);  // swizzle key of this row, as in panel_offset()
  auto release = [&]() {
    if (acc_free == nullptr) return;
    tc_fence_before();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(acc_free);
  };
  int ci = 0;
  for (; ci + 2 <= chunks; ci += 2) {  // two chunks per TMEM round trip
    int32_t v0[32], v1[32];
    tmem_ld64(tbase + (uint32_t)(ci * 32), v0, v1);
    if (ci + 2 >= chunks) release();
    fast_chunk<RELU1, KIND, WIDE>(p, fq, v0, ci, bias_row, io_base, panel_size, row_off, sw);
    fast_chunk<RELU1, KIND, WIDE>(p, fq, v1, ci + 1, bias_row, io_base, panel_size, row_off, sw);
  }
  if (ci < chunks) {
    int32_t v[32];
    tmem_ld32(tbase + (uint32_t)(ci * 32), v);
    release();
    fast_chunk<RELU1, KIND, WIDE>(p, fq, v, ci, bias_row, io_base, panel_size, row_off, sw);
  }
}

// Optional phase timers (development builds only, -DCVMK_CONV_TIMING): per CTA, cycles the elected
// lanes spend waiting and working.  Slots: 0 producer waits for a free stage, 1 MMA waits for a
// free accumulator, 2 MMA waits for operands, 3 MMA loop, 4+4g.. epilogue group g: wait for the
// accumulator, wait for the staging tile, TMEM loads + arithmetic, store phase; 12 whole kernel.
#ifdef CVMK_CONV_TIMING
__device__ long long g_conv_timing[148 * 16];
#define TSTART(var) long long var = clock64()
#define TSET(var) var = clock64()
#define TADD(slot, var) do { const long long now__ = clock64(); tacc[slot] += now__ - var; var = now__; } while (0)
#define TDECL long long tacc[16] = {0}
#define TFLUSH(slot) do { if (blockIdx.x < 148) g_conv_timing[blockIdx.x * 16 + (slot)] = tacc[slot]; } while (0)
// Event trace of CTA 0: g_conv_trace[role * 512 + seq] = clock of the seq-th event of that role.
__device__ long long g_conv_trace[17 * 512];
#define TRACE(role, seq) do { if (blockIdx.x == 0 && (seq) < 512) g_conv_trace[(role) * 512 + (seq)] = clock64(); } while (0)
#else
#define TRACE(role, seq) do {} while (0)
#define TSTART(var) do {} while (0)
#define TSET(var) do {} while (0)
#define TADD(slot, var) do {} while (0)
#define TDECL do {} while (0)
#define TFLUSH(slot) do {} while (0)
#endif

// Origin of a tile: first output channel, and either the first linear output row (modes 0, 1) or
// the corner (w, h, n) of the spatial patch (mode 2).
struct TileOrigin { int n0, m0, cw, ch, cn, nb, k0; };   // nb: first weight row, k0: first K byte (K slices)
__device__ __forceinline__ TileOrigin tile_origin(const ConvParams& p, int tile) {
  TileOrigin t;
  const int mt = fdiv(tile, p.fd_n_tiles);
  t.n0 = (tile - mt * p.num_n_tiles) * p.block_n;
  t.m0 = mt * BLOCK_M;
  t.nb = t.n0;
  t.k0 = 0;
  if (p.k_slices > 1) {
    const int s = t.n0 / p.oc_real;
    t.nb = t.n0 - s * p.oc_real;
    t.k0 = s * p.c;
  }
  t.cw = t.ch = t.cn = 0;
  if (p.a_mode >= 2) {
    const int r = fdiv(mt, p.fd_tiles_w);
    t.cw = (mt - r * p.tiles_w) * p.patch_w;
    const int tn = fdiv(r, p.fd_tiles_h);
    t.ch = (r - tn * p.tiles_h) * p.patch_h;
    t.cn = tn * p.patch_n;
  }
  return t;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_r,
               const __grid_constant__ ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[MAX_STAGES];
  __shared__ uint64_t bar_empty[MAX_STAGES];
  __shared__ uint64_t bar_acc_full[4];
  __shared__ uint64_t bar_acc_empty[4];
  __shared__ uint64_t bar_res[2][2];     // [group][buffer]: staging buffer free / operand tile landed in it
  __shared__ uint64_t bar_staged[2][2];  // [group][buffer]: the group has written its tile into the buffer
  __shared__ uint64_t bar_weights;       // a_mode 4: the resident weight matrix has landed
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  __shared__ __align__(16) int32_t bias_s[MAX_BIAS];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  // The warp index comes out of a shuffle so that the compiler knows it is the same for the whole
  // warp: the loops of the single-issuer roles below are then run by all 32 lanes on the uniform
  // datapath (loop counters, shared-memory addresses and descriptors stay in uniform registers, which
  // is where TMA and tcgen05 instructions take their operands from) and only the instructions with a
  // side effect are predicated on one elected lane.  Run by lane 0 alone, every operand had to be
  // moved from a per-thread register first, several hundred cycles per TMA / MMA instruction.
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) TRACE(16, 0);
  const int a_bytes = BLOCK_M * p.block_k;
  // (grouped: an N tile is gpt = block_n / c groups of c channels whose activations lie side by side
  //  in one halo of block_k = block_n bytes per pixel; a weight tile is the c x c block of one group)
  const int gpt = p.grouped ? p.block_n / p.c : 1;
  const int b_bytes = p.grouped ? p.c * p.c : p.block_n * p.block_k;
  // b_resident: a 1x1 layer whose N tiles divide the grid, so that every tile of a CTA has the same
  // first output channel: the K blocks of that N tile are loaded once and stay in front of the
  // ring, which then carries activations only.
  const bool b_resident = p.b_resident != 0;
  const int unit_bytes = a_bytes + (b_resident ? 0 : b_bytes);   // one A tile and the B tile that goes with it
  const int num_units = p.num_units;
  // Halo mode (a_mode 3): a ring stage is one channel block: the (patch_w + kw - 1) x
  // (patch_h + kh - 1) input pixels the patch touches, loaded once, then the kh * kw weight tiles.
  // Every filter tap multiplies a window of that halo: the descriptor starts (fy * halo_w + fx)
  // rows in and steps halo_w rows per 8-pixel group (the swizzle is a function of the shared-memory
  // address, so any 16-byte aligned start inside the swizzled halo reads consistently).
  // a_mode 4 is the halo mode with the whole weight matrix resident in shared memory (one or two
  // channel blocks, one N tile): the weights are loaded once per CTA in front of the ring and a
  // stage is the halo alone.
  const bool halo = p.a_mode >= 3;
  const bool w_resident = p.a_mode == 4;
  const int halo_w = p.patch_w + p.kw - 1;
  const int halo_bytes = halo_w * (p.patch_h + p.kh - 1) * p.block_k;
  const int halo_pad = (halo_bytes + 1023) & ~1023;
  const int taps = p.kh * p.kw;
  const int resident_bytes = w_resident ? (p.grouped ? gpt : p.num_kb) * taps * b_bytes   // [channel block | group][tap][tile]
                                        : (b_resident ? p.num_units * b_bytes : 0);   // [K block][block_n x block_k]
  uint8_t* const ring = smem + resident_bytes;
  const int stage_bytes = w_resident ? halo_pad : (halo ? halo_pad + taps * b_bytes : p.units * unit_bytes);
  const int num_kb = p.num_kb;  // ring stages consumed per tile
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const bool bias_in_smem = (p.bias != nullptr || p.fast_mode) && p.oc <= MAX_BIAS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 4; ++a) {
      mbar_init(&bar_acc_full[a], 1);
      mbar_init(&bar_acc_empty[a], NUM_EPI_WARPS / 2);
    }
    for (int a = 0; a < 2; ++a) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bar_res[a][b], 1);
        mbar_init(&bar_staged[a][b], NUM_EPI_WARPS / 2);
      }
    }
    mbar_init(&bar_weights, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, (uint32_t)p.tmem_cols);
  // Programmatic dependent launch: the next kernel of the stream may start its own prologue on SMs
  // this grid has left.  Until griddepcontrol.wait returns, the previous kernel of the stream may
  // still be running, so only memory that no kernel writes is touched before it: the tensor maps
  // and the parameter block (both in the kernel's own argument space), the weights, and the bias
  // when it is a model parameter.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp == IO_WARP) {
    // Warm the descriptor cache with the tensor maps.
    if (lane < 4) {
      const CUtensorMap* m = lane == 0 ? &tmap_a : (lane == 1 ? &tmap_b : (lane == 2 ? &tmap_y : &tmap_r));
      if (lane < 2 || (p.tma_out && (lane == 2 || p.res_step >= 0)))
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
    }
  } else if (warp == PRODUCER2_WARP && lane == 0) {
    // L2 warm-up: this CTA's share of the weight matrix (every CTA reads most of it soon).
    const unsigned per = ((p.w_bytes + gridDim.x - 1) / gridDim.x + 15u) & ~15u;
    const unsigned begin = blockIdx.x * per;
    if (begin < p.w_bytes) {
      const unsigned n = min(per, p.w_bytes - begin) & ~15u;
      if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.w + begin), "r"(n) : "memory");
    }
  }
  // The two producer warps need nothing of the set-up below but the barriers, which thread 0 (of
  // producer warp 0) has just initialised: they meet at a barrier of their own and go on to their
  // loads, whose latency then runs while the other ten warps allocate TMEM and stage the bias.
  // Warp 0 also ARRIVES (without waiting) at the barrier the other ten warps wait at, so that none
  // of them touches an mbarrier or the abort flag before thread 0 has initialised them.
  const bool two_issuers = p.two_issuers != 0;
  const bool is_producer = warp == 0 || (warp == PRODUCER2_WARP && !two_issuers);
  const int setup_threads = two_issuers ? NUM_THREADS : NUM_THREADS - 32;   // the waiting warps plus warp 0's arrival
  if (warp == 0) {
    __threadfence_block();
    asm volatile("bar.arrive 1, %0;" ::"r"(setup_threads) : "memory");
  }
  if (is_producer && !two_issuers) asm volatile("bar.sync 2, 64;" ::: "memory");
  auto stage_bias = [&]() {
    const int padded = min(MAX_BIAS, (p.oc + 31) & ~31);
    for (int i = (int)threadIdx.x - 32; i < padded; i += NUM_THREADS - 64) {   // warps 1..10
      const int32_t b = i < p.oc && p.bias ? __ldg(p.bias + i) : 0;
      // fast path: (bias + rounding addend) pre-multiplied by 2^(16 - shift), see fast_row()
      bias_s[i] = (p.fast_mode && !p.fast_wide) ? (int32_t)((uint32_t)(b + p.f_add) * (uint32_t)p.f_mul) : b;
    }
  };
  uint32_t tmem_base = 0;
  if (!is_producer) {
    if (bias_in_smem && p.bias_static) stage_bias();
    if (bias_in_smem && !p.bias_static) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      stage_bias();
    }
    // Every role below finishes its own set-up arithmetic first and executes griddepcontrol.wait just
    // before its loop, so that the set-up overlaps the tail of the previous kernel.
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"r"(setup_threads) : "memory");   // ten or eleven warps wait, warp 0 has arrived
    tc_fence_after();
    tmem_base = tmem_slot;
  }
  if (threadIdx.x == 0) TRACE(16, 2);

  if (is_producer) {
    // ------------------------------------------------------------------ TMA producers
    // Producer `which` issues the K blocks whose running number (over all tiles of this CTA) is
    // congruent to it modulo 2; both walk the same sequence of ring slots.
    {
      const bool leader = elect_one();
      const int which = warp == 0 ? 0 : 1;
      if (which == 0 && leader) TRACE(16, 6);
      int stage = which;  // the ring has at least two stages
      uint32_t phase = which >= p.stages ? 1u : 0u;
      int turn = which;  // 0: the next stage is this producer's
      bool live = true;
      int pseq = 0; (void)pseq;
      TDECL;
      TSTART(tk);
      // The loop below runs on one thread, so its own instruction latency bounds the rate of
      // loads: the filter taps are walked with nested counters (no divisions), and everything
      // that is constant for a tile is computed once per tile.
      const uint32_t smem_base = smem_u32(ring);
      const uint32_t full0 = smem_u32(&bar_full[0]);
      const TileOrigin to_first = tile_origin(p, (int)blockIdx.x);
      if (w_resident && which == 0) {  // the weight rows of this CTA's N tile, once (every tile of a CTA has the same n0)
        const uint32_t wb = smem_u32(&bar_weights);
        if (leader) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wb), "r"((uint32_t)resident_bytes) : "memory");
        uint32_t dst = smem_u32(smem);
        for (int cb = 0; cb < (p.grouped ? gpt : p.num_kb); ++cb) {
          int kcol = p.grouped ? 0 : cb * p.block_k;
          const int wrow = p.grouped ? to_first.n0 + cb * p.c : to_first.n0;
          for (int t = 0; t < taps; ++t) {
            if (leader) asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&tmap_b)), "r"(wb),
                "r"(kcol), "r"(wrow)
                : "memory");
            dst += (uint32_t)b_bytes;
            kcol += p.c;
          }
        }
      }
      if (b_resident && which == 0) {   // this CTA's N tile of the weights, once
        const uint32_t wb = smem_u32(&bar_weights);
        if (leader) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wb), "r"((uint32_t)resident_bytes) : "memory");
        uint32_t dst = smem_u32(smem);
        for (int u = 0; u < p.num_units; ++u, dst += (uint32_t)b_bytes)
          if (leader) asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
              " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&tmap_b)), "r"(wb),
              "r"(u * p.block_k), "r"(to_first.n0)
              : "memory");
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (which == 0 && leader) TRACE(16, 1);
      for (int tile = blockIdx.x; live && tile < num_tiles; tile += gridDim.x) {
        const TileOrigin to = tile == (int)blockIdx.x ? to_first : tile_origin(p, tile);
        const int m0 = to.m0;
        if (which == 0 && tile == (int)blockIdx.x && leader) TRACE(16, 7);
        int img = 0, base_w = 0, base_h = 0;
        if (p.a_mode == 1) {
          img = fdiv(m0, p.fd_ohow);
          const int rem = m0 - img * (p.oh * p.ow);
          const int oy = fdiv(rem, p.fd_ow);
          const int ox = rem - oy * p.ow;
          base_w = ox * p.stride_w - p.pad_w;
          base_h = oy * p.stride_h - p.pad_h;
        }
        if (halo) {
          for (int cb = 0; cb < num_kb; ++cb) {
            const bool my_stage = two_issuers || turn == 0;   // (a single producer takes every stage)
            turn ^= 1;
            if (!my_stage) continue;
            TSTART(tw);
            if (!mbar_wait(&bar_empty[stage], phase ^ 1, &abort_flag, 1)) { live = false; break; }
            TADD(0, tw);
            if (leader) TRACE(which * 2, pseq);
            const uint32_t sa = smem_base + (uint32_t)(stage * stage_bytes);
            const uint32_t bar = full0 + 8u * (uint32_t)stage;
            if (leader) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                         "r"((uint32_t)(halo_bytes + (w_resident ? 0 : taps * b_bytes))) : "memory");
            const int cc = cb * p.block_k;
            const int ca = p.grouped ? cc + to.n0 : cc;   // a group reads its own input channels
            if (leader) asm volatile(
                "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(sa), "l"(reinterpret_cast<uint64_t>(&tmap_a)),
                "r"(bar), "r"(ca), "r"(to.cw - p.pad_w), "r"(to.ch - p.pad_h), "r"(to.cn)
                : "memory");
            uint32_t sb = sa + (uint32_t)halo_pad;
            int kcol = cc;
            for (int t = 0; t < (w_resident ? 0 : taps); ++t) {   // (grouped convolutions always keep their weights)
              if (leader) asm volatile(
                  "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                  " [%0], [%1, {%3, %4}], [%2];" ::"r"(sb), "l"(reinterpret_cast<uint64_t>(&tmap_b)),
                  "r"(bar), "r"(kcol), "r"(to.n0)
                  : "memory");
              sb += (uint32_t)b_bytes;
              kcol += p.c;
            }
            if (leader) TRACE(which * 2 + 1, pseq);
            ++pseq;
            stage += two_issuers ? 1 : 2;
            if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
          }
          continue;
        }
        // Units (filter tap x channel block) in weight-matrix order; p.units of them share a stage.
        int kcol = 0, fy = 0, fx = 0, cc = 0, slot = 0;
        bool mine = false;
        uint32_t sa = 0, bar = 0;
        for (int unit = 0; unit < num_units; ++unit) {
          if (slot == 0) {
            mine = two_issuers || turn == 0;
            turn ^= 1;
            if (mine) {
              if (which == 0 && pseq == 0 && leader) TRACE(16, 8);
              TSTART(tw);
              if (!mbar_wait(&bar_empty[stage], phase ^ 1, &abort_flag, 1)) { live = false; break; }
              TADD(0, tw);
              if (leader) TRACE(which * 2, pseq);
              sa = smem_base + (uint32_t)(stage * stage_bytes);
              bar = full0 + 8u * (uint32_t)stage;
              const int in_stage = min(p.units, num_units - unit);
              if (leader) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                           "r"((uint32_t)(in_stage * unit_bytes)) : "memory");
            }
          }
          if (mine && leader) {
            const int off_w = fx * p.dil_w, off_h = fy * p.dil_h;
            if (p.a_mode == 2)  // the patch of this tile, shifted by the filter tap; zero fill outside the image
              asm volatile(
                  "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                  " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(sa), "l"(reinterpret_cast<uint64_t>(&tmap_a)),
                  "r"(bar), "r"(cc), "r"(to.cw + off_w - p.pad_w), "r"(to.ch + off_h - p.pad_h), "r"(to.cn)
                  : "memory");
            else if (p.a_mode == 1)
              asm volatile(
                  "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                  " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(sa),
                  "l"(reinterpret_cast<uint64_t>(&tmap_a)), "r"(bar), "r"(cc), "r"(base_w), "r"(base_h), "r"(img),
                  "h"((uint16_t)off_w), "h"((uint16_t)off_h)
                  : "memory");
            else
              asm volatile(
                  "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                  " [%0], [%1, {%3, %4}], [%2];" ::"r"(sa), "l"(reinterpret_cast<uint64_t>(&tmap_a)), "r"(bar),
                  "r"(cc + to.k0), "r"(m0)
                  : "memory");
            if (!b_resident) asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%3, %4}], [%2];" ::"r"(sa + (uint32_t)a_bytes), "l"(reinterpret_cast<uint64_t>(&tmap_b)),
                "r"(bar), "r"(kcol + to.k0), "r"(to.nb)
                : "memory");
          }
          if (mine) sa += (uint32_t)unit_bytes;
          // next unit
          kcol += p.block_k;
          cc += p.block_k;
          if (cc >= p.c) { cc = 0; if (++fx == p.kw) { fx = 0; ++fy; } }
          if (++slot == p.units || unit + 1 == num_units) {
            slot = 0;
            if (mine) {
              if (leader) TRACE(which * 2 + 1, pseq);
              ++pseq;
              stage += two_issuers ? 1 : 2;
              if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
            }
          }
        }
      }
      TADD(12, tk);
#ifdef CVMK_CONV_TIMING
      if (which == 0 && leader) { TFLUSH(0); TFLUSH(12); }
#endif
    }
  } else if (warp == 1 || warp == PRODUCER2_WARP) {
    // ------------------------------------------------------------------ MMA issuer(s)
    // One warp, or two that take the tiles of this CTA in turn (two_issuers): tiles are independent
    // of each other (own ring stages, own accumulator), so the two warps need no ordering between
    // them; each derives the stage and the accumulator of its tiles from the tile's running number.
    {
      const int issuers = two_issuers ? 2 : 1;
      const int me = warp == 1 ? 0 : 1;
      const bool leader = elect_one();
      const uint32_t idesc = umma_idesc_i8(p.grouped ? p.c : p.block_n);
      const uint64_t desc_a0 = umma_desc(smem_u32(ring), p.block_k);
      const uint64_t desc_w0 = umma_desc(smem_u32(smem), p.grouped ? p.c : p.block_k);  // resident weights (a_mode 4)
      const uint32_t w_lo0 = (uint32_t)desc_w0, w_hi = (uint32_t)(desc_w0 >> 32);
      // halo windows: 8-pixel groups are one halo row (halo_w pixels) apart
      const uint64_t desc_halo0 = (desc_a0 & ~((uint64_t)0x3FFF << 32)) |
                                  ((uint64_t)(((uint32_t)(halo_w * p.block_k)) >> 4) << 32);
      const int nk = p.block_k / 32;
      // descriptor halves and steps in 16-byte address units
      const uint32_t a_lo0 = (uint32_t)desc_a0, a_hi = (uint32_t)(desc_a0 >> 32);
      const uint32_t halo_hi = (uint32_t)(desc_halo0 >> 32);
      const uint32_t stage_q = (uint32_t)stage_bytes >> 4, unit_q = (uint32_t)unit_bytes >> 4;
      const uint32_t a_q = (uint32_t)a_bytes >> 4, b_q = (uint32_t)b_bytes >> 4;
      const uint32_t halo_pad_q = (uint32_t)halo_pad >> 4, halo_row_q = (uint32_t)(halo_w * p.block_k) >> 4;
      const uint32_t pix_q = (uint32_t)p.block_k >> 4;   // grouped: one pixel of the halo row
      // grouped: where filter column t of group g starts inside a halo row (16-byte units).  Without
      // folding that is halo pixel t, the group's own 32 channels.  With F sub-pixels per pixel the
      // group of sub-pixel a reads sub-pixel a + t - 1: the same halo pixel (1) for most, the last
      // sub-pixel of pixel 0 / the first of pixel 2 at the ends.
      uint32_t g_off[4][3];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int fold = p.group_fold > 1 ? p.group_fold : 1;
        const int cs = p.block_n / fold;          // channels per sub-pixel
        const int gps = cs >> 5;                  // 32-channel groups per sub-pixel
        const int a = p.group_fold > 1 ? g / gps : 0, h = p.group_fold > 1 ? g - a * gps : g;
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          int px = t, b = 0;
          if (p.group_fold > 1) {
            const int bp = a + t - 1;
            px = bp < 0 ? 0 : (bp >= fold ? 2 : 1);
            b = bp - (px - 1) * fold;
          }
          g_off[g][t] = (uint32_t)px * pix_q + (uint32_t)((b * cs + h * 32) >> 4);
        }
      }
      // this issuer's first tile is the CTA's tile number `me`: me * num_kb stages and me accumulators in
      int stage = (me * num_kb) % p.stages;
      uint32_t phase = (uint32_t)((me * num_kb) / p.stages) & 1u;
      int acc = me % p.acc_bufs;
      uint32_t acc_phase = (uint32_t)(me / p.acc_bufs) & 1u;
      bool live = true;
      // tcgen05.commit keeps this thread until the instructions queued before it have left the
      // queue, so after a commit the tensor pipe stands idle until the next instruction has been
      // issued -- through the loop overhead and the barrier checks of the next tile, if the commits
      // sit at the end of a tile.  So the commits a tile owes (its accumulator is complete, its ring
      // stage is free) are issued a few instructions INTO the next stage's instructions, where
      // nothing but the rest of that straight-line block follows them; they then also cover those
      // few instructions, which delays the signal by their run time.  Done in the halo modes, whose
      // stages are nine or more instructions and whose rings are deep.  Whenever the thread would
      // have to block on a barrier it pays its debts first (flush), so that an epilogue group or a
      // producer never waits for a commit that waits for them.
      int owed_stage = -1, owed_acc = -1;
      auto flush = [&]() {
        if (leader) {
          if (owed_acc >= 0) mma_commit(&bar_acc_full[owed_acc]);
          if (owed_stage >= 0) mma_commit(&bar_empty[owed_stage]);
        }
        owed_acc = owed_stage = -1;
      };
      auto ensure = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        if (mbar_test(bar, parity)) return true;
        flush();
        return mbar_wait(bar, parity, &abort_flag, code);
      };
      int mseq = 0, tseq = 0; (void)mseq; (void)tseq;
      TDECL;
      TSTART(tl);
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if ((w_resident || b_resident) && blockIdx.x < num_tiles && !mbar_wait(&bar_weights, 0u, &abort_flag, 7)) live = false;
      for (int tile = blockIdx.x + me * (int)gridDim.x; live && tile < num_tiles; tile += issuers * (int)gridDim.x) {
        TSTART(tw);
        if (!ensure(&bar_acc_empty[acc], acc_phase ^ 1, 2)) { live = false; break; }
        TADD(1, tw);
        if (leader) TRACE(6, tseq);
        ++tseq;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.block_n);
        int unit = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ensure(&bar_full[stage], phase, 3)) { live = false; break; }
          TADD(2, tw);
          if (leader) TRACE(4, mseq);
          tc_fence_after();
          const uint32_t st = a_lo0 + stage_q * (uint32_t)stage;
          if (halo) {
            TSTART(ti);
            if (p.grouped) {
              // every group of the N tile: its own columns of the halo rows, its own 9 weight tiles,
              // its own accumulator columns (the first tap overwrites them)
              uint32_t bl = w_lo0;
              uint32_t d_blk = d_tmem;
#pragma unroll
              for (int g = 0; g < 4; ++g) {   // 32 accumulator columns each
                if (g < gpt) {
#pragma unroll
                  for (int fy = 0; fy < 3; ++fy) {
                    const uint32_t al = st + (uint32_t)fy * halo_row_q;
#pragma unroll
                    for (int fx = 0; fx < 3; ++fx) {
                      if (leader) mma_i8_k<1>(d_blk, al + g_off[g][fx], halo_hi, bl, w_hi, idesc, (uint32_t)(fy | fx));
                      bl += b_q;
                    }
                    if (fy == 0 && g == 0) flush();
                  }
                  d_blk += 32u;
                }
              }
            } else {
              // 3 x 3 taps x two K slices of the 64-channel block, straight line
              uint32_t bl = w_resident ? w_lo0 + (uint32_t)(kb * 9) * b_q : st + halo_pad_q;
#pragma unroll
              for (int fy = 0; fy < 3; ++fy) {
                uint32_t al = st + (uint32_t)fy * halo_row_q;
#pragma unroll
                for (int fx = 0; fx < 3; ++fx) {
                  if (leader) mma_i8_k<2>(d_tmem, al, halo_hi, bl, a_hi, idesc, (uint32_t)(kb | fy | fx));
                  al += 4u;   // one pixel of 64 channels
                  bl += b_q;
                }
                if (fy == 0) flush();
              }
            }
            TADD(13, ti);
            owed_stage = stage;
            if (leader) TRACE(5, mseq);
            ++mseq;
            TADD(14, ti);
            TSET(tw);
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
            continue;
          }
          const int in_stage = min(p.units, num_units - unit);
          uint32_t al = st;
          // B next to A in the stage, or K block `unit` of the resident weights
          uint32_t bl = b_resident ? w_lo0 + (uint32_t)unit * b_q : st + a_q;
          const uint32_t b_step = b_resident ? b_q : unit_q;
          // (a stage of these modes is one to four instructions groups: its commit follows at once --
          //  deferring it would only take a stage out of a ring that is three deep)
          if (leader) {
            if (nk == 4) {
              for (int u = 0; u < in_stage; ++u, al += unit_q, bl += b_step) mma_i8_k<4>(d_tmem, al, a_hi, bl, a_hi, idesc, (uint32_t)(unit + u));
            } else if (nk == 2) {
              for (int u = 0; u < in_stage; ++u, al += unit_q, bl += b_step) mma_i8_k<2>(d_tmem, al, a_hi, bl, a_hi, idesc, (uint32_t)(unit + u));
            } else {
              for (int u = 0; u < in_stage; ++u, al += unit_q, bl += b_step) mma_i8_k<1>(d_tmem, al, a_hi, bl, a_hi, idesc, (uint32_t)(unit + u));
            }
            mma_commit(&bar_empty[stage]);
            TRACE(5, mseq);
          }
          unit += in_stage;
          ++mseq;
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!live) break;
        owed_acc = acc;
        if (!halo) flush();
        // on to this issuer's next tile: past the other issuer's stages and accumulator
        for (int k = 0; k < issuers; ++k)
          if (++acc == p.acc_bufs) { acc = 0; acc_phase ^= 1; }
        for (int k = 0; k < (issuers - 1) * num_kb; ++k)
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (live) flush();
      TADD(3, tl);
#ifdef CVMK_CONV_TIMING
      if (leader) { TFLUSH(1); TFLUSH(2); TFLUSH(3); TFLUSH(13); TFLUSH(14); }
#endif
    }
  } else if (warp < IO_WARP) {
    // ------------------------------------------------------------------ epilogue warps
    // Two groups of four warps; group g drains accumulator g, i.e. every second tile of this
    // CTA, so the waits of one group (TMEM loads, barriers) hide behind the other's work.  On the
    // TMA output path a group writes its tile into one of its staging buffers and hands it to the
    // IO warp; it never waits for a store itself.
    const int ew = warp - 2;         // 0..7
    const int quarter = warp & 3;    // TMEM lanes 32*quarter .. +31 belong to this warp
    const int group = ew >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const bool has_res = p.tma_out && p.res_step >= 0;
    const int pw = p.panel_bytes;
    const int panel_size = BLOCK_M * pw;
    const int buf_bytes = p.panels * panel_size;
    const bool leader = lane == 0 && (ew & 3) == 0;
    uint8_t* group_base = smem + p.ring_bytes + (size_t)group * p.io_bufs * buf_bytes;
    const bool vec_ok = (p.y_dtype == CVMK_I8) ? (p.oc % 16 == 0) : (p.oc % 4 == 0);
    const bool four_acc = p.acc_bufs == 4;
    const int stride_tiles = 2 * gridDim.x;
    const int first_tile = blockIdx.x + group * gridDim.x;
    // patch mode: this thread's pixel inside the patch
    int pr_w = 0, pr_h = 0, pr_n = 0;
    if (p.a_mode >= 2) {
      pr_w = row_in_tile & (p.patch_w - 1);
      const int r = row_in_tile >> p.patch_w_log2;
      pr_h = r & (p.patch_h - 1);
      pr_n = r >> p.patch_h_log2;
    }
    int k = 0;  // index of this group's tile
    TDECL;
    (void)leader;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int tile = first_tile; tile < num_tiles; tile += stride_tiles, ++k) {
      const TileOrigin to = tile_origin(p, tile);
      const int n0 = to.n0;
      int row = to.m0 + row_in_tile;  // linear output row; m_total marks a row outside the tensor
      if (p.a_mode >= 2) {
        const int ow = to.cw + pr_w, oh = to.ch + pr_h, on = to.cn + pr_n;
        row = (ow < p.ow && oh < p.oh && on * p.oh * p.ow < p.m_total) ? (on * p.oh + oh) * p.ow + ow : p.m_total;
      }
      const int buf = p.io_bufs == 2 ? (k & 1) : 0;
      const uint32_t use = (uint32_t)(p.io_bufs == 2 ? (k >> 1) : k);  // how often this buffer was used before
      uint8_t* io_base = group_base + (size_t)buf * buf_bytes;
      TSTART(tw);
      // this group's k-th tile: accumulator g, or g and g + 2 in turn
      const int acc = four_acc ? group + 2 * (k & 1) : group;
      bool ok = mbar_wait(&bar_acc_full[acc], (uint32_t)((four_acc ? k >> 1 : k) & 1), &abort_flag, 4);
      TADD(4 + 4 * group, tw);
      if (leader) TRACE(7 + 3 * group, k);
      tc_fence_after();
      // the staging buffer is ours: its previous store has been read, or the operand tile landed
      if (ok && p.tma_out) ok = mbar_wait(&bar_res[group][buf], use & 1u, &abort_flag, 5);
      TADD(5 + 4 * group, tw);
      if (leader) TRACE(8 + 3 * group, k);
      if (!ok) break;
      if (ok) {
        const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * p.block_n);
        if (p.fast_mode) {
          const int chunks = min(p.block_n, p.oc - n0) >> 5;  // OC is a multiple of 32 on this path
          const int32_t* brow = bias_s + n0;
          uint64_t* early_free = four_acc ? nullptr : &bar_acc_empty[acc];
          switch (p.fast_variant + 8 * p.fast_wide) {
            case 0: fast_row<0, 0, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 1: fast_row<1, 0, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 2: fast_row<0, 1, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 3: fast_row<1, 1, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 4: fast_row<0, 2, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 5: fast_row<1, 2, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 6: fast_row<0, 3, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 7: fast_row<1, 3, 0>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 8: fast_row<0, 0, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 9: fast_row<1, 0, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 10: fast_row<0, 1, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 11: fast_row<1, 1, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 12: fast_row<0, 2, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 13: fast_row<1, 2, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            case 14: fast_row<0, 3, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
            default: fast_row<1, 3, 1>(p, tbase, chunks, brow, io_base, panel_size, row_in_tile, pw, early_free); break;
          }
        } else {
        int32_t v[32];
        tmem_ld32(tbase, v);
        for (int c0 = 0; c0 < p.block_n; c0 += 32) {
          const int col0 = n0 + c0;
          if (col0 >= p.oc) break;  // uniform across the warp
          if (p.bias || p.fast_mode) {
            if (bias_in_smem) {
              const int4* bp = reinterpret_cast<const int4*>(bias_s + col0);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int4 b4 = bp[j];
                v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += (col0 + j < p.oc) ? __ldg(p.bias + col0 + j) : 0;
            }
          }
          const size_t lin = (size_t)row * p.oc + col0;
          if (p.tma_out) {
            uint8_t* pb = io_base + (size_t)(c0 >> 7) * panel_size;
            const int j0 = (c0 & 127) >> 4;  // first 16-byte chunk of this thread inside the panel row
            uint4* q0 = reinterpret_cast<uint4*>(pb + panel_offset(row_in_tile, j0, pw));
            uint4* q1 = reinterpret_cast<uint4*>(pb + panel_offset(row_in_tile, j0 + 1, pw));
            if (row < p.m_total) {
              if (has_res) {
                int32_t rv[32];
                const uint4 r0 = *q0, r1 = *q1;
                const int w[8] = {(int)r0.x, (int)r0.y, (int)r0.z, (int)r0.w, (int)r1.x, (int)r1.y, (int)r1.z, (int)r1.w};
#pragma unroll
                for (int e = 0; e < 32; ++e) rv[e] = (int32_t)(int8_t)(w[e >> 2] >> ((e & 3) * 8));
                apply_chain<32, true>(p.chain, v, lin, col0, 1, rv, p.res_step, p.first_step);
              } else {
                apply_chain<32>(p.chain, v, lin, col0, 1, nullptr, -1, p.first_step);
              }
            }
            uint4 a, b;
            a.x = pack4(v[0], v[1], v[2], v[3]);     a.y = pack4(v[4], v[5], v[6], v[7]);
            a.z = pack4(v[8], v[9], v[10], v[11]);   a.w = pack4(v[12], v[13], v[14], v[15]);
            b.x = pack4(v[16], v[17], v[18], v[19]); b.y = pack4(v[20], v[21], v[22], v[23]);
            b.z = pack4(v[24], v[25], v[26], v[27]); b.w = pack4(v[28], v[29], v[30], v[31]);
            *q0 = a;
            *q1 = b;
          } else if (row < p.m_total) {
            if (col0 + 32 <= p.oc && vec_ok) {
              apply_chain<32>(p.chain, v, lin, col0, 1, nullptr, -1, p.first_step);
              store_vals<32>(p, lin, v);
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (col0 + g * 8 < p.oc) {
                  int32_t t[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) t[j] = v[g * 8 + j];
                  apply_chain<8>(p.chain, t, lin + g * 8, col0 + g * 8, 1, nullptr, -1, p.first_step);
                  store_vals<8>(p, lin + g * 8, t);
                }
              }
            }
          }
          if (c0 + 32 < p.block_n && n0 + c0 + 32 < p.oc) tmem_ld32(tbase + (uint32_t)(c0 + 32), v);
        }
        }
      }
      tc_fence_before();
      if (p.tma_out) fence_async_smem();  // make the staged bytes visible to the TMA engine
      __syncwarp();
      if (lane == 0) {
        if (!p.fast_mode || four_acc) mbar_arrive(&bar_acc_empty[acc]);   // (else fast_row has handed it back already)
        if (p.tma_out) mbar_arrive(&bar_staged[group][buf]);
      }
      TADD(6 + 4 * group, tw);
      if (leader) TRACE(9 + 3 * group, k);
      if (abort_flag) break;
    }
#ifdef CVMK_CONV_TIMING
    if (leader) { TFLUSH(4 + 4 * group); TFLUSH(5 + 4 * group); TFLUSH(6 + 4 * group); TFLUSH(7 + 4 * group); }
#endif
  } else if (p.tma_out) {
    const bool leader = elect_one();
    // ------------------------------------------------------------------ IO warp
    // Moves the staged tiles: waits until a group has written a buffer, stores it with TMA, waits
    // until the TMA engine has read it, then hands the buffer back -- directly, or by loading the
    // int8 operand tile of the tile that will use it next (residual joins).
    const bool has_res = p.res_step >= 0;
    const int panel_size = BLOCK_M * p.panel_bytes;
    const int buf_bytes = p.panels * panel_size;
    uint8_t* io_all = smem + p.ring_bytes;
    auto buffer_of = [&](int g, int b) { return io_all + (size_t)(g * p.io_bufs + b) * buf_bytes; };
    auto hand_back = [&](int g, int b, int next_tile) {
      if (next_tile >= num_tiles) return;
      if (!has_res) { if (leader) mbar_arrive(&bar_res[g][b]); return; }
      const TileOrigin to = tile_origin(p, next_tile);
      uint8_t* dst = buffer_of(g, b);
      if (leader) {
        mbar_expect_tx(&bar_res[g][b], (uint32_t)buf_bytes);
        for (int q = 0; q < p.panels; ++q) {
          if (p.a_mode >= 2)
            tma_load_4d(dst + (size_t)q * panel_size, &tmap_r, &bar_res[g][b], to.n0 + q * 128, to.cw, to.ch, to.cn);
          else
            tma_load_2d(dst + (size_t)q * panel_size, &tmap_r, &bar_res[g][b], to.n0 + q * 128, to.m0);
        }
      }
    };
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // every buffer starts free (or with the operand of its first tile on the way)
    for (int g = 0; g < 2; ++g)
      for (int b = 0; b < p.io_bufs; ++b) hand_back(g, b, (int)blockIdx.x + (2 * b + g) * (int)gridDim.x);
    int i = 0;  // position in this CTA's tile sequence
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++i) {
      const int g = i & 1, k = i >> 1;
      const int b = p.io_bufs == 2 ? (k & 1) : 0;
      const uint32_t use = (uint32_t)(p.io_bufs == 2 ? (k >> 1) : k);
      if (!mbar_wait(&bar_staged[g][b], use & 1u, &abort_flag, 6)) break;
      if (leader) TRACE(13, i);
      const TileOrigin to = tile_origin(p, tile);
      const uint8_t* src = buffer_of(g, b);
      if (leader) {
        for (int q = 0; q < p.panels; ++q) {
          if (to.n0 + q * 128 >= p.oc) break;
          if (p.a_mode >= 2) tma_store_4d(&tmap_y, src + (size_t)q * panel_size, to.n0 + q * 128, to.cw, to.ch, to.cn);
          else tma_store_2d(&tmap_y, src + (size_t)q * panel_size, to.n0 + q * 128, to.m0);
        }
        tma_store_commit();
        tma_store_wait_read();
        TRACE(14, i);
      }
      __syncwarp();
      hand_back(g, b, tile + 2 * p.io_bufs * (int)gridDim.x);
      if (leader) TRACE(15, i);
    }
    // Every store has been read out of shared memory (wait_group.read above); the writes
    // themselves complete with the grid, which is what the next kernel's griddepcontrol.wait
    // (or the stream order) waits for.
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (threadIdx.x == 0) TRACE(16, 3);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TRACE(16, 4);
  if (abort_flag) {
    // Give copies that may still be in flight time to land before shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, 0x100 | abort_flag);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    if (lane == 0) TRACE(16, 5);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

void* driver_entry(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
    set_error("cudaGetDriverEntryPoint(%s) failed: %s", name, cudaGetErrorString(e));
    return nullptr;
  }
  return fn;
}

CUtensorMapSwizzle swizzle_for(int row_bytes) {
  return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

int pick_block_k(int c) { return c % 128 == 0 ? 128 : (c % 64 == 0 ? 64 : 32); }

int pick_block_n(int oc) {
  if (oc >= 256 && oc % 256 == 0) return 256;
  if (oc > 128) return (oc % 128 == 0 || oc > 256) ? 128 : 256;
  int n = 32;
  while (n < oc) n *= 2;  // 32, 64, 128
  return n;
}

bool is_pointwise(const cvmk_conv_desc& d) {
  return d.KH == 1 && d.KW == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_h == 0 &&
         d.pad_w == 0;
}

// 2-D int8 tensor map over a row-major [rows, cols] matrix with a {box_cols, box_rows} box.
CUresult encode_rows(EncodeTiledFn enc, CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                     int box_cols, int box_rows, CUtensorMapL2promotion promo) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(box_cols), promo,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

// 4-D int8 tensor map over an NHWC tensor [n, h, w, c] with a {box_c, box_w, box_h, box_n} box.
CUresult encode_nhwc(EncodeTiledFn enc, CUtensorMap* map, const void* base, int64_t n, int64_t h, int64_t w,
                     int64_t c, int box_c, int box_w, int box_h, int box_n, CUtensorMapL2promotion promo) {
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c, (cuuint64_t)(w * c), (cuuint64_t)(h * w * c)};
  cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)box_w, (cuuint32_t)box_h, (cuuint32_t)box_n};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(box_c), promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

// Spatial patches for stride-1 filters: an M tile of 128 output pixels is pw x ph pixels of pn
// images (powers of two, pw * ph * pn = 128), so that the activations of one filter tap are one
// plain tiled TMA box shifted by the tap.  Picks the split that wastes the fewest rows; false if
// even that needs over a quarter more tiles than the linear order.
bool pick_patch(const cvmk_conv_desc& d, int* pw, int* ph, int* pn) {
  const int64_t linear = ((int64_t)d.N * d.OH * d.OW + BLOCK_M - 1) / BLOCK_M;
  int64_t best = -1;
  for (int w = BLOCK_M; w >= 1; w >>= 1) {
    for (int h = 1; w * h <= BLOCK_M; h <<= 1) {
      const int n = BLOCK_M / (w * h);
      const int64_t tiles = (int64_t)((d.OW + w - 1) / w) * ((d.OH + h - 1) / h) * ((d.N + n - 1) / n);
      if (best < 0 || tiles < best) { best = tiles; *pw = w; *ph = h; *pn = n; }
    }
  }
#ifdef CVMK_CONV_TIMING
  if (const char* e = getenv("CVM_PATCH")) {  // development builds: force a patch shape "w,h,n"
    if (sscanf(e, "%d,%d,%d", pw, ph, pn) == 3 && *pw * *ph * *pn == BLOCK_M) return true;
  }
#endif
  return best > 0 && best * 4 <= linear * 5;
}

// Halo tiles are 8 x 16 output pixels of one image: taken when that needs at most 35 % more tiles
// than cutting the output rows linearly.
bool halo_tiles_fit(const cvmk_conv_desc& d) {
  const int64_t linear = ((int64_t)d.N * d.OH * d.OW + BLOCK_M - 1) / BLOCK_M;
  const int64_t tiles = (int64_t)((d.OW + 7) / 8) * ((d.OH + 15) / 16) * d.N;
  return tiles * 20 <= linear * 27;
}

// Grouped convolutions run in halo mode only, one group per N tile.
bool grouped_supported(const cvmk_conv_desc& d) {
  if (d.C % d.groups != 0 || d.OC % d.groups != 0) return false;
  const int cg = d.C / d.groups;
  if (cg != d.OC / d.groups || cg != 32) return false;
  if (d.KH != 3 || d.KW != 3 || d.stride_h != 1 || d.stride_w != 1 || d.dil_h != 1 || d.dil_w != 1) return false;
  if (d.group_fold > 1) {   // folded pixels: one N tile holds all sub-pixels; the real padding is one sub-pixel
    if ((d.group_fold != 2 && d.group_fold != 4) || d.C != 128 || d.pad_w != 1) return false;
    if (d.OH != d.H + 2 * d.pad_h - 2 || d.OW != d.W) return false;
    return halo_tiles_fit(d);
  }
  if (d.OH != d.H + 2 * d.pad_h - 2 || d.OW != d.W + 2 * d.pad_w - 2) return false;
  return halo_tiles_fit(d);
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_conv2d_tc_supported(const cvmk_conv_desc* d) {
  if (!d) return 0;
  if (d->C % 32 != 0 || d->OC % 8 != 0) return 0;
  if (d->groups > 1 && !grouped_supported(*d)) return 0;
  if (d->pad_h > 127 || d->pad_w > 127) return 0;
  if ((d->KH - 1) * d->dil_h > 255 || (d->KW - 1) * d->dil_w > 255) return 0;
  if ((d->KH - 1) * d->dil_h - d->pad_h > 128 || (d->KW - 1) * d->dil_w - d->pad_w > 128) return 0;
  if (d->stride_h > 8 || d->stride_w > 8) return 0;
  if ((int64_t)d->N * d->OH * d->OW > (int64_t)INT32_MAX - 256) return 0;
  return 1;
}

// K slices for a pointwise layer of at most one M tile: 1 = not cut.  The slice count divides
// the number of K blocks, leaves at least four blocks per slice, and is the smallest that makes
// the best use of the SMs (tiles / (waves x SMs)).
static int pick_k_slices(const cvmk_conv_desc& d, int bk, int bn) {
  if (!is_pointwise(d) || d.groups > 1 || (int64_t)d.N * d.OH * d.OW > BLOCK_M || d.OC % bn != 0 || d.C % bk != 0) return 1;
  if (dev_env("CVM_B200_NO_SPLIT_K")) return 1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaGetLastError();
  const int blocks = d.C / bk, nt = d.OC / bn;
  if (blocks < 8 || 2 * nt >= sms) return 1;
  int best = 1;
  double best_eff = (double)nt / sms;
  for (int s = 2; s * 4 <= blocks; ++s) {
    if (blocks % s) continue;
    const int tiles = nt * s;
    if (tiles > 4 * sms) break;
    const double eff = (double)tiles / (double)(((tiles + sms - 1) / sms) * sms);
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
  }
  return best;
}

extern "C" int64_t cvmk_conv2d_tc_workspace_bytes(const cvmk_conv_desc* d) {
  if (!d || !cvmk_conv2d_tc_supported(d)) return 0;
  const int s = pick_k_slices(*d, pick_block_k(d->C), pick_block_n(d->OC));
  return s > 1 ? (int64_t)d->N * d->OH * d->OW * s * d->OC * 4 : 0;
}

// Adds the k_slices partial sums of every output element and applies the chain.
__global__ void __launch_bounds__(256) splitk_finish_kernel(const int32_t* __restrict__ part, void* y, int y_dtype, int m,
                                                            int oc, int slices, const __grid_constant__ DevChain chain) {
  const int quads = oc / 4;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m * quads) return;
  const int row = i / quads, c0 = (i - row * quads) * 4;
  const int4* src = reinterpret_cast<const int4*>(part + ((size_t)row * slices) * oc + c0);
  int32_t v[4] = {0, 0, 0, 0};
  for (int s = 0; s < slices; ++s) {
    const int4 t = __ldg(src + (size_t)s * (oc / 4));
    v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
  }
  const size_t lin = (size_t)row * oc + c0;
  apply_chain<4>(chain, v, lin, c0, 1, nullptr, -1, 0);
  if (y_dtype == CVMK_I8) *reinterpret_cast<uint32_t*>(reinterpret_cast<int8_t*>(y) + lin) = pack4(v[0], v[1], v[2], v[3]);
  else *reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(y) + lin) = make_int4(v[0], v[1], v[2], v[3]);
}

extern "C" int cvmk_conv2d_tc_prepare(const cvmk_conv_desc* d, cvmk_conv_plan* plan) {
  if (!d || !plan) { set_error("conv2d_tc_prepare: null argument"); return CVMK_ERR_ARG; }
  if (!cvmk_conv2d_tc_supported(d)) {
    set_error("conv2d_tc_prepare: shape not supported by the tensor-core path");
    return CVMK_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)d->x & 15) || ((uintptr_t)d->w & 15) || ((uintptr_t)d->y & 15)) {
    set_error("conv2d_tc_prepare: operands must be 16-byte aligned");
    return CVMK_ERR_ARG;
  }
  static EncodeTiledFn enc_tiled = (EncodeTiledFn)driver_entry("cuTensorMapEncodeTiled");
  static EncodeIm2colFn enc_im2col = (EncodeIm2colFn)driver_entry("cuTensorMapEncodeIm2col");
  if (!enc_tiled || !enc_im2col) return CVMK_ERR_CUDA;

  memset(plan, 0, sizeof(*plan));
  plan->d = *d;
  const bool grouped = d->groups > 1;
  const int cg = grouped ? d->C / d->groups : d->C;   // channels one output channel reduces over
  if (grouped && d->y_dtype != CVMK_I8) {
    set_error("conv2d_tc_prepare: grouped convolutions write int8");
    return CVMK_ERR_UNSUPPORTED;
  }
  int bk = grouped ? cg : pick_block_k(d->C);   // (grouped: set to the N tile below)
  if (const char* e = grouped ? nullptr : dev_env("CVM_B200_BK")) {  // experiments: a smaller K block (must divide C)
    const int v = atoi(e);
    if ((v == 32 || v == 64 || v == 128) && d->C % v == 0 && v <= bk) bk = v;
  }
  // grouped: an N tile is as many whole groups as make the epilogue's work per tile worth its
  // fixed cost and still leave room for the groups' weights beside the ring (128 channels)
  int bn = pick_block_n(d->OC);
  if (grouped) {
    bn = cg;
    while (bn < 128 && d->OC % (2 * bn) == 0) bn *= 2;
    bk = bn;   // one halo holds the channels of all groups of the N tile
  }
  plan->block_n = bn;
  int patch_w = 0, patch_h = 0, patch_n = 0;
  plan->a_im2col = is_pointwise(*d) ? 0 : 1;
  if (plan->a_im2col && d->stride_h == 1 && d->stride_w == 1 && (grouped || !dev_env("CVM_B200_NO_PATCH")) &&
      (grouped || pick_patch(*d, &patch_w, &patch_h, &patch_n)))
    plan->a_im2col = 2;
  // Halo mode: 3x3 (or any small) stride-1 undilated filters over at most 128 channels and output
  // channels.  The M tile is an 8 x 16 pixel patch of one image; its 10 x 18 input halo is loaded
  // once per 64-channel block and every filter tap multiplies a window of it, so the activations
  // cross L2 -> shared memory about 1.4 times instead of kh * kw times.
  bool halo = false;
  if (grouped) {   // (shape and tile fit were checked by cvmk_conv2d_tc_supported)
    halo = true;
    plan->a_im2col = 3;
    patch_w = 8; patch_h = 16; patch_n = 1;
  } else if (plan->a_im2col == 2 && d->dil_h == 1 && d->dil_w == 1 && d->KH == 3 && d->KW == 3 && d->C % 64 == 0 &&
      d->C <= 128 && bn <= 128 && d->y_dtype == CVMK_I8 && d->OC % 32 == 0 && !dev_env("CVM_B200_NO_HALO")) {
    if (halo_tiles_fit(*d)) {
      halo = true;
      plan->a_im2col = 3;
      patch_w = 8; patch_h = 16; patch_n = 1;
      bk = 64;
    }
  }
  plan->reserved[0] = patch_w; plan->reserved[1] = patch_h; plan->reserved[2] = patch_n;

  // Output path: int8 tiles leave through shared memory and a TMA store; the first int8 tensor
  // operand of the chain (a residual join) comes in by TMA as well.
  // Reductions cut along K write int32 partial sums into the caller's scratch with plain stores.
  {
    const int ks = pick_k_slices(*d, bk, bn);
    const int64_t need = (int64_t)d->N * d->OH * d->OW * ks * d->OC * 4;
    plan->k_slices = (ks > 1 && d->workspace && d->workspace_bytes >= need && ((uintptr_t)d->workspace & 15) == 0) ? ks : 1;
  }
  plan->tma_out = plan->k_slices == 1 && d->y_dtype == CVMK_I8 && d->OC % 32 == 0 && !dev_env("CVM_B200_NO_TMA_STORE");
  plan->res_step = -1;
  if (plan->tma_out) {
    for (int i = 0; i < d->ep.n; ++i) {
      const cvmk_ep_step& s = d->ep.s[i];
      if ((s.op == CVMK_EP_ADD_T || s.op == CVMK_EP_SUB_T || s.op == CVMK_EP_RSUB_T) &&
          s.ptr_dtype == CVMK_I8 && s.ptr && ((uintptr_t)s.ptr & 15) == 0) {
        plan->res_step = i;
        break;
      }
    }
  }
  plan->panels = bn == 256 ? 2 : 1;
  plan->panel_bytes = bn < 128 ? bn : 128;
  // Staging: each epilogue group owns one buffer, or two when they fit beside an operand ring that
  // is still deep enough; short reductions (little work per output tile) may give up half of their
  // K block for it.
  const int group_bytes = plan->panels * BLOCK_M * plan->panel_bytes;
  const int64_t k_all = (int64_t)d->KH * d->KW * cg / plan->k_slices;   // per tile
  const int budget = SMEM_DYNAMIC_MAX - 1024;
  plan->io_bufs = 1;
  // Weights resident in shared memory: one N tile, i.e. every tile of the launch multiplies the
  // same 9 * bn * C bytes (up to 144 KB for 128 x 128 channels).  A ring stage is then the 12 KB
  // halo alone.
  const int halo_pad = ((10 * 18 * bk) + 1023) & ~1023;
  int resident = 0;
  int sms_all = 148;
  {
    int dev0 = 0;
    if (cudaGetDevice(&dev0) == cudaSuccess) cudaDeviceGetAttribute(&sms_all, cudaDevAttrMultiProcessorCount, dev0);
    cudaGetLastError();
  }
  // (grouped: the grid is cut to a multiple of the N tiles below, so that every tile of a CTA
  //  covers the same groups and their 9 weight tiles each can stay as well)
  if (halo && (d->OC <= bn || (grouped && d->OC / bn <= sms_all)) && !dev_env("CVM_B200_NO_RESIDENT_WEIGHTS")) {
    // all channel blocks (one or two) stay, if three halo stages and one staging buffer per group still fit
    const int all = grouped ? d->KH * d->KW * bn * cg : (cg / bk) * d->KH * d->KW * bn * bk;
    if (budget - all - 2 * group_bytes >= 3 * halo_pad) {
      resident = all;
      plan->a_im2col = 4;
    }
  }
  if (grouped && plan->a_im2col != 4) {
    set_error("conv2d_tc_prepare: the weights of a grouped convolution's N tile must fit shared memory");
    return CVMK_ERR_UNSUPPORTED;
  }
  const int halo_stage = halo ? (resident ? halo_pad : halo_pad + d->KH * d->KW * bn * bk) : 0;
  if (halo) {
    if (plan->tma_out && (budget - resident - 4 * group_bytes) / halo_stage >= 3) plan->io_bufs = 2;
  } else if (plan->tma_out && !dev_env("CVM_B200_SINGLE_STAGING")) {
    auto ring_depth = [&](int k) { return (budget - 4 * group_bytes) / ((BLOCK_M + bn) * k); };
    // Long reductions want the shared memory for operands in flight (three 128-byte K blocks
    // cover the load latency, three 64-byte ones do not), short ones for the second staging buffer
    // (their tiles are bound by the epilogue).
    const bool deep_ring_first = bk == 128 && k_all >= 256 && ring_depth(128) < 3 &&
                                 (budget - 2 * group_bytes) / ((BLOCK_M + bn) * 128) >= 3 && !dev_env("CVM_B200_DOUBLE_STAGING");
    if (deep_ring_first) plan->io_bufs = 1;
    else if (ring_depth(bk) >= 3) plan->io_bufs = 2;
    else if (bk == 128 && k_all <= 512 && ring_depth(64) >= 3) { plan->io_bufs = 2; bk = 64; }
  }
  plan->block_k = bk;
  // 1x1 layers: when the number of N tiles divides the grid, tile t + k * grid has the N tile of
  // tile t, so a CTA multiplies one block of output channels all along and can keep its weights
  // (K x block_n bytes) in shared memory; the ring then carries activations only, a third or a
  // fifth of the bytes.  Taken when the weights leave room for a ring of at least four A blocks.
  plan->b_resident = 0;
  if (plan->a_im2col == 0 && plan->k_slices == 1 && !dev_env("CVM_B200_NO_RESIDENT_B")) {
    int sms = 148, dev0 = 0;
    if (cudaGetDevice(&dev0) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev0);
    const int64_t m_tiles = ((int64_t)d->N * d->OH * d->OW + BLOCK_M - 1) / BLOCK_M;
    const int nt = (d->OC + bn - 1) / bn;
    const int64_t w_bytes = (int64_t)d->C * bn;
    const int io1 = plan->tma_out ? 2 * plan->io_bufs * group_bytes : 0;
    if (m_tiles * nt >= 2LL * sms && sms % nt == 0 && d->OC % bn == 0 &&
        budget - io1 - w_bytes >= 4LL * BLOCK_M * bk) {
      plan->b_resident = 1;
      resident = (int)w_bytes;
    }
  }
  const int io_bytes = plan->tma_out ? 2 * plan->io_bufs * group_bytes : 0;
  // Every hand-over of a ring stage (TMA completion -> MMA thread -> commit -> producer) costs a
  // fixed latency of several hundred cycles whatever the stage holds, so small (tap, channel block)
  // units are grouped: up to four per stage, about 48 KB, while the ring stays three deep.
  const int unit_bytes = (BLOCK_M + (plan->b_resident ? 0 : bn)) * bk;
  const int num_units = (int)(k_all / bk);
  int units = 48 * 1024 / unit_bytes;
  if (units > 4) units = 4;
  if (units > num_units) units = num_units;
  if (const char* e = dev_env("CVM_B200_UNITS")) units = atoi(e);
  while (units > 1 && (budget - io_bytes - resident) / (units * unit_bytes) < 3) --units;
  if (units < 1) units = 1;
  if (halo) units = d->KH * d->KW;
  plan->reserved[3] = units;
  const int stage_bytes = halo ? halo_stage : units * unit_bytes;
  int stages = (budget - io_bytes - resident) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) { set_error("conv2d_tc_prepare: tile does not fit shared memory"); return CVMK_ERR_UNSUPPORTED; }
  plan->stages = stages;
  plan->ring_bytes = resident + stages * stage_bytes;  // resident weights (a_im2col 4) sit in front of the ring
  plan->smem_bytes = plan->ring_bytes + io_bytes + 1024;

  const int64_t m_total = (int64_t)d->N * d->OH * d->OW;
  const int64_t k_total = (int64_t)d->KH * d->KW * cg;
  CUtensorMap* ta = reinterpret_cast<CUtensorMap*>(plan->tmap_a);
  CUtensorMap* tb = reinterpret_cast<CUtensorMap*>(plan->tmap_b);
  CUresult r;
  if (plan->a_im2col >= 3) {
    r = encode_nhwc(enc_tiled, ta, d->x, d->N, d->H, d->W, d->C, bk, patch_w + d->KW - 1, patch_h + d->KH - 1, 1,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  } else if (plan->a_im2col == 2) {
    r = encode_nhwc(enc_tiled, ta, d->x, d->N, d->H, d->W, d->C, bk, patch_w, patch_h, patch_n,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  } else if (plan->a_im2col) {
    cuuint64_t dims[4] = {(cuuint64_t)d->C, (cuuint64_t)d->W, (cuuint64_t)d->H, (cuuint64_t)d->N};
    cuuint64_t strides[3] = {(cuuint64_t)d->C, (cuuint64_t)d->W * d->C,
                             (cuuint64_t)d->H * d->W * d->C};
    int lower[2] = {-d->pad_w, -d->pad_h};
    int upper[2] = {d->pad_w - (d->KW - 1) * d->dil_w, d->pad_h - (d->KH - 1) * d->dil_h};
    cuuint32_t estr[4] = {1, (cuuint32_t)d->stride_w, (cuuint32_t)d->stride_h, 1};
    r = enc_im2col(ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d->x, dims, strides, lower, upper,
                   (cuuint32_t)bk, (cuuint32_t)BLOCK_M, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_for(bk), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    r = encode_rows(enc_tiled, ta, d->x, m_total, d->C, bk, BLOCK_M, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  }
  if (r != CUDA_SUCCESS) { set_error("conv2d_tc_prepare: activation tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
  r = encode_rows(enc_tiled, tb, d->w, d->OC, k_total, grouped ? cg : bk, grouped ? cg : bn, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (r != CUDA_SUCCESS) { set_error("conv2d_tc_prepare: weight tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
  if (plan->tma_out) {
    auto encode_out = [&](unsigned char* map, const void* base, CUtensorMapL2promotion promo) {
      CUtensorMap* m = reinterpret_cast<CUtensorMap*>(map);
      if (plan->a_im2col >= 2)
        return encode_nhwc(enc_tiled, m, base, d->N, d->OH, d->OW, d->OC, plan->panel_bytes, patch_w, patch_h,
                           patch_n, promo);
      return encode_rows(enc_tiled, m, base, m_total, d->OC, plan->panel_bytes, BLOCK_M, promo);
    };
    r = encode_out(plan->tmap_y, d->y, CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (r != CUDA_SUCCESS) { set_error("conv2d_tc_prepare: output tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
    if (plan->res_step >= 0) {
      r = encode_out(plan->tmap_r, d->ep.s[plan->res_step].ptr, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
      if (r != CUDA_SUCCESS) { set_error("conv2d_tc_prepare: operand tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
    }
  }
  int64_t num_m_tiles = (m_total + BLOCK_M - 1) / BLOCK_M;
  if (plan->a_im2col >= 2)
    num_m_tiles = (int64_t)((d->OW + patch_w - 1) / patch_w) * ((d->OH + patch_h - 1) / patch_h) *
                  ((d->N + patch_n - 1) / patch_n);
  const int64_t num_n_tiles = (d->OC + bn - 1) / bn;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t tiles = num_m_tiles * num_n_tiles * plan->k_slices;
  plan->grid = (int)(tiles < sms ? tiles : sms);
  if (grouped && plan->a_im2col == 4) plan->grid = (int)(plan->grid / num_n_tiles * num_n_tiles);   // tile t + k * grid: same group as t
  return CVMK_OK;
}

extern "C" int cvmk_conv2d_tc_launch(const cvmk_conv_plan* plan, cvmk_stream_t stream) {
  if (!plan) { set_error("conv2d_tc_launch: null plan"); return CVMK_ERR_ARG; }
  const cvmk_conv_desc& d = plan->d;
  ConvParams p;
  memset(&p, 0, sizeof(p));
  p.y = d.y;
  p.y_dtype = d.y_dtype;
  p.m_total = d.N * d.OH * d.OW;
  p.oc = d.OC;
  p.oh = d.OH; p.ow = d.OW;
  p.c = d.C; p.kh = d.KH; p.kw = d.KW;
  p.stride_h = d.stride_h; p.stride_w = d.stride_w;
  p.pad_h = d.pad_h; p.pad_w = d.pad_w;
  p.dil_h = d.dil_h; p.dil_w = d.dil_w;
  p.block_k = plan->block_k; p.block_n = plan->block_n;
  p.stages = plan->stages; p.a_mode = plan->a_im2col;
  p.b_resident = plan->b_resident;
  p.units = plan->reserved[3] > 0 ? plan->reserved[3] : 1;
  p.num_m_tiles = (p.m_total + BLOCK_M - 1) / BLOCK_M;
  if (p.a_mode >= 2) {
    p.patch_w = plan->reserved[0]; p.patch_h = plan->reserved[1]; p.patch_n = plan->reserved[2];
    p.tiles_w = (d.OW + p.patch_w - 1) / p.patch_w;
    p.tiles_h = (d.OH + p.patch_h - 1) / p.patch_h;
    while ((1 << p.patch_w_log2) < p.patch_w) ++p.patch_w_log2;
    while ((1 << p.patch_h_log2) < p.patch_h) ++p.patch_h_log2;
    p.num_m_tiles = p.tiles_w * p.tiles_h * ((d.N + p.patch_n - 1) / p.patch_n);
  }
  p.num_n_tiles = (d.OC + plan->block_n - 1) / plan->block_n;
  if (d.groups > 1) { p.grouped = 1; p.c = d.C / d.groups; p.group_fold = d.group_fold > 1 ? d.group_fold : 1; }
  p.num_units = p.grouped ? d.KH * d.KW : d.KH * d.KW * (p.c / plan->block_k);
  p.num_kb = p.a_mode >= 3 ? (p.grouped ? 1 : p.c / plan->block_k) : (p.num_units + p.units - 1) / p.units;
  p.fd_n_tiles = make_fastdiv(p.num_n_tiles);
  p.fd_tiles_w = make_fastdiv(p.tiles_w);
  p.fd_tiles_h = make_fastdiv(p.tiles_h);
  p.fd_ohow = make_fastdiv(d.OH * d.OW);
  p.fd_ow = make_fastdiv(d.OW);
  p.acc_bufs = (plan->block_n <= 128 && !dev_env("CVM_B200_TWO_ACCUMULATORS")) ? 4 : 2;
  int cols = p.acc_bufs * plan->block_n;
  int pow2 = 32;
  while (pow2 < cols) pow2 *= 2;
  p.tmem_cols = pow2;
  p.status = d.status;
  p.bias_static = d.bias_static;
  p.w = d.w;
  p.w_bytes = (unsigned)std::min<int64_t>((int64_t)d.OC * d.KH * d.KW * p.c, (int64_t)1 << 30);
  p.tma_out = plan->tma_out; p.res_step = plan->res_step;
  const int ks = plan->k_slices > 1 ? plan->k_slices : 1;
  if (ks > 1) {   // virtual columns (slice, real column); int32 partial sums, no chain in this kernel
    p.k_slices = ks;
    p.oc_real = d.OC;
    p.oc = ks * d.OC;
    p.c = d.C / ks;
    p.y = d.workspace;
    p.y_dtype = CVMK_I32;
    p.num_n_tiles *= ks;
    p.num_units = d.C / ks / plan->block_k;
    p.num_kb = (p.num_units + p.units - 1) / p.units;
    p.fd_n_tiles = make_fastdiv(p.num_n_tiles);
  }
  // Two issuing warps (and one producer) in the halo modes, where a tile takes one or two ring
  // stages and the ring has more: an issuer that waits for the first stage of its next tile is then
  // never more than one lap of that stage's barrier ahead of the producer, which is what a parity
  // wait can tell apart.  (The same rule applied to the short 1x1 reductions of the other modes
  // passed every single-kernel check and gained 12 % on 64 -> 64 and 256 -> 64 layers, but a
  // bounded wait ran out in ResNet-50's end-to-end loop, where per-chunk kernels follow each other
  // closely; it stays off until that is understood.)
  p.two_issuers = (p.a_mode >= 3 && p.num_kb < p.stages && !dev_env("CVM_B200_ONE_ISSUER")) ? 1 : 0;
#ifdef CVMK_CONV_TIMING
  p.dbg = getenv("CVM_DBG") ? atoi(getenv("CVM_DBG")) : 0;
  if (getenv("CVM_HINT")) {
    const uint32_t h = (uint32_t)atoi(getenv("CVM_HINT"));
    cudaMemcpyToSymbol(tc::g_wait_hint, &h, sizeof(h));
  }
#endif
  p.panels = plan->panels; p.panel_bytes = plan->panel_bytes;
  p.io_bufs = plan->io_bufs; p.ring_bytes = plan->ring_bytes;
  int rc = lower_chain(d.ep, &p.chain);
  if (rc != CVMK_OK) return rc;
  DevChain finish_chain = p.chain;
  if (ks > 1) p.chain.n = 0;
  // lower_chain() may merge steps: find the TMA-served operand again by its pointer.
  if (plan->res_step >= 0) {
    const void* want = d.ep.s[plan->res_step].ptr;
    p.res_step = -1;
    for (int i = 0; i < p.chain.n; ++i)
      if ((p.chain.s[i].op == K_ADD_T || p.chain.s[i].op == K_SUB_T || p.chain.s[i].op == K_RSUB_T) &&
          p.chain.s[i].ptr == want) { p.res_step = i; break; }
    if (p.res_step < 0) { set_error("conv2d_tc_launch: tensor operand lost while lowering the chain"); return CVMK_ERR_ARG; }
  }
  // A leading per-channel add is the bias: the kernel keeps it in shared memory.
  p.bias = nullptr;
  p.first_step = 0;
  if (p.chain.n > 0 && p.chain.s[0].op == K_ADD_C) {
    p.bias = reinterpret_cast<const int32_t*>(p.chain.s[0].ptr);
    p.first_step = 1;
  }

  // Packed requantisation: chain = [bias] rs_clamp [add_t|sub_t (the TMA-served operand) clip].
  p.fast_mode = 0;
  if (p.tma_out && d.acc_bound > 0 && d.OC <= MAX_BIAS && !dev_env("CVM_B200_NO_FAST_REQUANT")) {
    const int i0 = p.first_step;
    const int left = p.chain.n - i0;
    if (left >= 1 && p.chain.s[i0].op == K_RS_CLAMP) {
      const DevStep& rs = p.chain.s[i0];
      const int64_t add = rs.c;
      const int sh = rs.d;
      const int64_t lo1 = ((int64_t)rs.a + add) >> sh, hi1 = ((int64_t)rs.b + add) >> sh;
      const bool no_overflow = d.acc_bound + add < (int64_t)INT32_MAX;
      const bool fits16 = ((d.acc_bound + add) >> sh) < 32767;
      const bool clamp_ok = lo1 >= -32767 && hi1 <= 32767 && lo1 <= hi1 && sh <= 16;
      // Without fits16 the sum is clamped to [rs.a, rs.b] before it is scaled (fast_wide); the
      // clamped value plus the rounding addend then stays below 2^(15 + shift).
      const bool wide_ok = (int64_t)rs.b + add < ((int64_t)1 << (15 + sh)) && (int64_t)rs.a + add > -((int64_t)1 << (15 + sh));
      p.fast_wide = 0;
      if (no_overflow && (fits16 || wide_ok) && clamp_ok) {
        if (!fits16) { p.fast_wide = 1; p.f_pre_lo = rs.a; p.f_pre_hi = rs.b; }
        auto x2 = [](int64_t v) { return (uint32_t)((uint32_t)(uint16_t)(int16_t)v | ((uint32_t)(uint16_t)(int16_t)v << 16)); };
        if (left == 1) {
          p.fast_mode = 1;
        } else if (left == 3 && p.res_step == i0 + 1 && p.chain.s[i0 + 2].op == K_CLIP &&
                   (p.chain.s[i0 + 1].op == K_ADD_T || p.chain.s[i0 + 1].op == K_SUB_T) &&
                   p.chain.s[i0 + 2].a >= -32767 && p.chain.s[i0 + 2].b <= 32767 &&
                   std::max(std::abs(lo1), std::abs(hi1)) + 128 < 32767) {
          p.fast_mode = 2;
          p.f_sub = p.chain.s[i0 + 1].op == K_SUB_T;
          p.f_lo2 = x2(p.chain.s[i0 + 2].a);
          p.f_hi2 = x2(p.chain.s[i0 + 2].b);
        }
        if (p.fast_mode) {
          const int kind = p.fast_mode == 1 ? 0 : (p.f_sub ? 3 : (p.chain.s[i0 + 2].a == 0 ? 1 : 2));
          p.fast_variant = (lo1 == 0 ? 1 : 0) + 2 * kind;
          p.f_shift = sh;
          p.f_mul = 1 << (16 - sh);
          p.f_add = (int)add;
          p.f_lo1 = x2(lo1);
          p.f_hi1 = x2(hi1);
        }
      }
    }
  }

  static bool attr_set_dev[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_DYNAMIC_MAX);
    if (check_cuda(e, "cudaFuncSetAttribute(conv_tc_kernel)")) return CVMK_ERR_CUDA;
    attr_set = true;
  }
  CUtensorMap ta, tb, ty, tr;
  memcpy(&ta, plan->tmap_a, sizeof(ta));
  memcpy(&tb, plan->tmap_b, sizeof(tb));
  memcpy(&ty, plan->tmap_y, sizeof(ty));
  memcpy(&tr, plan->tmap_r, sizeof(tr));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)plan->grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = (size_t)plan->smem_bytes;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  static const bool pdl = dev_env("CVM_B200_NO_PDL") == nullptr;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  if (check_cuda(cudaLaunchKernelEx(&cfg, conv_tc_kernel, ta, tb, ty, tr, p), "conv_tc_kernel launch")) return CVMK_ERR_CUDA;
  if (ks > 1) {
    const int m = d.N * d.OH * d.OW;
    const int work = m * (d.OC / 4);
    splitk_finish_kernel<<<(work + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const int32_t*>(d.workspace), d.y, d.y_dtype, m, d.OC, ks, finish_chain);
    return check_cuda(cudaGetLastError(), "splitk_finish_kernel launch");
  }
  return CVMK_OK;
}

#ifdef CVMK_CONV_TIMING
extern "C" int cvmk_conv_timing_read(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_conv_timing, sizeof(long long) * (size_t)count);
}
extern "C" int cvmk_conv_trace_read(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_conv_trace, sizeof(long long) * (size_t)count);
}
extern "C" int cvmk_conv_trace_clear() {
  static long long zero[17 * 512];
  return (int)cudaMemcpyToSymbol(g_conv_trace, zero, sizeof(zero));
}
#endif
