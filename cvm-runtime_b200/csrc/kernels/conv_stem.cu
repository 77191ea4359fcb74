// conv2d for image stems (1..4 input channels, stride 1 or 2) on the tensor cores, straight from the
// NCHW input, without a patch matrix anywhere -- not in HBM and not in shared memory.
//
// Reference operator: cvm.runtime.cpu.conv2d, groups = 1 (cpu/ops/ops.cc:368-456), applied to the
// network input, whose values the runtime clamps to the declared precision first
// (graph_runtime.cc:379-386).
//
// The stride is folded into the channels: with stride S the S x S input pixels that share
// (iy + pad_h) / S and (ix + pad_w) / S become ONE staged pixel of C * S * S <= 16 channels, padded
// to 16 bytes, and the filter becomes a stride-1 filter of KH' x KW' = ceil(KH / S) x ceil(KW / S)
// taps over staged pixels (weights of the taps the folding adds are zero).  Output pixel ox of a
// row then reads staged pixels ox .. ox + KW' - 1 of staged rows oy .. oy + KH' - 1, so the A operand
// of filter tap (ky', kx') for 128 consecutive output pixels is the 128 consecutive staged pixels
// starting at pixel kx' of staged row oy + ky': 16 bytes each, 16 bytes apart.  That IS the
// tensor core's K-major layout without swizzle (core matrices of 8 rows x 16 bytes stored
// contiguously, 128 bytes from one 8-row group to the next), and a second core matrix along K that
// starts 16 bytes after the first is simply the next tap.  One tcgen05.mma (K = 32) therefore
// multiplies two taps of a filter row straight out of the staged input row; shared-memory
// descriptors that overlap stand in for the patch matrix.
//
// One CTA works on blocks of consecutive output rows of one image:
//   warps 0-3  one of their threads has TMA bring the planar input rows of a block (all channels),
//              zero-filled above and below the image, two blocks ahead; all of them fold the rows
//              that have landed: clamp, interleave channels and the S x S neighbours, zero left /
//              right of the image -> staged rows, 16 bytes per staged pixel;
//   warp 4     issues KH' * ceil(KW' / 2) tcgen05.mma (M = 128 pixels, N = OC, K = 32) per output row
//              segment into one of two TMEM accumulators;
//   warps 5-8  drain the accumulator, apply the fused chain (or the packed requantisation), write
//              int8 into a swizzled staging panel;
//   warp 9     stores the panels with TMA.
// Planar rows, staged rows, accumulators and panels are all double buffered; every mbarrier wait
// is bounded.
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include "tc_common.cuh"

namespace cvmk {
namespace {

using namespace tc;

constexpr int STEM_THREADS = 320;   // warps 0-3 load + fold, 4 MMA, 5-8 epilogue, 9 output stores
constexpr int FOLDERS = 128;
constexpr int MMA_WARP = 4;
constexpr int STORE_WARP = 9;
constexpr int PIX = 16;             // bytes per staged pixel
constexpr int MAX_OC = 128;
constexpr int STEM_SMEM_MAX = 110 * 1024;   // two CTAs per SM

struct StemConvParams {
  const int8_t* w;
  int N, H, W, C, OC, KH, KW, OH, OW, S, ph, pw;
  int clamp;
  int khp, kwp, nj;     // folded filter: rows, taps per row, MMAs per row (two taps each)
  int rows_per_block, blocks_per_image, num_blocks;
  int segs, seg_w;      // an output row is cut into `segs` tiles of seg_w <= 128 pixels
  int srows, xw, pitch; // staged rows per block, staged pixels per row, bytes per staged row
  int in_rows;          // planar input rows per block (S * srows)
  int wbox, nwb;        // columns per TMA box and boxes per input row (a box is at most 256 wide)
  int box_stride;       // bytes from one box to the next in shared memory (a multiple of 128)
  int lpad;             // columns of zero fill a box starts left of the image (0 or 16)
  int fold_words;       // 1: rows are folded four staged pixels at a time on 32-bit words
  int planar_bytes, staged_bytes, w_bytes;
  int tmem_cols;
  int off_planar, off_staged, off_out, off_bias;  // byte offsets of the shared-memory regions after the weights
  int* status;
  const int32_t* bias;
  int first_step;
  int fast_mode, fast_variant, f_mul, f_add;
  uint32_t f_lo1, f_hi1;
  DevChain chain;
};

// Named barrier that also tells every participant whether any of them raised `flag`.
__device__ __forceinline__ bool bar_any(int id, int count, bool flag) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %1, 0;\n"
      "bar.red.or.pred q, %2, %3, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)flag), "r"(id), "r"(count)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Shared-memory descriptor of a K-major operand WITHOUT swizzle: core matrices of 8 rows x 16
// bytes, `lbo` bytes from one core matrix to the next along K, `sbo` bytes from one 8-row group to
// the next.  Split into its two 32-bit halves (only the low one moves between instructions).
__device__ __forceinline__ uint32_t desc_lo_plain(uint32_t saddr, uint32_t lbo) {
  return ((saddr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
}
__device__ __forceinline__ uint32_t desc_hi_plain(uint32_t sbo) {
  return (sbo >> 4) | (1u << 14);   // bit 46 of the descriptor: version (sm_100)
}

// One staged pixel: the S x S input pixels of all C channels, byte (a * S + b) * C + c = channel c of
// the pixel at sub-row a, sub-column b; clamped to +-clamp; zero where the image ends.
template <int C, int S>
__device__ __forceinline__ uint4 fold_pixel(const StemConvParams& p, const uint8_t* planar, int R, int X) {
  uint32_t o[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int a = 0; a < S; ++a) {
    const int row = R * S + a;
#pragma unroll
    for (int b = 0; b < S; ++b) {
      const int ix = X * S + b - p.pw;
      const bool inside = ix >= 0 && ix < p.W;
      const int ixc = inside ? ix : 0;
      const int col = ixc + p.lpad;   // column inside the boxes
      const int wb = p.nwb == 1 ? 0 : col / p.wbox;
      const uint8_t* src = planar + (size_t)wb * p.box_stride + (size_t)row * p.wbox + (col - wb * p.wbox);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        int v = (int)(int8_t)src[(size_t)c * p.in_rows * p.wbox];
        v = inside ? max(min(v, p.clamp), -p.clamp) : 0;
        const int i = (a * S + b) * C + c;
        o[i >> 2] |= (uint32_t)(v & 0xff) << (8 * (i & 3));
      }
    }
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// The same on words, four staged pixels (X0 .. X0 + 3, X0 a multiple of 4) per call, for a single
// box that carries zero columns left and right of the image (so that no column needs a test) and a
// clamp to +-127 (only -128 moves).  Per sub-row and channel the 4 * S input bytes the pixels
// take come out of two or three aligned words and a funnel shift; one byte permute moves each
// byte into place.
__device__ __forceinline__ uint32_t clamp127(uint32_t x) {
  const uint32_t z = x ^ 0x80808080u;
  const uint32_t m = ~(((z & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | z) & 0x80808080u;   // 0x80 in every byte that is -128
  return x + (m >> 7);
}
template <int C, int S>
__device__ __forceinline__ void fold_four(const StemConvParams& p, const uint8_t* planar, uint8_t* dst, int R, int X0) {
  uint32_t o[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) o[j][q] = 0u;
  const int first = X0 * S - p.pw + p.lpad;          // first input column of the four pixels, inside the box
  const uint32_t sh = (uint32_t)(first & 3) * 8u;
#pragma unroll
  for (int a = 0; a < S; ++a) {
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(planar + ((size_t)c * p.in_rows + (R * S + a)) * p.wbox + (first & ~3));
      uint32_t s[S];   // the 4 * S bytes: pixel j, sub-column b at byte j * S + b
      const uint32_t w0 = w[0], w1 = w[1];
      s[0] = clamp127(__funnelshift_r(w0, w1, sh));
      if (S == 2) s[S - 1] = clamp127(__funnelshift_r(w1, w[2], sh));
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < S; ++b) {
          const int from = j * S + b;                 // byte of s[]
          const int to = (a * S + b) * C + c;         // byte of the staged pixel
          const uint32_t sel = (0x3210u & ~(0xFu << (4 * (to & 3)))) | ((uint32_t)(4 + (from & 3)) << (4 * (to & 3)));
          o[j][to >> 2] = __byte_perm(o[j][to >> 2], s[from >> 2], sel);
        }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(dst + (size_t)(X0 + j) * PIX) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
}

template <int C, int S>
__device__ __forceinline__ void fold_block(const StemConvParams& p, const uint8_t* planar, uint8_t* staged, int t) {
  if (p.fold_words) {
    const int quads = p.xw >> 2;   // xw is a multiple of 4 on this path
    for (int i = t; i < p.srows * quads; i += FOLDERS) {
      const int R = i / quads, X0 = (i - R * quads) * 4;
      fold_four<C, S>(p, planar, staged + (size_t)R * p.pitch, R, X0);
    }
    return;
  }
  for (int R = 0; R < p.srows; ++R)
    for (int X = t; X < p.xw; X += FOLDERS)
      *reinterpret_cast<uint4*>(staged + (size_t)R * p.pitch + X * PIX) = fold_pixel<C, S>(p, planar, R, X);
}

// Packed requantisation of one thread's row (see fast_requant): straight-line per 32 columns, two
// chunks per TMEM round trip.
template <int RELU1>
__device__ __forceinline__ void stem_fast_chunk(const FastQ& fq, int mul, int32_t (&v)[32], int ci, const int32_t* bias_s,
                                                uint8_t* panel, uint32_t sw_key) {
  const int4* bp = reinterpret_cast<const int4*>(bias_s + ci * 32);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int4 b4 = bp[j];
    v[4 * j] = v[4 * j] * mul + b4.x;
    v[4 * j + 1] = v[4 * j + 1] * mul + b4.y;
    v[4 * j + 2] = v[4 * j + 2] * mul + b4.z;
    v[4 * j + 3] = v[4 * j + 3] * mul + b4.w;
  }
  const uint4 z = make_uint4(0, 0, 0, 0);
  uint4 a, b;
  fast_requant<RELU1, 0>(fq, v, z, z, &a, &b);
  const uint32_t j0 = (uint32_t)(ci * 2);
  *reinterpret_cast<uint4*>(panel + ((j0 ^ sw_key) << 4)) = a;
  *reinterpret_cast<uint4*>(panel + (((j0 + 1) ^ sw_key) << 4)) = b;
}
template <int RELU1>
__device__ __forceinline__ void stem_fast_row(const FastQ& fq, int mul, uint32_t tbase, int chunks, const int32_t* bias_s,
                                              uint8_t* panel, uint32_t sw_key) {
  int ci = 0;
  for (; ci + 2 <= chunks; ci += 2) {
    int32_t v0[32], v1[32];
    tmem_ld64(tbase + (uint32_t)(ci * 32), v0, v1);
    stem_fast_chunk<RELU1>(fq, mul, v0, ci, bias_s, panel, sw_key);
    stem_fast_chunk<RELU1>(fq, mul, v1, ci + 1, bias_s, panel, sw_key);
  }
  if (ci < chunks) {
    int32_t v[32];
    tmem_ld32(tbase + (uint32_t)(ci * 32), v);
    stem_fast_chunk<RELU1>(fq, mul, v, ci, bias_s, panel, sw_key);
  }
}

#ifdef CVMK_STEM_TIMING
// Development builds: cycles per role and phase, per CTA.  Slots: 0 folders wait for the planar
// rows, 1 folders wait for a free staged buffer, 2 folding, 3 MMA waits for the accumulator, 4 MMA
// waits for the staged rows, 5 MMA issue, 6 epilogue waits for the accumulator, 7 epilogue waits
// for a panel, 12 epilogue TMEM load + arithmetic + staging stores, 13 tcgen05 fence, 14 proxy fence,
// 8 hand-over, 10 whole folder loop, 11 tiles.
__device__ long long g_stem_timing[296 * 16];
#define STSTART(var) long long var = clock64()
#define STADD(slot, var) do { const long long now__ = clock64(); stacc[slot] += now__ - var; var = now__; } while (0)
#define STDECL long long stacc[16] = {0}
#define STFLUSH(slot) do { if (blockIdx.x < 296) g_stem_timing[blockIdx.x * 16 + (slot)] = stacc[slot]; } while (0)
#else
#define STSTART(var) do {} while (0)
#define STADD(slot, var) do {} while (0)
#define STDECL do {} while (0)
#define STFLUSH(slot) do {} while (0)
#endif

__global__ void __launch_bounds__(STEM_THREADS, 2)
conv_stem_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                 const __grid_constant__ StemConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t planar_full[2], staged_full[2], staged_empty[2];
  __shared__ uint64_t acc_full[2], acc_empty[2], out_free[2], out_full[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* wq = smem;                        // [KH' * nj][2][OC][16]: two taps per MMA, no swizzle
  uint8_t* planar = smem + p.off_planar;     // [2][nwb][C][in_rows][wbox]
  uint8_t* staged = smem + p.off_staged;     // [2][srows][pitch]
  uint8_t* out_panels = smem + p.off_out;    // [2][128][OC], swizzle of width OC
  int32_t* bias_s = reinterpret_cast<int32_t*>(smem + p.off_bias);
  // warp index through a shuffle: provably uniform, so that the loops of the single-issuer roles
  // (loads, MMA, output stores) run on the uniform datapath with one elected lane issuing
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&planar_full[b], 1);
      mbar_init(&staged_full[b], FOLDERS / 32);
      mbar_init(&staged_empty[b], 1);
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
      mbar_init(&out_free[b], 1);
      mbar_init(&out_full[b], 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // weights -> shared memory, same byte order as in global memory
  for (int i = threadIdx.x; i < p.w_bytes / 16; i += STEM_THREADS)
    reinterpret_cast<uint4*>(wq)[i] = __ldg(reinterpret_cast<const uint4*>(p.w) + i);
  for (int i = threadIdx.x; i < p.OC; i += STEM_THREADS) {
    const int32_t b = p.bias ? __ldg(p.bias + i) : 0;
    bias_s[i] = p.fast_mode ? (int32_t)((uint32_t)(b + p.f_add) * (uint32_t)p.f_mul) : b;
  }
  fence_async_smem();
  if (warp == MMA_WARP) tmem_alloc(&tmem_slot, (uint32_t)p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) { mbar_arrive(&out_free[0]); mbar_arrive(&out_free[1]); }  // both panels start free
  const uint32_t tmem_base = tmem_slot;

  if (warp < MMA_WARP) {
    // ------------------------------------------------------------------ load planar rows (TMA), fold them
    const int t = threadIdx.x;
    const bool issuer = elect_one() && warp == 0;
    // all C planes x in_rows rows of a block; rows above and below the image arrive as zeros
    auto load_block = [&](int blk, int buf) {
      const int n = blk / p.blocks_per_image;
      const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
      mbar_expect_tx(&planar_full[buf], (uint32_t)(p.C * p.in_rows * p.wbox * p.nwb));
      for (int wb = 0; wb < p.nwb; ++wb)
        tma_load_3d(planar + (size_t)buf * p.planar_bytes + (size_t)wb * p.box_stride, &tmap_x, &planar_full[buf],
                    wb * p.wbox - p.lpad, oy0 * p.S - p.ph, n * p.C);
    };
    if (issuer) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
      if ((int)blockIdx.x < p.num_blocks) load_block(blockIdx.x, 0);
      if ((int)(blockIdx.x + gridDim.x) < p.num_blocks) load_block(blockIdx.x + gridDim.x, 1);
    }
    uint32_t bi = 0;
    STDECL;
    STSTART(tall);
    for (int blk = blockIdx.x; blk < p.num_blocks; blk += gridDim.x, ++bi) {
      const int buf = (int)(bi & 1u);
      const uint32_t par = (bi >> 1) & 1u;
      STSTART(tw);
      bool ok = mbar_wait(&planar_full[buf], par, &abort_flag, 2);
      STADD(0, tw);
      ok = ok && mbar_wait(&staged_empty[buf], par ^ 1u, &abort_flag, 3);
      STADD(1, tw);
      if (ok) {
        const uint8_t* src = planar + (size_t)buf * p.planar_bytes;
        uint8_t* dst = staged + (size_t)buf * p.staged_bytes;
        switch (p.C * 2 + p.S - 3) {   // (C, S) -> 2 * (C - 1) + (S - 1)
          case 0: fold_block<1, 1>(p, src, dst, t); break;
          case 1: fold_block<1, 2>(p, src, dst, t); break;
          case 2: fold_block<2, 1>(p, src, dst, t); break;
          case 3: fold_block<2, 2>(p, src, dst, t); break;
          case 4: fold_block<3, 1>(p, src, dst, t); break;
          case 5: fold_block<3, 2>(p, src, dst, t); break;
          case 6: fold_block<4, 1>(p, src, dst, t); break;
          default: fold_block<4, 2>(p, src, dst, t); break;
        }
      }
      fence_async_smem();   // the staged rows are read by the tensor core, the planar rows rewritten by TMA
      // every folder is done with the planar rows; if a wait ran out for anyone, all leave together
      if (bar_any(1, FOLDERS, !ok)) break;
      if (issuer && blk + 2 * (int)gridDim.x < p.num_blocks) load_block(blk + 2 * (int)gridDim.x, buf);
      __syncwarp();
      if (lane == 0) mbar_arrive(&staged_full[buf]);
      STADD(2, tw);
    }
#ifdef CVMK_STEM_TIMING
    STADD(10, tall);
    if (t == 0) { STFLUSH(0); STFLUSH(1); STFLUSH(2); STFLUSH(10); }
#endif
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    {
      const bool leader = elect_one();
      const uint32_t idesc = umma_idesc_i8(p.OC);
      const uint32_t a_hi = desc_hi_plain(128u), b_hi = desc_hi_plain(128u);
      const uint32_t b_lo0 = desc_lo_plain(smem_u32(wq), (uint32_t)p.OC * PIX);
      const uint32_t b_step = (uint32_t)(p.OC * 2 * PIX) >> 4;   // one MMA's weights: two taps x OC rows x 16 bytes
      const uint32_t row_step = (uint32_t)p.pitch >> 4;
      uint32_t tile = 0, bi = 0;
      bool live = true;
      STDECL;
      for (int blk = blockIdx.x; live && blk < p.num_blocks; blk += gridDim.x, ++bi) {
        const int n = blk / p.blocks_per_image;
        const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
        const int sbuf = (int)(bi & 1u);
        STSTART(tw);
        if (!mbar_wait(&staged_full[sbuf], (bi >> 1) & 1u, &abort_flag, 4)) { live = false; break; }
        STADD(4, tw);
        tc_fence_after();
        const uint32_t a_blk = desc_lo_plain(smem_u32(staged + (size_t)sbuf * p.staged_bytes), PIX);
        for (int rr = 0; live && rr < p.rows_per_block && oy0 + rr < p.OH; ++rr) {
          for (int sg = 0; sg < p.segs; ++sg, ++tile) {
            const int buf = (int)(tile & 1u);
            if (!mbar_wait(&acc_empty[buf], ((tile >> 1) & 1u) ^ 1u, &abort_flag, 5)) { live = false; break; }
            STADD(3, tw);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.OC);
            // tap (ky', 2j) of output pixel m of this segment: staged row rr + ky', staged pixel sg * seg_w + m + 2j
            uint32_t al_row = a_blk + (uint32_t)rr * row_step + (uint32_t)(sg * p.seg_w);
            uint32_t bl = b_lo0;
            if (leader) {
              uint32_t acc = 0;
              for (int ky = 0; ky < p.khp; ++ky, al_row += row_step) {
                uint32_t al = al_row;
                for (int j = 0; j < p.nj; ++j, al += 2u, bl += b_step, acc = 1u)
                  mma_i8_k<1>(d_tmem, al, a_hi, bl, b_hi, idesc, acc);
              }
              mma_commit(&acc_full[buf]);
            }
            STADD(5, tw);
          }
        }
        if (leader) mma_commit(&staged_empty[sbuf]);   // all MMAs that read this block's rows have finished
      }
#ifdef CVMK_STEM_TIMING
      if (leader) { stacc[11] = tile; STFLUSH(3); STFLUSH(4); STFLUSH(5); STFLUSH(11); }
#endif
    }
  } else if (warp < STORE_WARP) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const bool leader = warp == MMA_WARP + 1 && lane == 0;
    (void)leader;
    const int pw = p.OC;  // panel row = all output channels of a pixel
    const int panel_bytes = BLOCK_M * pw;
    const int chunks = p.OC >> 5;
    const uint32_t row_off = (uint32_t)row_in_tile * (uint32_t)pw;
    const uint32_t sw_key = (row_off >> 7) & (((uint32_t)pw - 1u) >> 4);
    const FastQ fq = {p.f_lo1, p.f_hi1, 0u, 0u};
    uint32_t tile = 0;
    bool live = true;
    STDECL;
    for (int blk = blockIdx.x; live && blk < p.num_blocks; blk += gridDim.x) {
      const int n = blk / p.blocks_per_image;
      const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
      for (int rr = 0; live && rr < p.rows_per_block && oy0 + rr < p.OH; ++rr) {
        const int oy = oy0 + rr;
        for (int sg = 0; sg < p.segs; ++sg, ++tile) {
          const int buf = (int)(tile & 1u);
          const uint32_t par = (tile >> 1) & 1u;
          STSTART(tw);
          if (!mbar_wait(&acc_full[buf], par, &abort_flag, 6)) { live = false; break; }
          STADD(6, tw);
          tc_fence_after();
          if (!mbar_wait(&out_free[buf], par, &abort_flag, 7)) { live = false; break; }
          STADD(7, tw);
          uint8_t* panel = out_panels + (size_t)buf * panel_bytes + row_off;
          const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.OC);
          const int ox = sg * p.seg_w + row_in_tile;
          const bool valid = row_in_tile < p.seg_w && ox < p.OW;
          const size_t lin0 = (((size_t)n * p.OH + oy) * p.OW + (valid ? ox : 0)) * p.OC;
          if (p.fast_mode) {
            if (p.fast_variant & 1) stem_fast_row<1>(fq, p.f_mul, tbase, chunks, bias_s, panel, sw_key);
            else stem_fast_row<0>(fq, p.f_mul, tbase, chunks, bias_s, panel, sw_key);
            STADD(12, tw);
          } else
          for (int ci = 0; ci < chunks; ++ci) {
            int32_t v[32];
            tmem_ld32(tbase + (uint32_t)(ci * 32), v);
            const int4* bp = reinterpret_cast<const int4*>(bias_s + ci * 32);
            uint4 a, b;
            {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int4 b4 = bp[j];
                v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
              }
              if (valid) apply_chain<32>(p.chain, v, lin0 + ci * 32, ci * 32, 1, nullptr, -1, p.first_step);
              a.x = pack4(v[0], v[1], v[2], v[3]);     a.y = pack4(v[4], v[5], v[6], v[7]);
              a.z = pack4(v[8], v[9], v[10], v[11]);   a.w = pack4(v[12], v[13], v[14], v[15]);
              b.x = pack4(v[16], v[17], v[18], v[19]); b.y = pack4(v[20], v[21], v[22], v[23]);
              b.z = pack4(v[24], v[25], v[26], v[27]); b.w = pack4(v[28], v[29], v[30], v[31]);
            }
            const uint32_t j0 = (uint32_t)(ci * 2);
            *reinterpret_cast<uint4*>(panel + ((j0 ^ sw_key) << 4)) = a;
            *reinterpret_cast<uint4*>(panel + (((j0 + 1) ^ sw_key) << 4)) = b;
          }
          tc_fence_before();
          STADD(13, tw);
          fence_async_smem();
          STADD(14, tw);
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&acc_empty[buf]);
            mbar_arrive(&out_full[buf]);
          }
          STADD(8, tw);
          if (abort_flag) { live = false; break; }
        }
      }
    }
#ifdef CVMK_STEM_TIMING
    if (leader) { STFLUSH(6); STFLUSH(7); STFLUSH(8); STFLUSH(9); STFLUSH(12); STFLUSH(13); STFLUSH(14); }
#endif
  } else {
    // ------------------------------------------------------------------ output stores
    // One elected thread: waits until the four epilogue warps have written a panel, stores it with
    // TMA, and hands the panel back once the engine has read it.
    const bool leader = elect_one();
    uint32_t tile = 0;
    bool live = true;
    const int panel_bytes = BLOCK_M * p.OC;
    for (int blk = blockIdx.x; live && blk < p.num_blocks; blk += gridDim.x) {
      const int n = blk / p.blocks_per_image;
      const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
      for (int rr = 0; live && rr < p.rows_per_block && oy0 + rr < p.OH; ++rr) {
        for (int sg = 0; sg < p.segs; ++sg, ++tile) {
          const int buf = (int)(tile & 1u);
          if (!mbar_wait(&out_full[buf], (tile >> 1) & 1u, &abort_flag, 8)) { live = false; break; }
          if (leader) {
            tma_store_3d(&tmap_y, out_panels + (size_t)buf * panel_bytes, 0, sg * p.seg_w, n * p.OH + oy0 + rr);
            tma_store_commit();
            tma_store_wait_read();  // the engine has read this panel: hand it back at once
            mbar_arrive(&out_free[buf]);
          }
          __syncwarp();
        }
      }
    }
    // the writes themselves complete with the grid
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // loads that were issued may still be landing in this CTA's shared memory: give them time
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, 0x200 | abort_flag);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct StemLayout {
  int S, khp, kwp, nj, rows_per_block, segs, seg_w, srows, xw, pitch, in_rows, wbox, nwb, box_stride, lpad, fold_words;
  int planar_bytes, staged_bytes, w_bytes, off_planar, off_staged, off_out, off_bias, smem_bytes;
};

bool stem_layout(const cvmk_stem_conv_desc& d, StemLayout* L) {
  const int S = d.stride_h;
  L->S = S;
  L->khp = (d.KH + S - 1) / S;
  L->kwp = (d.KW + S - 1) / S;
  L->nj = (L->kwp + 1) / 2;
  L->segs = (d.OW + BLOCK_M - 1) / BLOCK_M;
  L->seg_w = (d.OW + L->segs - 1) / L->segs;
  L->xw = L->segs * L->seg_w + 2 * L->nj;        // every tap of every real output pixel lies inside the row
  L->nwb = (d.W + 255) / 256;
  if (d.W % (16 * L->nwb) != 0) return false;
  L->wbox = d.W / L->nwb;
  L->lpad = 0;
  L->fold_words = 0;
  // One box with 16 zero columns on either side of the image, when that fits a box and covers every
  // column the staged pixels take (rounded up to whole words): the rows are then folded on words.
  {
    const int xw4 = (L->xw + 3) / 4 * 4;
    const int last = (xw4 - 1) * S + (S - 1) - d.pad_w + 16;   // last column read, inside the box
    if (d.W + 32 <= 256 && d.pad_w <= 16 && d.clamp == 127 && (last | 3) + 4 < d.W + 32 && !dev_env("CVM_B200_NO_FOLD_WORDS")) {
      L->lpad = 16;
      L->wbox = d.W + 32;
      L->fold_words = 1;
      L->xw = xw4;
    }
  }
  L->pitch = L->xw * PIX;
  L->w_bytes = L->khp * L->nj * 2 * d.OC * PIX;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaGetLastError();
  // Blocks of 8 output rows re-fold few rows (KH' - 1 per block); smaller blocks when the batch is
  // too small to give every CTA slot one, or when shared memory is short.
  for (int rpb = 8; rpb >= 1; rpb /= 2) {
    L->rows_per_block = std::min(rpb, (int)d.OH);
    const int64_t blocks = (int64_t)d.N * ((d.OH + L->rows_per_block - 1) / L->rows_per_block);
    L->srows = L->rows_per_block + L->khp - 1;
    L->in_rows = L->srows * S;
    L->box_stride = (d.C * L->in_rows * L->wbox + 127) / 128 * 128;   // (one box, or nwb boxes of wbox = W / nwb columns)
    L->planar_bytes = L->nwb * L->box_stride;
    L->staged_bytes = (L->srows * L->pitch + 127) / 128 * 128;
    L->off_planar = (L->w_bytes + 1023) / 1024 * 1024;
    L->off_staged = L->off_planar + 2 * L->planar_bytes;
    // rows of a tile past the segment's width read on past the staged row they start in: whatever
    // follows (the next rows, the panels) is inside this CTA's shared memory
    L->off_out = (L->off_staged + 2 * L->staged_bytes + 1023) / 1024 * 1024;
    L->off_bias = L->off_out + 2 * BLOCK_M * d.OC;
    L->smem_bytes = L->off_bias + d.OC * 4 + 1024;
    const bool fits = L->smem_bytes <= STEM_SMEM_MAX && L->in_rows <= 256;
    if (fits && (blocks >= 2 * sms || rpb <= 2)) return true;
    if (rpb == 1) return fits;
  }
  return false;
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_conv2d_stem_supported(const cvmk_stem_conv_desc* d) {
  if (!d) return 0;
  if (d->C < 1 || d->C > 4 || d->KH < 1 || d->KH > 8 || d->KW < 1 || d->KW > 8) return 0;
  if (d->OC != 32 && d->OC != 64 && d->OC != 128) return 0;
  if (d->stride_h != d->stride_w || d->stride_h < 1 || d->stride_h > 2) return 0;
  if (d->pad_h < 0 || d->pad_w < 0 || d->clamp < 1 || d->clamp > 127) return 0;
  if (d->W % 16 != 0 || d->H < 1 || d->OH < 1 || d->OW < 1) return 0;
  if ((int64_t)d->N * d->OH > INT32_MAX / 4 || (int64_t)d->N * d->OH * d->OW * d->OC > ((int64_t)1 << 40)) return 0;
  if ((int64_t)d->N * d->C > INT32_MAX / 2) return 0;
  StemLayout L;
  return stem_layout(*d, &L) ? 1 : 0;
}

extern "C" int64_t cvmk_conv2d_stem_weight_bytes(const cvmk_stem_conv_desc* d) {
  StemLayout L;
  if (!d || !cvmk_conv2d_stem_supported(d) || !stem_layout(*d, &L)) return -1;
  return L.w_bytes;
}

// OIHW int32 filter values -> the kernel's operand order: for filter row ky' and tap pair j, two
// blocks (taps 2j and 2j + 1) of OC rows x 16 bytes; byte (a * S + b) * C + c of a row is
// w[oc][c][S * ky' + a][S * kx' + b], zero where that lies outside the filter.
extern "C" int cvmk_conv2d_stem_pack_weights(const cvmk_stem_conv_desc* d, const int32_t* w_oihw, int8_t* packed) {
  StemLayout L;
  if (!d || !w_oihw || !packed || !cvmk_conv2d_stem_supported(d) || !stem_layout(*d, &L)) {
    set_error("conv2d_stem_pack_weights: unsupported shape");
    return CVMK_ERR_UNSUPPORTED;
  }
  memset(packed, 0, (size_t)L.w_bytes);
  const int S = L.S;
  for (int kyp = 0; kyp < L.khp; ++kyp)
    for (int kxp = 0; kxp < L.kwp; ++kxp)
      for (int oc = 0; oc < d->OC; ++oc)
        for (int a = 0; a < S; ++a)
          for (int b = 0; b < S; ++b)
            for (int c = 0; c < d->C; ++c) {
              const int ky = S * kyp + a, kx = S * kxp + b;
              if (ky >= d->KH || kx >= d->KW) continue;
              const size_t at = ((((size_t)kyp * L.nj + kxp / 2) * 2 + (kxp & 1)) * d->OC + oc) * PIX + (a * S + b) * d->C + c;
              packed[at] = (int8_t)w_oihw[(((size_t)oc * d->C + c) * d->KH + ky) * d->KW + kx];
            }
  return CVMK_OK;
}

extern "C" int cvmk_conv2d_stem_prepare(const cvmk_stem_conv_desc* d, cvmk_stem_conv_plan* plan) {
  if (!d || !plan || !cvmk_conv2d_stem_supported(d)) { set_error("conv2d_stem_prepare: unsupported shape"); return CVMK_ERR_UNSUPPORTED; }
  if (((uintptr_t)d->w & 15) || ((uintptr_t)d->y & 15) || ((uintptr_t)d->x & 15)) {
    set_error("conv2d_stem_prepare: operands must be 16-byte aligned");
    return CVMK_ERR_ARG;
  }
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !fn) {
    set_error("conv2d_stem_prepare: cuTensorMapEncodeTiled not available");
    return CVMK_ERR_CUDA;
  }
  memset(plan, 0, sizeof(*plan));
  plan->d = *d;
  StemLayout L;
  stem_layout(*d, &L);
  {
    cuuint64_t dims[3] = {(cuuint64_t)d->OC, (cuuint64_t)d->OW, (cuuint64_t)d->N * d->OH};
    cuuint64_t strides[2] = {(cuuint64_t)d->OC, (cuuint64_t)d->OW * d->OC};
    cuuint32_t box[3] = {(cuuint32_t)d->OC, (cuuint32_t)L.seg_w, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle swz = d->OC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : (d->OC == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = ((EncodeTiledFn)fn)(reinterpret_cast<CUtensorMap*>(plan->tmap_y), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                     d->y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("conv2d_stem_prepare: output tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
  }
  {
    // the input as planes of rows: [N * C][H][W]; a box is all C planes of an image x in_rows rows x wbox columns
    cuuint64_t dims[3] = {(cuuint64_t)d->W, (cuuint64_t)d->H, (cuuint64_t)d->N * d->C};
    cuuint64_t strides[2] = {(cuuint64_t)d->W, (cuuint64_t)d->W * d->H};
    cuuint32_t box[3] = {(cuuint32_t)L.wbox, (cuuint32_t)L.in_rows, (cuuint32_t)d->C};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ((EncodeTiledFn)fn)(reinterpret_cast<CUtensorMap*>(plan->tmap_x), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                     const_cast<int8_t*>(d->x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("conv2d_stem_prepare: input tensor map rejected (CUresult %d)", (int)r); return CVMK_ERR_CUDA; }
  }
  plan->smem_bytes = L.smem_bytes;
  const int blocks_per_image = (d->OH + L.rows_per_block - 1) / L.rows_per_block;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t blocks = (int64_t)d->N * blocks_per_image;
  plan->grid = (int)std::min<int64_t>(blocks, 2 * sms);
  return CVMK_OK;
}

extern "C" int cvmk_conv2d_stem_launch(const cvmk_stem_conv_plan* plan, cvmk_stream_t stream) {
  if (!plan) { set_error("conv2d_stem_launch: null plan"); return CVMK_ERR_ARG; }
  const cvmk_stem_conv_desc& d = plan->d;
  StemLayout L;
  stem_layout(d, &L);
  StemConvParams p;
  memset(&p, 0, sizeof(p));
  p.w = d.w;
  p.N = d.N; p.H = d.H; p.W = d.W; p.C = d.C; p.OC = d.OC; p.KH = d.KH; p.KW = d.KW; p.OH = d.OH; p.OW = d.OW;
  p.S = L.S; p.ph = d.pad_h; p.pw = d.pad_w;
  p.clamp = d.clamp;
  p.khp = L.khp; p.kwp = L.kwp; p.nj = L.nj;
  p.rows_per_block = L.rows_per_block;
  p.blocks_per_image = (d.OH + L.rows_per_block - 1) / L.rows_per_block;
  p.num_blocks = d.N * p.blocks_per_image;
  p.segs = L.segs; p.seg_w = L.seg_w; p.srows = L.srows; p.xw = L.xw; p.pitch = L.pitch;
  p.in_rows = L.in_rows; p.wbox = L.wbox; p.nwb = L.nwb; p.box_stride = L.box_stride;
  p.lpad = L.lpad; p.fold_words = L.fold_words;
  p.planar_bytes = L.planar_bytes; p.staged_bytes = L.staged_bytes; p.w_bytes = L.w_bytes;
  p.off_planar = L.off_planar; p.off_staged = L.off_staged; p.off_out = L.off_out; p.off_bias = L.off_bias;
  int cols = 2 * d.OC, pow2 = 32;
  while (pow2 < cols) pow2 *= 2;
  p.tmem_cols = pow2;
  p.status = d.status;
  int rc = lower_chain(d.ep, &p.chain);
  if (rc != CVMK_OK) return rc;
  p.bias = nullptr;
  p.first_step = 0;
  if (p.chain.n > 0 && p.chain.s[0].op == K_ADD_C) {
    p.bias = reinterpret_cast<const int32_t*>(p.chain.s[0].ptr);
    p.first_step = 1;
  }
  // packed requantisation: chain = [bias] rs_clamp, same proof obligations as the general kernel
  if (d.acc_bound > 0 && p.chain.n - p.first_step == 1 && p.chain.s[p.first_step].op == K_RS_CLAMP &&
      !dev_env("CVM_B200_NO_FAST_REQUANT")) {
    const DevStep& rs = p.chain.s[p.first_step];
    const int64_t add = rs.c;
    const int sh = rs.d;
    const int64_t lo1 = ((int64_t)rs.a + add) >> sh, hi1 = ((int64_t)rs.b + add) >> sh;
    if (d.acc_bound + add < (int64_t)INT32_MAX && ((d.acc_bound + add) >> sh) < 32767 && lo1 >= -32767 &&
        hi1 <= 32767 && lo1 <= hi1 && sh <= 16) {
      auto x2 = [](int64_t v) { return (uint32_t)((uint32_t)(uint16_t)(int16_t)v | ((uint32_t)(uint16_t)(int16_t)v << 16)); };
      p.fast_mode = 1;
      p.fast_variant = lo1 == 0 ? 1 : 0;
      p.f_mul = 1 << (16 - sh);
      p.f_add = (int)add;
      p.f_lo1 = x2(lo1);
      p.f_hi1 = x2(hi1);
    }
  }
  static bool attr_set_dev[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_stem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STEM_SMEM_MAX);
    if (check_cuda(e, "cudaFuncSetAttribute(conv_stem_kernel)")) return CVMK_ERR_CUDA;
    attr_set = true;
  }
  CUtensorMap tx, ty;
  memcpy(&tx, plan->tmap_x, sizeof(tx));
  memcpy(&ty, plan->tmap_y, sizeof(ty));
  conv_stem_kernel<<<plan->grid, STEM_THREADS, plan->smem_bytes, (cudaStream_t)stream>>>(tx, ty, p);
  return check_cuda(cudaGetLastError(), "conv_stem_kernel launch");
}

#ifdef CVMK_STEM_TIMING
extern "C" int cvmk_stem_timing_read(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_stem_timing, sizeof(long long) * (size_t)count);
}
#endif
