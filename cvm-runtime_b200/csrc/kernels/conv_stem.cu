// conv2d for image stems (1..4 input channels) on the tensor cores, straight from the NCHW input.
//
// Reference operator: cvm.runtime.cpu.conv2d, groups = 1 (cpu/ops/ops.cc:368-456), applied to the
// network input, whose values the runtime clamps to the declared precision first
// (graph_runtime.cc:379-386).  With so few channels a filter tap is too short for a K block, so the
// GEMM is built per filter ROW: K block ky holds the KW * C bytes (kx-major, then channel) of row
// ky of the window, zero padded to 32 bytes; the weights are packed to match ([KH][OC][32], zeros
// in the padding, so whatever input bytes sit there do not count).
//
// One CTA works on blocks of consecutive output rows of one image:
//   warps 0-3  stage the input rows of the block in shared memory (clamped, channel-interleaved,
//              zero padded left/right/top/bottom), then build the A tile of every output row:
//              thread t copies, for each ky, the 32 bytes starting at pixel (ox * stride_w) of
//              staged row (oy * stride_h + ky) into row t of K block ky (32-byte swizzle);
//   warp 4     issues KH tcgen05.mma (M = 128 pixels, N = OC, K = 32) per tile into one of two TMEM
//              accumulators;
//   warps 5-8  drain the accumulator, apply the fused chain (or the packed requantisation),
//              write int8 into a swizzled staging panel, and one of their threads stores it with TMA.
// A tiles and staging panels are double buffered; every mbarrier wait is bounded.
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include "tc_common.cuh"

namespace cvmk {
namespace {

using namespace tc;

constexpr int STEM_THREADS = 320;   // warps 0-3 build, 4 MMA, 5-8 epilogue, 9 output stores
constexpr int STORE_WARP = 9;
constexpr int BUILDERS = 128;
constexpr int MMA_WARP = 4;
constexpr int SLOT = 32;           // bytes of K per filter row
constexpr int A_BLOCK = BLOCK_M * SLOT;
constexpr int MAX_OC = 128;

struct StemConvParams {
  const int8_t* x;
  const int8_t* w;
  int N, H, W, C, OC, KH, KW, OH, OW, sh, sw, ph, pw;
  int clamp;
  int rows_per_block, blocks_per_image, num_blocks;
  int segs, seg_w;
  int srows, srow_bytes;
  int left;             // byte offset of image column 0 in a staged row (a multiple of 16)
  int tmem_cols;
  int off_a, off_in, off_out, off_bias;  // byte offsets of the shared-memory regions after the weights
  int* status;
  const int32_t* bias;
  int first_step;
  int fast_mode, fast_variant, f_mul, f_add;
  uint32_t f_lo1, f_hi1;
  DevChain chain;
};

__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
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
__device__ __forceinline__ void tma_store_wait_read1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}

// Input rows of a block -> shared memory, channel-interleaved.  One task = 16 pixels of one row:
// C 16-byte loads (one per channel plane), the clamp, a byte interleave in registers and C 16-byte
// stores.  The loads of all tasks of a thread are issued before anything depends on them (clamped
// row index; rows outside the image are written as zeros).
template <int C>
__device__ __forceinline__ void stage_rows(const StemConvParams& p, uint8_t* srow, int n, int iy0, int t) {
  constexpr int MAXT = 2;
  const int vpr = p.W / 16;
  const int tasks = p.srows * vpr;
  const uint32_t lo = (uint32_t)(uint8_t)(int8_t)(-p.clamp) * 0x01010101u;
  const uint32_t hi = (uint32_t)(uint8_t)(int8_t)p.clamp * 0x01010101u;
  for (int i0 = t; i0 < tasks; i0 += BUILDERS * MAXT) {
    uint4 raw[MAXT][C];
#pragma unroll
    for (int k = 0; k < MAXT; ++k) {
      const int i = min(i0 + k * BUILDERS, tasks - 1);
      const int vx = i % vpr;
      const int iy = min(max(iy0 + i / vpr, 0), p.H - 1);
#pragma unroll
      for (int c = 0; c < C; ++c)
        raw[k][c] = __ldg(reinterpret_cast<const uint4*>(p.x + (((int64_t)n * C + c) * p.H + iy) * p.W) + vx);
    }
#pragma unroll
    for (int k = 0; k < MAXT; ++k) {
      const int i = i0 + k * BUILDERS;
      if (i >= tasks) break;
      const int vx = i % vpr;
      const int r = i / vpr;
      const bool inside = iy0 + r >= 0 && iy0 + r < p.H;
      uint32_t w[C][4];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        w[c][0] = raw[k][c].x; w[c][1] = raw[k][c].y; w[c][2] = raw[k][c].z; w[c][3] = raw[k][c].w;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t x = inside ? w[c][q] : 0u;
          if (p.clamp == 127) {  // only -128 moves: add 1 to every byte equal to 0x80 (exact per-byte test)
            const uint32_t z = x ^ 0x80808080u;
            const uint32_t m = ~(((z & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | z) & 0x80808080u;
            x += m >> 7;
          } else {
            x = __vmins4(__vmaxs4(x, lo), hi);
          }
          w[c][q] = x;
        }
      }
      // output byte b of the 16 * C is channel b % C of pixel b / C
      uint32_t out[4 * C];
#pragma unroll
      for (int ow = 0; ow < 4 * C; ++ow) {
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int b = 4 * ow + j;
          const int pix = b / C, c = b % C;
          // byte (pix & 3) of the source word goes to byte j of acc
          const uint32_t sel = (0x3210u & ~(0xFu << (4 * j))) | ((uint32_t)(4 + (pix & 3)) << (4 * j));
          acc = __byte_perm(acc, w[c][pix >> 2], sel);
        }
        out[ow] = acc;
      }
      uint4* dst = reinterpret_cast<uint4*>(srow + (size_t)r * p.srow_bytes + p.left + vx * 16 * C);
#pragma unroll
      for (int q = 0; q < C; ++q) dst[q] = make_uint4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
    }
  }
}

// Packed requantisation of one thread's row (see fast_requant): straight-line per 32 columns.
template <int RELU1>
__device__ __forceinline__ void stem_fast_row(const FastQ& fq, int mul, uint32_t tbase, int chunks, const int32_t* bias_s,
                                              uint8_t* panel, uint32_t sw_key) {
  for (int ci = 0; ci < chunks; ++ci) {
    int32_t v[32];
    tmem_ld32(tbase + (uint32_t)(ci * 32), v);
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
}

#ifdef CVMK_STEM_TIMING
// Development builds: cycles per role and phase, per CTA.  Slots: 0 builders stage, 1 builders wait
// for a free A tile, 2 builders build, 3 MMA waits for the accumulator, 4 MMA waits for A, 5 MMA
// issue, 6 epilogue waits for the accumulator, 7 epilogue waits for a panel, 8 epilogue compute,
// 9 epilogue store hand-over, 10 whole builder loop, 11 tiles.
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
conv_stem_kernel(const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ StemConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t a_full[2], a_empty[2], acc_full[2], acc_empty[2], out_free[2], out_full[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* wq = smem;                    // [KH][OC][32], 32-byte swizzle
  uint8_t* a_tiles = smem + p.off_a;     // [2][KH][128][32], 32-byte swizzle
  uint8_t* srow = smem + p.off_in;       // [srows][srow_bytes]
  uint8_t* out_panels = smem + p.off_out;  // [2][128][OC], swizzle of width OC
  int32_t* bias_s = reinterpret_cast<int32_t*>(smem + p.off_bias);
  // warp index through a shuffle: provably uniform, so that the loops of the single-issuer roles
  // (MMA, output stores) run on the uniform datapath with one elected lane issuing
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&a_full[b], BUILDERS / 32);
      mbar_init(&a_empty[b], 1);
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
      mbar_init(&out_free[b], 1);
      mbar_init(&out_full[b], 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // weights -> shared memory (row r of K block ky at ky * OC * 32 + r * 32, chunks swapped in rows 4..7 of 8)
  for (int i = threadIdx.x; i < p.KH * p.OC * 2; i += STEM_THREADS) {
    const int chunk = i & 1, r = (i >> 1) % p.OC, ky = (i >> 1) / p.OC;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.w) + i);
    *reinterpret_cast<uint4*>(wq + (size_t)ky * p.OC * SLOT + r * SLOT + ((chunk ^ ((r >> 2) & 1)) << 4)) = v;
  }
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
    // ------------------------------------------------------------------ stage + build
    const int t = threadIdx.x;
    const int wp_cols = p.srow_bytes;
    uint32_t tile = 0;
    bool live = true;
    STDECL;
    STSTART(tall);
    for (int blk = blockIdx.x; blk < p.num_blocks; blk += gridDim.x) {
      const int n = blk / p.blocks_per_image;
      const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
      const int iy0 = oy0 * p.sh - p.ph;
      STSTART(tw);
      // everybody is done reading the previous block's rows; if a wait ran out for anyone, all
      // builders leave together (nobody may be left alone at a barrier)
      if (bar_any(1, BUILDERS, !live)) break;
      for (int i = t; i < p.srows * wp_cols / 4; i += BUILDERS) reinterpret_cast<uint32_t*>(srow)[i] = 0;
      bar_sync(1, BUILDERS);
      if (p.W % 16 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
        switch (p.C) {
          case 1: stage_rows<1>(p, srow, n, iy0, t); break;
          case 2: stage_rows<2>(p, srow, n, iy0, t); break;
          case 3: stage_rows<3>(p, srow, n, iy0, t); break;
          default: stage_rows<4>(p, srow, n, iy0, t); break;
        }
      } else {
        const int total = p.srows * p.C * p.W;
        for (int i = t; i < total; i += BUILDERS) {
          const int ix = i % p.W;
          const int c = (i / p.W) % p.C;
          const int r = i / (p.W * p.C);
          const int iy = iy0 + r;
          if (iy < 0 || iy >= p.H) continue;
          int v = __ldg(p.x + (((int64_t)n * p.C + c) * p.H + iy) * p.W + ix);
          v = max(min(v, p.clamp), -p.clamp);
          srow[(size_t)r * wp_cols + p.left + ix * p.C + c] = (uint8_t)(int8_t)v;
        }
      }
      bar_sync(1, BUILDERS);
      STADD(0, tw);
      for (int rr = 0; live && rr < p.rows_per_block && oy0 + rr < p.OH; ++rr) {
        for (int sg = 0; sg < p.segs; ++sg, ++tile) {
          const int buf = (int)(tile & 1u);
          if (!mbar_wait(&a_empty[buf], ((tile >> 1) & 1u) ^ 1u, &abort_flag, 1)) { live = false; break; }
          STADD(1, tw);
          const int ox = sg * p.seg_w + t;
          if (t < p.seg_w && ox < p.OW) {
            uint8_t* arow = a_tiles + (size_t)buf * p.KH * A_BLOCK + t * SLOT;
            const uint32_t sw_key = (uint32_t)((t >> 2) & 1);
            const uint32_t off = (uint32_t)(p.left - p.pw * p.C + ox * p.sw * p.C);
            const uint32_t shift = (off & 3u) * 8u;
            const uint8_t* src0 = srow + (size_t)(rr * p.sh) * wp_cols + (off & ~3u);
            for (int ky = 0; ky < p.KH; ++ky) {
              const uint32_t* src = reinterpret_cast<const uint32_t*>(src0 + (size_t)ky * wp_cols);
              uint32_t l[9];
#pragma unroll
              for (int j = 0; j < 9; ++j) l[j] = src[j];
              uint32_t o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = __funnelshift_r(l[j], l[j + 1], shift);
              uint8_t* dst = arow + (size_t)ky * A_BLOCK;
              *reinterpret_cast<uint4*>(dst + ((0u ^ sw_key) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(dst + ((1u ^ sw_key) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[buf]);
          STADD(2, tw);
        }
      }
    }
#ifdef CVMK_STEM_TIMING
    STADD(10, tall);
    if (t == 0) { stacc[11] = tile; STFLUSH(0); STFLUSH(1); STFLUSH(2); STFLUSH(10); STFLUSH(11); }
#endif
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    {
      const bool leader = elect_one();
      const uint32_t idesc = umma_idesc_i8(p.OC);
      const uint64_t desc_b0 = umma_desc(smem_u32(wq), SLOT);
      const uint64_t desc_a0 = umma_desc(smem_u32(a_tiles), SLOT);
      const uint64_t b_step = (uint64_t)((uint32_t)(p.OC * SLOT) >> 4);
      const uint64_t a_step = (uint64_t)((uint32_t)A_BLOCK >> 4);
      uint32_t tile = 0;
      bool live = true;
      STDECL;
      for (int blk = blockIdx.x; live && blk < p.num_blocks; blk += gridDim.x) {
        const int n = blk / p.blocks_per_image;
        const int oy0 = (blk - n * p.blocks_per_image) * p.rows_per_block;
        for (int rr = 0; live && rr < p.rows_per_block && oy0 + rr < p.OH; ++rr) {
          for (int sg = 0; sg < p.segs; ++sg, ++tile) {
            const int buf = (int)(tile & 1u);
            const uint32_t par = (tile >> 1) & 1u;
            STSTART(tw);
            if (!mbar_wait(&acc_empty[buf], par ^ 1u, &abort_flag, 2)) { live = false; break; }
            STADD(3, tw);
            if (!mbar_wait(&a_full[buf], par, &abort_flag, 3)) { live = false; break; }
            STADD(4, tw);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.OC);
            // one 32-bit add per operand and instruction (only the low descriptor word moves)
            uint32_t al = (uint32_t)desc_a0 + (uint32_t)buf * (uint32_t)p.KH * (uint32_t)a_step;
            uint32_t bl = (uint32_t)desc_b0;
            const uint32_t a_hi = (uint32_t)(desc_a0 >> 32), b_hi = (uint32_t)(desc_b0 >> 32);
            if (leader) {
              for (int ky = 0; ky < p.KH; ++ky, al += (uint32_t)a_step, bl += (uint32_t)b_step)
                mma_i8_k<1>(d_tmem, al, a_hi, bl, b_hi, idesc, (uint32_t)ky);
              mma_commit(&a_empty[buf]);
              mma_commit(&acc_full[buf]);
            }
            STADD(5, tw);
          }
        }
      }
#ifdef CVMK_STEM_TIMING
      if (leader) { STFLUSH(3); STFLUSH(4); STFLUSH(5); }
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
          if (!mbar_wait(&acc_full[buf], par, &abort_flag, 4)) { live = false; break; }
          STADD(6, tw);
          tc_fence_after();
          if (!mbar_wait(&out_free[buf], par, &abort_flag, 5)) { live = false; break; }
          STADD(7, tw);
          uint8_t* panel = out_panels + (size_t)buf * panel_bytes + row_off;
          const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.OC);
          const int ox = sg * p.seg_w + row_in_tile;
          const bool valid = row_in_tile < p.seg_w && ox < p.OW;
          const size_t lin0 = (((size_t)n * p.OH + oy) * p.OW + (valid ? ox : 0)) * p.OC;
          if (p.fast_mode) {
            if (p.fast_variant & 1) stem_fast_row<1>(fq, p.f_mul, tbase, chunks, bias_s, panel, sw_key);
            else stem_fast_row<0>(fq, p.f_mul, tbase, chunks, bias_s, panel, sw_key);
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
          fence_async_smem();
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
    if (leader) { STFLUSH(6); STFLUSH(7); STFLUSH(8); STFLUSH(9); }
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
          if (!mbar_wait(&out_full[buf], (tile >> 1) & 1u, &abort_flag, 6)) { live = false; break; }
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
  int rows_per_block, segs, seg_w, srows, srow_bytes, left, off_a, off_in, off_out, off_bias, smem_bytes;
};

bool stem_layout(const cvmk_stem_conv_desc& d, StemLayout* L) {
  L->segs = (d.OW + BLOCK_M - 1) / BLOCK_M;
  L->seg_w = (d.OW + L->segs - 1) / L->segs;
  L->rows_per_block = 4;
  if (L->rows_per_block > d.OH) L->rows_per_block = d.OH;
  L->srows = (L->rows_per_block - 1) * d.stride_h + d.KH;
  // a window may start at the last output pixel and is read as nine 32-bit words
  L->left = (d.pad_w * d.C + 15) / 16 * 16;  // image column 0 starts 16-byte aligned in a staged row
  const int reach = L->left - d.pad_w * d.C + ((d.OW - 1) * d.stride_w) * d.C + 40;
  int row = L->left + (d.W + d.pad_w) * d.C;
  if (row < reach) row = reach;
  L->srow_bytes = (row + 15) / 16 * 16;
  const int w_bytes = d.KH * d.OC * SLOT;
  L->off_a = (w_bytes + 1023) / 1024 * 1024;
  L->off_in = L->off_a + 2 * d.KH * A_BLOCK;
  L->off_out = (L->off_in + L->srows * L->srow_bytes + 1023) / 1024 * 1024;
  L->off_bias = L->off_out + 2 * BLOCK_M * d.OC;
  L->smem_bytes = L->off_bias + d.OC * 4 + 1024;
  return L->smem_bytes <= 110 * 1024;
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_conv2d_stem_supported(const cvmk_stem_conv_desc* d) {
  if (!d) return 0;
  if (d->C < 1 || d->C > 4 || d->KW * d->C > SLOT || d->KH < 1 || d->KH > 8) return 0;
  if (d->OC % 32 != 0 || d->OC > MAX_OC || (d->OC != 32 && d->OC != 64 && d->OC != 128)) return 0;
  if (d->stride_h < 1 || d->stride_w < 1 || d->stride_h > 4 || d->stride_w > 4) return 0;
  if (d->pad_h < 0 || d->pad_w < 0 || d->clamp < 1 || d->clamp > 127) return 0;
  if ((int64_t)d->N * d->OH > INT32_MAX / 4 || (int64_t)d->N * d->OH * d->OW * d->OC > ((int64_t)1 << 40)) return 0;
  StemLayout L;
  return stem_layout(*d, &L) ? 1 : 0;
}

extern "C" int cvmk_conv2d_stem_prepare(const cvmk_stem_conv_desc* d, cvmk_stem_conv_plan* plan) {
  if (!d || !plan || !cvmk_conv2d_stem_supported(d)) { set_error("conv2d_stem_prepare: unsupported shape"); return CVMK_ERR_UNSUPPORTED; }
  if (((uintptr_t)d->w & 15) || ((uintptr_t)d->y & 15)) { set_error("conv2d_stem_prepare: operands must be 16-byte aligned"); return CVMK_ERR_ARG; }
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
  p.x = d.x; p.w = d.w;
  p.N = d.N; p.H = d.H; p.W = d.W; p.C = d.C; p.OC = d.OC; p.KH = d.KH; p.KW = d.KW; p.OH = d.OH; p.OW = d.OW;
  p.sh = d.stride_h; p.sw = d.stride_w; p.ph = d.pad_h; p.pw = d.pad_w;
  p.clamp = d.clamp;
  p.rows_per_block = L.rows_per_block;
  p.blocks_per_image = (d.OH + L.rows_per_block - 1) / L.rows_per_block;
  p.num_blocks = d.N * p.blocks_per_image;
  p.segs = L.segs; p.seg_w = L.seg_w; p.srows = L.srows; p.srow_bytes = L.srow_bytes; p.left = L.left;
  p.off_a = L.off_a; p.off_in = L.off_in; p.off_out = L.off_out; p.off_bias = L.off_bias;
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
    cudaError_t e = cudaFuncSetAttribute(conv_stem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    if (check_cuda(e, "cudaFuncSetAttribute(conv_stem_kernel)")) return CVMK_ERR_CUDA;
    attr_set = true;
  }
  CUtensorMap ty;
  memcpy(&ty, plan->tmap_y, sizeof(ty));
  conv_stem_kernel<<<plan->grid, STEM_THREADS, plan->smem_bytes, (cudaStream_t)stream>>>(ty, p);
  return check_cuda(cudaGetLastError(), "conv_stem_kernel launch");
}

#ifdef CVMK_STEM_TIMING
extern "C" int cvmk_stem_timing_read(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_stem_timing, sizeof(long long) * (size_t)count);
}
#endif
