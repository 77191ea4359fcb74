// conv2d on CUDA cores: grouped / depthwise convolutions and the shapes the tensor-core kernel
// does not take (channel counts that are not a multiple of 32, e.g. a 3-channel stem).
//
// Reproduces groupwise_conv2d (src/runtime/cpu/ops/ops.cc:333-366) for groups > 1 and the
// im2col + matrix_mul path (:204-246, :148-200, :368-456) for groups = 1.  Accumulation is int32
// and exact, so the summation order is free.
#include <cuda_runtime.h>
#include <string.h>
#include "common.cuh"

namespace cvmk {
namespace {

struct DirectParams {
  const void* x; const int8_t* w; void* y;
  int xd, yd, narrow_x;
  int N, H, W, C, OC, KH, KW, OH, OW, groups;
  int sh, sw, ph, pw, dh, dw;
  int64_t total;
  DevChain chain;
};

__device__ __forceinline__ void store_one(void* y, int yd, int64_t i, int32_t v) {
  if (yd == CVMK_I8) reinterpret_cast<int8_t*>(y)[i] = (int8_t)v;
  else reinterpret_cast<int32_t*>(y)[i] = v;
}

// One thread per output element; consecutive threads walk the output channels of one pixel, so
// activation reads are warp-broadcast and weight reads are contiguous per thread.
template <int XD>
__global__ void __launch_bounds__(256) conv_direct_kernel(const __grid_constant__ DirectParams p) {
  const int icg = p.C / p.groups;
  const int ocg = p.OC / p.groups;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    const int oc = (int)(i % p.OC);
    int64_t pix = i / p.OC;
    const int ox = (int)(pix % p.OW); pix /= p.OW;
    const int oy = (int)(pix % p.OH);
    const int n = (int)(pix / p.OH);
    const int ic0 = (oc / ocg) * icg;
    int32_t acc = 0;
    for (int fy = 0; fy < p.KH; ++fy) {
      const int iy = oy * p.sh + fy * p.dh - p.ph;
      if (iy < 0 || iy >= p.H) continue;
      for (int fx = 0; fx < p.KW; ++fx) {
        const int ix = ox * p.sw + fx * p.dw - p.pw;
        if (ix < 0 || ix >= p.W) continue;
        const int64_t xb = (((int64_t)n * p.H + iy) * p.W + ix) * p.C + ic0;
        const int8_t* wp = p.w + (((int64_t)oc * p.KH + fy) * p.KW + fx) * icg;
        if (XD == CVMK_I8) {
          const int8_t* xp = reinterpret_cast<const int8_t*>(p.x) + xb;
          int ic = 0;
          if (((reinterpret_cast<uintptr_t>(xp) | reinterpret_cast<uintptr_t>(wp)) & 3) == 0) {
            for (; ic + 4 <= icg; ic += 4)
              acc = __dp4a(*reinterpret_cast<const int*>(xp + ic), *reinterpret_cast<const int*>(wp + ic), acc);
          }
          for (; ic < icg; ++ic) acc += (int32_t)xp[ic] * (int32_t)wp[ic];
        } else {
          const int32_t* xp = reinterpret_cast<const int32_t*>(p.x) + xb;
          if (p.narrow_x) {
            for (int ic = 0; ic < icg; ++ic) acc += (int32_t)(int8_t)xp[ic] * (int32_t)wp[ic];
          } else {
            for (int ic = 0; ic < icg; ++ic)
              acc = (int32_t)((uint32_t)acc + (uint32_t)xp[ic] * (uint32_t)(int32_t)wp[ic]);
          }
        }
      }
    }
    int32_t v[1] = {acc};
    apply_chain<1>(p.chain, v, (size_t)i, oc);
    store_one(p.y, p.yd, i, v[0]);
  }
}

// Depthwise, int8 NHWC, channels a multiple of 16: one thread owns 16 channels of PX consecutive
// output pixels of a row.  Weights are [KH, KW, C]; the per-channel products come from byte
// extraction of the packed words.
template <int PX>
__global__ void __launch_bounds__(128) depthwise_kernel(const __grid_constant__ DirectParams p) {
  const int cvec = p.C / 16;
  const int oxg = (p.OW + PX - 1) / PX;
  const int64_t total = (int64_t)p.N * p.OH * oxg * cvec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int cv = (int)(i % cvec);
    int64_t r = i / cvec;
    const int ox0 = (int)(r % oxg) * PX; r /= oxg;
    const int oy = (int)(r % p.OH);
    const int n = (int)(r / p.OH);
    int32_t acc[PX][16];
#pragma unroll
    for (int q = 0; q < PX; ++q)
#pragma unroll
      for (int k = 0; k < 16; ++k) acc[q][k] = 0;
    for (int fy = 0; fy < p.KH; ++fy) {
      const int iy = oy * p.sh + fy * p.dh - p.ph;
      if (iy < 0 || iy >= p.H) continue;
      for (int fx = 0; fx < p.KW; ++fx) {
        const int4 wv = __ldg(reinterpret_cast<const int4*>(p.w + ((int64_t)fy * p.KW + fx) * p.C) + cv);
        const int ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int q = 0; q < PX; ++q) {
          const int ix = (ox0 + q) * p.sw + fx * p.dw - p.pw;
          if (ix < 0 || ix >= p.W || ox0 + q >= p.OW) continue;
          const int4 xv = __ldg(reinterpret_cast<const int4*>(reinterpret_cast<const int8_t*>(p.x) +
                                                                (((int64_t)n * p.H + iy) * p.W + ix) * p.C) + cv);
          const int xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const int32_t a = (int32_t)(int8_t)(xw[k >> 2] >> ((k & 3) * 8));
            const int32_t b = (int32_t)(int8_t)(ww[k >> 2] >> ((k & 3) * 8));
            acc[q][k] += a * b;
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < PX; ++q) {
      if (ox0 + q >= p.OW) continue;
      const int64_t lin = ((((int64_t)n * p.OH + oy) * p.OW + ox0 + q) * p.C) + cv * 16;
      apply_chain<16>(p.chain, acc[q], (size_t)lin, cv * 16);
      if (p.yd == CVMK_I8) {
        int4 o;
        o.x = (int)pack4(acc[q][0], acc[q][1], acc[q][2], acc[q][3]);
        o.y = (int)pack4(acc[q][4], acc[q][5], acc[q][6], acc[q][7]);
        o.z = (int)pack4(acc[q][8], acc[q][9], acc[q][10], acc[q][11]);
        o.w = (int)pack4(acc[q][12], acc[q][13], acc[q][14], acc[q][15]);
        *reinterpret_cast<int4*>(reinterpret_cast<int8_t*>(p.y) + lin) = o;
      } else {
        int4* dst = reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(p.y) + lin);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          dst[g] = make_int4(acc[q][4 * g], acc[q][4 * g + 1], acc[q][4 * g + 2], acc[q][4 * g + 3]);
      }
    }
  }
}


// Depthwise 3x3, int8 NHWC, channels a multiple of 4, no dilation, stride S in {1, 2}: one thread
// owns 4 channels (one 32-bit word per pixel) of a whole output row and walks it in strips of 4
// pixels.  Its 36 weights (and the bias, when the chain starts with one) are unpacked into
// registers once per row; every input word is unpacked once per strip and feeds all the outputs
// it belongs to, so the inner loop is one multiply-add per product.
template <int S>
__global__ void __launch_bounds__(256) depthwise3x3_kernel(const __grid_constant__ DirectParams p) {
  constexpr int PX = 4;
  constexpr int IN = (PX - 1) * S + 3;  // input pixels of a row that a strip touches
  const int cw = p.C / 4;
  const int64_t total = (int64_t)p.N * p.OH * cw;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool has_bias = p.chain.n > 0 && p.chain.s[0].op == K_ADD_C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int cv = (int)(i % cw);
    const int row = (int)(i / cw);
    const int oy = row % p.OH;
    const int n = row / p.OH;
    int32_t wgt[9][4];
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      const int w = __ldg(reinterpret_cast<const int*>(p.w + (int64_t)t * p.C) + cv);
#pragma unroll
      for (int k = 0; k < 4; ++k) wgt[t][k] = (int32_t)(int8_t)(w >> (k * 8));
    }
    int32_t bias[4] = {0, 0, 0, 0};
    if (has_bias) {
      const int4 b4 = __ldg(reinterpret_cast<const int4*>(p.chain.s[0].ptr) + cv);
      bias[0] = b4.x; bias[1] = b4.y; bias[2] = b4.z; bias[3] = b4.w;
    }
    // Rows and columns outside the image are read from a clamped (valid) address and masked to
    // zero, so that all loads of a strip are independent and in flight together.
    const int* rows[3];
    bool row_ok[3];
#pragma unroll
    for (int fy = 0; fy < 3; ++fy) {
      const int iy = oy * S + fy - p.ph;
      row_ok[fy] = iy >= 0 && iy < p.H;
      const int iyc = min(max(iy, 0), p.H - 1);
      rows[fy] = reinterpret_cast<const int*>(reinterpret_cast<const int8_t*>(p.x) + ((int64_t)n * p.H + iyc) * p.W * p.C) + cv;
    }
    const int64_t out_row = ((int64_t)n * p.OH + oy) * p.OW;
    for (int ox0 = 0; ox0 < p.OW; ox0 += PX) {
      int32_t acc[PX][4];
#pragma unroll
      for (int q = 0; q < PX; ++q)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[q][k] = bias[k];
      const int ix0 = ox0 * S - p.pw;
      int xin[3][IN];
#pragma unroll
      for (int fy = 0; fy < 3; ++fy) {
#pragma unroll
        for (int j = 0; j < IN; ++j) {
          const int ix = ix0 + j;
          const int v = __ldg(rows[fy] + min(max(ix, 0), p.W - 1) * cw);
          xin[fy][j] = (row_ok[fy] && ix >= 0 && ix < p.W) ? v : 0;
        }
      }
#pragma unroll
      for (int fy = 0; fy < 3; ++fy) {
#pragma unroll
        for (int j = 0; j < IN; ++j) {
          const int xw = xin[fy][j];
          int32_t xv[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) xv[k] = (int32_t)(int8_t)(xw >> (k * 8));
#pragma unroll
          for (int fx = 0; fx < 3; ++fx) {
            if ((j - fx) % S != 0 || j - fx < 0 || (j - fx) / S >= PX) continue;  // resolved at compile time
            const int q = (j - fx) / S;
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[q][k] += xv[k] * wgt[fy * 3 + fx][k];
          }
        }
      }
#pragma unroll
      for (int q = 0; q < PX; ++q) {
        if (ox0 + q >= p.OW) continue;
        const int64_t lin = (out_row + ox0 + q) * p.C + cv * 4;
        apply_chain<4>(p.chain, acc[q], (size_t)lin, cv * 4, 1, nullptr, -1, has_bias ? 1 : 0);
        if (p.yd == CVMK_I8)
          *reinterpret_cast<uint32_t*>(reinterpret_cast<int8_t*>(p.y) + lin) = pack4(acc[q][0], acc[q][1], acc[q][2], acc[q][3]);
        else
          *reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(p.y) + lin) = make_int4(acc[q][0], acc[q][1], acc[q][2], acc[q][3]);
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Depthwise 3x3 (stride 1 or 2), int8 in / int8 out, tiled through shared memory.
//
// A CTA takes one image, a band of R output rows (all columns) and a block of CB = 32 / 64 / 128
// channels.  The input rows of the band are copied into shared memory once with 16-byte
// asynchronous copies (zeros where the filter reaches outside the image), so every input byte
// crosses L2 -> SM once per band instead of three times, and all boundary handling is done there.
// A thread then owns 4 channels (one 32-bit word per pixel) and walks strips of 4 output pixels.
// The words of four neighbouring pixels are transposed in registers (eight byte permutes) into
// four words that each hold ONE channel at four consecutive pixels; a funnel shift moves the
// window of an output pixel to byte 0, and one dp4a against the word (w[fy][0], w[fy][1],
// w[fy][2], 0) of that channel multiplies a whole filter row: three multiply instructions per
// output element instead of nine, on a part whose integer multiply pipe runs at half rate and was
// the limit of the form that multiplied tap by tap.  A warp covers CB/4
// consecutive channel words of 32*4/CB rows; the row pitch is padded so that those rows fall into
// different banks.  The requantisation is the packed form of the tensor-core kernels (multiply-add
// into the upper half word, clamp on s16x2, byte permutes).
// Reproduces groupwise_conv2d with groups = C (src/runtime/cpu/ops/ops.cc:333-366).
// Division of a non-negative 31-bit number by a divisor fixed at launch: q = umulhi(n, mul) >> shr
// (mul = ceil(2^(31 + ceil(log2 d)) / d)); d = 1 is flagged by mul = 0.
struct DwDiv { uint32_t mul, shr; };
__device__ __forceinline__ int dw_div(int n, const DwDiv& d) { return d.mul ? (int)(__umulhi((uint32_t)n, d.mul) >> d.shr) : n; }
static DwDiv make_dw_div(int d) {
  DwDiv f = {0, 0};
  if (d <= 1) return f;
  int lg = 0;
  while ((1LL << lg) < d) ++lg;
  f.mul = (uint32_t)((((uint64_t)1 << (31 + lg)) + (uint64_t)d - 1) / (uint64_t)d);
  f.shr = (uint32_t)(lg - 1);
  return f;
}

struct Dw3Params {
  const int8_t* x; const int8_t* w; const int32_t* bias; int8_t* y;
  DwDiv div_per_row, div_strips;   // by xw * (cb_words / 4) and by strips
  int vec_log2;                    // log2(cb_words / 4)
  int N, H, W, C, OH, OW, ph, pw;
  int cb_words;        // channel words per block (CB / 4): 8, 16 or 32
  int rows_per_tile;   // R
  int tiles_y, tiles_c;
  int xw;              // staged pixels per input row
  int pitch;           // words between staged rows
  int strips;          // ceil(OW / 4)
  int mul, add;        // requantisation: ((acc + bias + add) * mul) >> 16, mul = 2^(16 - shift)
  uint32_t lo, hi;     // clamp, replicated into both halves of an s16x2 word
  int relu;            // the clamp's lower bound is 0
};

// 4 x 4 byte transpose: words a, b, c, d (4 bytes each) -> t[k] = (a.k, b.k, c.k, d.k)
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&t)[4]) {
  const uint32_t ab01 = __byte_perm(a, b, 0x5140), cd01 = __byte_perm(c, d, 0x5140);   // (a0 b0 a1 b1), (c0 d0 c1 d1)
  const uint32_t ab23 = __byte_perm(a, b, 0x7362), cd23 = __byte_perm(c, d, 0x7362);   // (a2 b2 a3 b3), (c2 d2 c3 d3)
  t[0] = __byte_perm(ab01, cd01, 0x5410);
  t[1] = __byte_perm(ab01, cd01, 0x7632);
  t[2] = __byte_perm(ab23, cd23, 0x5410);
  t[3] = __byte_perm(ab23, cd23, 0x7632);
}

template <int S>
__global__ void __launch_bounds__(256) dw3x3_tile_kernel(const __grid_constant__ Dw3Params p) {
  extern __shared__ __align__(16) uint32_t tile[];
  constexpr int PX = 4;
  constexpr int IN = (PX - 1) * S + 3;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int t = blockIdx.x;
  const int tc = t % p.tiles_c; t /= p.tiles_c;
  const int ty = t % p.tiles_y;
  const int n = t / p.tiles_y;
  const int oy0 = ty * p.rows_per_tile;
  const int rows_here = min(p.rows_per_tile, p.OH - oy0);
  const int cbw = p.cb_words;
  const int c0 = tc * cbw * 4;
  // ---- stage the input rows of the band
  const int in_rows = (rows_here - 1) * S + 3;
  const int iy0 = oy0 * S - p.ph;
  const int vecs = cbw / 4;                     // 16-byte vectors per pixel
  const int per_row = p.xw * vecs;
  for (int idx = tid; idx < in_rows * per_row; idx += 256) {
    const int r = dw_div(idx, p.div_per_row), rem = idx - r * per_row;
    const int xs = rem >> p.vec_log2, v = rem - (xs << p.vec_log2);
    const int iy = iy0 + r, ix = xs - p.pw;
    uint32_t* dst = tile + (size_t)r * p.pitch + xs * cbw + v * 4;
    if (iy >= 0 && iy < p.H && ix >= 0 && ix < p.W) {
      const int8_t* src = p.x + (((int64_t)n * p.H + iy) * p.W + ix) * p.C + c0 + v * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  // ---- weights and bias of this thread's four channels (meanwhile)
  const int cw = lane % cbw, rr = lane / cbw, rows_per_warp = 32 / cbw;
  uint32_t wrow[3][4];   // wrow[fy][k] = (w[fy][0], w[fy][1], w[fy][2], 0) of channel k
#pragma unroll
  for (int fy = 0; fy < 3; ++fy) {
    uint32_t w3[3];
#pragma unroll
    for (int fx = 0; fx < 3; ++fx)
      w3[fx] = (uint32_t)__ldg(reinterpret_cast<const int*>(p.w + (int64_t)(fy * 3 + fx) * p.C + c0) + cw);
    transpose4x4(w3[0], w3[1], w3[2], 0u, wrow[fy]);
  }
  int bq[4] = {0, 0, 0, 0};   // (bias + rounding addend) * mul
  {
    int4 b4 = make_int4(0, 0, 0, 0);
    if (p.bias) b4 = __ldg(reinterpret_cast<const int4*>(p.bias + c0) + cw);
    bq[0] = (b4.x + p.add) * p.mul; bq[1] = (b4.y + p.add) * p.mul;
    bq[2] = (b4.z + p.add) * p.mul; bq[3] = (b4.w + p.add) * p.mul;
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();
  // ---- compute: warp items = (group of rows_per_warp rows, strip of 4 pixels)
  const int groups = (rows_here + rows_per_warp - 1) / rows_per_warp;
  for (int item = warp; item < groups * p.strips; item += 8) {
    const int g = dw_div(item, p.div_strips), sidx = item - g * p.strips;
    const int orow = g * rows_per_warp + rr;
    if (orow >= rows_here) continue;
    const int ox0 = sidx * PX;
    const uint32_t* base = tile + (size_t)(orow * S) * p.pitch + (ox0 * S) * cbw + cw;
    int acc[PX][4];
#pragma unroll
    for (int q = 0; q < PX; ++q)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[q][k] = 0;
#pragma unroll
    for (int fy = 0; fy < 3; ++fy) {
      uint32_t xin[12];
#pragma unroll
      for (int j = 0; j < 12; ++j) xin[j] = j < IN ? base[(size_t)fy * p.pitch + j * cbw] : 0u;
      // t[g][k]: channel k at input pixels 4g .. 4g + 3 of the strip
      uint32_t t[3][4];
      transpose4x4(xin[0], xin[1], xin[2], xin[3], t[0]);
      transpose4x4(xin[4], xin[5], xin[6], xin[7], t[1]);
      if (S == 2) {
#pragma unroll
        for (int k = 0; k < 4; ++k) t[2][k] = __byte_perm(xin[8], 0u, 0x4440 + k);   // pixel 8 alone
      }
#pragma unroll
      for (int q = 0; q < PX; ++q) {
        const int first = q * S;            // first input pixel of this output's window
        const int g = first >> 2, sh = (first & 3) * 8;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t win = sh ? __funnelshift_r(t[g][k], t[g + 1][k], sh) : t[g][k];
          acc[q][k] = __dp4a((int)win, (int)wrow[fy][k], acc[q][k]);
        }
      }
    }
    int8_t* yrow = p.y + (((int64_t)n * p.OH + oy0 + orow) * p.OW + ox0) * p.C + c0 + cw * 4;
#pragma unroll
    for (int q = 0; q < PX; ++q) {
      if (ox0 + q >= p.OW) break;
      const uint32_t v0 = (uint32_t)(acc[q][0] * p.mul + bq[0]), v1 = (uint32_t)(acc[q][1] * p.mul + bq[1]);
      const uint32_t v2 = (uint32_t)(acc[q][2] * p.mul + bq[2]), v3 = (uint32_t)(acc[q][3] * p.mul + bq[3]);
      uint32_t h0 = __byte_perm(v0, v1, 0x7632), h1 = __byte_perm(v2, v3, 0x7632);   // the upper halves
      if (p.relu) { h0 = __vimin_s16x2_relu(h0, p.hi); h1 = __vimin_s16x2_relu(h1, p.hi); }
      else { h0 = __vmaxs2(__vmins2(h0, p.hi), p.lo); h1 = __vmaxs2(__vmins2(h1, p.hi), p.lo); }
      *reinterpret_cast<uint32_t*>(yrow + (int64_t)q * p.C) = __byte_perm(h0, h1, 0x6420);
    }
  }
}

// Patch gather: one thread builds 16 consecutive bytes of one row of A.  The (fy, fx, c) split
// of every k is looked up in a shared-memory table built once per block.
struct PackParams {
  const int8_t* x; int8_t* a;
  int N, H, W, C, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, Kp, K;
  int64_t total;  // rows * Kp / 16
};
__global__ void __launch_bounds__(256) im2col_pack_kernel(const __grid_constant__ PackParams p) {
  extern __shared__ int lut[];  // per k: (fy*dh) << 20 | (fx*dw) << 8 | c
  for (int k = threadIdx.x; k < p.K; k += blockDim.x) {
    const int fy = k / (p.KW * p.C), r = k - fy * (p.KW * p.C);
    const int fx = r / p.C, c = r - fx * p.C;
    lut[k] = ((fy * p.dh) << 20) | ((fx * p.dw) << 8) | c;
  }
  __syncthreads();
  const int chunks = p.Kp / 16;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    const int q = (int)(i % chunks);
    int64_t m = i / chunks;
    const int ox = (int)(m % p.OW);
    int64_t t = m / p.OW;
    const int oy = (int)(t % p.OH);
    const int n = (int)(t / p.OH);
    const int iy0 = oy * p.sh - p.ph, ix0 = ox * p.sw - p.pw;
    const int8_t* xn = p.x + (int64_t)n * p.H * p.W * p.C;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int k = q * 16 + j;
      if (k < p.K) {
        const int e = lut[k];
        const int iy = iy0 + (e >> 20), ix = ix0 + ((e >> 8) & 0xfff), c = e & 0xff;
        if (iy >= 0 && iy < p.H && ix >= 0 && ix < p.W) {
          const uint32_t b = (uint8_t)__ldg(xn + ((int64_t)iy * p.W + ix) * p.C + c);
          w[j >> 2] |= b << ((j & 3) * 8);
        }
      }
    }
    *reinterpret_cast<uint4*>(p.a + m * p.Kp + q * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}


// Patch gather straight from the NCHW network input.  One CTA per (image, output row): the KH
// input rows of every channel are staged (clamped, zero-padded left and right) in shared memory,
// then warp q builds the q-th 16-byte chunk of the A rows of that output row, 32 pixels at a time.
struct StemParams {
  const int8_t* x; int8_t* a;
  int N, H, W, C, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, Kp, K, clamp, wp;
};
__global__ void __launch_bounds__(512) stem_pack_kernel(const __grid_constant__ StemParams p) {
  extern __shared__ __align__(16) int8_t srow[];  // [KH][C][wp], wp = W + 2 * pw
  const int n = blockIdx.x / p.OH, oy = blockIdx.x % p.OH;
  const int iy0 = oy * p.sh - p.ph;
  const int total = p.KH * p.C * p.wp;
  const bool vec = (p.W % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
  if (vec) {
    // zero everything (padding columns, rows outside the image), then one 16-byte global load per
    // thread and row piece: all loads of a CTA are in flight together
    for (int i = threadIdx.x; i < (total + 3) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(srow)[i] = 0;
    __syncthreads();
    const int vpr = p.W / 16;  // vectors per input row
    const int tasks = p.KH * p.C * vpr;
    for (int i = threadIdx.x; i < tasks; i += blockDim.x) {
      const int vx = i % vpr;
      const int c = (i / vpr) % p.C;
      const int r = i / (vpr * p.C);
      const int iy = iy0 + r * p.dh;
      if (iy < 0 || iy >= p.H) continue;
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.x + (((int64_t)n * p.C + c) * p.H + iy) * p.W) + vx);
      const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
      int8_t* dst = srow + (r * p.C + c) * p.wp + p.pw + vx * 16;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int v = (int)(int8_t)(w4[j >> 2] >> ((j & 3) * 8));
        dst[j] = (int8_t)max(min(v, p.clamp), -p.clamp);
      }
    }
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int xx = i % p.wp - p.pw;
      const int c = (i / p.wp) % p.C;
      const int iy = iy0 + (i / (p.wp * p.C)) * p.dh;
      int v = 0;
      if (xx >= 0 && xx < p.W && iy >= 0 && iy < p.H) {
        v = __ldg(p.x + (((int64_t)n * p.C + c) * p.H + iy) * p.W + xx);
        v = max(min(v, p.clamp), -p.clamp);
      }
      srow[i] = (int8_t)v;
    }
  }
  __syncthreads();
  // blockDim.x is a multiple of the chunk count, so a thread always builds the same chunk q and
  // consecutive threads write consecutive 16-byte pieces of the (contiguous) A rows of this
  // output row.
  const int chunks = p.Kp / 16;
  const int q = threadIdx.x % chunks;
  const int ox_step = blockDim.x / chunks;
  int off[16];  // shared-memory offset of byte j of this chunk for output pixel 0, -1: zero
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int k = q * 16 + j;
    if (k < p.K) {
      const int fy = k / (p.KW * p.C), r = k - fy * (p.KW * p.C);
      const int fx = r / p.C, c = r - fx * p.C;
      off[j] = (fy * p.C + c) * p.wp + fx * p.dw;
    } else {
      off[j] = -1;
    }
  }
  int8_t* arow = p.a + (((int64_t)n * p.OH + oy) * p.OW) * p.Kp + q * 16;
  for (int ox = threadIdx.x / chunks; ox < p.OW; ox += ox_step) {
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (off[j] >= 0) w[j >> 2] |= (uint32_t)(uint8_t)srow[off[j] + ox * p.sw] << ((j & 3) * 8);
    *reinterpret_cast<uint4*>(arow + (int64_t)ox * p.Kp) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Plans and launches dw3x3_tile_kernel when the layer and its chain qualify; returns -1 when they
// do not (the caller then uses the register kernel).
int try_dw3x3_tile(const cvmk_conv_direct_desc* d, const DevChain& chain, cudaStream_t s) {
  if (d->y_dtype != CVMK_I8 || d->C % 32 != 0 || d->acc_bound <= 0 || d->OW < 1) return -1;
  if (d->pad_h > 1 || d->pad_w > 1) return -1;
  // chain = [bias] rs_clamp, with a sum that cannot overflow and fits 16 bits after the shift
  int i0 = 0;
  const int32_t* bias = nullptr;
  if (chain.n > 0 && chain.s[0].op == K_ADD_C) { bias = reinterpret_cast<const int32_t*>(chain.s[0].ptr); i0 = 1; }
  if (chain.n - i0 != 1 || chain.s[i0].op != K_RS_CLAMP) return -1;
  const DevStep& rs = chain.s[i0];
  const int64_t add = rs.c;
  const int sh = rs.d;
  const int64_t lo1 = ((int64_t)rs.a + add) >> sh, hi1 = ((int64_t)rs.b + add) >> sh;
  if (sh > 16 || d->acc_bound + add >= (int64_t)INT32_MAX || ((d->acc_bound + add) >> sh) >= 32767 ||
      lo1 < -32767 || hi1 > 32767 || lo1 > hi1)
    return -1;
  // The kernel clamps after the shift; the chain clamps the sum to [rs.a, rs.b] first.  Both give
  // the same value because the shift is monotone (the argument of the tensor-core kernels).
  Dw3Params p;
  memset(&p, 0, sizeof(p));
  p.x = reinterpret_cast<const int8_t*>(d->x); p.w = d->w; p.bias = bias; p.y = reinterpret_cast<int8_t*>(d->y);
  p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C; p.OH = d->OH; p.OW = d->OW; p.ph = d->pad_h; p.pw = d->pad_w;
  const int S = d->stride_h;
  const int cb = d->C % 128 == 0 ? 128 : (d->C % 64 == 0 ? 64 : 32);
  p.cb_words = cb / 4;
  p.tiles_c = d->C / cb;
  p.strips = (d->OW + 3) / 4;
  p.xw = (p.strips * 4 - 1) * S + 3;
  // rows of a warp must land in different banks: pitch = multiple of 32 words + cb_words / S
  p.pitch = (p.xw * p.cb_words + 31) / 32 * 32 + p.cb_words / S;
  const int rows_per_warp = 32 / p.cb_words;
  int R = d->OH;
  auto smem_of = [&](int r) { return ((r - 1) * S + 3) * p.pitch * 4; };
  // up to 44 KB a CTA (four or five per SM); wide images whose shortest band needs more take up to 100 KB
  while (R > rows_per_warp && smem_of(R) > 44 * 1024) --R;
  if (smem_of(R) > 100 * 1024) return -1;
  // enough tiles to fill the GPU a few times over
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  while (R > 2 * rows_per_warp && (int64_t)d->N * ((d->OH + R - 1) / R) * p.tiles_c < 6LL * sms) R = (R + 1) / 2;
  if (R > rows_per_warp) R = R / rows_per_warp * rows_per_warp;   // whole warp row groups
  if (smem_of(R) > 100 * 1024) return -1;
  p.rows_per_tile = R;
  p.tiles_y = (d->OH + R - 1) / R;
  p.div_per_row = make_dw_div(p.xw * (p.cb_words / 4));
  p.div_strips = make_dw_div(p.strips);
  p.vec_log2 = p.cb_words == 8 ? 1 : (p.cb_words == 16 ? 2 : 3);
  p.mul = 1 << (16 - sh);
  p.add = (int)add;
  auto x2 = [](int64_t v) { return (uint32_t)((uint32_t)(uint16_t)(int16_t)v | ((uint32_t)(uint16_t)(int16_t)v << 16)); };
  p.lo = x2(lo1); p.hi = x2(hi1);
  p.relu = lo1 == 0;
  const int64_t tiles = (int64_t)d->N * p.tiles_y * p.tiles_c;
  if (tiles > INT32_MAX) return -1;
  const int smem = smem_of(R);
  if (smem > 48 * 1024) {
    static bool attr_set_dev[64] = {false};
    bool& attr_set = attr_set_dev[dev & 63];
    if (!attr_set) {
      if (check_cuda(cudaFuncSetAttribute(dw3x3_tile_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024), "cudaFuncSetAttribute(dw3x3_tile_kernel)") ||
          check_cuda(cudaFuncSetAttribute(dw3x3_tile_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024), "cudaFuncSetAttribute(dw3x3_tile_kernel)"))
        return CVMK_ERR_CUDA;
      attr_set = true;
    }
  }
  if (S == 1) dw3x3_tile_kernel<1><<<(unsigned)tiles, 256, smem, s>>>(p);
  else dw3x3_tile_kernel<2><<<(unsigned)tiles, 256, smem, s>>>(p);
  return check_cuda(cudaGetLastError(), "dw3x3_tile_kernel launch");
}

int grid_sized(int64_t work, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t blocks = (work + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  const int64_t cap = (int64_t)sms * 16;
  if (blocks > cap) blocks = cap;
  else if (blocks > sms) blocks = (blocks + sms - 1) / sms * sms;
  return (int)blocks;
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_conv2d_direct(const cvmk_conv_direct_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->w || !d->y || d->groups < 1 || d->C % d->groups || d->OC % d->groups) {
    set_error("conv2d_direct: bad argument");
    return CVMK_ERR_ARG;
  }
  DirectParams p;
  memset(&p, 0, sizeof(p));
  p.x = d->x; p.w = d->w; p.y = d->y;
  p.xd = d->x_dtype; p.yd = d->y_dtype; p.narrow_x = d->narrow_x;
  p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C; p.OC = d->OC; p.KH = d->KH; p.KW = d->KW;
  p.OH = d->OH; p.OW = d->OW; p.groups = d->groups;
  p.sh = d->stride_h; p.sw = d->stride_w; p.ph = d->pad_h; p.pw = d->pad_w; p.dh = d->dil_h; p.dw = d->dil_w;
  p.total = (int64_t)d->N * d->OH * d->OW * d->OC;
  int rc = lower_chain(d->ep, &p.chain);
  if (rc != CVMK_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (d->depthwise) {
    if (d->groups != d->C || d->OC != d->C || d->C % 16 || d->x_dtype != CVMK_I8 ||
        ((uintptr_t)d->x & 15) || ((uintptr_t)d->w & 15) || ((uintptr_t)d->y & 15)) {
      set_error("conv2d_direct: depthwise path needs int8 NHWC, C %% 16 == 0, 16-byte aligned operands");
      return CVMK_ERR_UNSUPPORTED;
    }
    if (d->KH == 3 && d->KW == 3 && d->dil_h == 1 && d->dil_w == 1 && d->stride_h == d->stride_w &&
        (d->stride_h == 1 || d->stride_h == 2)) {
      const int rc_tile = try_dw3x3_tile(d, p.chain, s);
      if (rc_tile >= 0) return rc_tile;
      const int64_t work3 = (int64_t)d->N * d->OH * (d->C / 4);
      if (d->stride_h == 1) depthwise3x3_kernel<1><<<grid_sized(work3, 256), 256, 0, s>>>(p);
      else depthwise3x3_kernel<2><<<grid_sized(work3, 256), 256, 0, s>>>(p);
      return check_cuda(cudaGetLastError(), "depthwise3x3_kernel launch");
    }
    const int64_t work = (int64_t)d->N * d->OH * ((d->OW + 3) / 4) * (d->C / 16);
    depthwise_kernel<4><<<grid_sized(work, 128), 128, 0, s>>>(p);
    return check_cuda(cudaGetLastError(), "depthwise_kernel launch");
  }
  if (d->x_dtype == CVMK_I8) conv_direct_kernel<CVMK_I8><<<grid_sized(p.total, 256), 256, 0, s>>>(p);
  else conv_direct_kernel<CVMK_I32><<<grid_sized(p.total, 256), 256, 0, s>>>(p);
  return check_cuda(cudaGetLastError(), "conv_direct_kernel launch");
}

extern "C" int cvmk_im2col_pack(const cvmk_im2col_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->a || d->Kp % 16 || d->C > 255 || (d->KW - 1) * d->dil_w > 4095 ||
      (d->KH - 1) * d->dil_h > 2047 || d->KH * d->KW * d->C > d->Kp || d->KH * d->KW * d->C > 8192 ||
      ((uintptr_t)d->a & 15)) {
    set_error("im2col_pack: bad argument");
    return CVMK_ERR_ARG;
  }
  PackParams p;
  p.x = d->x; p.a = d->a;
  p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C; p.KH = d->KH; p.KW = d->KW; p.OH = d->OH; p.OW = d->OW;
  p.sh = d->stride_h; p.sw = d->stride_w; p.ph = d->pad_h; p.pw = d->pad_w; p.dh = d->dil_h; p.dw = d->dil_w;
  p.Kp = d->Kp; p.K = d->KH * d->KW * d->C;
  p.total = (int64_t)d->N * d->OH * d->OW * (d->Kp / 16);
  im2col_pack_kernel<<<grid_sized(p.total, 256), 256, p.K * sizeof(int), (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "im2col_pack_kernel launch");
}

extern "C" int cvmk_stem_pack_supported(const cvmk_stem_pack_desc* d) {
  if (!d) return 0;
  if (d->C < 1 || d->C > 4 || d->Kp % 16 || d->KH * d->KW * d->C > d->Kp) return 0;
  if ((int64_t)d->KH * d->C * (d->W + 2 * d->pad_w) > 48 * 1024) return 0;
  if ((int64_t)d->N * d->OH > INT32_MAX) return 0;
  return 1;
}

extern "C" int cvmk_stem_pack(const cvmk_stem_pack_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->a || !cvmk_stem_pack_supported(d) || ((uintptr_t)d->a & 15)) {
    set_error("stem_pack: bad argument");
    return CVMK_ERR_ARG;
  }
  StemParams p;
  p.x = d->x; p.a = d->a;
  p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C; p.KH = d->KH; p.KW = d->KW; p.OH = d->OH; p.OW = d->OW;
  p.sh = d->stride_h; p.sw = d->stride_w; p.ph = d->pad_h; p.pw = d->pad_w; p.dh = d->dil_h; p.dw = d->dil_w;
  p.Kp = d->Kp; p.K = d->KH * d->KW * d->C; p.clamp = d->clamp;
  // right padding also covers the taps of the last output pixel
  const int reach = (d->OW - 1) * d->stride_w + (d->KW - 1) * d->dil_w + 1;
  p.wp = d->W + 2 * d->pad_w;
  if (reach > p.wp) p.wp = reach;
  const int smem = d->KH * d->C * p.wp;
  if (smem > 48 * 1024) { set_error("stem_pack: input rows do not fit shared memory"); return CVMK_ERR_UNSUPPORTED; }
  const int chunks = d->Kp / 16;
  int threads = chunks * 32;             // a multiple of the chunk count, see the kernel
  while (threads > 512) threads -= chunks;
  if (chunks > 512) { set_error("stem_pack: Kp too large"); return CVMK_ERR_UNSUPPORTED; }
  stem_pack_kernel<<<d->N * d->OH, threads, smem, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "stem_pack_kernel launch");
}
