// Bandwidth-bound operators: element chains, strided copies / broadcasts, reductions, max pooling.
// All are coalesced grid-stride kernels sized to the SM count; the int8 paths move 16 bytes per
// thread per access.
#include <cuda_runtime.h>
#include <string.h>
#include "common.cuh"

namespace cvmk {
namespace {

int sm_count() {
  static thread_local int cached_dev = -1, cached = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return cached;
}

// Grid for a grid-stride loop over `work` items with `threads` per block: whole multiples of the
// SM count, at most 8 blocks per SM.
int grid_for(int64_t work, int threads) {
  const int sms = sm_count();
  int64_t blocks = (work + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  const int64_t cap = (int64_t)sms * 8;
  if (blocks > cap) blocks = cap;
  else if (blocks > sms) blocks = (blocks + sms - 1) / sms * sms;
  return (int)blocks;
}

__device__ __forceinline__ void unpack16(const int4& raw, int32_t* v) {
  const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 16; ++k) v[k] = (int32_t)(int8_t)(w[k >> 2] >> ((k & 3) * 8));
}
__device__ __forceinline__ int4 pack16(const int32_t* v) {
  int4 r;
  r.x = (int)pack4(v[0], v[1], v[2], v[3]);
  r.y = (int)pack4(v[4], v[5], v[6], v[7]);
  r.z = (int)pack4(v[8], v[9], v[10], v[11]);
  r.w = (int)pack4(v[12], v[13], v[14], v[15]);
  return r;
}

// y = chain(x), 16 elements per thread per step.
template <int XD, int YD>
__global__ void __launch_bounds__(256) elemwise_kernel(const void* __restrict__ x, void* __restrict__ y,
                                                       int64_t n, const __grid_constant__ DevChain chain) {
  const int64_t nvec = n / 16;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    int32_t v[16];
    if (XD == CVMK_I8) {
      unpack16(__ldg(reinterpret_cast<const int4*>(x) + i), v);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        int4 r = __ldg(reinterpret_cast<const int4*>(x) + i * 4 + q);
        v[4 * q] = r.x; v[4 * q + 1] = r.y; v[4 * q + 2] = r.z; v[4 * q + 3] = r.w;
      }
    }
    apply_chain<16>(chain, v, (size_t)i * 16, 0, 0);
    if (YD == CVMK_I8) {
      reinterpret_cast<int4*>(y)[i] = pack16(v);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        reinterpret_cast<int4*>(y)[i * 4 + q] = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
  }
  // tail (n % 16 elements)
  const int64_t tail0 = nvec * 16;
  for (int64_t i = tail0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int32_t v[1];
    v[0] = XD == CVMK_I8 ? (int32_t) reinterpret_cast<const int8_t*>(x)[i] : reinterpret_cast<const int32_t*>(x)[i];
    apply_chain<1>(chain, v, (size_t)i, 0, 0);
    if (YD == CVMK_I8) reinterpret_cast<int8_t*>(y)[i] = (int8_t)v[0];
    else reinterpret_cast<int32_t*>(y)[i] = v[0];
  }
}

// Division of a non-negative 31-bit number by a divisor fixed at launch: q = umulhi(n, mul) >> shr
// (mul = ceil(2^(31 + ceil(log2 d)) / d)); d = 1 is flagged by mul = 0.  The index split of the
// strided kernels is one such division per dimension and element; the 64-bit hardware-emulated
// divisions it replaces cost more than the copy itself.
struct IdxDiv { uint32_t mul, shr; };
__device__ __forceinline__ uint32_t idx_div(uint32_t n, const IdxDiv& d) { return d.mul ? __umulhi(n, d.mul) >> d.shr : n; }
static IdxDiv make_idx_div(int64_t d) {
  IdxDiv f = {0, 0};
  if (d <= 1) return f;
  int lg = 0;
  while ((1LL << lg) < d) ++lg;
  f.mul = (uint32_t)((((uint64_t)1 << (31 + lg)) + (uint64_t)d - 1) / (uint64_t)d);
  f.shr = (uint32_t)(lg - 1);
  return f;
}

struct StridedParams {
  int op, ndim;
  int64_t total;
  int64_t extent[6];
  IdxDiv fd[6];
  int idx32;          // total < 2^31: the index is split with 32-bit multiply-shifts
  int64_t as[6], bs[6], ys[6];
  const void* a; const void* b; void* y;
  int ad, bd, yd;
  int64_t a_off, b_off, y_off;
  DevChain chain;
};

__device__ __forceinline__ int32_t load_elem(const void* p, int dt, int64_t off) {
  return dt == CVMK_I8 ? (int32_t) reinterpret_cast<const int8_t*>(p)[off]
                       : reinterpret_cast<const int32_t*>(p)[off];
}

__global__ void __launch_bounds__(256) strided_kernel(const __grid_constant__ StridedParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t ao = p.a_off, bo = p.b_off, yo = p.y_off;
    if (p.idx32) {
      uint32_t rem = (uint32_t)i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const uint32_t q = idx_div(rem, p.fd[k]);
          const int64_t c = (int64_t)(rem - q * (uint32_t)p.extent[k]);
          rem = q;
          ao += c * p.as[k];
          bo += c * p.bs[k];
          yo += c * p.ys[k];
        }
      }
    } else {
      int64_t rem = i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const int64_t c = rem % p.extent[k];
          rem /= p.extent[k];
          ao += c * p.as[k];
          bo += c * p.bs[k];
          yo += c * p.ys[k];
        }
      }
    }
    int32_t v[1];
    const int32_t a = load_elem(p.a, p.ad, ao);
    if (p.op == CVMK_OP_COPY) {
      v[0] = a;
    } else {
      const int32_t b = load_elem(p.b, p.bd, bo);
      switch (p.op) {
        case CVMK_OP_ADD: v[0] = (int32_t)((uint32_t)a + (uint32_t)b); break;
        case CVMK_OP_SUB: v[0] = (int32_t)((uint32_t)a - (uint32_t)b); break;
        case CVMK_OP_MUL: v[0] = (int32_t)((uint32_t)a * (uint32_t)b); break;
        case CVMK_OP_MAX: v[0] = a > b ? a : b; break;
        case CVMK_OP_DIV: v[0] = b == 0 ? 0 : (b == -1 ? (int32_t)(0u - (uint32_t)a) : a / b); break;
        default: v[0] = a > b ? 1 : 0; break;
      }
    }
    apply_chain<1>(p.chain, v, (size_t)yo, 0, 0);
    if (p.yd == CVMK_I8) reinterpret_cast<int8_t*>(p.y)[yo] = (int8_t)v[0];
    else reinterpret_cast<int32_t*>(p.y)[yo] = v[0];
  }
}

// COPY fast path: the innermost extent is contiguous in a and y, dtypes equal, everything 16-byte
// aligned: move 16-byte vectors.
struct StridedVecParams {
  int ndim;
  int idx32;
  int64_t total_vec;
  int64_t extent[6];   // innermost extent counted in vectors
  IdxDiv fd[6];
  int64_t as[6], ys[6];  // strides in vectors (innermost = 1)
  const int4* a; int4* y;
};
__device__ __forceinline__ void strided_vec_body(const StridedVecParams& p, int64_t first, int64_t stride) {
  for (int64_t i = first; i < p.total_vec; i += stride) {
    int64_t ao = 0, yo = 0;
    if (p.idx32) {
      uint32_t rem = (uint32_t)i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const uint32_t q = idx_div(rem, p.fd[k]);
          const int64_t c = (int64_t)(rem - q * (uint32_t)p.extent[k]);
          rem = q;
          ao += c * p.as[k];
          yo += c * p.ys[k];
        }
      }
    } else {
      int64_t rem = i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const int64_t c = rem % p.extent[k];
          rem /= p.extent[k];
          ao += c * p.as[k];
          yo += c * p.ys[k];
        }
      }
    }
    p.y[yo] = __ldg(p.a + ao);
  }
}
__global__ void __launch_bounds__(256) strided_vec_kernel(const __grid_constant__ StridedVecParams p) {
  strided_vec_body(p, (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
}
// Several element-wise copies in one launch, any strides and either element type on either side.
struct StridedCopyItem {
  int ndim, idx32;
  int64_t total;
  int64_t extent[6];
  IdxDiv fd[6];
  int64_t as[6], ys[6];
  const void* a; void* y;
  int ad, yd;
  int64_t a_off, y_off;
};
constexpr int STRIDED_BATCH_MAX = 8;
struct StridedCopyBatch { StridedCopyItem item[STRIDED_BATCH_MAX]; };
__global__ void __launch_bounds__(256) strided_copy_batch_kernel(const __grid_constant__ StridedCopyBatch b) {
  const StridedCopyItem& p = b.item[blockIdx.y];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t ao = p.a_off, yo = p.y_off;
    if (p.idx32) {
      uint32_t rem = (uint32_t)i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const uint32_t q = idx_div(rem, p.fd[k]);
          const int64_t c = (int64_t)(rem - q * (uint32_t)p.extent[k]);
          rem = q;
          ao += c * p.as[k];
          yo += c * p.ys[k];
        }
      }
    } else {
      int64_t rem = i;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.ndim) {
          const int64_t c = rem % p.extent[k];
          rem /= p.extent[k];
          ao += c * p.as[k];
          yo += c * p.ys[k];
        }
      }
    }
    const int32_t v = load_elem(p.a, p.ad, ao);
    if (p.yd == CVMK_I8) reinterpret_cast<int8_t*>(p.y)[yo] = (int8_t)v;
    else reinterpret_cast<int32_t*>(p.y)[yo] = v;
  }
}
// Several vector copies in one launch (the inputs of a concatenate): blockIdx.y picks the copy.
struct StridedVecBatch { StridedVecParams item[STRIDED_BATCH_MAX]; };
__global__ void __launch_bounds__(256) strided_vec_batch_kernel(const __grid_constant__ StridedVecBatch b) {
  strided_vec_body(b.item[blockIdx.y], (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
}

struct ReduceParams {
  int is_max, init_zero, n_keep, n_red;
  int64_t total, red_total;
  int64_t ke[6], ks[6], re[6], rs[6];
  const void* x; void* y;
  int xd, yd;
  DevChain chain;
};
__global__ void __launch_bounds__(256) reduce_kernel(const __grid_constant__ ReduceParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t rem = i, base = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < p.n_keep) {
        base += (rem % p.ke[k]) * p.ks[k];
        rem /= p.ke[k];
      }
    }
    int32_t acc = p.init_zero ? 0 : load_elem(p.x, p.xd, base);
    for (int64_t r = p.init_zero ? 0 : 1; r < p.red_total; ++r) {
      int64_t rr = r, off = base;
#pragma unroll
      for (int k = 5; k >= 0; --k) {
        if (k < p.n_red) {
          off += (rr % p.re[k]) * p.rs[k];
          rr /= p.re[k];
        }
      }
      const int32_t val = load_elem(p.x, p.xd, off);
      if (p.is_max) acc = acc < val ? val : acc;
      else acc = (int32_t)((uint32_t)acc + (uint32_t)val);
    }
    int32_t v[1] = {acc};
    apply_chain<1>(p.chain, v, (size_t)i, 0, 0);
    if (p.yd == CVMK_I8) reinterpret_cast<int8_t*>(p.y)[i] = (int8_t)v[0];
    else reinterpret_cast<int32_t*>(p.y)[i] = v[0];
  }
}

// max_pool2d, NHWC.  int8: one thread owns 16 channels of one output pixel (vmax4 on packed
// bytes); int32: 4 channels.  Taps outside the image are skipped, which equals a max with INT_MIN
// because the reference guarantees at least one tap inside (pad < pool size).
// One thread per 16 neighbouring outputs (innermost kept extent, counted in groups of 16 here).
__global__ void __launch_bounds__(128) reduce_vec16_kernel(const __grid_constant__ ReduceParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t rem = i, base = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < p.n_keep) {
        const int64_t c = rem % p.ke[k];
        rem /= p.ke[k];
        base += c * (k == p.n_keep - 1 ? 16 : p.ks[k]);
      }
    }
    const int8_t* src = reinterpret_cast<const int8_t*>(p.x) + base;
    int32_t acc[16];
    int64_t r0 = 0;
    if (p.init_zero) {
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = 0;
    } else {
      const int4 raw = __ldg(reinterpret_cast<const int4*>(src));
      const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = (int32_t)(int8_t)(w[j >> 2] >> ((j & 3) * 8));
      r0 = 1;
    }
#pragma unroll 4
    for (int64_t r = r0; r < p.red_total; ++r) {
      const int4 raw = __ldg(reinterpret_cast<const int4*>(src + r * p.rs[0]));
      const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int32_t val = (int32_t)(int8_t)(w[j >> 2] >> ((j & 3) * 8));
        if (p.is_max) acc[j] = acc[j] < val ? val : acc[j];
        else acc[j] = (int32_t)((uint32_t)acc[j] + (uint32_t)val);
      }
    }
    apply_chain<16>(p.chain, acc, (size_t)i * 16, 0, 0);
    if (p.yd == CVMK_I8) {
      reinterpret_cast<int4*>(p.y)[i] = pack16(acc);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        reinterpret_cast<int4*>(p.y)[i * 4 + q] = make_int4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    }
  }
}

struct PoolParams {
  const void* x; void* y;
  int N, H, W, C, OH, OW, KH, KW, sh, sw, ph, pw;
  int64_t total;  // output vectors
  int cvec;       // vectors per pixel
  IdxDiv d_cvec, d_ow, d_oh;   // multiply-shift forms of the three divisions of the index split
};
// IDX32: the output has fewer than 2^31 vectors, so the index split runs on 32-bit divisions (the
// 64-bit ones cost more instructions than the nine taps of a 3x3 window).
template <int DT, bool IDX32>
__global__ void __launch_bounds__(256) pool_vec_kernel(const __grid_constant__ PoolParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int cv, ox, oy, n;
    if (IDX32) {
      const uint32_t u = (uint32_t)i;
      const uint32_t pix = idx_div(u, p.d_cvec);
      cv = (int)(u - pix * (uint32_t)p.cvec);
      const uint32_t r1 = idx_div(pix, p.d_ow);
      ox = (int)(pix - r1 * (uint32_t)p.OW);
      const uint32_t r2 = idx_div(r1, p.d_oh);
      oy = (int)(r1 - r2 * (uint32_t)p.OH);
      n = (int)r2;
    } else {
      cv = (int)(i % p.cvec);
      int64_t pix = i / p.cvec;
      ox = (int)(pix % p.OW); pix /= p.OW;
      oy = (int)(pix % p.OH);
      n = (int)(pix / p.OH);
    }
    // Taps outside the image are read from a clamped (valid) address and replaced by the
    // identity of max, so the loads of a window are independent of each other.  Signed bytes are
    // compared as s16x2: even and odd bytes are moved into the high byte of each half.
    int4 m;
    if (DT == CVMK_I8) {
      uint32_t me[4], mo[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) { me[q] = 0x80008000u; mo[q] = 0x80008000u; }
      for (int fy = 0; fy < p.KH; ++fy) {
        const int iy = oy * p.sh + fy - p.ph;
        const bool row_ok = iy >= 0 && iy < p.H;
        const int iyc = min(max(iy, 0), p.H - 1);
        const int4* row = reinterpret_cast<const int4*>(p.x) + ((int64_t)n * p.H + iyc) * p.W * p.cvec + cv;
#pragma unroll 3
        for (int fx = 0; fx < p.KW; ++fx) {
          const int ix = ox * p.sw + fx - p.pw;
          const bool ok = row_ok && ix >= 0 && ix < p.W;
          int4 v = __ldg(row + (int64_t)min(max(ix, 0), p.W - 1) * p.cvec);
          if (!ok) v = make_int4(0x80808080, 0x80808080, 0x80808080, 0x80808080);
          const uint32_t w[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {   // one byte permute each: (0, b0, 0, b2) and (0, b1, 0, b3)
            me[q] = __vmaxs2(me[q], __byte_perm(w[q], 0u, 0x2404));
            mo[q] = __vmaxs2(mo[q], __byte_perm(w[q], 0u, 0x3414));
          }
        }
      }
      uint32_t r[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) r[q] = __byte_perm(me[q], mo[q], 0x7351);   // (me.b1, mo.b1, me.b3, mo.b3)
      m = make_int4((int)r[0], (int)r[1], (int)r[2], (int)r[3]);
    } else {
      m = make_int4(INT32_MIN, INT32_MIN, INT32_MIN, INT32_MIN);
      for (int fy = 0; fy < p.KH; ++fy) {
        const int iy = oy * p.sh + fy - p.ph;
        const bool row_ok = iy >= 0 && iy < p.H;
        const int iyc = min(max(iy, 0), p.H - 1);
        const int4* row = reinterpret_cast<const int4*>(p.x) + ((int64_t)n * p.H + iyc) * p.W * p.cvec + cv;
#pragma unroll 3
        for (int fx = 0; fx < p.KW; ++fx) {
          const int ix = ox * p.sw + fx - p.pw;
          const bool ok = row_ok && ix >= 0 && ix < p.W;
          int4 v = __ldg(row + (int64_t)min(max(ix, 0), p.W - 1) * p.cvec);
          if (!ok) v = make_int4(INT32_MIN, INT32_MIN, INT32_MIN, INT32_MIN);
          m.x = max(m.x, v.x); m.y = max(m.y, v.y); m.z = max(m.z, v.z); m.w = max(m.w, v.w);
        }
      }
    }
    reinterpret_cast<int4*>(p.y)[i] = m;
  }
}
// Any channel count: one thread per output element.
__global__ void __launch_bounds__(256) pool_scalar_kernel(const __grid_constant__ PoolParams p, int dt) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t total = (int64_t)p.N * p.OH * p.OW * p.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % p.C);
    int64_t pix = i / p.C;
    const int ox = (int)(pix % p.OW); pix /= p.OW;
    const int oy = (int)(pix % p.OH);
    const int n = (int)(pix / p.OH);
    int32_t m = INT32_MIN;
    for (int fy = 0; fy < p.KH; ++fy) {
      const int iy = oy * p.sh + fy - p.ph;
      if (iy < 0 || iy >= p.H) continue;
      for (int fx = 0; fx < p.KW; ++fx) {
        const int ix = ox * p.sw + fx - p.pw;
        if (ix < 0 || ix >= p.W) continue;
        m = max(m, load_elem(p.x, dt, (((int64_t)n * p.H + iy) * p.W + ix) * p.C + c));
      }
    }
    if (dt == CVMK_I8) reinterpret_cast<int8_t*>(p.y)[i] = (int8_t)m;
    else reinterpret_cast<int32_t*>(p.y)[i] = m;
  }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_elemwise(const void* x, int x_dtype, void* y, int y_dtype, int64_t n,
                             const cvmk_epilogue* ep, cvmk_stream_t stream) {
  if (!x || !y || n < 0 || (x_dtype != CVMK_I8 && x_dtype != CVMK_I32) ||
      (y_dtype != CVMK_I8 && y_dtype != CVMK_I32)) {
    set_error("elemwise: bad argument");
    return CVMK_ERR_ARG;
  }
  if (n == 0) return CVMK_OK;
  DevChain chain;
  cvmk_epilogue none;
  memset(&none, 0, sizeof(none));
  int rc = lower_chain(ep ? *ep : none, &chain);
  if (rc != CVMK_OK) return rc;
  if (!aligned16(x) || !aligned16(y)) {
    // Unaligned views go through the strided kernel (one element per thread).
    cvmk_strided_desc d;
    memset(&d, 0, sizeof(d));
    d.op = CVMK_OP_COPY; d.ndim = 1; d.extent[0] = n;
    d.a = x; d.a_dtype = x_dtype; d.a_stride[0] = 1;
    d.y = y; d.y_dtype = y_dtype; d.y_stride[0] = 1;
    if (ep) d.ep = *ep;
    return cvmk_strided(&d, stream);
  }
  const int threads = 256;
  const int grid = grid_for((n + 15) / 16, threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dtype == CVMK_I8 && y_dtype == CVMK_I8) elemwise_kernel<CVMK_I8, CVMK_I8><<<grid, threads, 0, s>>>(x, y, n, chain);
  else if (x_dtype == CVMK_I8) elemwise_kernel<CVMK_I8, CVMK_I32><<<grid, threads, 0, s>>>(x, y, n, chain);
  else if (y_dtype == CVMK_I8) elemwise_kernel<CVMK_I32, CVMK_I8><<<grid, threads, 0, s>>>(x, y, n, chain);
  else elemwise_kernel<CVMK_I32, CVMK_I32><<<grid, threads, 0, s>>>(x, y, n, chain);
  return check_cuda(cudaGetLastError(), "elemwise_kernel launch");
}

// Fills `p` when `d` is a plain copy whose innermost run is contiguous and 16-byte aligned on both
// sides (the vector kernels); false otherwise.
static bool strided_as_vectors(const cvmk_strided_desc* d, int64_t total, StridedVecParams* p) {
  const int in = d->ndim - 1;
  const int es = d->a_dtype;
  const int vec = 16 / es;
  bool fast = d->op == CVMK_OP_COPY && d->ep.n == 0 && d->a_dtype == d->y_dtype &&
              d->a_stride[in] == 1 && d->y_stride[in] == 1 && d->extent[in] % vec == 0 &&
              d->a_off % vec == 0 && d->y_off % vec == 0 && aligned16(d->a) && aligned16(d->y);
  for (int k = 0; fast && k < in; ++k) fast = d->a_stride[k] % vec == 0 && d->y_stride[k] % vec == 0;
  if (!fast) return false;
  memset(p, 0, sizeof(*p));
  p->ndim = d->ndim;
  p->total_vec = total / vec;
  p->idx32 = p->total_vec < ((int64_t)1 << 31);
  for (int k = 0; k < d->ndim; ++k) {
    p->extent[k] = k == in ? d->extent[k] / vec : d->extent[k];
    p->fd[k] = make_idx_div(p->extent[k]);
    p->as[k] = k == in ? 1 : d->a_stride[k] / vec;
    p->ys[k] = k == in ? 1 : d->y_stride[k] / vec;
  }
  p->a = reinterpret_cast<const int4*>(reinterpret_cast<const char*>(d->a) + d->a_off * es);
  p->y = reinterpret_cast<int4*>(reinterpret_cast<char*>(d->y) + d->y_off * es);
  return true;
}

static bool strided_total(const cvmk_strided_desc* d, int64_t* total) {
  if (!d || !d->a || !d->y || d->ndim < 1 || d->ndim > 6 || (d->op != CVMK_OP_COPY && !d->b)) {
    set_error("strided: bad argument");
    return false;
  }
  *total = 1;
  for (int k = 0; k < d->ndim; ++k) {
    if (d->extent[k] < 1) { set_error("strided: empty extent"); return false; }
    *total *= d->extent[k];
  }
  return true;
}

// `n` copies: one launch per group of STRIDED_BATCH_MAX when all of them are vector copies, or all
// plain copies without a chain; else one cvmk_strided() each.
extern "C" int cvmk_strided_batch(const cvmk_strided_desc* d, int32_t n, cvmk_stream_t stream) {
  if (!d || n < 1) { set_error("strided_batch: bad argument"); return CVMK_ERR_ARG; }
  cudaStream_t s = (cudaStream_t)stream;
  {
    // element-wise form: every input a plain copy, but not all of them whole vectors
    bool plain = n > 1, vectors = true;
    for (int32_t i = 0; i < n && plain; ++i) {
      int64_t total;
      if (!strided_total(&d[i], &total)) return CVMK_ERR_ARG;
      plain = d[i].op == CVMK_OP_COPY && d[i].ep.n == 0;
      StridedVecParams tmp;
      vectors = vectors && strided_as_vectors(&d[i], total, &tmp);
    }
    if (plain && !vectors) {
      for (int32_t first = 0; first < n; first += STRIDED_BATCH_MAX) {
        const int m = std::min<int32_t>(STRIDED_BATCH_MAX, n - first);
        StridedCopyBatch b;
        memset(&b, 0, sizeof(b));
        int64_t largest = 0;
        for (int i = 0; i < m; ++i) {
          const cvmk_strided_desc& e = d[first + i];
          StridedCopyItem& it = b.item[i];
          it.ndim = e.ndim;
          it.total = 1;
          for (int k = 0; k < e.ndim; ++k) {
            it.extent[k] = e.extent[k];
            it.fd[k] = make_idx_div(e.extent[k]);
            it.as[k] = e.a_stride[k];
            it.ys[k] = e.y_stride[k];
            it.total *= e.extent[k];
          }
          it.idx32 = it.total < ((int64_t)1 << 31);
          it.a = e.a; it.y = e.y; it.ad = e.a_dtype; it.yd = e.y_dtype; it.a_off = e.a_off; it.y_off = e.y_off;
          largest = std::max(largest, it.total);
        }
        strided_copy_batch_kernel<<<dim3((unsigned)grid_for(largest, 256), (unsigned)m), 256, 0, s>>>(b);
        if (check_cuda(cudaGetLastError(), "strided_copy_batch_kernel launch")) return CVMK_ERR_CUDA;
      }
      return CVMK_OK;
    }
  }
  StridedVecBatch b;
  bool all = true;
  for (int32_t first = 0; first < n && all; first += STRIDED_BATCH_MAX) {
    const int m = std::min<int32_t>(STRIDED_BATCH_MAX, n - first);
    int64_t largest = 0;
    for (int i = 0; i < m && all; ++i) {
      int64_t total;
      if (!strided_total(&d[first + i], &total)) return CVMK_ERR_ARG;
      all = strided_as_vectors(&d[first + i], total, &b.item[i]);
      largest = std::max(largest, b.item[i].total_vec);
    }
    if (!all) {
      if (first == 0) break;   // nothing launched yet: fall through to the one-by-one form
      for (int32_t i = first; i < n; ++i) {
        const int rc = cvmk_strided(&d[i], stream);
        if (rc != CVMK_OK) return rc;
      }
      return CVMK_OK;
    }
    strided_vec_batch_kernel<<<dim3((unsigned)grid_for(largest, 256), (unsigned)m), 256, 0, s>>>(b);
    if (check_cuda(cudaGetLastError(), "strided_vec_batch_kernel launch")) return CVMK_ERR_CUDA;
  }
  if (all) return CVMK_OK;
  for (int32_t i = 0; i < n; ++i) {
    const int rc = cvmk_strided(&d[i], stream);
    if (rc != CVMK_OK) return rc;
  }
  return CVMK_OK;
}

extern "C" int cvmk_strided(const cvmk_strided_desc* d, cvmk_stream_t stream) {
  int64_t total = 1;
  if (!strided_total(d, &total)) return CVMK_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  {
    StridedVecParams p;
    if (strided_as_vectors(d, total, &p)) {
      strided_vec_kernel<<<grid_for(p.total_vec, threads), threads, 0, s>>>(p);
      return check_cuda(cudaGetLastError(), "strided_vec_kernel launch");
    }
  }
  StridedParams p;
  memset(&p, 0, sizeof(p));
  p.op = d->op; p.ndim = d->ndim; p.total = total;
  p.idx32 = total < ((int64_t)1 << 31);
  for (int k = 0; k < d->ndim; ++k) {
    p.extent[k] = d->extent[k];
    p.fd[k] = make_idx_div(d->extent[k]);
    p.as[k] = d->a_stride[k]; p.bs[k] = d->b_stride[k]; p.ys[k] = d->y_stride[k];
  }
  p.a = d->a; p.b = d->b; p.y = d->y;
  p.ad = d->a_dtype; p.bd = d->b_dtype; p.yd = d->y_dtype;
  p.a_off = d->a_off; p.b_off = d->b_off; p.y_off = d->y_off;
  int rc = lower_chain(d->ep, &p.chain);
  if (rc != CVMK_OK) return rc;
  strided_kernel<<<grid_for(total, threads), threads, 0, s>>>(p);
  return check_cuda(cudaGetLastError(), "strided_kernel launch");
}

extern "C" int cvmk_reduce(const cvmk_reduce_desc* d, cvmk_stream_t stream) {
  // Channels-last reductions over the spatial extents (global pooling as sum + shift): int8 input,
  // one run of reduced elements at a constant stride, kept innermost extent contiguous -> each
  // thread owns 16 neighbouring outputs and reads 16-byte vectors.
  if (d && d->x && d->y && d->x_dtype == CVMK_I8 && d->n_keep >= 1 && d->n_keep <= 6 && d->n_red >= 1) {
    int64_t re = d->red_extent[d->n_red - 1], rs = d->red_stride[d->n_red - 1];
    bool one_run = true;
    for (int k = d->n_red - 2; k >= 0 && one_run; --k) {
      one_run = d->red_stride[k] == rs * re;
      re *= d->red_extent[k];
    }
    const int in = d->n_keep - 1;
    bool ok = one_run && d->keep_stride[in] == 1 && d->keep_extent[in] % 16 == 0 && rs % 16 == 0 && aligned16(d->x) &&
              (d->y_dtype == CVMK_I32 ? aligned16(d->y) : aligned16(d->y));
    for (int k = 0; ok && k < in; ++k) ok = d->keep_stride[k] % 16 == 0;
    if (ok) {
      ReduceParams p;
      memset(&p, 0, sizeof(p));
      p.is_max = d->is_max; p.init_zero = d->init_zero; p.n_keep = d->n_keep; p.n_red = 1;
      p.total = 1;
      for (int k = 0; k < d->n_keep; ++k) { p.ke[k] = d->keep_extent[k]; p.ks[k] = d->keep_stride[k]; p.total *= p.ke[k]; }
      p.ke[in] /= 16;
      p.total /= 16;
      p.re[0] = re; p.rs[0] = rs; p.red_total = re;
      p.x = d->x; p.y = d->y; p.xd = d->x_dtype; p.yd = d->y_dtype;
      int rc = lower_chain(d->ep, &p.chain);
      if (rc != CVMK_OK) return rc;
      reduce_vec16_kernel<<<grid_for(p.total, 128), 128, 0, (cudaStream_t)stream>>>(p);
      return check_cuda(cudaGetLastError(), "reduce_vec16_kernel launch");
    }
  }
  if (!d || !d->x || !d->y || d->n_keep < 0 || d->n_keep > 6 || d->n_red < 0 || d->n_red > 6) {
    set_error("reduce: bad argument");
    return CVMK_ERR_ARG;
  }
  ReduceParams p;
  memset(&p, 0, sizeof(p));
  p.is_max = d->is_max; p.init_zero = d->init_zero; p.n_keep = d->n_keep; p.n_red = d->n_red;
  p.total = 1; p.red_total = 1;
  for (int k = 0; k < d->n_keep; ++k) { p.ke[k] = d->keep_extent[k]; p.ks[k] = d->keep_stride[k]; p.total *= p.ke[k]; }
  for (int k = 0; k < d->n_red; ++k) { p.re[k] = d->red_extent[k]; p.rs[k] = d->red_stride[k]; p.red_total *= p.re[k]; }
  p.x = d->x; p.y = d->y; p.xd = d->x_dtype; p.yd = d->y_dtype;
  int rc = lower_chain(d->ep, &p.chain);
  if (rc != CVMK_OK) return rc;
  const int threads = 256;
  reduce_kernel<<<grid_for(p.total, threads), threads, 0, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "reduce_kernel launch");
}

// int8 max pooling with a 3 x 3 or 2 x 2 window whose every position holds at least one pixel of
// the image in each direction (padding smaller than the window, the usual case).  Taps outside
// the image are then read from the nearest pixel inside it, which lies in the same window, so
// the maximum does not change and no tap needs a select.  The signed bytes of a 16-byte channel
// vector are compared as s16x2 (even and odd bytes moved into the high byte of each half), three
// values per instruction: a row of taps is one __vimax3_s16x2, the rows another.
template <int K, bool IDX32>
__global__ void __launch_bounds__(256) pool_window_kernel(const __grid_constant__ PoolParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int cv, ox, oy, n;
    if (IDX32) {
      const uint32_t u = (uint32_t)i;
      const uint32_t pix = idx_div(u, p.d_cvec);
      cv = (int)(u - pix * (uint32_t)p.cvec);
      const uint32_t r1 = idx_div(pix, p.d_ow);
      ox = (int)(pix - r1 * (uint32_t)p.OW);
      const uint32_t r2 = idx_div(r1, p.d_oh);
      oy = (int)(r1 - r2 * (uint32_t)p.OH);
      n = (int)r2;
    } else {
      cv = (int)(i % p.cvec);
      int64_t pix = i / p.cvec;
      ox = (int)(pix % p.OW); pix /= p.OW;
      oy = (int)(pix % p.OH);
      n = (int)(pix / p.OH);
    }
    int xo[K];   // vector offsets of the window's columns inside a row
#pragma unroll
    for (int fx = 0; fx < K; ++fx) xo[fx] = min(max(ox * p.sw + fx - p.pw, 0), p.W - 1) * p.cvec;
    uint32_t re[K][4], ro[K][4];
#pragma unroll
    for (int fy = 0; fy < K; ++fy) {
      const int iy = min(max(oy * p.sh + fy - p.ph, 0), p.H - 1);
      const int4* row = reinterpret_cast<const int4*>(p.x) + ((int64_t)n * p.H + iy) * p.W * p.cvec + cv;
      uint32_t te[K][4], to[K][4];
#pragma unroll
      for (int fx = 0; fx < K; ++fx) {
        const int4 v = __ldg(row + xo[fx]);
        const uint32_t w[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {   // (0, b0, 0, b2) and (0, b1, 0, b3)
          te[fx][q] = __byte_perm(w[q], 0u, 0x2404);
          to[fx][q] = __byte_perm(w[q], 0u, 0x3414);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (K == 3) {
          re[fy][q] = __vimax3_s16x2(te[0][q], te[1][q], te[2][q]);
          ro[fy][q] = __vimax3_s16x2(to[0][q], to[1][q], to[2][q]);
        } else {
          re[fy][q] = __vmaxs2(te[0][q], te[1][q]);
          ro[fy][q] = __vmaxs2(to[0][q], to[1][q]);
        }
      }
    }
    uint32_t r[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t me = K == 3 ? __vimax3_s16x2(re[0][q], re[1][q], re[2][q]) : __vmaxs2(re[0][q], re[1][q]);
      const uint32_t mo = K == 3 ? __vimax3_s16x2(ro[0][q], ro[1][q], ro[2][q]) : __vmaxs2(ro[0][q], ro[1][q]);
      r[q] = __byte_perm(me, mo, 0x7351);   // (me.b1, mo.b1, me.b3, mo.b3)
    }
    reinterpret_cast<int4*>(p.y)[i] = make_int4((int)r[0], (int)r[1], (int)r[2], (int)r[3]);
  }
}

extern "C" int cvmk_max_pool2d(const cvmk_pool_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->y || (d->dtype != CVMK_I8 && d->dtype != CVMK_I32)) {
    set_error("max_pool2d: bad argument");
    return CVMK_ERR_ARG;
  }
  PoolParams p;
  p.x = d->x; p.y = d->y;
  p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C; p.OH = d->OH; p.OW = d->OW;
  p.KH = d->KH; p.KW = d->KW; p.sh = d->stride_h; p.sw = d->stride_w; p.ph = d->pad_h; p.pw = d->pad_w;
  const int vec = 16 / d->dtype;
  const int threads = 256;
  cudaStream_t s = (cudaStream_t)stream;
  if (d->C % vec == 0 && aligned16(d->x) && aligned16(d->y)) {
    p.cvec = d->C / vec;
    p.total = (int64_t)d->N * d->OH * d->OW * p.cvec;
    p.d_cvec = make_idx_div(p.cvec); p.d_ow = make_idx_div(d->OW); p.d_oh = make_idx_div(d->OH);
    const bool idx32 = p.total < ((int64_t)1 << 31);
    // every window position holds a pixel of the image in both directions
    const bool inside = d->pad_h < d->KH && d->pad_w < d->KW && (d->OH - 1) * d->stride_h - d->pad_h <= d->H - 1 &&
                        (d->OW - 1) * d->stride_w - d->pad_w <= d->W - 1;
    const bool window = d->dtype == CVMK_I8 && d->KH == d->KW && (d->KH == 3 || d->KH == 2) && inside &&
                        !dev_env("CVM_B200_NO_POOL_WINDOW");
    if (window) {
      const int grid = grid_for(p.total, threads);
      if (d->KH == 3) {
        if (idx32) pool_window_kernel<3, true><<<grid, threads, 0, s>>>(p);
        else pool_window_kernel<3, false><<<grid, threads, 0, s>>>(p);
      } else {
        if (idx32) pool_window_kernel<2, true><<<grid, threads, 0, s>>>(p);
        else pool_window_kernel<2, false><<<grid, threads, 0, s>>>(p);
      }
    } else if (d->dtype == CVMK_I8) {
      if (idx32) pool_vec_kernel<CVMK_I8, true><<<grid_for(p.total, threads), threads, 0, s>>>(p);
      else pool_vec_kernel<CVMK_I8, false><<<grid_for(p.total, threads), threads, 0, s>>>(p);
    } else {
      if (idx32) pool_vec_kernel<CVMK_I32, true><<<grid_for(p.total, threads), threads, 0, s>>>(p);
      else pool_vec_kernel<CVMK_I32, false><<<grid_for(p.total, threads), threads, 0, s>>>(p);
    }
  } else {
    p.cvec = 0;
    p.total = (int64_t)d->N * d->OH * d->OW * d->C;
    pool_scalar_kernel<<<grid_for(p.total, threads), threads, 0, s>>>(p, d->dtype);
  }
  return check_cuda(cudaGetLastError(), "max_pool2d launch");
}
