// Index-driven transforms: take / cvm_lut (gather through an index tensor) and where (select).
// The pure index-map transforms (transpose, strided_slice, slice_like, repeat, tile) need no kernel
// of their own: the host expresses them as strided copies.
#include "common.cuh"

namespace cvmk {
namespace {

__device__ __forceinline__ int32_t load_any(const void* p, int dt, int64_t off) {
  return dt == CVMK_I8 ? (int32_t) reinterpret_cast<const int8_t*>(p)[off]
                       : __ldg(reinterpret_cast<const int32_t*>(p) + off);
}
__device__ __forceinline__ void store_any(void* p, int dt, int64_t off, int32_t v) {
  if (dt == CVMK_I8) reinterpret_cast<int8_t*>(p)[off] = (int8_t)v;
  else reinterpret_cast<int32_t*>(p)[off] = v;
}

struct TakeParams {
  const void* x; const void* idx; void* y;
  int xd, id, yd;
  int64_t count, inner, extent, total;
};

// y[o, m, n] = x[o, clamp(idx[m], 0, extent - 1), n]; one thread per output element, consecutive
// threads along n (then m), so writes are coalesced and reads are coalesced runs of `inner`.
__global__ void __launch_bounds__(256) take_kernel(const __grid_constant__ TakeParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    const int64_t n = i % p.inner, t = i / p.inner;
    const int64_t m = t % p.count, o = t / p.count;
    int64_t k = load_any(p.idx, p.id, m);
    k = k < 0 ? 0 : (k > p.extent - 1 ? p.extent - 1 : k);
    store_any(p.y, p.yd, i, load_any(p.x, p.xd, (o * p.extent + k) * p.inner + n));
  }
}

struct WhereParams {
  const void* c; const void* x; const void* y; void* out;
  int cd, xd, yd, od;
  int64_t total, inner;
};

__global__ void __launch_bounds__(256) where_kernel(const __grid_constant__ WhereParams p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    const int32_t c = load_any(p.c, p.cd, p.inner == 1 ? i : i / p.inner);
    store_any(p.out, p.od, i, c == 0 ? load_any(p.y, p.yd, i) : load_any(p.x, p.xd, i));
  }
}

// Batched matrix transpose through shared memory: y[b][c][r] = clamp(x[b][r][c]) for b < batch,
// r < rows, c < cols.  This is the NCHW <-> NHWC change of a 4-D tensor (rows = C, cols = H * W or
// the other way round).  A CTA moves a TILE x TILE block: reads and writes are both runs along
// the contiguous dimension of their side (int8: 4 bytes per thread, 64-byte runs per row of the
// tile), where the generic strided copy reads single bytes a whole plane apart.
struct TransposeParams {
  const void* x; void* y;
  int rows, cols;
  int tiles_r, tiles_c;
  int64_t total_tiles;
  int lo, hi, clamp;
};
template <typename T, int TILE>
__global__ void __launch_bounds__(256) transpose_kernel(const __grid_constant__ TransposeParams p) {
  __shared__ T tile[TILE][TILE + (sizeof(T) == 1 ? 4 : 1)];
  const T* x = reinterpret_cast<const T*>(p.x);
  T* y = reinterpret_cast<T*>(p.y);
  for (int64_t t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
    const int tc = (int)(t % p.tiles_c);
    const int64_t q = t / p.tiles_c;
    const int tr = (int)(q % p.tiles_r);
    const int64_t b = q / p.tiles_r;
    const int r0 = tr * TILE, c0 = tc * TILE;
    const T* xb = x + b * (int64_t)p.rows * p.cols;
    T* yb = y + b * (int64_t)p.rows * p.cols;
    for (int e = threadIdx.x; e < TILE * TILE; e += 256) {   // consecutive threads along cols
      const int r = e / TILE, c = e % TILE;
      if (r0 + r < p.rows && c0 + c < p.cols) {
        T v = xb[(int64_t)(r0 + r) * p.cols + c0 + c];
        if (p.clamp) v = (T)min(max((int)v, p.lo), p.hi);
        tile[r][c] = v;
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < TILE * TILE; e += 256) {   // consecutive threads along rows
      const int c = e / TILE, r = e % TILE;
      if (r0 + r < p.rows && c0 + c < p.cols) yb[(int64_t)(c0 + c) * p.rows + r0 + r] = tile[r][c];
    }
    __syncthreads();
  }
}

int grid_for(int64_t total, int threads) {
  const int64_t want = (total + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

bool dtype_ok(int dt) { return dt == CVMK_I8 || dt == CVMK_I32; }

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" int cvmk_take(const cvmk_take_desc* d, cvmk_stream_t stream) {
  if (!d || !d->x || !d->indices || !d->y || !dtype_ok(d->x_dtype) || !dtype_ok(d->idx_dtype) ||
      !dtype_ok(d->y_dtype) || d->outer < 1 || d->count < 1 || d->inner < 1 || d->extent < 1) {
    set_error("take: bad argument");
    return CVMK_ERR_ARG;
  }
  TakeParams p;
  p.x = d->x; p.idx = d->indices; p.y = d->y;
  p.xd = d->x_dtype; p.id = d->idx_dtype; p.yd = d->y_dtype;
  p.count = d->count; p.inner = d->inner; p.extent = d->extent;
  p.total = d->outer * d->count * d->inner;
  take_kernel<<<grid_for(p.total, 256), 256, 0, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "take_kernel launch");
}

extern "C" int cvmk_where(const cvmk_where_desc* d, cvmk_stream_t stream) {
  if (!d || !d->cond || !d->x || !d->y || !d->out || !dtype_ok(d->cond_dtype) || !dtype_ok(d->x_dtype) ||
      !dtype_ok(d->y_dtype) || !dtype_ok(d->out_dtype) || d->n < 1 || d->inner < 1) {
    set_error("where: bad argument");
    return CVMK_ERR_ARG;
  }
  WhereParams p;
  p.c = d->cond; p.x = d->x; p.y = d->y; p.out = d->out;
  p.cd = d->cond_dtype; p.xd = d->x_dtype; p.yd = d->y_dtype; p.od = d->out_dtype;
  p.total = d->n; p.inner = d->inner;
  where_kernel<<<grid_for(p.total, 256), 256, 0, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "where_kernel launch");
}

extern "C" int cvmk_transpose_batched(const void* x, void* y, int32_t dtype, int64_t batch, int32_t rows,
                                      int32_t cols, int32_t clamp, int32_t lo, int32_t hi, cvmk_stream_t stream) {
  if (!x || !y || !dtype_ok(dtype) || batch < 1 || rows < 1 || cols < 1) {
    set_error("transpose_batched: bad argument");
    return CVMK_ERR_ARG;
  }
  TransposeParams p;
  p.x = x; p.y = y; p.rows = rows; p.cols = cols;
  p.lo = lo; p.hi = hi; p.clamp = clamp;
  const int tile = dtype == CVMK_I8 ? 64 : 32;
  p.tiles_r = (rows + tile - 1) / tile;
  p.tiles_c = (cols + tile - 1) / tile;
  p.total_tiles = batch * p.tiles_r * p.tiles_c;
  const int64_t cap = 148 * 8;
  const int grid = (int)(p.total_tiles < cap ? p.total_tiles : cap);
  if (dtype == CVMK_I8) transpose_kernel<int8_t, 64><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else transpose_kernel<int32_t, 32><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  return check_cuda(cudaGetLastError(), "transpose_kernel launch");
}
