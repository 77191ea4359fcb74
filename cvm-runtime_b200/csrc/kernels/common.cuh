// Shared device helpers: the fused element chain and small utilities used by every kernel file.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "cvmk_kernels.h"

namespace cvmk {

// Environment variables that re-route operators or resize tiles exist for experiments only: they
// are honoured in builds made with -DCVM_B200_DEV_SWITCHES and ignored by the shipped library, whose
// results and code paths must not depend on the environment of the process that loads it.
inline const char* dev_env(const char* name) {
#ifdef CVM_B200_DEV_SWITCHES
  return getenv(name);
#else
  (void)name;
  return nullptr;
#endif
}

void set_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

// The chain as the kernels see it: host-resolved steps (RSHIFT is split into its CPU branches).
enum : int {
  K_NOP = 0, K_RELU, K_RS_ZERO, K_RS_SIGN, K_RS_NOCLIP, K_RS_CLIP, K_LSHIFT, K_CLIP,
  K_ADD_T, K_SUB_T, K_RSUB_T, K_ADD_C, K_MUL_S, K_ADD_S, K_RSUB_S, K_MAX_S, K_DIV_S, K_RDIV_S,
  K_GT_S, K_LT_S, K_ABS, K_NEG, K_PRECISION, K_RS_CLAMP
};

struct DevStep {
  int op;
  int a;
  int b;
  int dt;
  int c;   // K_RS_CLAMP: rounding addend
  int d;   // K_RS_CLAMP: shift
  const void* ptr;
};
struct DevChain {
  int n;
  int pad;
  DevStep s[CVMK_MAX_EP_STEPS];
};

// Host: translate the public chain into the device form.  Returns CVMK_OK or CVMK_ERR_ARG.
int lower_chain(const cvmk_epilogue& in, DevChain* out);

// Bit length of |x| with the reference's x = 0 -> 1 rule (cpu/ops/ops.cc:525-542).
__device__ __forceinline__ int32_t precision_of(int32_t x) {
  uint32_t a = x < 0 ? (uint32_t)(-(int64_t)x) : (uint32_t)x;
  return a == 0 ? 1 : 32 - __clz(a);
}

// Apply the chain to V consecutive elements held in registers.
//   lin0  linear index (in the output tensor's physical layout) of v[0]; v[j] is lin0 + j
//   ch0   channel index of v[0] when the V elements run along the channel axis
//         (ADD_C uses ch0 + j); pass cstride = 0 if all V elements share channel ch0.
//   pre / pre_step: when PRE, the tensor operand of step `pre_step` has already been fetched by
//         the caller (e.g. from a shared-memory tile) into pre[0..V).
template <int V, bool PRE = false>
__device__ __forceinline__ void apply_chain(const DevChain& c, int32_t (&v)[V], size_t lin0,
                                            int ch0, int cstride = 1, const int32_t* pre = nullptr,
                                            int pre_step = -1, int first_step = 0) {
  for (int si = first_step; si < c.n; ++si) {
    const DevStep st = c.s[si];
    switch (st.op) {
      case K_RELU:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = max(v[j], 0);
        break;
      case K_RS_ZERO:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = 0;
        break;
      case K_RS_SIGN:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = v[j] >> 31;
        break;
      case K_RS_NOCLIP: {
        const int sh = st.a - 1;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          int32_t t = v[j] >> sh;
          v[j] = ((int32_t)((uint32_t)t + 1u)) >> 1;  // the CPU's int32 "+1" wraps
        }
      } break;
      case K_RS_CLIP: {
        const int sh = st.a - 1;
        const int hi = st.b, lo = -st.b;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          int32_t t = v[j] >> sh;
          t = (t >> 1) + (t & 1);  // == (t + 1) >> 1 without overflow
          v[j] = min(max(t, lo), hi);
        }
      } break;
      case K_RS_CLAMP: {
        // clip(round_shift(x)) == round_shift(clamp(x, a, b)) because the rounding shift is
        // monotone; the clamp also keeps the addition below from overflowing.
        const int lo = st.a, hi = st.b, add = st.c, sh = st.d;
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = (min(max(v[j], lo), hi) + add) >> sh;
      } break;
      case K_LSHIFT: {
        const int hi = st.b, lo = -st.b;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          int32_t t = (int32_t)((uint32_t)v[j] << st.a);
          v[j] = max(min(t, hi), lo);
        }
      } break;
      case K_CLIP:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = max(min(v[j], st.b), st.a);
        break;
      case K_ADD_T:
      case K_SUB_T:
      case K_RSUB_T: {
        int32_t t[V];
        if (PRE && si == pre_step) {
#pragma unroll
          for (int j = 0; j < V; ++j) t[j] = pre[j];
        } else if (st.dt == CVMK_I8) {
          const int8_t* p = reinterpret_cast<const int8_t*>(st.ptr) + lin0;
          if (V % 16 == 0 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
            for (int q = 0; q < V / 16; ++q) {
              int4 raw = __ldg(reinterpret_cast<const int4*>(p) + q);
              const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int k = 0; k < 16; ++k) t[q * 16 + k] = (int32_t)(int8_t)(w[k >> 2] >> ((k & 3) * 8));
            }
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j) t[j] = p[j];
          }
        } else {
          const int32_t* p = reinterpret_cast<const int32_t*>(st.ptr) + lin0;
          if (V % 4 == 0 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
            for (int q = 0; q < V / 4; ++q) {
              int4 raw = __ldg(reinterpret_cast<const int4*>(p) + q);
              t[q * 4 + 0] = raw.x; t[q * 4 + 1] = raw.y; t[q * 4 + 2] = raw.z; t[q * 4 + 3] = raw.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j) t[j] = p[j];
          }
        }
        if (st.op == K_ADD_T) {
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] = v[j] + t[j];
        } else if (st.op == K_SUB_T) {
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] = v[j] - t[j];
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] = t[j] - v[j];
        }
      } break;
      case K_ADD_C: {
        const int32_t* p = reinterpret_cast<const int32_t*>(st.ptr);
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] += __ldg(p + ch0 + j * cstride);
      } break;
      case K_MUL_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = (int32_t)((uint32_t)v[j] * (uint32_t)st.a);
        break;
      case K_ADD_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = (int32_t)((uint32_t)v[j] + (uint32_t)st.a);
        break;
      case K_RSUB_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = (int32_t)((uint32_t)st.a - (uint32_t)v[j]);
        break;
      case K_MAX_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = max(v[j], st.a);
        break;
      case K_DIV_S:
#pragma unroll
        for (int j = 0; j < V; ++j)
          v[j] = st.a == 0 ? 0 : (st.a == -1 ? (int32_t)(0u - (uint32_t)v[j]) : v[j] / st.a);
        break;
      case K_RDIV_S:
#pragma unroll
        for (int j = 0; j < V; ++j)
          v[j] = v[j] == 0 ? 0 : (v[j] == -1 ? (int32_t)(0u - (uint32_t)st.a) : st.a / v[j]);
        break;
      case K_GT_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = v[j] > st.a ? 1 : 0;
        break;
      case K_LT_S:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = st.a > v[j] ? 1 : 0;
        break;
      case K_ABS:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = v[j] < 0 ? (int32_t)(0u - (uint32_t)v[j]) : v[j];
        break;
      case K_NEG:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = (int32_t)(0u - (uint32_t)v[j]);
        break;
      case K_PRECISION:
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = precision_of(v[j]);
        break;
      default:
        break;
    }
  }
}

// Pack four int32 (already within int8 range, or to be truncated like static_cast<int8_t>) into
// one 32-bit word, element 0 in the low byte.
__device__ __forceinline__ uint32_t pack4(int32_t a, int32_t b, int32_t c, int32_t d) {
  const uint32_t lo = __byte_perm((uint32_t)a, (uint32_t)b, 0x0040);  // a.b0, b.b0
  const uint32_t hi = __byte_perm((uint32_t)c, (uint32_t)d, 0x0040);  // c.b0, d.b0
  return __byte_perm(lo, hi, 0x5410);
}

}  // namespace cvmk
