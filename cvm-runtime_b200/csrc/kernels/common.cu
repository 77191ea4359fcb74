// Host-side helpers shared by the launchers: error text, CUDA status mapping, chain lowering.
#include <stdarg.h>
#include <stdio.h>
#include <stdint.h>
#include "common.cuh"

namespace cvmk {

static thread_local char g_err[512] = {0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return CVMK_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return CVMK_ERR_CUDA;
}

// Peephole simplification of a lowered chain.  Every rewrite is an identity on int32 values:
//   relu ; clip(a, b), b >= 0             ->  clip(max(a, 0), b)
//   rshift_clip(b, alpha)                 ->  rs_clamp: ((clamp(x, lo, hi) + 2^(b-1)) >> b) with
//                                             lo = -2*alpha << (b-1), hi = (2*alpha-1) << (b-1)
//   relu ; rs_clamp(lo, hi)               ->  rs_clamp(max(lo, 0), hi)
//   rs_clamp(.., alpha) ; clip(a, b) with [-alpha, alpha] inside [a, b]  ->  rs_clamp
static void simplify_chain(DevChain* c) {
  DevStep out[CVMK_MAX_EP_STEPS];
  int alpha_of[CVMK_MAX_EP_STEPS];
  int n = 0;
  for (int i = 0; i < c->n; ++i) {
    DevStep s = c->s[i];
    int alpha = -1;
    if (s.op == K_RS_CLIP) {
      const int b = s.a;
      alpha = s.b;
      const long long lo = (-2LL * alpha) * (1LL << (b - 1)), hi = (2LL * alpha - 1) * (1LL << (b - 1));
      if (lo >= INT32_MIN && hi <= INT32_MAX && hi + (1LL << (b - 1)) <= INT32_MAX) {
        s.op = K_RS_CLAMP;
        s.a = (int)lo; s.b = (int)hi; s.c = (int)(1LL << (b - 1)); s.d = b;
      }
    }
    if (n > 0 && out[n - 1].op == K_RELU) {
      if (s.op == K_CLIP && s.b >= 0) { s.a = s.a > 0 ? s.a : 0; --n; }
      else if (s.op == K_RS_CLAMP && s.b >= 0) { s.a = s.a > 0 ? s.a : 0; --n; }
    }
    if (n > 0 && out[n - 1].op == K_RS_CLAMP && s.op == K_CLIP && alpha_of[n - 1] >= 0 &&
        s.a <= -alpha_of[n - 1] && s.b >= alpha_of[n - 1])
      continue;  // the clip cannot change anything
    alpha_of[n] = alpha;
    out[n++] = s;
  }
  c->n = n;
  for (int i = 0; i < n; ++i) c->s[i] = out[i];
}

int lower_chain(const cvmk_epilogue& in, DevChain* out) {
  if (in.n < 0 || in.n > CVMK_MAX_EP_STEPS) {
    set_error("element chain has %d steps (max %d)", in.n, CVMK_MAX_EP_STEPS);
    return CVMK_ERR_ARG;
  }
  out->n = in.n;
  out->pad = 0;
  for (int i = 0; i < in.n; ++i) {
    const cvmk_ep_step& s = in.s[i];
    DevStep d;
    d.op = K_NOP; d.a = s.a; d.b = s.b; d.dt = s.ptr_dtype; d.c = 0; d.d = 0; d.ptr = s.ptr;
    switch (s.op) {
      case CVMK_EP_RELU: d.op = K_RELU; break;
      case CVMK_EP_RSHIFT: {
        // Branch order of cvm.runtime.cpu.cvm_right_shift (cpu/ops/elemwise.cc:129-147).
        const int b = s.a, p = s.b;
        if (b < 1 || b > 32 || p < 1 || p > 32) { set_error("cvm_right_shift: bad attributes"); return CVMK_ERR_ARG; }
        const int64_t alpha = ((int64_t)1 << (p - 1)) - 1;
        if (alpha == 0) d.op = K_RS_ZERO;
        else if (b >= 31) d.op = K_RS_SIGN;
        else if (p + b >= 32) { d.op = K_RS_NOCLIP; d.a = b; }
        else { d.op = K_RS_CLIP; d.a = b; d.b = (int)alpha; }
      } break;
      case CVMK_EP_LSHIFT: {
        const int b = s.a, p = s.b;
        if (b < 1 || b > 32 || p < 1 || p > 32) { set_error("cvm_left_shift: bad attributes"); return CVMK_ERR_ARG; }
        const int64_t alpha = ((int64_t)1 << (p - 1)) - 1;
        if (b >= 32) d.op = K_RS_ZERO;
        else { d.op = K_LSHIFT; d.a = b; d.b = (int)alpha; }
      } break;
      case CVMK_EP_CLIP: d.op = K_CLIP; break;
      case CVMK_EP_ADD_T: d.op = K_ADD_T; break;
      case CVMK_EP_SUB_T: d.op = K_SUB_T; break;
      case CVMK_EP_RSUB_T: d.op = K_RSUB_T; break;
      case CVMK_EP_ADD_C: d.op = K_ADD_C; break;
      case CVMK_EP_MUL_S: d.op = K_MUL_S; break;
      case CVMK_EP_ADD_S: d.op = K_ADD_S; break;
      case CVMK_EP_RSUB_S: d.op = K_RSUB_S; break;
      case CVMK_EP_MAX_S: d.op = K_MAX_S; break;
      case CVMK_EP_DIV_S: d.op = K_DIV_S; break;
      case CVMK_EP_RDIV_S: d.op = K_RDIV_S; break;
      case CVMK_EP_GT_S: d.op = K_GT_S; break;
      case CVMK_EP_LT_S: d.op = K_LT_S; break;
      case CVMK_EP_ABS: d.op = K_ABS; break;
      case CVMK_EP_NEG: d.op = K_NEG; break;
      case CVMK_EP_PRECISION: d.op = K_PRECISION; break;
      default:
        set_error("element chain: unknown step %d", s.op);
        return CVMK_ERR_ARG;
    }
    if ((d.op == K_ADD_T || d.op == K_SUB_T || d.op == K_RSUB_T || d.op == K_ADD_C) && !d.ptr) {
      set_error("element chain: step %d needs a tensor operand", i);
      return CVMK_ERR_ARG;
    }
    out->s[i] = d;
  }
  simplify_chain(out);
  return CVMK_OK;
}

}  // namespace cvmk

extern "C" const char* cvmk_last_error(void) { return cvmk::g_err; }
