/*
 * Kernel-level C-ABI of the B200 CVM operator library (libcvm_runtime.so).
 *
 * This is the layer the graph executor dispatches to: one launcher per operator family, plain
 * pointers and sizes, a CUDA stream, an int status.  No launcher allocates device memory, throws,
 * or synchronises; every pointer is a device pointer unless stated otherwise.
 *
 * It replaces the reference's per-operator registry bodies
 *   CVM_REGISTER_GLOBAL("cvm.runtime.<device>.<op>")  (include/cvm/runtime/registry.h:129-131),
 * which the reference executor resolves in CvmRuntime::CreateCVMOp
 *   (src/runtime/graph_runtime.cc:630-698) and calls with (DLTensor*..., NodeAttrs*).
 * Each launcher below cites the CPU operator body whose results it reproduces bit for bit.
 *
 * Storage convention.  The reference keeps every tensor as int32.  Here a tensor is stored as int8
 * when its values are provably within [-127, 127] and as int32 otherwise ("dtype" arguments:
 * CVMK_I8 / CVMK_I32).  4-D activations may be held channels-last (NHWC); the launchers say
 * which layout they expect.
 */
#ifndef CVMK_KERNELS_H_
#define CVMK_KERNELS_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CVMK_API
#define CVMK_API __attribute__((visibility("default")))
#endif

typedef void* cvmk_stream_t; /* a cudaStream_t */

enum { CVMK_OK = 0, CVMK_ERR_ARG = 1, CVMK_ERR_CUDA = 2, CVMK_ERR_UNSUPPORTED = 3 };
enum { CVMK_I8 = 1, CVMK_I32 = 4 }; /* element size in bytes */

/* ------------------------------------------------------------------------------------------------
 * Fused element chain ("epilogue").  A short program of int32 -> int32 steps applied, in order, to
 * every element a kernel produces before it is stored.  It is how relu / cvm_right_shift /
 * cvm_clip / clip / elemwise_add ... that the reference runs as separate graph nodes are folded
 * into the producing kernel.  Semantics per step follow the reference CPU operators:
 *   RELU      src/runtime/cpu/ops/ops.cc:12-26
 *   RSHIFT    src/runtime/cpu/ops/elemwise.cc:114-147  (all four branches of the CPU body)
 *   LSHIFT    src/runtime/formal/ops/elemwise.cc:173-199 (the CPU body always throws)
 *   CLIP      src/runtime/cpu/ops/elemwise.cc:47-62 and :88-112
 *   ADD_T/SUB_T/RSUB_T  src/runtime/cpu/ops/elemwise.cc:20-45 (other operand read from `ptr`,
 *             same shape and physical layout as the output, dtype in `ptr_dtype`)
 *   ADD_C     per-channel int32 vector (bias), index = channel of the element
 *   MUL_S/ADD_S/... scalar forms of broadcast_* src/runtime/cpu/ops/broadcast.cc:33-36
 *   ABS/NEG/PRECISION  src/runtime/cpu/ops/ops.cc:525-553, :632-642
 * ---------------------------------------------------------------------------------------------- */
enum {
  CVMK_EP_RELU = 1,
  CVMK_EP_RSHIFT = 2,    /* a = shift_bit, b = precision */
  CVMK_EP_LSHIFT = 3,    /* a = shift_bit, b = precision */
  CVMK_EP_CLIP = 4,      /* a = min, b = max */
  CVMK_EP_ADD_T = 5,     /* x + t[i] */
  CVMK_EP_SUB_T = 6,     /* x - t[i] */
  CVMK_EP_RSUB_T = 7,    /* t[i] - x */
  CVMK_EP_ADD_C = 8,     /* x + c[channel]  (ptr: int32[channels]) */
  CVMK_EP_MUL_S = 9,     /* x * a */
  CVMK_EP_ADD_S = 10,    /* x + a */
  CVMK_EP_RSUB_S = 11,   /* a - x */
  CVMK_EP_MAX_S = 12,    /* max(x, a) */
  CVMK_EP_DIV_S = 13,    /* a == 0 ? 0 : x / a  (truncating) */
  CVMK_EP_RDIV_S = 14,   /* x == 0 ? 0 : a / x */
  CVMK_EP_GT_S = 15,     /* x > a */
  CVMK_EP_LT_S = 16,     /* a > x */
  CVMK_EP_ABS = 17,
  CVMK_EP_NEG = 18,
  CVMK_EP_PRECISION = 19
};
#define CVMK_MAX_EP_STEPS 8

typedef struct {
  int32_t op;
  int32_t a;
  int32_t b;
  int32_t ptr_dtype; /* CVMK_I8 / CVMK_I32 for *_T steps */
  const void* ptr;
} cvmk_ep_step;

typedef struct {
  int32_t n;
  int32_t reserved;
  cvmk_ep_step s[CVMK_MAX_EP_STEPS];
} cvmk_epilogue;

/* ------------------------------------------------------------------------------------------------
 * conv2d, groups = 1, and dense, on the tcgen05 int8 tensor cores.
 * Reproduces cvm.runtime.cpu.conv2d (src/runtime/cpu/ops/ops.cc:368-456: im2col_cpu :204-246 +
 * matrix_mul :148-200) and cvm.runtime.cpu.dense (:34-75) followed by the fused chain.
 *
 *   x : int8 NHWC [N, H, W, C]      (dense: N = rows, H = W = 1, C = K)
 *   w : int8 [OC, KH, KW, C]        (OIHW weights re-packed once at load; dense: [units, K])
 *   y : NHWC [N, OH, OW, OC], int8 or int32 (y_dtype)
 * Requirements: C % 32 == 0, x/w/y 16-byte aligned.  The chain's ADD_C step carries the bias.
 *
 * cvmk_conv2d_tc_prepare() encodes the TMA tensor maps into `plan` (host memory owned by the
 * caller, 64-byte aligned; it has to be repeated if x or w move).  cvmk_conv2d_tc_launch() only
 * enqueues the kernel.  `status` is a device int32 the kernel ORs a non-zero code into if one of
 * its bounded waits runs out; the host reads it after synchronising.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const int8_t* x;
  const int8_t* w;
  void* y;
  int32_t y_dtype;
  int32_t N, H, W, C;
  int32_t OC, KH, KW;
  int32_t OH, OW;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t* status;
  cvmk_epilogue ep;
} cvmk_conv_desc;

typedef struct __attribute__((aligned(64))) {
  unsigned char tmap_a[128];
  unsigned char tmap_b[128];
  cvmk_conv_desc d;
  int32_t block_k;    /* bytes of K per pipeline stage: 32, 64 or 128 */
  int32_t block_n;    /* output channels per tile: 32..256 */
  int32_t a_im2col;   /* 1: A through an im2col-mode tensor map, 0: plain 2-D tiles */
  int32_t stages;
  int32_t grid;
  int32_t smem_bytes;
  int32_t reserved[10];
} cvmk_conv_plan;

CVMK_API int cvmk_conv2d_tc_supported(const cvmk_conv_desc* d);
CVMK_API int cvmk_conv2d_tc_prepare(const cvmk_conv_desc* d, cvmk_conv_plan* plan);
CVMK_API int cvmk_conv2d_tc_launch(const cvmk_conv_plan* plan, cvmk_stream_t stream);

/* Text of the last CUDA / argument error seen by a launcher on this thread. */
CVMK_API const char* cvmk_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CVMK_KERNELS_H_ */
