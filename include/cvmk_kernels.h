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
 * conv2d, groups = 1, and dense, on the tcgen05 int8 tensor cores; grouped 3 x 3 convolutions with
 * 32 channels per group as well (`groups` below; depthwise layers, i.e. the groups > 1 branch
 * cpu/ops/ops.cc:417-425 with depthwise_conv2d :248-277, are given to it with block-diagonal weights).
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
  /* Upper bound on |sum + bias| over every output element, proven by the caller from the operand
   * ranges (0 = unknown).  When it shows that the rounding shift cannot overflow and that its
   * result fits 16 bits, the kernel requantises two elements per instruction. */
  int64_t acc_bound;
  /* 1: the ADD_C vector of the chain (the bias) is a model parameter that no kernel ever writes,
   * like w.  The kernel may then read both before the previous kernel of the stream has finished
   * (it stages the bias and warms L2 with the weights while it waits for its turn). */
  int32_t bias_static;
  /* 0 or 1: an ordinary convolution.  > 1: a grouped convolution whose groups are C / groups = OC /
   * groups = 32 channels wide, 3 x 3, stride 1, no dilation, int8 output; w is then
   * [OC, KH, KW, 32].  A depthwise layer runs this way with block-diagonal weights (channel c of a
   * group multiplies only row c of that group): an N tile is up to four groups side by side, one
   * input halo serves all of them and each group is nine M128 N32 K32 instructions into its own
   * accumulator columns.  Only the diagonal of every 32 x 32 block is used, and it is still faster
   * than the CUDA-core form for 128 channels and more, which is bound by instruction issue.
   * cvmk_conv2d_tc_supported() says whether the 8 x 16 pixel tiles fit the image. */
  int32_t groups;
  /* Grouped mode only, 0 or 1 = off.  F = 2 or 4: x and y are views of tensors F times as wide with
   * C / F channels: a pixel here is F neighbouring pixels ("sub-pixels") of the real image side by
   * side, and the 3 x 3 filter of an output channel moves in sub-pixel steps (C = OC = 128,
   * pad_w = 1 real pixel; W and OW count folded pixels).  That is how a depthwise layer over 32 or
   * 64 channels fills 128-column tiles: the group of sub-pixel a reads the 32-channel groups of
   * sub-pixels a - 1, a, a + 1, the outer ones from the neighbouring folded pixel at the edges. */
  int32_t group_fold;
  int32_t reserved1;
  /* Optional scratch for reductions cut along K (dense layers of a few rows over a long K, whose
   * few output tiles would leave most SMs idle): cvmk_conv2d_tc_workspace_bytes() says how much the
   * shape wants (0: it is not cut).  With at least that much here, K slices run as separate tiles
   * that write int32 partial sums, and a second small kernel adds them and applies the chain.
   * Sums of integers: the result is the same bit for bit. */
  void* workspace;
  int64_t workspace_bytes;
  cvmk_epilogue ep;
} cvmk_conv_desc;

typedef struct __attribute__((aligned(64))) {
  unsigned char tmap_a[128];
  unsigned char tmap_b[128];
  unsigned char tmap_y[128];   /* output tiles, when they leave through shared memory + TMA */
  unsigned char tmap_r[128];   /* int8 operand of a fused tensor add/sub, fetched with TMA */
  cvmk_conv_desc d;
  int32_t block_k;    /* bytes of K per pipeline stage: 32, 64 or 128 */
  int32_t block_n;    /* output channels per tile: 32..256 */
  int32_t a_im2col;   /* activations: 0 plain 2-D tiles, 1 im2col-mode tensor map, 2 spatial patches (4-D tiled map), 3 patches with the input halo staged once per channel block, 4 the same with the weights resident in shared memory */
  int32_t stages;
  int32_t grid;
  int32_t smem_bytes;
  int32_t tma_out;    /* 1: int8 output staged in shared memory and stored with TMA */
  int32_t res_step;   /* chain step served by tmap_r, -1 if none */
  int32_t panels, panel_bytes;  /* staging: 128-column panels per tile, bytes per panel row */
  int32_t io_bufs;    /* staging buffers per epilogue group: 1 or 2 */
  int32_t ring_bytes; /* bytes of the operand ring in shared memory */
  int32_t reserved[4];  /* [0..2] patch width / height / images (a_im2col = 2, 3), [3] (tap, channel block) units per ring stage */
  int32_t k_slices;   /* > 1: the reduction is cut into this many slices (see cvmk_conv_desc.workspace) */
  int32_t b_resident; /* 1: 1x1 layer, every CTA keeps its N tile of the weights in shared memory */
  int32_t pad_[2];
} cvmk_conv_plan;

CVMK_API int cvmk_conv2d_tc_supported(const cvmk_conv_desc* d);
CVMK_API int64_t cvmk_conv2d_tc_workspace_bytes(const cvmk_conv_desc* d);
CVMK_API int cvmk_conv2d_tc_prepare(const cvmk_conv_desc* d, cvmk_conv_plan* plan);
CVMK_API int cvmk_conv2d_tc_launch(const cvmk_conv_plan* plan, cvmk_stream_t stream);


/* ------------------------------------------------------------------------------------------------
 * y = chain(x) over n contiguous elements (any layout, x and y share it).
 * Stand-alone form of relu (ops.cc:12-26), clip / cvm_clip / cvm_right_shift / cvm_left_shift
 * (elemwise.cc:47-62, :88-193), abs / negative / cvm_precision (ops.cc:525-553, :632-642) and,
 * through the chain's *_T steps, elemwise_add / elemwise_sub (elemwise.cc:8-45).
 * ---------------------------------------------------------------------------------------------- */
CVMK_API int cvmk_elemwise(const void* x, int x_dtype, void* y, int y_dtype, int64_t n,
                           const cvmk_epilogue* ep, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Strided element kernel: for every point c of an iteration space of up to 6 extents,
 *     y[y_off + sum c_k * ys_k] = chain( op( a[a_off + sum c_k * as_k], b[b_off + sum c_k * bs_k] ) )
 * Strides are in elements; a stride of 0 broadcasts.  With op = COPY (b unused) it is the layout
 * converter (NCHW <-> NHWC, int8 <-> int32), flatten / reshape of a channels-last tensor
 * (elemwise.cc:64-86), concatenate (ops.cc:567-602; one call per input), upsampling
 * (ops.cc:958-989; iteration space N,H,s,W,s,C) and expand_dims / squeeze.  With a binary op it
 * is broadcast_add/sub/mul/max/div/greater (cpu/ops/broadcast.cc:6-124).
 * ---------------------------------------------------------------------------------------------- */
enum { CVMK_OP_COPY = 0, CVMK_OP_ADD, CVMK_OP_SUB, CVMK_OP_MUL, CVMK_OP_MAX, CVMK_OP_DIV, CVMK_OP_GREATER };
typedef struct {
  int32_t op;
  int32_t ndim;
  int64_t extent[6];
  const void* a; int32_t a_dtype; int32_t pad0; int64_t a_off; int64_t a_stride[6];
  const void* b; int32_t b_dtype; int32_t pad1; int64_t b_off; int64_t b_stride[6];
  void* y;       int32_t y_dtype; int32_t pad2; int64_t y_off; int64_t y_stride[6];
  cvmk_epilogue ep;
} cvmk_strided_desc;
CVMK_API int cvmk_strided(const cvmk_strided_desc* d, cvmk_stream_t stream);
/* n strided copies at once (the inputs of a concatenate): one launch when every one of them moves
 * whole 16-byte vectors, otherwise one cvmk_strided() each. */
CVMK_API int cvmk_strided_batch(const cvmk_strided_desc* d, int32_t n, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * sum / max reduce (cpu/ops/reduce.cc:34-140).  Output point c (up to 6 kept extents, strides into
 * x given per extent) reduces over up to 6 reduced extents.  init_zero = 1 reproduces the
 * reduce-over-everything path, whose accumulator starts at 0 (reduce.cc:41-47); otherwise the
 * accumulator starts at the first element (reduce.cc:90-100).  y is written contiguously.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t is_max;
  int32_t init_zero;
  int32_t n_keep, n_red;
  int64_t keep_extent[6], keep_stride[6];
  int64_t red_extent[6], red_stride[6];
  const void* x; int32_t x_dtype; int32_t pad0;
  void* y;       int32_t y_dtype; int32_t pad1;
  cvmk_epilogue ep;
} cvmk_reduce_desc;
CVMK_API int cvmk_reduce(const cvmk_reduce_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * max_pool2d on channels-last tensors (cpu/ops/ops.cc:466-523): window max, taps outside the image
 * count as INT32_MIN.  x: NHWC [N,H,W,C], y: NHWC [N,OH,OW,C], same dtype for both.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x; void* y; int32_t dtype;
  int32_t N, H, W, C, OH, OW, KH, KW, stride_h, stride_w, pad_h, pad_w;
} cvmk_pool_desc;
CVMK_API int cvmk_max_pool2d(const cvmk_pool_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * conv2d on CUDA cores for the shapes the tensor-core path does not take: groups > 1
 * (groupwise_conv2d, cpu/ops/ops.cc:333-366), depthwise, and small or odd channel counts.
 *   x : NHWC [N,H,W,C], int8 or int32 (x_dtype)
 *   w : int8 [OC, KH, KW, C/groups]   (depthwise = 1: int8 [KH, KW, C])
 *   y : NHWC [N,OH,OW,OC] int8 or int32, chain applied (ADD_C carries the bias)
 * With x_dtype = CVMK_I32 and narrow_x = 1 each input is truncated like static_cast<int8_t>
 * (ops.cc:234), which is what the groups = 1 reference path does; the grouped path multiplies the
 * int32 values as they are.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x; int32_t x_dtype; int32_t narrow_x;
  const int8_t* w;
  void* y; int32_t y_dtype;
  int32_t N, H, W, C, OC, KH, KW, OH, OW, groups;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t depthwise;
  int32_t reserved0;
  /* Upper bound on |sum + bias| over every output element (0 = unknown), as in cvmk_conv_desc: lets
   * the depthwise kernels requantise with packed 16-bit arithmetic. */
  int64_t acc_bound;
  cvmk_epilogue ep;
} cvmk_conv_direct_desc;
CVMK_API int cvmk_conv2d_direct(const cvmk_conv_direct_desc* d, cvmk_stream_t stream);


/* ------------------------------------------------------------------------------------------------
 * Patch gather for convolutions whose channel count is not a multiple of 32 (image stems):
 * writes A[m][k], m = (n, oy, ox) row-major, k = (fy, fx, c) row-major, zero outside the image
 * and for K <= k < Kp, so that the convolution becomes a [M, Kp] x [OC, Kp]^T product for the
 * tensor-core kernel (weights padded the same way).  Same values as im2col_cpu
 * (cpu/ops/ops.cc:204-246), transposed.  x: int8 NHWC; a: int8 [N*OH*OW, Kp], Kp % 16 == 0.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const int8_t* x;
  int8_t* a;
  int32_t N, H, W, C, KH, KW, OH, OW;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t Kp;
} cvmk_im2col_desc;
CVMK_API int cvmk_im2col_pack(const cvmk_im2col_desc* d, cvmk_stream_t stream);

/* Same gather, reading the network input as the C-ABI delivers it: int8 NCHW [N, C, H, W] with
 * C <= 4, each value clamped to [-clamp, clamp] on the way (the input clamp of
 * CvmRuntime::SetInput, src/runtime/graph_runtime.cc:379-386).  One CTA stages the KH input rows
 * of one output row in shared memory; needs KH * C * (W + 2 * pad_w) <= 48 KB. */
typedef struct {
  const int8_t* x;
  int8_t* a;
  int32_t N, H, W, C, KH, KW, OH, OW;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t Kp;
  int32_t clamp;
} cvmk_stem_pack_desc;
CVMK_API int cvmk_stem_pack_supported(const cvmk_stem_pack_desc* d);
CVMK_API int cvmk_stem_pack(const cvmk_stem_pack_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * take (cpu/ops/ops.cc:868-945) and cvm_lut (:947-956) on row-major tensors:
 *     y[o, m, n] = x[o, clamp(indices[m], 0, extent - 1), n]
 * with o < outer (product of x's dims before the axis), m < count (elements of `indices`),
 * n < inner (product of x's dims after the axis).  Without an axis, and for cvm_lut, the tensor is
 * taken flat: outer = inner = 1 and extent = its element count.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;       int32_t x_dtype;   int32_t pad0;
  const void* indices; int32_t idx_dtype; int32_t pad1;
  void* y;             int32_t y_dtype;   int32_t pad2;
  int64_t outer, count, inner, extent;
} cvmk_take_desc;
CVMK_API int cvmk_take(const cvmk_take_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * where (cpu/ops/ops.cc:1049-1075): out[i] = cond[i / inner] == 0 ? y[i] : x[i] over n elements.
 * inner = 1 is the element-wise form (condition shaped like x); inner = elements per leading row
 * is the form with a 1-D condition over the first dimension.  x, y and out share one layout.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* cond; int32_t cond_dtype; int32_t pad0;
  const void* x;    int32_t x_dtype;    int32_t pad1;
  const void* y;    int32_t y_dtype;    int32_t pad2;
  void* out;        int32_t out_dtype;  int32_t pad3;
  int64_t n, inner;
} cvmk_where_desc;
CVMK_API int cvmk_where(const cvmk_where_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * conv2d of the network input itself when it has 1..4 channels (image stems), groups = 1
 * (cpu/ops/ops.cc:368-456 after the input clamp of graph_runtime.cc:379-386), on the tensor cores
 * without an intermediate patch matrix.  Stride 1 or 2 (the same in both directions), filters up to
 * 8 x 8, W a multiple of 16, no dilation.
 *   x : the input as the C-ABI delivers it, NCHW int8 [N, C, H, W], 16-byte aligned; values are
 *       clamped to +-clamp
 *   w : the filter in the kernel's own operand order, cvmk_conv2d_stem_weight_bytes() bytes written
 *       by cvmk_conv2d_stem_pack_weights() (a host function: OIHW int32 values in, bytes out)
 *   y : NHWC int8 [N, OH, OW, OC], OC in {32, 64, 128}; chain as for cvmk_conv2d_tc_*
 * prepare() encodes the tensor maps of x and y; the plan must be 64-byte aligned.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const int8_t* x;
  const int8_t* w;
  void* y;
  int32_t N, H, W, C;
  int32_t OC, KH, KW;
  int32_t OH, OW;
  int32_t stride_h, stride_w, pad_h, pad_w;
  int32_t clamp;
  int32_t* status;
  int64_t acc_bound;   /* as in cvmk_conv_desc */
  cvmk_epilogue ep;
} cvmk_stem_conv_desc;

typedef struct __attribute__((aligned(64))) {
  unsigned char tmap_y[128];
  unsigned char tmap_x[128];
  cvmk_stem_conv_desc d;
  int32_t grid;
  int32_t smem_bytes;
  int32_t reserved[6];
} cvmk_stem_conv_plan;

CVMK_API int cvmk_conv2d_stem_supported(const cvmk_stem_conv_desc* d);
CVMK_API int64_t cvmk_conv2d_stem_weight_bytes(const cvmk_stem_conv_desc* d);
CVMK_API int cvmk_conv2d_stem_pack_weights(const cvmk_stem_conv_desc* d, const int32_t* w_oihw, int8_t* packed);
CVMK_API int cvmk_conv2d_stem_prepare(const cvmk_stem_conv_desc* d, cvmk_stem_conv_plan* plan);
CVMK_API int cvmk_conv2d_stem_launch(const cvmk_stem_conv_plan* plan, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * get_valid_counts (cpu/ops/nms.cc:42-63): per batch keep rows with row[1] > score_threshold in
 * their original order, write their number to valid_count[b], fill the remaining rows with -1.
 * x, y: int32 [B, N, K]; valid_count: int32 [B].
 * non_max_suppression (cpu/ops/nms.cc:65-140, iou :4-40), K = 6, corner boxes at columns 2..5,
 * score at column 1, class id at column 0.  x is read only unless x_writeback is set; `scratch` needs
 * cvmk_nms_scratch_bytes(B, N) bytes (16-byte aligned) and is clobbered.
 * ---------------------------------------------------------------------------------------------- */
CVMK_API int cvmk_get_valid_counts(const int32_t* x, int32_t* y, int32_t* valid_count, int32_t B,
                                   int32_t N, int32_t K, int32_t score_threshold,
                                   cvmk_stream_t stream);
/* The same with every element of x first clamped to [-clamp, clamp] (clamp > 0): for rows that are
 * the network input itself, which the runtime clamps to the declared precision on entry
 * (src/runtime/graph_runtime.cc:379-386); clamp = 0 reads x as it is. */
CVMK_API int cvmk_get_valid_counts_clamped(const int32_t* x, int32_t* y, int32_t* valid_count, int32_t B,
                                           int32_t N, int32_t K, int32_t score_threshold, int32_t clamp,
                                           cvmk_stream_t stream);
typedef struct {
  const int32_t* x;
  const int32_t* valid_count;
  int32_t* y;
  int32_t B, N;
  int32_t max_output_size, iou_threshold, top_k, force_suppress;
  void* scratch;
  int64_t scratch_bytes;
  /* The CPU implementation overwrites, in its INPUT, the rows that fall outside the top_k best
   * scores with -1 (cpu/ops/nms.cc:93-97).  A caller whose graph reads that tensor again after the
   * operator passes x here to get the same side effect; NULL leaves x untouched. */
  int32_t* x_writeback;
} cvmk_nms_desc;
CVMK_API int64_t cvmk_nms_scratch_bytes(int32_t B, int32_t N);
CVMK_API int cvmk_non_max_suppression(const cvmk_nms_desc* d, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * non_max_suppression for callers that cannot allocate device memory.  No counterpart in the
 * reference.
 *
 * Some callers of this library are not allowed to call cudaMalloc at the point where they need
 * NMS: code running between cudaStreamBeginCapture and EndCapture, real-time loops that forbid
 * anything that may synchronise the device, and hosts that hand this library a fixed memory
 * budget and no allocator.  cvmk_non_max_suppression() asks such callers for a scratch buffer;
 * this variant brings its own: a fixed array of CVMK_NMS_STATIC_SCRATCH_BYTES that lives in the
 * library's device image (every GPU that loads the library holds it until the process exits).
 *
 *   - The caller still passes x, valid_count and y (device pointers, as for the entry point above).
 *   - Problems that need more than CVMK_NMS_STATIC_SCRATCH_BYTES of scratch
 *     (cvmk_nms_scratch_bytes(B, N) tells how much) are refused with CVMK_ERR_ARG and a message in
 *     cvmk_last_error(); nothing is launched.
 *   - The first call on each device resolves the device address of the array (one
 *     cudaGetSymbolAddress); make that first call before starting a stream capture.  No call
 *     allocates or frees memory.
 *   - x is never written: the variant has no x_writeback (the top_k side effect of the CPU operator
 *     on its input, see cvmk_nms_desc); a caller that needs it uses cvmk_non_max_suppression().
 *   - All calls on a device share the one array and it keeps whatever the previous call left.
 *     The kernel writes every scratch word before reading it, so nothing has to be cleared, but
 *     two calls whose kernels overlap on the GPU (different streams) race on it: serialise them.
 * ---------------------------------------------------------------------------------------------- */
#define CVMK_NMS_STATIC_SCRATCH_BYTES (8u << 20)
CVMK_API int cvmk_non_max_suppression_static(const int32_t* x, const int32_t* valid_count, int32_t* y,
                                             int32_t B, int32_t N, int32_t max_output_size,
                                             int32_t iou_threshold, int32_t top_k,
                                             int32_t force_suppress, cvmk_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Batched matrix transpose, y[b][c][r] = x[b][r][c] (optionally clamped to [lo, hi] on the way):
 * the NCHW <-> NHWC change of layout of a 4-D tensor (rows = C, cols = H * W, or the reverse).
 * No operator of the reference corresponds to it; the executor uses it where a tensor enters or
 * leaves the channels-last layout the convolution kernels work in.
 * ---------------------------------------------------------------------------------------------- */
CVMK_API int cvmk_transpose_batched(const void* x, void* y, int32_t dtype, int64_t batch, int32_t rows,
                                    int32_t cols, int32_t clamp, int32_t lo, int32_t hi, cvmk_stream_t stream);

/* Text of the last CUDA / argument error seen by a launcher on this thread. */
CVMK_API const char* cvmk_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CVMK_KERNELS_H_ */
