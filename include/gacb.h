/* gacb.h -- C ABI of the B200 (sm_100a) deformable-sampling kernels.
 *
 * This is the drop-in boundary for the two operators GAC dispatches as
 * generated kernels today:
 *
 *   MSDeformableAttention / gac.ms_deform_attn[_offsets]
 *   gac.deform_conv2d (MMCVModulatedDeformConv2d, DCNv2)
 *
 * Conventions (all entry points):
 *   - every tensor pointer is DEVICE memory owned by the caller, dense
 *     row-major (C-contiguous), 16-byte aligned, and no output aliases an input;
 *   - small shape tables (spatial_hw) are HOST memory, read before return;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream);
 *     work is enqueued asynchronously and the call returns without waiting;
 *   - the return value is GACB_OK or a negative gacb_status; nothing throws;
 *     gacb_last_error_string() gives the text for the calling thread;
 *   - the library is re-entrant across streams and threads unless an entry
 *     point says otherwise, and allocates device memory only where stated.
 */
#ifndef GACB_H_
#define GACB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GACB_ABI_VERSION 1

typedef enum gacb_status {
  GACB_OK = 0,
  GACB_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive extent, bad enum        */
  GACB_ERR_SHAPE_MISMATCH = -2,   /* S != sum(H_l*W_l), channel/group divisibility, ... */
  GACB_ERR_UNSUPPORTED = -3,      /* legal for the operator, outside this build's limits */
  GACB_ERR_CUDA = -4,             /* a CUDA runtime call or launch failed                */
  GACB_ERR_NO_DEVICE = -5,        /* no CUDA device / not compute capability 10.x        */
  GACB_ERR_DEVICE_TIMEOUT = -6    /* a bounded in-kernel wait expired (status word set)  */
} gacb_status;

typedef enum gacb_dtype { GACB_F32 = 0, GACB_BF16 = 1 } gacb_dtype;

/* How DCNv2 multiplies on the tensor cores: all modes accumulate in float32.
 * Shapes whose channel counts do not fit the tensor-core tiling run a float32
 * CUDA-core kernel instead, whatever the mode. */
typedef enum gacb_dcn_math {
  GACB_DCN_F32X3 = 0, /* fp32-faithful: both operands split into bf16 hi + lo, three products
                         (hi*hi in one accumulator, hi*lo + lo*hi in a second), summed at the end */
  GACB_DCN_TF32 = 1,  /* single TF32 product                                             */
  GACB_DCN_BF16 = 2   /* single product of operands rounded to bf16                      */
} gacb_dcn_math;

/* Flags that may be OR-ed into the `math_mode` argument of the DCNv2 / Conv2D calls that take a workspace.  They
 * let a caller that runs the same layer again and again skip work whose result is still in its workspace; the
 * library cannot check the promise, a stale workspace gives wrong results.
 *   GACB_DCN_REUSE_WEIGHTS  the workspace still holds the packed weights written by an earlier call with the same
 *                           W contents, shapes, groups and math mode (inference: weights never change);
 *   GACB_DCN_REUSE_INPUT    the workspace still holds the channel-last copy of the same X (same images
 *                           [n_begin, n_end) or pixel range, same math mode's element type) written by an earlier
 *                           call -- e.g. the DCNv2 call that follows `conv_offset` on the same input and workspace.
 * The workspace layout is [channel-last copy | packed weights]; the copy's size depends only on X and the mode's
 * element type (fp32 for F32X3/TF32, bf16 for BF16), so calls on the same X share it.  Ignored when the shape runs
 * on the CUDA-core kernel (workspace size 0). */
#define GACB_DCN_REUSE_WEIGHTS 0x100
#define GACB_DCN_REUSE_INPUT 0x200
/*   GACB_DCN_INPUT_AT_END   the workspace layout is [packed weights | ... | channel-last copy] with the copy in the
 *                           LAST input_copy_bytes of the workspace (workspace_bytes then a multiple of 256).  Two
 *                           layers that read the same X -- `conv_offset` and the DCNv2 it feeds -- can then share
 *                           one copy and still keep their own packed weights: give both calls workspaces that END
 *                           at the same address (the second one starts after the first one's weights), let the
 *                           first call make the copy and pass GACB_DCN_REUSE_INPUT to the second; with
 *                           GACB_DCN_REUSE_WEIGHTS on both, a steady-state block pays one copy and no packing.
 *                           gacb_dcnv2_workspace_parts gives the two sizes. */
#define GACB_DCN_INPUT_AT_END 0x800

int gacb_version(void);
const char *gacb_last_error_string(void);

/* Number of CUDA devices, and (major*10+minor) of `device`; negative status on failure. */
int gacb_device_count(void);
int gacb_device_capability(int device);

/* Multi-scale deformable attention, forward.
 *
 * Replaces: the NVRTC kernel generated from src/gac/targets/cuda/compiler.py:521-557
 * (`gac_kernel_<i>(const float* p0, const float* p1, const float* p2, float* out)`)
 * and the native `gac_op_<idx>` produced by native/lib/DeviceLowering.cpp:755-802;
 * semantics are those of src/gac/core/ops.py:787-851.
 *
 *   value  [B, S, H, D]        value_dtype = GACB_F32 or GACB_BF16 (storage only)
 *   loc    [B, Q, H, L, P, 2]  float32, (x, y) normalised to [0,1], align_corners=False
 *   attn   [B, Q, H, L, P]     float32
 *   out    [B, Q, H*D]         float32 (always accumulated and stored in float32)
 *   spatial_hw                 HOST int32 [L][2] = {H_l, W_l}; S must equal sum H_l*W_l
 *
 * Only queries q_begin <= q < q_end are computed (for every batch entry); other
 * rows of `out` are left untouched.  Pass 0, Q for the whole tensor.  A rank
 * that holds only its own slice of loc/attn/out passes that slice with Q = the
 * slice length.  Limits: L <= 32, P <= 64, every tensor < 2^31 elements.
 * No device memory is allocated. */
int gacb_msda_forward(const void *value, int value_dtype, const float *loc, const float *attn,
                      float *out, const int32_t *spatial_hw, int L, int B, int S, int Q, int H,
                      int D, int P, int q_begin, int q_end, void *stream);

/* Same operator with the coordinate arithmetic folded in
 * (gac.ms_deform_attn_offsets, native/lib/GraphPasses.cpp:206-271,
 * native/lib/DeviceLowering.cpp:763-775):
 *
 *   loc[i] = offsets[i] / normalizer[bcast(i)]  (+)  reference[bcast(i)]
 *
 * `offsets` has the location shape [B,Q,H,L,P,2]; `normalizer` is described by
 * norm_shape[6] (each extent 1 or the matching location extent); the quotient
 * is viewed as coord_shape[coord_rank] (same element count, rank <= 8) and
 * `reference` is described by ref_shape[coord_rank] (each extent 1 or the
 * matching coord extent).  reference_first != 0 computes reference + quotient,
 * else quotient + reference; divide and add are separately rounded. */
int gacb_msda_offsets_forward(const void *value, int value_dtype, const float *offsets,
                              const float *attn, const float *normalizer, const float *reference,
                              float *out, const int32_t *spatial_hw, int L, int B, int S, int Q,
                              int H, int D, int P, const int32_t *norm_shape,
                              const int32_t *coord_shape, const int32_t *ref_shape, int coord_rank,
                              int reference_first, int q_begin, int q_end, void *stream);

/* The two entry points above with the attention softmax folded in: `logits` [B,Q,H,L,P] are the raw scores and
 * the weights are softmax over the L*P scores of each (b,q,h), computed in the kernel as exp(x - max) / sum like
 * the reference's Softmax node (src/gac/core/ops.py:1119-1125) that feeds MSDeformableAttention in the
 * BEVFormer graphs (src/gac/models/bevformer/spatial.py:172-174, temporal.py:334-341).  The reference has no such
 * fused op; outputs equal Softmax followed by the unfused op to float32 rounding. */
int gacb_msda_logits_forward(const void *value, int value_dtype, const float *loc, const float *logits,
                             float *out, const int32_t *spatial_hw, int L, int B, int S, int Q, int H,
                             int D, int P, int q_begin, int q_end, void *stream);
int gacb_msda_offsets_logits_forward(const void *value, int value_dtype, const float *offsets,
                                     const float *logits, const float *normalizer, const float *reference,
                                     float *out, const int32_t *spatial_hw, int L, int B, int S, int Q,
                                     int H, int D, int P, const int32_t *norm_shape,
                                     const int32_t *coord_shape, const int32_t *ref_shape, int coord_rank,
                                     int reference_first, int q_begin, int q_end, void *stream);

/* Every MSDA option in one call, plus the reductions that follow the operator in BEVFormer's attention blocks.
 * (No counterpart as one op in the reference: GAC runs Mul, ReduceSum, Clamp, Div / ReduceMean as separate
 * dispatches after MSDeformableAttention: src/gac/models/bevformer/spatial.py:183-188, temporal.py:374-389.)
 *
 *   normalizer/reference   both NULL: `locations` are sampling locations; else the fused-coordinate form
 *   attention_is_logits    softmax over each row's L*P scores is formed in the kernel
 *   visibility             optional [B,Q] (the graph's [b,cam,Q,1]): rows of a (batch entry, query) whose value
 *                          is 0 are skipped -- no gathers, and `out` is not written there
 *   group, reduce_mode     batch entries n = g*group + r form groups (cameras of one sample, or the two queue
 *                          frames).  reduce_mode 0: none.  1: reduce_out[g,q,:] = sum_r visibility[n,q]*out[n,q,:]
 *                          / max(sum_r visibility[n,q], 1)  (spatial cross-attention).  2: mean over r (temporal
 *                          self-attention).  `out` [B,Q,H*D] is then the per-entry scratch the caller provides and
 *                          `reduce_out` [B/group,Q,H*D] the result; the sum runs over r in order, in float32. */
typedef struct gacb_msda_desc {
  const void *value; int value_dtype;
  const float *locations, *attention, *normalizer, *reference, *visibility;
  float *out, *reduce_out;
  const int32_t *spatial_hw, *norm_shape, *coord_shape, *ref_shape;
  int L, B, S, Q, H, D, P;
  int coord_rank, reference_first, attention_is_logits;
  int group, reduce_mode;
  int q_begin, q_end;
  void *compact_scratch;       /* optional device scratch of (B*Q + 4) * 4 bytes: with `visibility` the visible  */
  size_t compact_scratch_bytes;/* rows are compacted first so that the gather kernel runs dense CTAs over them   */
} gacb_msda_desc;
int gacb_msda_run(const gacb_msda_desc *desc, void *stream);

/* Kernel choice for one-level "query grid = texel grid" calls (temporal self-attention over the BEV map:
 * src/gac/models/bevformer/temporal.py:366-373).  When value is float32 with D = 32, there is one level with
 * Q = H_0*W_0 (query q sits on texel q), L*P <= 8 and no visibility mask, the MSDA entry points above can run
 * a kernel that stages each 16 x 16 query block's window of the value map in shared memory and gathers from there,
 * falling back to global memory, sample by sample, for samples outside the window.  Results are bit-identical to
 * the general kernel.  It is off by default: on B200 it trades L2 traffic (4.6 times less) for shared-memory
 * traffic of the same volume and ends level with the general kernel.  No reference counterpart (a tuning knob):
 *   gacb_msda_tile_path(mode)      mode 0 = never use that kernel (default), 1 = use it where it applies, any
 *                                  other value = leave unchanged; returns the previous mode.  Process-wide. */
int gacb_msda_tile_path(int mode);

/* DCNv2 modulated deformable convolution, forward.
 *
 * Replaces: the native `gac_op_<idx>` for gac.deform_conv2d produced by
 * native/lib/DeviceLowering.cpp:605-743 (operand order X, offset, mask, W[, bias]);
 * shape contract of native/lib/Dialect.cpp:272-360.
 *
 *   x      [N, Cin, H, W]              offset [N, 2*dg*Kh*Kw, Ho, Wo]  (dy, dx per kernel point)
 *   mask   [N, dg*Kh*Kw, Ho, Wo]       w      [Cout, Cin/groups, Kh, Kw]
 *   bias   [Cout] or NULL              y      [N, Cout, Ho, Wo]
 *   Ho = (H + 2*ph - dh*(Kh-1) - 1)/sh + 1, likewise Wo.
 *
 * Only images n_begin <= n < n_end are computed.  `workspace` is caller-owned
 * device scratch of at least gacb_dcnv2_workspace_bytes(...) bytes, 256-byte
 * aligned (it may be NULL when that function returns 0); its contents are
 * overwritten.
 * `status_word` is an optional device int32 that a kernel sets non-zero if one
 * of its bounded waits expires (pass NULL to ignore). */
int gacb_dcnv2_forward(const float *x, const float *offset, const float *mask, const float *w,
                       const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                       int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                       int deform_groups, int n_begin, int n_end, int math_mode, void *workspace,
                       size_t workspace_bytes, int32_t *status_word, void *stream);

/* DCNv2 with its neighbours in the R101-DCN bottleneck folded in (GAC runs them as separate dispatches: Sigmoid
 * native/lib/DeviceLowering.cpp:387-394, BatchNorm :858-866, ReLU; its own fusion pass only joins Conv+ReLU):
 *   mask_is_logits != 0   `mask` holds pre-sigmoid scores; the sigmoid is applied while sampling;
 *   bn_* != NULL          inference BatchNorm per output channel after the bias:
 *                         (v - mean) / sqrt(var + epsilon) * scale + bn_bias, in that order (all four or none);
 *   relu != 0             max(v, 0) last.
 * Everything else is as in gacb_dcnv2_forward. */
int gacb_dcnv2_fused_forward(const float *x, const float *offset, const float *mask, int mask_is_logits,
                             const float *w, const float *bias, const float *bn_scale, const float *bn_bias,
                             const float *bn_mean, const float *bn_var, float bn_epsilon, int relu, float *y,
                             int N, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int ph,
                             int pw, int dh, int dw, int groups, int deform_groups, int n_begin, int n_end,
                             int math_mode, void *workspace, size_t workspace_bytes, int32_t *status_word,
                             void *stream);

/* Plain 2-D convolution through the same kernels (offset and mask absent: integer taps, coefficient 1), for the
 * convolutions next to DCNv2 in the R101-DCN bottleneck -- above all the 3x3 `conv_offset` that produces the
 * offsets and the mask scores.  Replaces GAC's Conv2D / conv2d_relu dispatch
 * (native/lib/DeviceLowering.cpp:605-698, non-deformable branch :666-688; contract src/gac/core/ops.py:615-645):
 *   Y[n,co,oy,ox] = bias[co] + sum_{ci,kh,kw} W[co,ci,kh,kw] * X[n, g*Cin_g+ci, oy*sh - pad_top + kh*dh,
 *                                                                 ox*sw - pad_left + kw*dw],
 * taps outside the image contribute nothing; `relu != 0` applies max(v, 0) last (conv2d_relu).
 * Split output: with `y_split != NULL`, channels [0, split_at) are written to y [N, split_at, Ho, Wo] and channels
 * [split_at, Cout) to y_split [N, Cout - split_at, Ho, Wo] -- for conv_offset, split_at = 2*dg*K gives the DCNv2
 * `offset` and (pre-sigmoid) `mask` operands as two contiguous tensors without a slicing pass; pass
 * mask_is_logits = 1 to gacb_dcnv2_fused_forward to fold the sigmoid in.  Otherwise y is [N, Cout, Ho, Wo] and
 * split_at must be 0.
 * Ho = (H + pad_top + pad_bottom - dh*(Kh-1) - 1)/sh + 1, Wo likewise.  Output-channel counts that are not a
 * multiple of 16 (27 for conv_offset) run on the tensor cores with zero-padded weight rows.
 * math_mode, workspace (size from gacb_conv2d_workspace_bytes), status_word, n_begin/n_end and stream are as in
 * gacb_dcnv2_forward.  With non-finite weights a padding tap yields NaN on the tensor-core path where GAC skips
 * the multiply. */
int gacb_conv2d_forward(const float *x, const float *w, const float *bias, int relu, float *y, float *y_split,
                        int split_at, int N, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw,
                        int pad_top, int pad_left, int pad_bottom, int pad_right, int dh, int dw, int groups,
                        int n_begin, int n_end, int math_mode, void *workspace, size_t workspace_bytes,
                        int32_t *status_word, void *stream);
size_t gacb_conv2d_workspace_bytes(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw,
                                   int pad_top, int pad_left, int pad_bottom, int pad_right, int dh, int dw,
                                   int groups, int math_mode);

/* Kernel choice for plain convolutions with few output channels.  A whole-image call with groups = 1,
 * stride = dilation = 1, Cout <= 64 (32 in F32X3 mode), Cin a multiple of 64 (32 in TF32 mode) and no BatchNorm
 * runs a persistent kernel that stages each 16 x 8 pixel tile's input window in shared memory once and feeds the
 * tensor core shifted views of it, one per kernel point, instead of gathering every tap (the 27-channel convolution
 * that produces DCNv2's offsets and mask scores in an R101-DCN bottleneck; to the reference it is an ordinary
 * Conv2D, src/gac/core/ops.py:1045-1076).  Operands and products are those of the gather
 * kernel in the same math mode, with two differences: the order of the float32 additions, and in TF32 mode the
 * activations are truncated to tf32 (the tensor core reads the upper 19 bits of the float32 copy) where the gather
 * kernel rounds them to nearest.  The packed weights in the workspace have this kernel's own layout, so
 * GACB_DCN_REUSE_WEIGHTS calls must run under the mode the weights were packed under.  No reference counterpart
 * (a tuning knob):
 *   gacb_conv_window_path(mode)    mode 0 = always the gather kernel, 1 = the window kernel where it applies
 *                                  (default), any other value = leave unchanged; returns the previous mode.
 *                                  Process-wide. */
int gacb_conv_window_path(int mode);

/* gacb_dcnv2_forward restricted to the output rows [row_begin, row_end) of every image in [n_begin, n_end): the
 * unit of the balanced multi-GPU split, where 6 cameras are spread over 4 or 8 GPUs as (camera, row block) pieces.
 * Deformable offsets are unbounded, so a piece still reads its whole input image (and the workspace still holds
 * the whole images' channel-last copy); only the sampling, the product and the stores are limited to the rows.
 * Rows outside the range are not written.  Each output element is computed exactly as in the unrestricted call.
 * No reference counterpart: GAC runs one GPU. */
int gacb_dcnv2_rows_forward(const float *x, const float *offset, const float *mask, const float *w,
                            const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                            int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                            int deform_groups, int n_begin, int n_end, int row_begin, int row_end,
                            int math_mode, void *workspace, size_t workspace_bytes, int32_t *status_word,
                            void *stream);

/* gacb_dcnv2_forward restricted to the output pixels [pixel_begin, pixel_end) of the flattened (image, oy, ox)
 * space, 0 <= pixel_begin <= pixel_end <= N*Ho*Wo: the balanced multi-GPU split as ONE launch per GPU (a rank's
 * share may start and end in the middle of a camera).  The images the range touches are
 * [pixel_begin / (Ho*Wo), ceil(pixel_end / (Ho*Wo))); the workspace must hold that many images
 * (gacb_dcnv2_workspace_bytes).  Pixels outside the range are not written; each output element is computed
 * exactly as in the unrestricted call.  No reference counterpart. */
int gacb_dcnv2_pixels_forward(const float *x, const float *offset, const float *mask, const float *w,
                              const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                              int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                              int deform_groups, long long pixel_begin, long long pixel_end, int math_mode,
                              void *workspace, size_t workspace_bytes, int32_t *status_word, void *stream);

/* Scratch bytes gacb_dcnv2_forward needs for these extents (n = n_end - n_begin
 * images per call); a negative gacb_status (cast to size_t it is huge) never
 * occurs: invalid shapes return 0 and the forward call reports the error. */
size_t gacb_dcnv2_workspace_bytes(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh,
                                  int sw, int ph, int pw, int dh, int dw, int groups,
                                  int deform_groups, int math_mode);

/* The two parts of the workspace of gacb_dcnv2_forward (plain = 0; pad_bottom/pad_right = pad_top/pad_left) or
 * gacb_conv2d_forward (plain = 1) for n images: the channel-last copy of the images and the packed weights, both 0
 * when the shape runs on the CUDA-core kernel.  Their sum is what the *_workspace_bytes functions return. */
int gacb_dcnv2_workspace_parts(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int pad_top,
                               int pad_left, int pad_bottom, int pad_right, int dh, int dw, int groups,
                               int deform_groups, int math_mode, int plain, size_t *input_copy_bytes,
                               size_t *weights_bytes);

/* DCNv2 forward for callers that may not allocate device memory.  (No counterpart in the reference: GAC's
 * runners allocate whatever a dispatch needs when they build their arena.)
 *
 * Same operator, arguments and results as gacb_dcnv2_forward, but without the workspace pair: the scratch for the
 * NHWC image copy and the packed weights is an array built into the library, GACB_DCNV2_STATIC_SCRATCH_BYTES
 * (40 MiB) of global memory that every GPU which loads libgacb.so holds until the process exits.  It is meant for
 * hosts whose device memory is fully planned before the first inference -- an arena sized at model-load time, a
 * plugin slot inside somebody else's engine, a real-time loop where cudaMalloc's implicit device synchronisation
 * is not acceptable -- and who therefore cannot hand over a workspace that was not in the plan.  This entry point
 * calls no cudaMalloc/cudaFree and no allocating library routine.
 *
 * Limits and rules:
 *   - a call whose scratch need (gacb_dcnv2_workspace_bytes for n_end - n_begin images) exceeds the built-in size
 *     is rejected with GACB_ERR_UNSUPPORTED before anything is launched; split the images over several calls.
 *     BEVFormer-base's stage shapes fit with all six cameras (38.0 MB and 27.3 MB);
 *   - the first call on each device looks up the array's device address (with that device current) and keeps it
 *     for the life of the process: make that first call before any stream capture, have the device that owns
 *     `stream` current at every call (the address is looked up for the CURRENT device), and do not reset the device
 *     or destroy its primary context between calls (the remembered address would then be stale);
 *   - all calls on a device share the one array and it keeps whatever the last call left.  Nothing in it has to
 *     be zero beforehand (every byte a call reads is written by that call first), but two calls that overlap in
 *     time on the same GPU -- different streams, or different host threads -- race on it: serialise them. */
#define GACB_DCNV2_STATIC_SCRATCH_BYTES (40u << 20)
int gacb_dcnv2_forward_static(const float *x, const float *offset, const float *mask, const float *w,
                              const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                              int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                              int deform_groups, int n_begin, int n_end, int math_mode,
                              int32_t *status_word, void *stream);

/* The launch the library makes for a problem, without making it: which kernel, grid, block, dynamic shared memory
 * and how many work units (MSDA: (batch, query, head) rows; convolutions: output pixels) one thread block covers.
 * Pure host functions (no CUDA call, no device needed).  They replace the launch metadata GAC's compiler attaches to
 * its generated kernels (`KernelLaunch.grid/block`, src/gac/targets/cuda/compiler.py:40-55; `grid_size`, `block_size`
 * of a plan.json dispatch, native/lib/DeviceLowering.cpp:1641-1656): here the kernels are precompiled, so the
 * library is the one place that knows their shapes.  `sm_count` (<= 0: 148) matters because convolutions with
 * narrow channel tiles switch to a two-CTAs-per-SM shape when the grid exceeds one wave.  The MSDA answer is for
 * the plain entry points (no visibility, no fused coordinates) under the current gacb_msda_tile_path mode. */
typedef struct gacb_launch_geometry {
  int grid[3], block[3];
  size_t dynamic_smem_bytes;
  int units_per_cta;
  char kernel[64];
} gacb_launch_geometry;
int gacb_msda_launch_geometry(int value_dtype, const int32_t *spatial_hw, int L, int B, int S, int Q, int H, int D,
                              int P, int q_begin, int q_end, gacb_launch_geometry *out);
int gacb_dcnv2_launch_geometry(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int ph, int pw,
                               int dh, int dw, int groups, int deform_groups, int math_mode, int plain, int sm_count,
                               gacb_launch_geometry *out);

/* Checked build.  A library compiled with -DGACB_CHECKED=1 (general_ai_compiler_b200.build.build_native(
 * extra_flags=("-DGACB_CHECKED=1",), output=...)) range-checks every gather offset, record-table slot and output
 * index inside its kernels against the extent of the tensor or table it addresses; an index outside is counted and
 * the access is redirected to element 0 (or, for a store, dropped), so nothing faults.  *count = violations on
 * the current device since the library was loaded, *last_site = the code of the last failing site (the source
 * files list them).  Synchronises the device.  The normal build returns GACB_ERR_UNSUPPORTED.  It stands in for
 * the static guards of the reference (guarded loads as control flow, native/lib/DeviceLowering.cpp:251-286;
 * launch and lifetime validation, native/runtime/dispatch-plan.h:609-627) and for a memory checker. */
int gacb_checked_violations(unsigned int *count, unsigned int *last_site);

/* The device status word of the calls above, turned into a status.  (GAC reports a failed device step as a
 * `failed` session / a `status:"failed"` report with the failing stage: src/gac/execution/cuda.py:457-464,
 * native/runtime/cuda-run.cpp:685-703.)
 *   gacb_status_from_word   pure host function: GACB_OK for 0, else GACB_ERR_DEVICE_TIMEOUT with a message;
 *   gacb_read_status_word   copies the word from the device on `stream`, waits for the stream (so every kernel
 *                           enqueued before it has finished) and returns gacb_status_from_word of it.  After
 *                           GACB_ERR_DEVICE_TIMEOUT the outputs of the calls that shared the word are incomplete;
 *                           the context stays usable (the kernels returned by themselves) and the caller clears
 *                           the word before reusing it. */
int gacb_status_from_word(int32_t word);
int gacb_read_status_word(const int32_t *status_word, void *stream);

/* Peer-memory plumbing for the multi-GPU form (one process per GPU on one node).  No reference counterpart: GAC
 * runs one device.  Query-sharded MSDA needs the whole value tensor in each GPU's own memory; these calls let the
 * ranks bring a sharded value together with COPY-ENGINE peer copies over NVLink, which -- unlike a collective's
 * kernels -- take no SM and run beside the gather kernel.  The MSDA kernels themselves only ever read local memory.
 *   gacb_ipc_alloc    cudaMalloc `bytes` (zeroed) and export a CUDA IPC handle (GACB_IPC_HANDLE_BYTES bytes) for it
 *   gacb_ipc_open     map a buffer another process exported (peer access is enabled on demand); the result is
 *                     valid as a copy source or destination in this process
 *   gacb_ipc_close    unmap what gacb_ipc_open returned;  gacb_ipc_free  release what gacb_ipc_alloc returned
 *   gacb_copy_async   cudaMemcpyAsync between any two addresses mapped in this process, on `stream`
 *   gacb_peer_barrier enqueue on `stream` a one-block kernel that tells every rank "this rank has got here" and
 *                     waits until every rank has: peer_flags[r] = rank r's flag array (world uint32, mapped here;
 *                     peer_flags[rank] = local_flags), local_step = one device uint32 the kernel increments (so a
 *                     captured launch keeps working).  The wait is bounded (about half a second); when it runs out
 *                     *status_word is set to 2 and the kernel returns.  All ranks must enqueue the same number of
 *                     barriers.  world <= 16. */
#define GACB_IPC_HANDLE_BYTES 64
int gacb_ipc_alloc(size_t bytes, void **ptr, unsigned char *handle);
int gacb_ipc_open(const unsigned char *handle, void **ptr);
int gacb_ipc_close(void *ptr);
int gacb_ipc_free(void *ptr);
int gacb_copy_async(void *dst, const void *src, size_t bytes, void *stream);
int gacb_peer_barrier(void *const *peer_flags, void *local_flags, void *local_step, int world, int rank,
                      int32_t *status_word, void *stream);

/* float32 -> bfloat16 (round to nearest even) for the bf16-storage value variant. */
int gacb_cast_f32_to_bf16(const float *src, void *dst, size_t count, void *stream);

/* Measurement helper, no reference counterpart: launches one kernel in which every group of lanes reads
 * `loads_per_thread` pseudo-random 128-byte lines of `buffer`, sixteen loads in flight per lane, nothing else.
 * lane_bytes = 16: eight lanes share a line, four lines per warp-wide load -- the access shape of the MSDA tap
 * gather; lane_bytes = 4: the 32 lanes of a warp share a line, one line per load.  The caller times it with events
 * on `stream`; *bytes_gathered (host, optional) receives blocks * 256 * loads_per_thread * lane_bytes.  `buffer` is
 * 128-byte aligned device memory of `bytes` bytes, a power-of-two number of 128-byte lines up to 1 GiB (a few KB:
 * L1-resident; tens of MB: L2-resident), `sink` one
 * device word that is practically never written, `loads_per_thread` a positive multiple of 16. */
int gacb_gather_probe(const void *buffer, size_t bytes, int blocks, int loads_per_thread, int lane_bytes,
                      uint32_t seed, uint32_t *sink, size_t *bytes_gathered, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GACB_H_ */
