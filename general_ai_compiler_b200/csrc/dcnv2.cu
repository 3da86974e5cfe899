// DCNv2 modulated deformable convolution (forward) for sm_100a.
//
// Operator semantics: native/lib/DeviceLowering.cpp:605-698 of the reference
// (deform branch :645-664) with its bilinear helper Scalar::bilinear
// (:251-286); shape contract native/lib/Dialect.cpp:272-360.
//
//   Y[n,co,oy,ox] = bias[co] + sum_{ci,kh,kw} W[co,ci,kh,kw] *
//                   ( mask[n,dg*K+k,oy,ox] * bilinear(X[n,g*Cin_g+ci]; y, x) )
//   y = oy*sh - ph + kh*dh + offset[n,2*(dg*K+k),oy,ox],  x likewise with channel +1.
//
// Two paths:
//
// 1. dcn_direct_kernel -- any legal shape.  One thread per output element walks
//    the reduction in the reference's order (input channel, kernel row, kernel
//    column) with separately rounded multiplies and adds.
//
// 2. Tensor-core implicit GEMM (tcgen05 + TMEM) when the channel counts allow:
//    D[M=pixels, N=Cout] = A[M, K'] * B[N, K']^T with K' = (channel block, kernel
//    point, channel in block): one bilinear sample position serves a run of
//    consecutive channels, and K blocks that are in flight together sample the
//    same channels at neighbouring kernel points.
//      dcn_nhwc_(vec_)kernel X (NCHW) -> X_t (NHWC, fp32 or bf16) in the caller's
//                           workspace, so a tap of one pixel is a contiguous run
//                           of channels;
//      dcn_pack_weights     W (OIHW fp32) -> per (N-tile, K-block) images of the
//                           swizzled K-major shared-memory tile: bf16 hi (+ lo),
//                           or tf32 words;
//      dcn_umma_kernel      per 128-pixel tile: the producers turn offsets and
//                           mask into a table of tap records (once per tile when
//                           it fits), then four independent producer groups of
//                           four warps gather X_t, blend, and store A tiles
//                           straight into the swizzled UMMA layout, K block kb
//                           into stage kb mod 6 of the A ring; one thread streams
//                           B tiles through a ring of two with cp.async.bulk; one
//                           thread issues tcgen05.mma into TMEM accumulators; the
//                           producers then read TMEM back, apply bias / BatchNorm /
//                           ReLU and store NCHW.
//    The same kernels run plain convolutions (no offset/mask operands: one integer
//    tap per sample) for the layers next to DCNv2, above all conv_offset.
//    Math modes: F32X3 = both operands split into bf16 hi + lo, three products;
//    TF32 = one product of tf32-rounded operands; BF16 = one product of
//    bf16-rounded operands.  All accumulate in float32 in TMEM.  The tensor
//    core's accumulator update is not correctly rounded, so the error of a long
//    reduction grows with the number of tcgen05.mma steps that touch one
//    accumulator (measured: three tf32 products per 8-wide step were LESS
//    accurate than three bf16 products per 16-wide step).  F32X3 therefore uses
//    bf16 pairs (fewest steps) and keeps the two small cross products
//    (lo*hi, hi*lo) in a second TMEM accumulator that the epilogue adds.
//    Every mbarrier wait is bounded: on expiry the kernel raises a shared abort
//    flag, sets the caller's status word, drains what it issued, frees TMEM and
//    returns.
#include <cuda.h>   // CUtensorMap and its enums only; the encoder is looked up through the runtime

#include <algorithm>
#include <atomic>
#include <mutex>
#include <type_traits>

#include "gacb_common.cuh"

namespace gacb {
namespace {

GACB_CHECK_RECORD;
// Sites of the checked build in this file: 11 tap-record table, 12 gathers from the channel-last copy,
// 13 offset / mask operands, 14 output elements, 15 packed-weight stages.

// Scratch of gacb_dcnv2_forward_static: lives in the module's global memory on every GPU that loads the library,
// from load until the process exits.  Host code must not pass this name to a kernel (on the host it is only a
// stand-in for the symbol); the device address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_dcn_static_scratch[GACB_DCNV2_STATIC_SCRATCH_BYTES];

struct DcnArgs {
  const float *x, *offset, *mask, *w, *bias;
  float *y;
  int N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups, dgroups, Ho, Wo;
  int n_begin, n_end;
  int row_begin, row_end;   // output rows [row_begin, row_end) of every image of the call; the whole plane by default
  // The call computes m_count "selected pixels" starting at number m_first, where selected pixel f is pixel
  // row_begin*Wo + f % plane_sel of image n_begin + f / plane_sel, plane_sel = (row_end - row_begin) * Wo.
  int m_first, m_count;
  // optional neighbours of the convolution in the R101-DCN bottleneck, folded in (all off when zero/NULL):
  int mask_is_logits;                                 // mask operand holds pre-sigmoid scores
  const float *bn_scale, *bn_bias, *bn_mean, *bn_var;  // inference BatchNorm over output channels
  float bn_eps;
  int relu;
  // Plain convolution (offset == NULL: integer taps, no mask) may split its output channels over two tensors:
  // channels [0, split_at) go to y [N, split_at, Ho, Wo], the rest to y_split [N, Cout - split_at, Ho, Wo].
  float *y_split;
  int split_at;
};

// Address of output element (image n, channel co, pixel pix).
__device__ __forceinline__ float *dcn_out_ptr(const DcnArgs &a, int n, int co, long long plane_out, int pix) {
  if (a.y_split == nullptr) return a.y + ((long long)n * a.Cout + co) * plane_out + pix;
  if (co < a.split_at) return a.y + ((long long)n * a.split_at + co) * plane_out + pix;
  return a.y_split + ((long long)n * (a.Cout - a.split_at) + (co - a.split_at)) * plane_out + pix;
}

// The reference's Sigmoid (native/lib/DeviceLowering.cpp:387-394; src/gac/core/ops.py:916-924): the stable form.
__device__ __forceinline__ float sigmoid_ref(float x) {
  const float e = expf(-fabsf(x));
  const float den = __fadd_rn(1.0f, e);
  return x >= 0.0f ? __fdiv_rn(1.0f, den) : __fdiv_rn(e, den);
}

// conv + bias -> BatchNorm ((v - mean) / sqrt(var + eps) * scale + bias, the reference's operation order:
// native/lib/DeviceLowering.cpp:858-866, src/gac/core/ops.py:1084-1089) -> ReLU.
__device__ __forceinline__ float dcn_epilogue(const DcnArgs &a, float v, int co) {
  if (a.bias) v = __fadd_rn(v, __ldg(a.bias + co));
  if (a.bn_scale) {
    const float sd = __fsqrt_rn(__fadd_rn(__ldg(a.bn_var + co), a.bn_eps));
    v = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v, __ldg(a.bn_mean + co)), sd), __ldg(a.bn_scale + co)),
                  __ldg(a.bn_bias + co));
  }
  if (a.relu) v = fmaxf(v, 0.0f);
  return v;
}

// ----------------------------------------------------------------------------------------------
// Shared sampling arithmetic
// ----------------------------------------------------------------------------------------------

// Scalar::bilinear of the reference on one NCHW plane (guards are real branches; (a+c)+(d+e)).
__device__ __forceinline__ float bilinear_nchw(const float *plane, int height, int width, float x, float y) {
  if (!(x > -1.0f && x < (float)width && y > -1.0f && y < (float)height)) return 0.0f;
  const int tx = (int)x, ty = (int)y;
  const int x0 = (x < (float)tx) ? tx - 1 : tx;
  const int y0 = (y < (float)ty) ? ty - 1 : ty;
  const float dx = __fsub_rn(x, (float)x0), dy = __fsub_rn(y, (float)y0);
  const bool x0in = x0 >= 0 && x0 < width, x1in = x0 + 1 >= 0 && x0 + 1 < width;
  const bool y0in = y0 >= 0 && y0 < height, y1in = y0 + 1 >= 0 && y0 + 1 < height;
  const float v00 = (x0in && y0in) ? __ldg(plane + y0 * width + x0) : 0.0f;
  const float v01 = (x1in && y0in) ? __ldg(plane + y0 * width + x0 + 1) : 0.0f;
  const float v10 = (x0in && y1in) ? __ldg(plane + (y0 + 1) * width + x0) : 0.0f;
  const float v11 = (x1in && y1in) ? __ldg(plane + (y0 + 1) * width + x0 + 1) : 0.0f;
  const float gx = __fsub_rn(1.0f, dx), gy = __fsub_rn(1.0f, dy);
  const float a = __fmul_rn(v00, __fmul_rn(gx, gy));
  const float c = __fmul_rn(v01, __fmul_rn(dx, gy));
  const float d = __fmul_rn(v10, __fmul_rn(gx, dy));
  const float e = __fmul_rn(v11, __fmul_rn(dx, dy));
  return __fadd_rn(__fadd_rn(a, c), __fadd_rn(d, e));
}

__global__ void __launch_bounds__(256) dcn_direct_kernel(const __grid_constant__ DcnArgs a) {
  const long long plane_out = (long long)a.Ho * a.Wo;
  const int plane_sel = (a.row_end - a.row_begin) * a.Wo;   // pixels of the selected rows of one image
  const long long total = (long long)a.Cout * a.m_count;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int co = (int)(i / a.m_count);                      // consecutive threads: consecutive pixels
  const int f = a.m_first + (int)(i - (long long)co * a.m_count);
  const int n = a.n_begin + f / plane_sel;
  const int pix = a.row_begin * a.Wo + f % plane_sel;
  const int oy = pix / a.Wo, ox = pix % a.Wo;
  const int K = a.Kh * a.Kw, cin_g = a.Cin / a.groups, cout_g = a.Cout / a.groups, cin_dg = a.Cin / a.dgroups;
  const int g = co / cout_g;
  const float *wrow = a.w + (long long)co * cin_g * K;
  float acc = 0.0f;
  for (int ci = 0; ci < cin_g; ++ci) {
    const int channel = g * cin_g + ci;
    const int dgi = channel / cin_dg;
    const float *plane = a.x + ((long long)n * a.Cin + channel) * a.H * a.W;
    for (int kh = 0; kh < a.Kh; ++kh)
      for (int kw = 0; kw < a.Kw; ++kw) {
        if (a.offset == nullptr) {
          // plain convolution (native/lib/DeviceLowering.cpp:666-688): a padding tap skips the multiply entirely
          const int sy = oy * a.sh + kh * a.dh - a.ph, sx = ox * a.sw + kw * a.dw - a.pw;
          if (sy >= 0 && sy < a.H && sx >= 0 && sx < a.W)
            acc = __fadd_rn(acc, __fmul_rn(__ldg(plane + sy * a.W + sx), __ldg(wrow + ci * K + kh * a.Kw + kw)));
          continue;
        }
        const int mch = dgi * K + kh * a.Kw + kw;
        const float *off = a.offset + ((long long)n * 2 * a.dgroups * K + 2 * mch) * plane_out + pix;
        const float fy = __fadd_rn((float)(oy * a.sh + kh * a.dh - a.ph), __ldg(off));
        const float fx = __fadd_rn((float)(ox * a.sw + kw * a.dw - a.pw), __ldg(off + plane_out));
        float m = __ldg(a.mask + ((long long)n * a.dgroups * K + mch) * plane_out + pix);
        if (a.mask_is_logits) m = sigmoid_ref(m);
        const float sample = __fmul_rn(bilinear_nchw(plane, a.H, a.W, fx, fy), m);
        acc = __fadd_rn(acc, __fmul_rn(sample, __ldg(wrow + ci * K + kh * a.Kw + kw)));
      }
  }
  *dcn_out_ptr(a, n, co, plane_out, pix) = dcn_epilogue(a, acc, co);
}

// ----------------------------------------------------------------------------------------------
// Tensor-core path: layout constants
// ----------------------------------------------------------------------------------------------

constexpr int kTileM = 128;          // pixels per CTA tile = TMEM lanes
#ifndef GACB_DCN_BLOCK_H
#define GACB_DCN_BLOCK_H 8           // rows of the pixel blocks a whole-image call walks (0 = plain row-major order)
#endif
#ifndef GACB_DCN_BATCH_BF16
#define GACB_DCN_BATCH_BF16 2
#endif
#ifndef GACB_DCN_BATCH_PLAIN
#define GACB_DCN_BATCH_PLAIN 8
#endif
#ifndef GACB_DCN_BATCH_F32
#define GACB_DCN_BATCH_F32 2
#endif
// Pipeline shape.  Four producer groups fill a ring of kAStages A tiles (16 KB each in every mode); K block kb goes
// to A stage kb % kAStages whichever group makes it, so a group that has finished a tile starts the next one at
// once instead of waiting for the tensor core to drain "its" stage: the two spare stages absorb the hand-off
// latency (arrive -> MMA issue -> commit -> visible to the producer, ~1400 cycles measured).  B tiles (32 KB each
// at 256 output channels) stream through their own, shorter ring: two stages are enough (measured), and the 32 KB a
// third one would take serve better as L1 for the gathers, which share L2 bandwidth with the B stream.
#ifndef GACB_DCN_GROUPS
#define GACB_DCN_GROUPS 4
#endif
constexpr int kGroups = GACB_DCN_GROUPS;
#ifndef GACB_DCN_A_STAGES
#define GACB_DCN_A_STAGES 6
#endif
#ifndef GACB_DCN_B_STAGES
#define GACB_DCN_B_STAGES 2
#endif
constexpr int kAStages = GACB_DCN_A_STAGES;
constexpr int kBStages = GACB_DCN_B_STAGES;
constexpr int kProducerWarps = 4 * kGroups;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kLoaderWarp = kProducerWarps;      // streams B tiles
constexpr int kMmaWarp = kProducerWarps + 1;     // owns TMEM, issues tcgen05.mma
constexpr int kMma2Warp = kProducerWarps + 2;    // second issuer, used by narrow channel tiles only (see UmmaArgs::dual)
constexpr int kUmmaThreads = (kProducerWarps + 3) * 32;
// Shape of one CTA.  The wide shape (above) fills an SM by itself.  Channel tiles of at most 64 columns take the
// narrow shape: half the producer groups, four A stages and about 104 KB of shared memory, so that TWO CTAs share an
// SM.  Such a tile's time is mostly fixed cost (launch, prologue, pipeline fill, drain, epilogue: 7.5 us against
// 0.33 us per K block for the 27-channel conv_offset) and the one thread that issues its MMAs; two resident CTAs
// overlap both, and a problem of up to 296 tiles runs as one wave instead of two.
#ifndef GACB_DCN_NARROW_A_STAGES
#define GACB_DCN_NARROW_A_STAGES 4
#endif
template <bool NARROW>
struct CtaShape {
  static constexpr int kGroups = NARROW ? 2 : gacb::kGroups;
  static constexpr int kAStages = NARROW ? GACB_DCN_NARROW_A_STAGES : gacb::kAStages;
  static constexpr int kProducerWarps = 4 * kGroups;
  static constexpr int kProducerThreads = kProducerWarps * 32;
  static constexpr int kLoaderWarp = kProducerWarps;
  static constexpr int kMmaWarp = kProducerWarps + 1;
  static constexpr int kMma2Warp = kProducerWarps + 2;
  static constexpr int kThreads = (kProducerWarps + 3) * 32;
  static constexpr int kMinCtas = NARROW ? 2 : 1;
};
constexpr double kMinTensorFlopsPerImage = 12e6;
// Bounded mbarrier polling (each poll may block ~us in hardware).  GACB_DCN_SPIN_LIMIT shortens it in the test
// build that makes a wait run out on purpose (GACB_DCN_FAULT_INJECT, see UmmaArgs::drop_weight_copies).
#ifndef GACB_DCN_SPIN_LIMIT
#define GACB_DCN_SPIN_LIMIT (1u << 22)
#endif
#ifndef GACB_DCN_FAULT_INJECT
#define GACB_DCN_FAULT_INJECT 0
#endif
constexpr uint32_t kSpinLimit = GACB_DCN_SPIN_LIMIT;
// math_mode flag of the test build only: the weight loader issues none of its copies, so the tensor-core thread's
// wait for the first weight stage runs out and the kernel has to unwind through its abort path.
constexpr int kTestDropWeightCopies = 0x400;

enum { MODE_F32X3 = GACB_DCN_F32X3, MODE_TF32 = GACB_DCN_TF32, MODE_BF16 = GACB_DCN_BF16 };

// kElemBytes: operand element in shared memory; kParts: hi (+lo); kBlockK: channels per tile row (kRowBytes bytes);
// kUmmaK: K of one tcgen05.mma; kXtBytes: element size of the NHWC copy the producers gather from.
template <int MODE>
struct ModeTraits;
template <>
struct ModeTraits<MODE_BF16> {
  static constexpr int kElemBytes = 2, kParts = 1, kBlockK = 64, kUmmaK = 16, kXtBytes = 2, kRowBytes = 128;
};
template <>
struct ModeTraits<MODE_F32X3> {
  // 64-byte rows (32 channels per K block): a stage is 48 KB, so four stages fit like in the other modes
  static constexpr int kElemBytes = 2, kParts = 2, kBlockK = 32, kUmmaK = 16, kXtBytes = 4, kRowBytes = 64;
};
template <>
struct ModeTraits<MODE_TF32> {
  static constexpr int kElemBytes = 4, kParts = 1, kBlockK = 32, kUmmaK = 8, kXtBytes = 4, kRowBytes = 128;
};

__host__ __device__ inline int block_k_of(int mode) { return mode == MODE_BF16 ? 64 : 32; }
__host__ __device__ inline int row_bytes_of(int mode) { return mode == MODE_F32X3 ? 64 : 128; }
__host__ __device__ inline int parts_of(int mode) { return mode == MODE_F32X3 ? 2 : 1; }
__host__ __device__ inline int xt_bytes_of(int mode) { return mode == MODE_BF16 ? 2 : 4; }

// Byte offset of the 16-byte chunk `chunk` of row `row` inside a K-major swizzled tile whose rows are 128 bytes
// (128-byte swizzle: chunk bits ^= byte-offset bits 7..9) or 64 bytes (64-byte swizzle: chunk bits ^= bits 7..8).
// Rows are stored densely; eight rows form one swizzle atom.
__host__ __device__ inline uint32_t swizzled_chunk(uint32_t row, uint32_t chunk, int row_bytes) {
  if (row_bytes == 128) return row * 128u + ((chunk ^ (row & 7u)) << 4);
  return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
}

// Round to the nearest tf32 (10-bit mantissa), returned as an fp32 bit pattern with the low 13 bits clear.
__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

struct UmmaPlan {
  int tile_n;        // output channels per CTA tile (multiple of 16, <= 256, divides Cout/groups)
  int n_tiles;       // tiles along Cout per group
  int k_blocks;      // K' / block_k per group
  int chan_blocks;   // block_k-channel runs per kernel point
  int m_tiles;       // pixel tiles
  long long m_total; // selected pixels of the images [n_begin, n_end)
  size_t xt_bytes, blob_bytes, b_stage_bytes;
};

bool plan_umma(const DcnArgs &a, int mode, UmmaPlan &p) {
  const int cin_g = a.Cin / a.groups, cout_g = a.Cout / a.groups, cin_dg = a.Cin / a.dgroups;
  const int bk = block_k_of(mode);
  if (cin_g % bk || cin_dg % bk) return false;
  // Small problems stay on the CUDA-core kernel: a handful of tiles cannot fill 148 SMs, and that kernel keeps
  // the reference's reduction order and rounding.  The test is per image so that a call restricted to some of
  // the images takes the same path as the whole call (shards stay bit-identical to one launch).
  const double image_flops = 2.0 * a.Cout * cin_g * a.Kh * a.Kw * (double)a.Ho * a.Wo;
  if (image_flops < kMinTensorFlopsPerImage) return false;
  // Output-channel tile: the whole group when it fits one accumulator, else the largest multiple of 16 that
  // divides it.  A group that is not a multiple of 16 (the 27-channel offset/mask convolution) gets tiles padded
  // with zero weight rows; the epilogue never stores the padding columns.
  int tn;
  if (cout_g % 16 == 0) {
    tn = cout_g <= 256 ? cout_g : 256;
    while (tn >= 16 && (cout_g % tn || tn % 16)) tn -= 16;
    if (tn < 16) return false;
  } else {
    tn = cout_g <= 256 ? (cout_g + 15) / 16 * 16 : 256;
  }
  const long long m_total = a.m_count;
  if (m_total <= 0 || m_total > 2147483647LL - kTileM) return false;
  if ((long long)a.N * a.Cin * a.H * a.W > 2147483647LL) return false;
  p.tile_n = tn;
  p.n_tiles = (cout_g + tn - 1) / tn;
  p.chan_blocks = cin_g / bk;
  p.k_blocks = a.Kh * a.Kw * p.chan_blocks;
  p.m_total = m_total;
  p.m_tiles = (int)((m_total + kTileM - 1) / kTileM);
  p.b_stage_bytes = (size_t)parts_of(mode) * tn * row_bytes_of(mode);
  p.blob_bytes = (size_t)a.groups * p.n_tiles * p.k_blocks * p.b_stage_bytes;
  if (a.groups == 1 && a.Cout <= 64) {
    // room for the window kernel's weight layout, which pads the output channels to a multiple of 32
    const size_t windowed = (size_t)((a.Cout + 31) / 32 * 32) * a.Cin * a.Kh * a.Kw * (mode == MODE_TF32 ? 4 : 2) * parts_of(mode);
    p.blob_bytes = std::max(p.blob_bytes, windowed);
  }
  p.xt_bytes = ((size_t)(a.n_end - a.n_begin) * a.Cin * a.H * a.W * xt_bytes_of(mode) + 1023) / 1024 * 1024;
  return true;
}

// X [n][c][h*w] -> X_t [n][h*w][c] for the images of the call (32x32 tiles through shared memory).
template <typename OutT>
__global__ void __launch_bounds__(256) dcn_nhwc_kernel(const float *__restrict__ x, OutT *__restrict__ xt, int C,
                                                       int HW, int n_begin) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const float *src = x + (long long)(n_begin + n) * C * HW;
  OutT *dst = xt + (long long)n * C * HW;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, p = p0 + tx;
    tile[r][tx] = (c < C && p < HW) ? __ldg(src + (long long)c * HW + p) : 0.0f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int p = p0 + r, c = c0 + tx;
    if (p < HW && c < C) dst[(long long)p * C + c] = static_cast<OutT>(tile[tx][r]);
  }
}

// The same copy with vector accesses, for C % 32 == 0 and H*W % V == 0 (V = 4 or 2 pixels per load): tiles of
// 32 channels x 128 pixels; V-pixel loads along the pixels, 4-channel stores along the channels.
__device__ __forceinline__ void store4(float *dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4 *>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16 *dst, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
}
template <typename OutT, int V>
__global__ void __launch_bounds__(256) dcn_nhwc_vec_kernel(const float *__restrict__ x, OutT *__restrict__ xt, int C,
                                                           int HW, int n_begin) {
  constexpr int kPix = 128, kCh = 32, kStride = kPix + 1;
  __shared__ float tile[kCh * kStride];
  const int n = blockIdx.z;
  const float *src = x + (long long)(n_begin + n) * C * HW;
  OutT *dst = xt + (long long)n * C * HW;
  const int p0 = blockIdx.x * kPix, c0 = blockIdx.y * kCh;
  constexpr int kVecPerRow = kPix / V;
#pragma unroll
  for (int i = 0; i < kCh * kVecPerRow / 256; ++i) {
    const int idx = threadIdx.x + 256 * i;
    const int c_l = idx / kVecPerRow, q = idx - c_l * kVecPerRow;
    const int p = p0 + V * q;
    float v[V];
#pragma unroll
    for (int e = 0; e < V; ++e) v[e] = 0.0f;
    if (p < HW) {   // H*W is a multiple of V, so a vector is inside or outside as a whole
      const float *g = src + (long long)(c0 + c_l) * HW + p;
      if constexpr (V == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(g));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
        const float2 t = __ldg(reinterpret_cast<const float2 *>(g));
        v[0] = t.x; v[1] = t.y;
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) tile[c_l * kStride + V * q + e] = v[e];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kPix * (kCh / 4) / 256; ++i) {
    const int idx = threadIdx.x + 256 * i;
    const int p_l = idx >> 3, cg = idx & 7;
    if (p0 + p_l < HW) {
      const float *t = tile + (4 * cg) * kStride + p_l;
      store4(dst + (long long)(p0 + p_l) * C + c0 + 4 * cg, t[0], t[kStride], t[2 * kStride], t[3 * kStride]);
    }
  }
}

// W [Cout][Cin_g][Kh*Kw] -> blob[g][n_tile][k_block][part][tile_n rows][128 B swizzled], k' = kp*Cin_g + ci.
__global__ void __launch_bounds__(256) dcn_pack_weights(const float *__restrict__ w, unsigned char *__restrict__ blob,
                                                        int Cout, int cin_g, int K, int groups, int tile_n,
                                                        int n_tiles, int k_blocks, int mode) {
  const int bk = block_k_of(mode), parts = parts_of(mode);
  const int cout_g = Cout / groups;
  const int cout_pad = n_tiles * tile_n;                  // rows of a group's tiles, padding rows included
  const long long total = (long long)groups * cout_pad * cin_g * K;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int kprime = (int)(i % ((long long)cin_g * K));   // kp*cin_g + ci: consecutive threads -> consecutive k'
  const int row_all = (int)(i / ((long long)cin_g * K));
  const int kp = kprime / cin_g, ci = kprime - kp * cin_g;
  const int g = row_all / cout_pad, cog = row_all - g * cout_pad;
  const float v = cog < cout_g ? __ldg(w + ((long long)(g * cout_g + cog) * cin_g + ci) * K + kp) : 0.0f;
  const int nt = cog / tile_n, row = cog - nt * tile_n;
  // K blocks run channel-block-major, kernel-point-minor: consecutive blocks sample the same channels at
  // neighbouring kernel points, so their taps overlap in L1.
  const int cblk = ci / bk, kk = ci - cblk * bk;
  const int kb = cblk * K + kp;
  const int row_bytes = row_bytes_of(mode);
  const size_t part_bytes = (size_t)tile_n * row_bytes;
  unsigned char *stage = blob + (((size_t)g * n_tiles + nt) * k_blocks + kb) * (parts * part_bytes);
  if (mode == MODE_TF32) {
    const uint32_t byte = swizzled_chunk(row, kk >> 2, row_bytes) + (kk & 3) * 4;
    *reinterpret_cast<float *>(stage + byte) = tf32_round(v);
  } else {
    const uint32_t byte = swizzled_chunk(row, kk >> 3, row_bytes) + (kk & 7) * 2;
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    *reinterpret_cast<__nv_bfloat16 *>(stage + byte) = hi;
    if (parts == 2)
      *reinterpret_cast<__nv_bfloat16 *>(stage + part_bytes + byte) = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
}

// ----------------------------------------------------------------------------------------------
// PTX wrappers (sm_100a)
// ----------------------------------------------------------------------------------------------

// Bounded wait for two barriers at once: both are polled in every round, so the two shared-memory round trips
// overlap instead of following each other.
__device__ __forceinline__ bool mbar_wait2(uint32_t bar0, uint32_t parity0, uint32_t bar1, uint32_t parity1,
                                           volatile int *abort_flag);
// Bounded wait.  Returns false when the abort flag is (or becomes) set.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait2(uint32_t bar0, uint32_t parity0, uint32_t bar1, uint32_t parity1,
                                           volatile int *abort_flag) {
  bool done0 = false, done1 = false;
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    const bool t0 = done0 || mbar_try_wait(bar0, parity0);
    const bool t1 = done1 || mbar_try_wait(bar1, parity1);
    done0 = t0;
    done1 = t1;
    if (done0 && done1) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// Bounded wait for a whole warp: lane 0 polls (pausing between polls, so that idle roles leave the shared-memory
// pipe to the tensor core's operand reads) and the outcome is broadcast.  All lanes must call it.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane) {
  int ok = 0;
  if (lane == 0) {
    ok = -1;
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
      if (mbar_try_wait(bar, parity)) { ok = 1; break; }
      if (*abort_flag) { ok = 0; break; }
      __nanosleep(40);
    }
    if (ok < 0) { *abort_flag = 1; ok = 0; }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// The same for a warp that must not lose time: lane 0 polls without pausing.  The result is warp-uniform.
__device__ __forceinline__ bool mbar_wait_uniform(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane) {
  int ok = 0;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// One lane of a converged warp (the same one every time): the lane that executes tcgen05.mma / tcgen05.commit.
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(chosen));
  return chosen != 0;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool TF32>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if (TF32)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major swizzled operand: 8-row atoms (8 * ROW_BYTES) stacked along M/N; 128- or 64-byte swizzle.
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)((8 * ROW_BYTES) >> 4) << 32;         // stride byte offset between 8-row atoms
  d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
  d |= (uint64_t)(ROW_BYTES == 128 ? 2 : 4) << 61;     // SWIZZLE_128B / SWIZZLE_64B
  return d;
}
// D = f32, A/B K-major; format 1 = bf16 (kind::f16), 2 = tf32 (kind::tf32).
__device__ __forceinline__ uint32_t umma_idesc(int format, int m, int n) {
  return (1u << 4) | ((uint32_t)format << 7) | ((uint32_t)format << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// ----------------------------------------------------------------------------------------------
// The implicit-GEMM kernel
// ----------------------------------------------------------------------------------------------

struct UmmaArgs {
  DcnArgs d;
  const void *xt;              // NHWC copy of images [n_begin, n_end): fp32, or bf16 in BF16 mode
  const unsigned char *blob;   // packed weights
  int32_t *status;             // optional device status word
  int tile_n, n_tiles, k_blocks, chan_blocks, m_tiles, tmem_cols;
  int cross_col;               // first TMEM column of the cross-product accumulator (F32X3)
  // Narrow channel tiles (the 27-channel conv_offset): one thread needs ~900 cycles per K block to see the barriers,
  // issue and commit, whatever the size of the products, and that paces the tile.  Two threads then take alternate
  // K blocks, each into its own accumulator set (acc2_col columns apart); the epilogue adds the two.
  int dual, acc2_col;
  int m_total;
  int record_slots;            // slots of the tap-record table
  int precomputed;             // the table holds every (kernel point, deformable group) record of a tile
  unsigned b_stage_bytes;
  int drop_weight_copies;      // test build only (GACB_DCN_FAULT_INJECT): the loader skips every copy
  int block_h, block_w;        // blocked pixel order of whole-image calls (PixelOrder); 0 = plain order
};

// Tap records live in shared memory as two arrays of record_slots x 128 entries: a packed geometry word and the
// four tap coefficients (20 bytes per record).  With up to kMaxRecordSlots (kernel point, deformable group) pairs
// per CTA the whole table is built once per tile; otherwise each of the four producer groups owns one slot.
constexpr int kMaxRecordSlots = 9;
// Per output channel of the tile, staged in shared memory once: bias, BatchNorm mean, sqrt(variance + epsilon),
// scale, BatchNorm bias (the epilogue would otherwise fetch them -- and take the square root -- per element).
constexpr int kEpilogueParams = 5;
constexpr int kRecordBytes = sizeof(uint32_t) + sizeof(float4);

template <int MODE>
struct SmemLayout {
  using T = ModeTraits<MODE>;
  static constexpr int kATile = kTileM * T::kRowBytes;   // per part
  static size_t a_stage_bytes() { return (size_t)T::kParts * kATile; }
  static size_t b_stage_bytes(int tile_n) { return (size_t)T::kParts * tile_n * T::kRowBytes; }
  // ep_rows = rows of the epilogue parameter table: kEpilogueParams with BatchNorm folded in, else 0; every KB not
  // taken here stays L1 for the gathers
  static size_t total(int tile_n, int record_slots, int a_stages = kAStages, int ep_rows = kEpilogueParams) {
    return 1024 /*alignment slack*/ + a_stages * a_stage_bytes() + kBStages * b_stage_bytes(tile_n) +
           (size_t)record_slots * kTileM * kRecordBytes + 256 /*barriers, tmem slot, abort flag*/ +
           (size_t)ep_rows * ((tile_n + 31) / 32 * 32) * sizeof(float);
  }
};

// CH consecutive channels of one tap as they sit in the NHWC copy.  A lane takes 16 bytes per load where it can: a
// warp-wide load then covers whole 128-byte lines (one L1 wavefront per line) instead of half of each of twice as many.
template <int XT_BYTES, int CH>
struct Texels;
template <>
struct Texels<4, 4> {
  typedef float4 Raw;
  __device__ static __forceinline__ Raw load(const void *base, long long elem) {
    return __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem));
  }
  __device__ static __forceinline__ void accumulate(float (&o)[4], const Raw &v, float c) {
    o[0] = fmaf(v.x, c, o[0]); o[1] = fmaf(v.y, c, o[1]); o[2] = fmaf(v.z, c, o[2]); o[3] = fmaf(v.w, c, o[3]);
  }
};
template <>
struct Texels<2, 8> {
  typedef uint4 Raw;
  __device__ static __forceinline__ Raw load(const void *base, long long elem) {
    return __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(base) + elem));
  }
  __device__ static __forceinline__ void accumulate(float (&o)[8], const Raw &v, float c) {
    o[0] = fmaf(bf16_lo(v.x), c, o[0]); o[1] = fmaf(bf16_hi(v.x), c, o[1]);
    o[2] = fmaf(bf16_lo(v.y), c, o[2]); o[3] = fmaf(bf16_hi(v.y), c, o[3]);
    o[4] = fmaf(bf16_lo(v.z), c, o[4]); o[5] = fmaf(bf16_hi(v.z), c, o[5]);
    o[6] = fmaf(bf16_lo(v.w), c, o[6]); o[7] = fmaf(bf16_hi(v.w), c, o[7]);
  }
};

// BF16 mode only: blend four taps of eight bf16 channels in packed bf16x2 arithmetic (the result is going to be
// rounded to bf16 for the tensor core anyway; this replaces 32 fp32 FMAs + 16 unpacks + 8 converts by 16 HFMA2).
// c01 / c23 hold the four tap coefficients as bf16 pairs (c0 in the low half of c01, ...).
__device__ __forceinline__ uint4 blend_bf16x2(const uint4 (&v)[4], uint32_t c01, uint32_t c23) {
  auto as2 = [](uint32_t w) { return *reinterpret_cast<const __nv_bfloat162 *>(&w); };
  const __nv_bfloat162 c0 = as2(__byte_perm(c01, 0u, 0x1010)), c1 = as2(__byte_perm(c01, 0u, 0x3232));
  const __nv_bfloat162 c2 = as2(__byte_perm(c23, 0u, 0x1010)), c3 = as2(__byte_perm(c23, 0u, 0x3232));
  auto lane = [&](uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    __nv_bfloat162 acc = __hmul2(as2(a), c0);
    acc = __hfma2(as2(b), c1, acc);
    acc = __hfma2(as2(c), c2, acc);
    acc = __hfma2(as2(d), c3, acc);
    return *reinterpret_cast<uint32_t *>(&acc);
  };
  return make_uint4(lane(v[0].x, v[1].x, v[2].x, v[3].x), lane(v[0].y, v[1].y, v[2].y, v[3].y),
                    lane(v[0].z, v[1].z, v[2].z, v[3].z), lane(v[0].w, v[1].w, v[2].w, v[3].w));
}

__device__ __forceinline__ uint32_t pack_bf16x2(__nv_bfloat16 lo, __nv_bfloat16 hi) {
  return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

// Order of the output pixels along the M dimension of the implicit GEMM.  A call that covers whole images
// (block_h > 0) walks every image in blocks of block_h rows x block_w columns, row-major inside a block, blocks
// row-major over the image, ragged blocks at the right and bottom edges: a 128-row tile is then a compact
// 8 x 16 patch of pixels whose taps fall on a small neighbourhood of the input (the nine kernel points and the
// neighbouring pixels share texels), which is what L1 can hold.  A call restricted to rows or to a pixel run
// keeps the plain (image, row, column) order.  Each output element is computed the same way in both orders.
struct PixelOrder {
  int plane_sel, pix_first, m_first;   // plain order: selected pixel f = m_first + m -> image f / plane_sel, ...
  int block_h, block_w, Ho, Wo;        // blocked order when block_h > 0
};

__device__ __forceinline__ void pixel_of(const PixelOrder &o, int m, int &img, int &pix) {
  if (o.block_h == 0) {
    const int f = o.m_first + m;
    img = f / o.plane_sel;
    pix = o.pix_first + f - img * o.plane_sel;
    return;
  }
  const int plane = o.Ho * o.Wo;
  img = m / plane;
  int r = m - img * plane;
  const int strip_px = o.block_h * o.Wo;                   // pixels of a full strip of block_h rows
  const int strip = r / strip_px;
  r -= strip * strip_px;
  const int rows = min(o.block_h, o.Ho - strip * o.block_h);   // rows of this strip (the last one may be short)
  const int block_px = rows * o.block_w;                   // pixels of a full-width block of this strip
  const int block = r / block_px;
  r -= block * block_px;
  const int cols = min(o.block_w, o.Wo - block * o.block_w);   // columns of this block (the last one may be narrow)
  const int y = r / cols;
  pix = (strip * o.block_h + y) * o.Wo + block * o.block_w + (r - y * cols);
}

// Epilogue parameter table of one tile's output channels (BatchNorm calls only); padding columns get neutral values.
__device__ __noinline__ void fill_epilogue_table(const DcnArgs &a, float *table, int pitch, int group, int n_tile, int tile_n) {
  const int cout_g = a.Cout / a.groups;
  const int cols = min(tile_n, cout_g - n_tile * tile_n);
  for (int c = threadIdx.x; c < pitch; c += blockDim.x) {
    const int co = group * cout_g + n_tile * tile_n + c;
    const bool live = c < cols;
    table[0 * pitch + c] = (live && a.bias) ? __ldg(a.bias + co) : 0.0f;
    table[1 * pitch + c] = live ? __ldg(a.bn_mean + co) : 0.0f;
    table[2 * pitch + c] = live ? __fsqrt_rn(__fadd_rn(__ldg(a.bn_var + co), a.bn_eps)) : 1.0f;
    table[3 * pitch + c] = live ? __ldg(a.bn_scale + co) : 1.0f;
    table[4 * pitch + c] = live ? __ldg(a.bn_bias + co) : 0.0f;
  }
}

// PLAIN = plain convolution (no offset/mask operands): every sample is one texel at an integer position, so the
// producers fetch one tap instead of four and copy instead of blending.
template <int MODE, bool PLAIN, bool NARROW>
__global__ void __launch_bounds__(CtaShape<NARROW>::kThreads, CtaShape<NARROW>::kMinCtas)
    dcn_umma_kernel(const __grid_constant__ UmmaArgs u) {
  using T = ModeTraits<MODE>;
  // this CTA's shape; the names shadow the wide shape's namespace-level constants
  using Shape = CtaShape<NARROW>;
  constexpr int kGroups = Shape::kGroups, kAStages = Shape::kAStages, kProducerWarps = Shape::kProducerWarps;
  constexpr int kProducerThreads = Shape::kProducerThreads, kLoaderWarp = Shape::kLoaderWarp;
  constexpr int kMmaWarp = Shape::kMmaWarp;
  constexpr int S = kGroups;      // producer groups; group g makes K blocks g, g+S, ...
  constexpr int SA = kAStages, SB = kBStages;
  constexpr int kRowBytes = T::kRowBytes;
  constexpr int kATile = kTileM * kRowBytes;
  // channels a producer lane blends at once: 16 bytes of the NHWC copy (8 bf16 or 4 fp32)
  constexpr int kChanPerLane = 16 / T::kXtBytes;
  constexpr int kLanesPerRow = kRowBytes / (kChanPerLane * T::kElemBytes);  // 8
  using Quad = Texels<T::kXtBytes, kChanPerLane>;

  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const DcnArgs &a = u.d;
  const size_t b_part = (size_t)u.tile_n * kRowBytes;
  constexpr size_t a_stage = (size_t)T::kParts * kATile;     // A stage: [part0][part1?]
  const size_t b_stage = (size_t)T::kParts * b_part;         // B stage: [part0][part1?]
  unsigned char *a_stages = smem;
  unsigned char *b_stages = smem + SA * a_stage;
  float4 *rec_cf = reinterpret_cast<float4 *>(b_stages + SB * b_stage);            // [record_slots][kTileM]
  uint32_t *rec_geo = reinterpret_cast<uint32_t *>(rec_cf + u.record_slots * kTileM);
  uint64_t *bars = reinterpret_cast<uint64_t *>(rec_geo + u.record_slots * kTileM);
  // bars: full_a[SA] | empty_a[SA] | full_b[SB] | empty_b[SB] | acc_full
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * SA + 2 * SB + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // epilogue parameter table [rows][ep_stride] right after the barrier block (recomputed where it is used, so that
  // nothing of it stays live through the K loop)
  auto ep_table = [&]() { return reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(bars) + 256); };
  auto ep_pitch = [&]() { return (u.tile_n + 31) / 32 * 32; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m_tile = blockIdx.x, n_tile = blockIdx.y, group = blockIdx.z;
  const int m0 = m_tile * kTileM;
  const int plane_out = a.Ho * a.Wo;
  PixelOrder order;
  order.plane_sel = (a.row_end - a.row_begin) * a.Wo;        // tile rows enumerate the selected output rows only
  order.pix_first = a.row_begin * a.Wo;
  order.m_first = a.m_first;
  order.block_h = u.block_h;
  order.block_w = u.block_w;
  order.Ho = a.Ho;
  order.Wo = a.Wo;
  const int K = a.Kh * a.Kw;
  const int cin_g = a.Cin / a.groups, cin_dg = a.Cin / a.dgroups;
  const int k_blocks = u.k_blocks;
  const void *const xt = u.xt;

  const uint32_t bar_base = smem_u32(bars);
  auto full_a = [&](int s) { return bar_base + 8u * s; };
  auto empty_a = [&](int s) { return bar_base + 8u * (SA + s); };
  auto full_b = [&](int s) { return bar_base + 8u * (2 * SA + s); };
  auto empty_b = [&](int s) { return bar_base + 8u * (2 * SA + SB + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * SA + 2 * SB);

  if (tid == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(full_a(s), kProducerWarps / S);   // one arrival per warp of the producer group that fills it
      mbar_init(empty_a(s), 1);
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(full_b(s), 1);
      mbar_init(empty_b(s), 1);
    }
    mbar_init(acc_full, u.dual ? 2 : 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_slot), (uint32_t)u.tmem_cols);
  // BatchNorm folded in: per output channel of the tile {bias, mean, sqrt(variance + epsilon), scale, BatchNorm bias}
  // go to shared memory once, instead of five loads and a square root per element in the epilogue
  if (a.bn_scale != nullptr) fill_epilogue_table(a, ep_table(), ep_pitch(), group, n_tile, u.tile_n);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // F32X3 keeps the cross products in a second accumulator right after the main one.
  const uint32_t tmem_cross = tmem_base + (uint32_t)u.cross_col;

  if (warp < kProducerWarps) {
    // ------------------------------------------------------------------ A producers
    // Four independent groups of four warps; group g produces the A tiles of K blocks g, g+4, g+8, ..., K block kb
    // into A stage kb % SA.  Nothing synchronises the groups with each other, so while one group waits for its
    // gathers another blends or stores: the latencies of different K blocks overlap without extra registers.
    constexpr int kGroupThreads = kProducerThreads / S;          // 128: one thread per tile row for the records
    static_assert(kGroupThreads == kTileM, "one record per thread when a group rebuilds its K block's records");
    // items whose gathers are in flight together (a plain convolution loads a quarter as much per item)
    constexpr int kBatch = PLAIN ? GACB_DCN_BATCH_PLAIN : (T::kXtBytes == 2) ? GACB_DCN_BATCH_BF16 : GACB_DCN_BATCH_F32;
    constexpr int kItems = kLanesPerRow;                          // (row, channel slice) items per thread and K block
    constexpr int kRowsPerStep = kGroupThreads / kLanesPerRow;    // rows covered by the group per item step
    const int g = warp / (kProducerWarps / S);
    const int gt = tid - g * kGroupThreads;                       // thread within the group
    const int lane_in_row = gt % kLanesPerRow;
    const int row_base = gt / kLanesPerRow;
    const int image_elems = a.H * a.W * a.Cin;                    // X_t has fewer than 2^31 elements
    const int dg_first = (group * cin_g) / cin_dg;                // first deformable group this CTA's channels use
    const int dg_last = (group * cin_g + cin_g - 1) / cin_dg;     // and the last one

    // Tap record of (tile row, kernel point kp, deformable group dgi), written to slot `slot` of the table:
    //   geo = element offset in X_t of the (clamped) top-left texel, channel 0 | bit 0: the x1 column is one
    //         texel to the right | bit 1: the y1 row is one row down (offsets are multiples of Cin >= 32);
    //   cf  = mask * bilinear coefficient per tap, 0 for a tap outside the image.
    // Padding rows of the last tile and samples outside the image get zero coefficients at texel 0.
    // The record is made in two steps so that a thread can have the offset/mask loads of several records in
    // flight before it computes any of them.
    struct RawTap { float dy, dx, mk; int img, pix; };
    auto fetch_raw = [&](int row, int kp, int dgi) -> RawTap {
      RawTap t = {0.0f, 0.0f, 1.0f, -1, 0};
      const int m = m0 + row;
      if (m < u.m_total) {
        pixel_of(order, m, t.img, t.pix);
        if constexpr (!PLAIN) {
          const int n = a.n_begin + t.img;
          const int mch = dgi * K + kp;
          const long long mask_elems = (long long)a.N * a.dgroups * K * plane_out;
          const float *off = a.offset + GACB_INDEX(((long long)n * 2 * a.dgroups * K + 2 * mch) * plane_out + t.pix,
                                                   2 * mask_elems - plane_out, 13);
          t.dy = __ldg(off);
          t.dx = __ldg(off + plane_out);
          t.mk = __ldg(a.mask + GACB_INDEX(((long long)n * a.dgroups * K + mch) * plane_out + t.pix, mask_elems, 13));
        }
      }
      return t;
    };
    auto finish_record = [&](int slot, int row, int kp, const RawTap &t) {
      uint32_t geo = 0;
      float4 cf = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (t.img >= 0) {
        const int img = t.img, pix = t.pix;
        const int oy = pix / a.Wo, ox = pix - oy * a.Wo;
        const float dy = t.dy, dx = t.dx;
        float mk = t.mk;
        if constexpr (!PLAIN) {
          if (a.mask_is_logits) mk = sigmoid_ref(mk);
        }
        const int kh = kp / a.Kw, kw = kp - kh * a.Kw;
        const float y = __fadd_rn((float)(oy * a.sh + kh * a.dh - a.ph), dy);
        const float x = __fadd_rn((float)(ox * a.sw + kw * a.dw - a.pw), dx);
        if (x > -1.0f && x < (float)a.W && y > -1.0f && y < (float)a.H) {
          const int tx = (int)x, ty = (int)y;
          const int x0 = (x < (float)tx) ? tx - 1 : tx;
          const int y0 = (y < (float)ty) ? ty - 1 : ty;
          const float fx = x - (float)x0, fy = y - (float)y0;
          const float gx = 1.0f - fx, gy = 1.0f - fy;
          const bool x0in = x0 >= 0, x1in = x0 + 1 < a.W;   // the sample guard already bounds the other side
          const bool y0in = y0 >= 0, y1in = y0 + 1 < a.H;
          const int cx0 = x0in ? x0 : 0, cy0 = y0in ? y0 : 0;
          geo = (uint32_t)(img * image_elems + (cy0 * a.W + cx0) * a.Cin);
          // x1 = x0+1 is a +1 step only when x0 itself is inside; when x0 == -1 the x1 column IS cx0.
          geo |= (x0in && x1in) ? 1u : 0u;
          geo |= (y0in && y1in) ? 2u : 0u;
          const float wx0 = x0in ? gx : 0.0f, wx1 = x1in ? fx : 0.0f;
          const float wy0 = y0in ? gy : 0.0f, wy1 = y1in ? fy : 0.0f;
          cf = make_float4(wx0 * wy0 * mk, wx1 * wy0 * mk, wx0 * wy1 * mk, wx1 * wy1 * mk);
        }
      }
      if constexpr (MODE == MODE_BF16) {
        // BF16 mode blends in bf16x2, so its record carries the coefficients already rounded to bf16 and is one
        // 16-byte word: {geometry, c0 | c1 << 16, c2 | c3 << 16, unused} -- one shared-memory read per item
        reinterpret_cast<uint4 *>(rec_cf)[GACB_INDEX(slot * kTileM + row, u.record_slots * kTileM, 11)] =
            make_uint4(geo, pack_bf16x2(__float2bfloat16_rn(cf.x), __float2bfloat16_rn(cf.y)),
                       pack_bf16x2(__float2bfloat16_rn(cf.z), __float2bfloat16_rn(cf.w)), 0u);
      } else {
        rec_geo[GACB_INDEX(slot * kTileM + row, u.record_slots * kTileM, 11)] = geo;
        rec_cf[GACB_INDEX(slot * kTileM + row, u.record_slots * kTileM, 11)] = cf;
      }
    };
    // group-only barrier (ids 1..4), 128 threads
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "n"(kGroupThreads) : "memory"); };

    // When the records of every (kernel point, deformable group) this CTA needs fit the table, they are all made
    // once, before the first K block: the channel blocks then reuse them and the K loop has no barrier at all.
    // Otherwise (many kernel points or deformable groups) each group rebuilds the records of its K block in its
    // own slot, between two group barriers.
    const bool pre = u.precomputed != 0;
    if (pre) {
      // up to kMaxRecordSlots * 128 / 512 = 2.25 records per thread: three at a time, loads first
      constexpr int kAhead = 3;
      const int total = u.record_slots * kTileM;
      for (int i0 = tid; i0 < total; i0 += kAhead * kProducerThreads) {
        RawTap raw[kAhead];
#pragma unroll
        for (int q = 0; q < kAhead; ++q) {
          const int i = i0 + q * kProducerThreads;
          const int slot = i / kTileM, dgl = slot / K;
          // slots past this group's last deformable group are never read (other groups span more)
          if (i < total) raw[q] = fetch_raw(i - slot * kTileM, slot - dgl * K, min(dg_first + dgl, dg_last));
        }
#pragma unroll
        for (int q = 0; q < kAhead; ++q) {
          const int i = i0 + q * kProducerThreads;
          const int slot = i / kTileM, dgl = slot / K;
          if (i < total) finish_record(slot, i - slot * kTileM, slot - dgl * K, raw[q]);
        }
      }
      asm volatile("bar.sync 15, %0;" ::"n"(kProducerThreads) : "memory");   // ids 1..kGroups belong to the groups
    }
    // slot of a K block's records in the precomputed table: the kernel point when all of this CTA's channels
    // share one deformable group (the usual case), else (deformable group, kernel point)
    const bool one_dg = dg_first == dg_last;

    // (channel block, kernel point) of this group's K blocks, advanced incrementally: kb = cb*K + kp = g, g+S, ...
    // Consecutive K blocks -- the ones the four groups work on at the same time -- are neighbouring kernel
    // points of one channel block: their taps fall on the same or adjacent texels, which is what makes L1 useful.
    int cb = g / K, kp = g - cb * K;
    auto dgi_of = [&](int cblock) { return (group * cin_g + cblock * T::kBlockK) / cin_dg; };
    // After an expired wait `alive` turns false: the thread keeps walking the loop (so the group barriers still
    // see every thread) but touches neither the pipeline nor memory.
    bool alive = true;
    const int step_x = a.Cin, step_y = a.W * a.Cin;
    for (int kb = g; kb < k_blocks; kb += S) {
      const int sa = kb % SA;
      const int chan0 = group * cin_g + cb * T::kBlockK;     // first input channel of this K block
      int slot = g;
      if (pre) {
        slot = one_dg ? kp : (dgi_of(cb) - dg_first) * K + kp;
      } else {
        finish_record(g, gt, kp, fetch_raw(gt, kp, dgi_of(cb)));
        group_sync();                                         // this block's records are complete
      }
      const uint32_t *geo_row = rec_geo + GACB_INDEX(slot, u.record_slots, 11) * kTileM;
      const float4 *cf_row = rec_cf + GACB_INDEX(slot, u.record_slots, 11) * kTileM;
      if (alive) alive = mbar_wait(empty_a(sa), ((kb / SA) & 1) ^ 1, abort_flag);
      if (alive) {
        unsigned char *a_hi = a_stages + sa * a_stage;
        unsigned char *a_lo = a_hi + kATile;
        const int lane_elem = chan0 + lane_in_row * kChanPerLane;
#pragma unroll 1
        for (int it = 0; it < kItems; it += kBatch) {
          typename Quad::Raw v[kBatch][4];
          float4 cf[kBatch];
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            const int row = row_base + (it + b) * kRowsPerStep;
            uint32_t geo;
            if constexpr (MODE == MODE_BF16) {
              const uint4 r = reinterpret_cast<const uint4 *>(cf_row)[row];
              geo = r.x;
              cf[b] = make_float4(__uint_as_float(r.y), __uint_as_float(r.z), 0.0f, 0.0f);   // packed bf16 pairs
            } else {
              geo = geo_row[row];
              cf[b] = cf_row[row];
            }
            const int e = lane_elem + (int)(geo & ~3u);
#if GACB_CHECKED
            const long long xt_last = (long long)(a.n_end - a.n_begin) * image_elems - kChanPerLane + 1;
#endif
            v[b][0] = Quad::load(xt, GACB_INDEX(e, xt_last, 12));
            if constexpr (!PLAIN) {
              const int sx = (geo & 1u) ? step_x : 0, sy = (geo & 2u) ? step_y : 0;
              v[b][1] = Quad::load(xt, GACB_INDEX(e + sx, xt_last, 12));
              v[b][2] = Quad::load(xt, GACB_INDEX(e + sy, xt_last, 12));
              v[b][3] = Quad::load(xt, GACB_INDEX(e + sy + sx, xt_last, 12));
            }
          }
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            const int row = row_base + (it + b) * kRowsPerStep;
            if constexpr (MODE == MODE_BF16) {
              uint4 packed;
              const uint32_t c01 = __float_as_uint(cf[b].x), c23 = __float_as_uint(cf[b].y);
              if constexpr (PLAIN) packed = (c01 & 0xffffu) != 0u ? v[b][0] : make_uint4(0u, 0u, 0u, 0u);
              else packed = blend_bf16x2(v[b], c01, c23);
              *reinterpret_cast<uint4 *>(a_hi + swizzled_chunk((uint32_t)row, (uint32_t)lane_in_row, kRowBytes)) = packed;
            } else {
            float o[kChanPerLane];
#pragma unroll
            for (int c = 0; c < kChanPerLane; ++c) o[c] = 0.0f;
            Quad::accumulate(o, v[b][0], cf[b].x);
            if constexpr (!PLAIN) {
              Quad::accumulate(o, v[b][1], cf[b].y);
              Quad::accumulate(o, v[b][2], cf[b].z);
              Quad::accumulate(o, v[b][3], cf[b].w);
            }
            // this lane's bytes of the tile row start at lane_in_row * kLaneBytes; 16-byte chunks are swizzled
            constexpr int kLaneBytes = kChanPerLane * T::kElemBytes;
            const uint32_t first = (uint32_t)(lane_in_row * kLaneBytes);
            if (T::kElemBytes == 4) {
#pragma unroll
              for (int c = 0; c < kChanPerLane; c += 4) {
                const uint32_t byte = swizzled_chunk((uint32_t)row, first / 16 + c / 4, kRowBytes);
                *reinterpret_cast<float4 *>(a_hi + byte) =
                    make_float4(tf32_round(o[c]), tf32_round(o[c + 1]), tf32_round(o[c + 2]), tf32_round(o[c + 3]));
              }
            } else {
              const uint32_t byte = swizzled_chunk((uint32_t)row, first / 16, kRowBytes) + (first & 15u);
              uint32_t hi[kChanPerLane / 2], lo[kChanPerLane / 2];
#pragma unroll
              for (int c = 0; c < kChanPerLane; c += 2) {
                const __nv_bfloat16 h0 = __float2bfloat16_rn(o[c]), h1 = __float2bfloat16_rn(o[c + 1]);
                hi[c / 2] = pack_bf16x2(h0, h1);
                lo[c / 2] = pack_bf16x2(__float2bfloat16_rn(o[c] - __bfloat162float(h0)),
                                        __float2bfloat16_rn(o[c + 1] - __bfloat162float(h1)));
              }
              if constexpr (kChanPerLane == 8) {
                *reinterpret_cast<uint4 *>(a_hi + byte) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                if (T::kParts == 2) *reinterpret_cast<uint4 *>(a_lo + byte) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
              } else {
                *reinterpret_cast<uint2 *>(a_hi + byte) = make_uint2(hi[0], hi[1]);
                if (T::kParts == 2) *reinterpret_cast<uint2 *>(a_lo + byte) = make_uint2(lo[0], lo[1]);
              }
            }
            }
          }
        }
        fence_proxy_async_smem();   // this thread's generic-proxy writes -> visible to the tensor core's async proxy
      }
      // one arrival per warp, after every lane's writes are fenced
      const bool warp_alive = __all_sync(0xffffffffu, alive);
      if (warp_alive && lane == 0) mbar_arrive(full_a(sa));
      if (!pre) group_sync();                                 // every thread is done reading this block's records
      kp += S;
      while (kp >= K) { kp -= K; ++cb; }
    }
    // ------------------------------------------------------------------ epilogue (same warps)
    bool go = alive && mbar_wait(acc_full, 0, abort_flag);
    go = __all_sync(0xffffffffu, go);   // tcgen05.ld is warp-collective: all lanes or none
    if (go) {
      tc_fence_after();
      const int quad = warp & 3;                  // TMEM lanes [32*quad, 32*quad+32)
      const int m = m0 + quad * 32 + lane;
      const bool row_ok = m < u.m_total;
      int img = 0, pix = 0;
      if (row_ok) pixel_of(order, m, img, pix);
      const int cout_g = a.Cout / a.groups;
      const int co_base = group * cout_g + n_tile * u.tile_n;
      const int tile_n = u.tile_n;
      const int cols = min(tile_n, cout_g - n_tile * tile_n);   // the last tile of a group may carry padding columns
      // Everything the store loop needs, in registers: per-channel parameters are fetched for the whole slab before
      // the stores, so that no load sits between two stores.
      const float *bias = a.bias, *bn_scale = a.bn_scale;
      const bool relu = a.relu != 0;
      const int n_img = a.n_begin + img;
      const int split_at = a.y_split != nullptr ? a.split_at : a.Cout;      // channels below it go to y
      float *const y_lo = a.y + (long long)n_img * split_at * plane_out + pix;
      float *const y_hi = a.y_split != nullptr
                              ? a.y_split + ((long long)n_img * (a.Cout - split_at) - split_at) * plane_out + pix
                              : nullptr;
      // the four warps of a lane quadrant take 32-column slabs round-robin
      for (int col = (warp >> 2) * 32; col < tile_n; col += (kProducerWarps / 4) * 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col, r);
        tmem_ld_wait();
        if (T::kParts == 2) {
          uint32_t x[32];
          tmem_ld32(tmem_cross + ((uint32_t)(quad * 32) << 16) + (uint32_t)col, x);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(x[j]));
        }
        if (u.dual) {
          // the second issuer's accumulators (main, then cross) hold the other half of the K blocks
          for (int part = 0; part < T::kParts; ++part) {
            uint32_t x[32];
            tmem_ld32((part == 0 ? tmem_base : tmem_cross) + (uint32_t)u.acc2_col + ((uint32_t)(quad * 32) << 16) + (uint32_t)col, x);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(x[j]));
          }
        }
        // bias, then BatchNorm ((v - mean) / sqrt(var + eps) * scale + bias), then ReLU: dcn_epilogue's arithmetic
        if (bn_scale != nullptr) {
          // bias, (v - mean) / sqrt(var + eps) * scale + BatchNorm bias, per-channel values from the table
          const float *ep_params = ep_table();
          const int ep_stride = ep_pitch();
          const float *bs = ep_params + col, *mean = bs + ep_stride, *sd = mean + ep_stride, *scale = sd + ep_stride,
                      *shift = scale + ep_stride;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = __uint_as_float(r[j]);
            if (bias != nullptr) v = __fadd_rn(v, bs[j]);
            v = __fdiv_rn(__fsub_rn(v, mean[j]), sd[j]);
            r[j] = __float_as_uint(__fadd_rn(__fmul_rn(v, scale[j]), shift[j]));
          }
        } else if (bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float b = col + j < cols ? __ldg(bias + co_base + col + j) : 0.0f;
            r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), b));
          }
        }
        if (relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(fmaxf(__uint_as_float(r[j]), 0.0f));
        }
        if (row_ok) {
          const int co0 = co_base + col;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col + j < cols) {
              const int co = co0 + j;
              float *dst = (co < split_at ? y_lo : y_hi) + (long long)co * plane_out;
#if GACB_CHECKED
              // the element must lie inside the tensor it goes to: y [N, split_at, plane] or y_split [N, Cout - split_at, plane]
              const long long rel = co < split_at ? dst - a.y : dst - a.y_split;
              const long long lim = (long long)a.N * (co < split_at ? split_at : a.Cout - split_at) * plane_out;
              if (GACB_INDEX(rel, lim, 14) != rel) continue;
#endif
              __stcs(dst, __uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
    }
  } else if (warp == kLoaderWarp) {
    // ------------------------------------------------------------------ B loader (one lane)
    if (lane == 0) {
      const uint32_t b_bytes = u.b_stage_bytes;
      const unsigned char *src = u.blob + ((size_t)group * u.n_tiles + n_tile) * k_blocks * (size_t)b_bytes;
      int issued = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % SB;
        if (!mbar_wait(empty_b(s), ((kb / SB) & 1) ^ 1, abort_flag)) break;
        if (GACB_DCN_FAULT_INJECT && u.drop_weight_copies) continue;   // nothing issued: nothing to drain later
        mbar_arrive_expect_tx(full_b(s), b_bytes);
        bulk_copy_g2s(smem_u32(b_stages + s * b_stage), src + (size_t)GACB_INDEX(kb, k_blocks, 15) * b_bytes, b_bytes, full_b(s));
        issued = kb + 1;
      }
      if (*abort_flag) {
        // drain: every copy this thread issued must have landed before shared memory is released
        for (int kb = issued > SB ? issued - SB : 0; kb < issued; ++kb) {
          const uint32_t bar = full_b(kb % SB), parity = (kb / SB) & 1;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_try_wait(bar, parity); ++it) {
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer(s) (one lane each)
    const int issuer = warp - kMmaWarp;             // 0, or 1 for the second issuer of a narrow tile
    if (lane == 0 && (issuer == 0 || u.dual)) {
      constexpr bool kTf32 = T::kElemBytes == 4;
      const uint32_t idesc = umma_idesc(kTf32 ? 2 : 1, kTileM, u.tile_n);
      const uint32_t acc_main = tmem_base + (uint32_t)(issuer * u.acc2_col);
      const uint32_t acc_cross = tmem_cross + (uint32_t)(issuer * u.acc2_col);
      const int kb_step = u.dual ? 2 : 1;
      bool ok = true;
      for (int kb = issuer; kb < k_blocks && ok; kb += kb_step) {
        const int sa = kb % SA, sb = kb % SB;
        ok = mbar_wait2(full_a(sa), (kb / SA) & 1, full_b(sb), (kb / SB) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_hi = smem_u32(a_stages + sa * a_stage);
        const uint32_t a_lo = a_hi + kATile;
        const uint32_t b_hi = smem_u32(b_stages + sb * b_stage);
        const uint32_t b_lo = b_hi + (uint32_t)b_part;
#pragma unroll
        for (int k = 0; k < T::kBlockK / T::kUmmaK; ++k) {
          const uint32_t koff = (uint32_t)k * T::kUmmaK * T::kElemBytes;   // 32 bytes per MMA along K
          const uint32_t first = (kb == issuer && k == 0) ? 0u : 1u;
          umma_ss<kTf32>(acc_main, umma_smem_desc<kRowBytes>(a_hi + koff), umma_smem_desc<kRowBytes>(b_hi + koff), idesc, first);
          if (T::kParts == 2) {
            // the two small cross products go to their own accumulator
            umma_ss<kTf32>(acc_cross, umma_smem_desc<kRowBytes>(a_lo + koff), umma_smem_desc<kRowBytes>(b_hi + koff), idesc, first);
            umma_ss<kTf32>(acc_cross, umma_smem_desc<kRowBytes>(a_hi + koff), umma_smem_desc<kRowBytes>(b_lo + koff), idesc, 1u);
          }
        }
        umma_commit(empty_a(sa));   // frees the stages once these MMAs have read them
        umma_commit(empty_b(sb));
      }
      umma_commit(acc_full);     // accumulators complete (or, after an abort, everything issued has retired)
      if (!ok) {
        for (uint32_t it = 0; it < kSpinLimit && !mbar_try_wait(acc_full, 0); ++it) {
        }
      }
    }
  }

  __syncthreads();
  if (tid == 0 && *abort_flag && u.status) atomicExch(u.status, 1);
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)u.tmem_cols);
  }
}

// ----------------------------------------------------------------------------------------------
// Plain convolution with few output channels (the 27-channel conv_offset) from a staged input window
// ----------------------------------------------------------------------------------------------
// A plain stride-1 convolution gathers nothing: the A operand of kernel point (ky, kx) is the input window shifted
// by (ky, kx).  A persistent CTA therefore stages, per 16 x 8 pixel tile and per group of 8 or 16 16-byte chunks of
// input channels, the (16 + Kh - 1) x (8 + Kw - 1) window of the channel-last copy ONCE in shared memory and issues
// one tcgen05.mma per (kernel point, two chunks) whose A descriptor simply starts (ky * window width + kx) texels
// further on: the eight pixels of a tile row are eight consecutive texels of a window row (one 8-row group of the
// K-major operand), the next tile row is one window row further (the descriptor's stride byte offset).  There are
// no producer warps and no A ring: the next windows are copied while the tensor core works on the current one (by
// one thread's tensor copies, or in F32X3 mode by eight converting warps, see below), one thread streams the packed
// weights of a few kernel points at a time through a ring, four warps store finished accumulators.  Taps outside
// the image are zero texels of the window.
//
// With 32 output columns an MMA is a few cycles of tensor work, but a thread issues one only every ~100 cycles,
// whatever its shape (measured: the same with N = 16 or M = 64, and with independent accumulators).  So kWinAccs
// warps issue side by side, each the two-chunk slices k ≡ j (mod kWinAccs) of every kernel point into its own
// accumulator (a partial sum); the epilogue adds the partial sums.  Two such sets sit in tensor memory, so that a
// tile's stores overlap the next tile's products.
//
// Whole images, groups = 1, stride = dilation = 1, at most 64 output channels (32 in F32X3 mode), bias and ReLU
// only.  The three math modes differ in what a window holds:
//   BF16   the bf16 channel-last copy as it is (8 channels per 16-byte chunk, K = 16 per MMA);
//   TF32   the float32 channel-last copy as it is (4 channels per chunk, K = 8 per MMA); the tensor core reads the
//          upper 19 bits of each float, i.e. the activations are truncated to tf32 here where the gather kernel
//          rounds them to nearest (the weights are rounded to nearest in both);
//   F32X3  two windows made by the fill from the float32 copy, hi = bf16(x) and lo = bf16(x - hi), and three
//          products per slice, hi*Whi into a main accumulator, lo*Whi + hi*Wlo into a cross accumulator: the gather
//          kernel's arithmetic.  Eight warps make them, in the un-swizzled K-major layout [chunk][texel][16 bytes]
//          (a core matrix = eight consecutive texels of a window row x 16 bytes; leading byte offset = one chunk).
// In BF16 and TF32 mode nothing touches the texels on their way, so ONE thread brings a window with tensor copies
// (TMA, cp.async.bulk.tensor; zero fill outside the image comes with it) and the fill warps are not launched.  The
// window then has the tensor copy's 128-byte-swizzled K-major layout: a texel is one 128-byte row (8 chunks, XOR-ed
// with the row's position in its 1 KB), the texels of the window follow each other densely, 16 chunks of channels
// are two such sub-windows.  The swizzle is a function of the shared-memory ADDRESS (measured: a descriptor whose
// start address is any multiple of 128 bytes, with a stride between 8-row groups that is no multiple of 1 KB, and
// base offset 0, reads the right rows; filling in the base offset gives wrong ones), so the shifted views work
// exactly as in the un-swizzled layout: start address + (ky * window width + kx) * 128.
template <int MODE>
struct WinTraits;
// kTma: the windows are brought by tensor copies (TMA) in the 128-byte-swizzled layout; otherwise eight warps make
// them (F32X3: the float32 texels have to be split into bf16 pairs on the way) in the un-swizzled chunked layout.
template <>
struct WinTraits<MODE_BF16> {
  using Xt = __nv_bfloat16;
  static constexpr int kChunkCh = 8, kParts = 1;
  static constexpr bool kTf32 = false, kTma = true;
};
template <>
struct WinTraits<MODE_TF32> {
  using Xt = float;
  static constexpr int kChunkCh = 4, kParts = 1;
  static constexpr bool kTf32 = true, kTma = true;
};
template <>
struct WinTraits<MODE_F32X3> {
  using Xt = float;
  static constexpr int kChunkCh = 8, kParts = 2;
  static constexpr bool kTf32 = false, kTma = false;
};
__host__ __device__ inline int win_chunk_channels(int mode) { return mode == MODE_TF32 ? 4 : 8; }
constexpr int kWinTileH = 16, kWinTileW = 8;          // pixels of a tile: 16 rows x 8 columns = 128 MMA rows
constexpr int kWinFillWarps = 8, kWinEpiWarps = 4;
constexpr int kWinAccs = 4;                           // accumulators per tile = issuing threads (one warp each)
constexpr int kWinLoaderWarp = kWinEpiWarps, kWinMmaWarp = kWinEpiWarps + 1, kWinFirstFillWarp = kWinMmaWarp + kWinAccs;
constexpr int kWinThreads = (kWinEpiWarps + 1 + kWinAccs + kWinFillWarps) * 32;
constexpr int kWinMaxBufs = 4, kWinMaxBStages = 8;    // sizes of the barrier arrays
constexpr int kWinStageBytes = 24 * 1024;             // target size of one weight stage
static_assert(kWinTileH * kWinTileW == kTileM, "a tile is one 128-row MMA");

struct ConvWinArgs {
  DcnArgs d;
  const void *xt;               // channel-last copy of images [n_begin, n_end): bf16 in BF16 mode, else float32
  const unsigned char *blob;    // packed weights: [channel group][kernel point][part][chunk][n_pad rows][16 bytes]
  int32_t *status;
  int n_pad;                    // MMA N: output channels rounded up to 32
  int tiles_x, tiles_y, tiles_total;
  int cgroups, cg_channels;     // channel groups per tile and channels per group (8 or 16 chunks)
  int chunks;                   // 16-byte chunks per texel of a window
  int win_h, win_w, win_texels;
  int chunk_stride;             // bytes between the 8-channel chunks of a window: an odd number of 16-byte units, so
                                // that the fill's 16 lanes of one texel (one per chunk) spread over all banks
  int stage_kps, cg_stages;     // kernel points per weight stage; stages per channel group
  int win_bufs, b_stages;       // ring depths
  unsigned win_part_bytes, win_bytes;      // one part of a window (hi or lo); all parts
  unsigned kp_part_bytes, kp_bytes;        // weights of one kernel point: one part; all parts
  unsigned b_stage_bytes;
  int tmem_cols;
  int drop_weight_copies;       // test build only (GACB_DCN_FAULT_INJECT): the loader skips every copy
  // TMA windows (BF16 and TF32): a tensor copy brings a box of {128 bytes of channels, win_w texels, win_h rows}
  unsigned tma_sub_bytes;       // bytes from the sub-window of channels [0, 8 chunks) to that of the next 8 chunks
};

// Un-swizzled K-major operand: core matrices of 8 rows x 16 bytes, `lbo` bytes between the two core matrices an MMA
// reads along K, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_smem_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;                              // descriptor version of sm_100; layout type 0 = no swizzle
  return d;
}

// K-major operand in the 128-byte swizzle whose first row may start at any multiple of 128 bytes: rows of 128
// bytes, `sbo` bytes (any multiple of 128) between 8-row groups.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128_at(uint32_t smem_addr, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B; base offset 0: the swizzle follows the address
  return d;
}
// One tiled tensor copy global -> this CTA's shared memory (4-D map); completion is counted in bytes on `bar`.
// No cluster multicast.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(256) conv_window_pack_weights(const float *__restrict__ w, unsigned char *__restrict__ blob,
                                                               int Cout, int Cin, int K, int n_pad, int cg_channels) {
  using T = WinTraits<MODE>;
  const long long total = (long long)n_pad * Cin * K;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int ci = (int)(i % Cin);
  const int kp = (int)((i / Cin) % K);
  const int n = (int)(i / ((long long)Cin * K));
  const float v = n < Cout ? __ldg(w + ((long long)n * Cin + ci) * K + kp) : 0.0f;
  const int cg = ci / cg_channels, cc = ci - cg * cg_channels;
  const size_t part = (size_t)(cg_channels / T::kChunkCh) * n_pad * 16;
  unsigned char *at = blob + ((size_t)cg * K + kp) * (T::kParts * part) + ((size_t)(cc / T::kChunkCh) * n_pad + n) * 16;
  if (T::kTf32) {
    reinterpret_cast<float *>(at)[cc % T::kChunkCh] = tf32_round(v);
  } else {
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    reinterpret_cast<__nv_bfloat16 *>(at)[cc % T::kChunkCh] = hi;
    if (T::kParts == 2) reinterpret_cast<__nv_bfloat16 *>(at + part)[cc % T::kChunkCh] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
}

template <int MODE>
__global__ void __launch_bounds__(kWinThreads, 1) conv_window_kernel(const __grid_constant__ ConvWinArgs u, const __grid_constant__ CUtensorMap xt_map) {
  using T = WinTraits<MODE>;
  using Xt = typename T::Xt;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const DcnArgs &a = u.d;
  unsigned char *windows = smem;
  unsigned char *b_ring = smem + (size_t)u.win_bufs * u.win_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(b_ring + (size_t)u.b_stages * u.b_stage_bytes);
  // bars: win_full[] | win_empty[] | b_full[] | b_empty[] | acc_full[2] | acc_empty[2] | drain[kWinAccs]
  constexpr int kBars = 2 * kWinMaxBufs + 2 * kWinMaxBStages + 4 + kWinAccs;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kBars);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *bias_s = reinterpret_cast<float *>(tmem_slot + 4);       // n_pad floats (zeros without a bias)
  const uint32_t bar_base = smem_u32(bars);
  auto win_full = [&](int b) { return bar_base + 8u * b; };
  auto win_empty = [&](int b) { return bar_base + 8u * (kWinMaxBufs + b); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * kWinMaxBufs + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * kWinMaxBufs + kWinMaxBStages + s); };
  auto acc_full = [&](int s) { return bar_base + 8u * (2 * kWinMaxBufs + 2 * kWinMaxBStages + s); };
  auto acc_empty = [&](int s) { return bar_base + 8u * (2 * kWinMaxBufs + 2 * kWinMaxBStages + 2 + s); };
  auto drain = [&](int j) { return bar_base + 8u * (2 * kWinMaxBufs + 2 * kWinMaxBStages + 4 + j); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = a.Kh * a.Kw;
  const int plane_out = a.Ho * a.Wo;
  const int tiles_per_image = u.tiles_x * u.tiles_y;
  if (tid == 0) {
    for (int i = 0; i < kWinMaxBufs; ++i) {
      mbar_init(win_full(i), T::kTma ? 1 : kWinFillWarps);
      mbar_init(win_empty(i), kWinAccs);      // one commit per issuing thread
    }
    for (int i = 0; i < kWinMaxBStages; ++i) {
      mbar_init(b_full(i), 1);
      mbar_init(b_empty(i), kWinAccs);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full(i), kWinAccs);
      mbar_init(acc_empty(i), kWinEpiWarps);
    }
    for (int i = 0; i < kWinAccs; ++i) mbar_init(drain(i), 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (tid < u.n_pad) bias_s[tid] = (a.bias != nullptr && tid < a.Cout) ? __ldg(a.bias + tid) : 0.0f;
  if (warp == kWinMmaWarp) tmem_alloc(smem_u32(tmem_slot), (uint32_t)u.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int set_cols = T::kParts * kWinAccs * u.n_pad;      // tensor-memory columns of one tile's accumulators

  if (warp >= kWinFirstFillWarp) {
    if constexpr (T::kTma) {
      // ---------------------------------------------------------------- window fill by tensor copies (one thread)
      if (warp == kWinFirstFillWarp && lane == 0) {
        const int subs = u.chunks / 8;                         // one tensor copy per 128 bytes of channels
        int buf = 0, round = 0, issued = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < u.tiles_total && ok; t += gridDim.x) {
          const int img = t / tiles_per_image, r = t - img * tiles_per_image;
          const int ty = r / u.tiles_x, tx = r - ty * u.tiles_x;
          const int y0 = ty * kWinTileH - a.ph, x0 = tx * kWinTileW - a.pw;   // may be negative: the copy fills zeros there
          for (int cg = 0; cg < u.cgroups; ++cg) {
            if (!mbar_wait(win_empty(buf), (round & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(win_full(buf), (uint32_t)subs * 128u * (uint32_t)u.win_texels);
            for (int sub = 0; sub < subs; ++sub)
              tma_load_4d(smem_u32(windows + (size_t)buf * u.win_bytes + (size_t)sub * u.tma_sub_bytes), &xt_map,
                          cg * u.cg_channels + sub * 8 * T::kChunkCh, x0, y0, img, win_full(buf));
            ++issued;
            if (++buf == u.win_bufs) { buf = 0; ++round; }
          }
        }
        if (*abort_flag && issued > 0) {
          // drain: every copy issued must have landed before shared memory is released (as in the weight loader)
          for (int back = 1; back <= u.win_bufs && back <= issued; ++back) {
            int pb = buf - back, pr = round;
            if (pb < 0) { pb += u.win_bufs; --pr; }
            for (uint32_t poll = 0; poll < kSpinLimit && !mbar_try_wait(win_full(pb), pr & 1); ++poll) {
            }
          }
        }
      }
    } else {
      // ---------------------------------------------------------------- window fill (eight warps), F32X3
      // A thread makes the 16-byte pieces (texel, chunk) with chunk = ft % 8 (neighbouring lanes read one texel's
      // channels) and texel = ft / 8, + 32, ...: eight float32 channels become a bf16 hi piece and a bf16 lo piece.
      const int ft = tid - kWinFirstFillWarp * 32;                    // 0 .. 255
      const int c = ft & 7, tt0 = ft >> 3, tt_step = (kWinFillWarps * 32) >> 3;
      const int wy0 = tt0 / u.win_w, wx0 = tt0 - wy0 * u.win_w;
      bool alive = true;
      int buf = 0, round = 0;                                         // ring position: step % win_bufs, step / win_bufs
      for (int t = blockIdx.x; t < u.tiles_total; t += gridDim.x) {
        const int img = t / tiles_per_image, r = t - img * tiles_per_image;
        const int ty = r / u.tiles_x, tx = r - ty * u.tiles_x;
        const int y0 = ty * kWinTileH - a.ph, x0 = tx * kWinTileW - a.pw;     // input position of window texel (0, 0)
        const Xt *image = static_cast<const Xt *>(u.xt) + (size_t)img * a.H * a.W * a.Cin;
        for (int cg = 0; cg < u.cgroups; ++cg) {
          if (alive) alive = mbar_wait_warp(win_empty(buf), (round & 1) ^ 1, abort_flag, lane);
          if (alive) {
            unsigned char *win = windows + (size_t)buf * u.win_bytes;
            unsigned char *dst = win + (size_t)c * u.chunk_stride + (size_t)tt0 * 16;
            const Xt *src = image + cg * u.cg_channels + c * T::kChunkCh;
            int wy = wy0, wx = wx0;
            for (int tt = tt0; tt < u.win_texels; tt += tt_step, dst += tt_step * 16) {
              const int gy = y0 + wy, gx = x0 + wx;
              uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;         // zero padding outside the image
              if (gy >= 0 && gy < a.H && gx >= 0 && gx < a.W) {
                const int e = (int)GACB_INDEX((gy * a.W + gx) * a.Cin, (long long)a.H * a.W * a.Cin, 12);
                const float4 v0 = __ldg(reinterpret_cast<const float4 *>(src + e));
                const float4 v1 = __ldg(reinterpret_cast<const float4 *>(src + e) + 1);
                const float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                uint32_t h[4], l[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const __nv_bfloat16 h0 = __float2bfloat16_rn(x[2 * k]), h1 = __float2bfloat16_rn(x[2 * k + 1]);
                  h[k] = pack_bf16x2(h0, h1);
                  l[k] = pack_bf16x2(__float2bfloat16_rn(x[2 * k] - __bfloat162float(h0)),
                                     __float2bfloat16_rn(x[2 * k + 1] - __bfloat162float(h1)));
                }
                hi = make_uint4(h[0], h[1], h[2], h[3]);
                lo = make_uint4(l[0], l[1], l[2], l[3]);
              }
              *reinterpret_cast<uint4 *>(dst) = hi;
              *reinterpret_cast<uint4 *>(dst + u.win_part_bytes) = lo;
              wx += tt_step;
              while (wx >= u.win_w) { wx -= u.win_w; ++wy; }
            }
            fence_proxy_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
          }
          // one arrival per warp, after every lane's writes are fenced
          const bool warp_alive = __all_sync(0xffffffffu, alive);
          if (warp_alive && lane == 0) mbar_arrive(win_full(buf));
          if (++buf == u.win_bufs) { buf = 0; ++round; }
        }
      }
    }
  } else if (warp == kWinLoaderWarp) {
    // ------------------------------------------------------------------ weight loader (one lane)
    if (lane == 0) {
      int s = 0, round = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < u.tiles_total && ok; t += gridDim.x)
        for (int cg = 0; cg < u.cgroups && ok; ++cg)
          for (int k0 = 0; k0 < K; k0 += u.stage_kps) {
            if (!mbar_wait(b_empty(s), (round & 1) ^ 1, abort_flag)) { ok = false; break; }
            const uint32_t bytes = (uint32_t)min(u.stage_kps, K - k0) * u.kp_bytes;
            mbar_arrive_expect_tx(b_full(s), bytes);
            if (!(GACB_DCN_FAULT_INJECT && u.drop_weight_copies)) {
              bulk_copy_g2s(smem_u32(b_ring + (size_t)s * u.b_stage_bytes), u.blob + ((size_t)cg * K + k0) * u.kp_bytes,
                            bytes, b_full(s));
              ++issued;
            }
            if (++s == u.b_stages) { s = 0; ++round; }
          }
      if (*abort_flag && issued > 0) {
        // drain: every copy issued must have landed before shared memory is released.  Stage s, round `round` is the
        // next one that would have been issued; the b_stages before it may still be in flight.
        for (int back = 1; back <= u.b_stages && back <= issued; ++back) {
          int ps = s - back, pr = round;
          if (ps < 0) { ps += u.b_stages; --pr; }
          for (uint32_t poll = 0; poll < kSpinLimit && !mbar_try_wait(b_full(ps), pr & 1); ++poll) {
          }
        }
      }
    }
  } else if (warp >= kWinMmaWarp) {
    // ------------------------------------------------------------------ MMA issuers (kWinAccs warps)
    // The whole warp runs the loop with warp-uniform values (the warp's number comes out of a shuffle, so the
    // compiler knows it is uniform) and one elected lane executes each tcgen05 instruction: descriptors and
    // addresses then live in uniform registers instead of being moved there one MMA at a time.
    {
      const int issuer = __shfl_sync(0xffffffffu, warp - kWinMmaWarp, 0);   // takes the slices issuer, issuer + kWinAccs, ...
      const uint32_t idesc = umma_idesc(T::kTf32 ? 2 : 1, kTileM, u.n_pad);
      constexpr bool tma = T::kTma;
      // bytes from a texel to the next one, and texels per window row, in the window's layout
      const uint32_t texel_bytes = tma ? 128u : 16u, row_texels = (uint32_t)u.win_w;
      const uint32_t a_lbo = (uint32_t)u.chunk_stride, a_sbo = row_texels * texel_bytes;
      const uint32_t b_lbo = (uint32_t)u.n_pad * 16u, b_sbo = 128u;
      // descriptors with a zero start address; a start address is added in 16-byte units
      const uint64_t a_desc0 = umma_smem_desc_plain(0, a_lbo, a_sbo), b_desc0 = umma_smem_desc_plain(0, b_lbo, b_sbo);
      // one slice = the two chunks an MMA reads along K (16 channels, 8 in TF32 mode), in 16-byte units
      const uint32_t a_k16 = tma ? 2u : (2u * a_lbo) >> 4, b_k16 = (2u * b_lbo) >> 4;   // TMA rows: 32 bytes along the row
      const int k16_quads = u.chunks / (2 * kWinAccs);
      const uint32_t a_lo = u.win_part_bytes >> 4, b_lo = u.kp_part_bytes >> 4;     // F32X3: from the hi part to the lo part
      const uint32_t windows_addr = smem_u32(windows), ring_addr = smem_u32(b_ring);
      bool ok = true;
      int buf = 0, wround = 0, s = 0, bround = 0, it = 0;
      for (int t = blockIdx.x; t < u.tiles_total && ok; t += gridDim.x, ++it) {
        const int set = it & 1, use = it >> 1;
        ok = mbar_wait_uniform(acc_empty(set), (use & 1) ^ 1, abort_flag, lane);   // the epilogue has read this set's last tile
        const uint32_t acc = tmem_base + (uint32_t)(set * set_cols + issuer * u.n_pad);
        const uint32_t acc_cross = acc + (uint32_t)(kWinAccs * u.n_pad);   // F32X3 only
        uint32_t accumulate = 0;                                      // 0 for the first MMA into the accumulator
        for (int cg = 0; cg < u.cgroups && ok; ++cg) {
          ok = mbar_wait_uniform(win_full(buf), wround & 1, abort_flag, lane);
          const uint32_t win = windows_addr + (uint32_t)buf * u.win_bytes;
          int ky = 0, kx = 0;
          for (int k0 = 0; k0 < K && ok; k0 += u.stage_kps) {
            ok = mbar_wait_uniform(b_full(s), bround & 1, abort_flag, lane);
            if (!ok) break;
            tc_fence_after();
            const int k1 = min(K, k0 + u.stage_kps);
            uint64_t bd = b_desc0 + (uint64_t)((ring_addr + (uint32_t)s * u.b_stage_bytes) >> 4) + issuer * b_k16;
            for (int kp = k0; kp < k1; ++kp) {
              const uint32_t tap = win + ((uint32_t)ky * row_texels + (uint32_t)kx) * texel_bytes;   // first row of this kernel point
              // TMA layout: the q-th group of kWinAccs slices is the q-th sub-window; chunked layout: 2 * kWinAccs chunks on
              uint64_t ad = (tma ? umma_smem_desc_sw128_at(tap, a_sbo) : a_desc0 + (uint64_t)(tap >> 4)) + issuer * a_k16;
              const uint32_t a_next = tma ? (u.tma_sub_bytes >> 4) : kWinAccs * a_k16;
              for (int q = 0; q < k16_quads; ++q) {
                if (elect_one()) {
                  umma_ss<T::kTf32>(acc, ad, bd, idesc, accumulate);
                  if constexpr (T::kParts == 2) {
                    umma_ss<false>(acc_cross, ad + a_lo, bd, idesc, accumulate);
                    umma_ss<false>(acc_cross, ad, bd + b_lo, idesc, 1u);
                  }
                }
                accumulate = 1u;
                ad += a_next;
                bd += kWinAccs * b_k16;      // after the last slice of a kernel point: the next point's first slice
              }
              if constexpr (T::kParts == 2) bd += b_lo;   // ... which lies behind this point's lo part
              if (++kx == a.Kw) { kx = 0; ++ky; }
            }
            if (elect_one()) umma_commit(b_empty(s));       // the stage is free once these MMAs have read it
            if (++s == u.b_stages) { s = 0; ++bround; }
          }
          if (ok && elect_one()) umma_commit(win_empty(buf));
          if (++buf == u.win_bufs) { buf = 0; ++wround; }
        }
        if (ok && elect_one()) umma_commit(acc_full(set));
      }
      if (!ok) {
        // after an abort: everything this warp issued must have retired before shared and tensor memory are released
        if (elect_one()) umma_commit(drain(issuer));
        if (lane == 0)
          for (uint32_t poll = 0; poll < kSpinLimit && !mbar_try_wait(drain(issuer), 0); ++poll) {
          }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (four warps, one per TMEM lane quadrant)
    const int quad = warp & 3;
    const int m = quad * 32 + lane;                 // tile row: pixel (m / 8, m % 8) of the tile
    const int split_at = a.y_split != nullptr ? a.split_at : a.Cout;      // channels below it go to y
    const bool relu = a.relu != 0;
    int it = 0;
    for (int t = blockIdx.x; t < u.tiles_total; t += gridDim.x, ++it) {
      const int set = it & 1, use = it >> 1;
      const bool go = mbar_wait_warp(acc_full(set), use & 1, abort_flag, lane);   // tcgen05.ld is warp-collective
      if (!go) break;
      tc_fence_after();
      const int img = t / tiles_per_image, r = t - img * tiles_per_image;
      const int ty = r / u.tiles_x, tx = r - ty * u.tiles_x;
      const int oy = ty * kWinTileH + (m >> 3), ox = tx * kWinTileW + (m & 7);
      const bool row_ok = oy < a.Ho && ox < a.Wo;
      const int n_img = a.n_begin + img;
      const int pix = oy * a.Wo + ox;
      float *const y_lo = a.y + (long long)n_img * split_at * plane_out + pix;
      float *const y_hi = a.y_split != nullptr
                              ? a.y_split + ((long long)n_img * (a.Cout - split_at) - split_at) * plane_out + pix
                              : nullptr;
      const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(set * set_cols);
      for (int col = 0; col < u.n_pad; col += 32) {
        // the tile's value is the sum of its partial accumulators (main ones first, then F32X3's cross ones)
        uint32_t rr[32], xa[32];
        tmem_ld32(lane_base + (uint32_t)col, rr);
        tmem_ld32(lane_base + (uint32_t)(u.n_pad + col), xa);
        tmem_ld_wait();
#pragma unroll
        for (int p = 2; p < T::kParts * kWinAccs; ++p) {
#pragma unroll
          for (int j = 0; j < 32; ++j) rr[j] = __float_as_uint(__fadd_rn(__uint_as_float(rr[j]), __uint_as_float(xa[j])));
          tmem_ld32(lane_base + (uint32_t)(p * u.n_pad + col), xa);
          tmem_ld_wait();
        }
        if (col + 32 >= u.n_pad) {
          // everything of this tile has been read: the issuing thread may start the tile after next in this set
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(set));
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) rr[j] = __float_as_uint(__fadd_rn(__uint_as_float(rr[j]), __uint_as_float(xa[j])));
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int co = col + j;
            if (co < a.Cout) {
              float v = __fadd_rn(__uint_as_float(rr[j]), bias_s[co]);
              if (relu) v = fmaxf(v, 0.0f);
              float *dst = (co < split_at ? y_lo : y_hi) + (long long)co * plane_out;
#if GACB_CHECKED
              const long long rel = co < split_at ? dst - a.y : dst - a.y_split;
              const long long lim = (long long)a.N * (co < split_at ? split_at : a.Cout - split_at) * plane_out;
              if (GACB_INDEX(rel, lim, 14) != rel) continue;
#endif
              __stcs(dst, v);
            }
          }
        }
      }
    }
  }

  __syncthreads();
  if (tid == 0 && *abort_flag && u.status) atomicExch(u.status, 1);
  if (warp == kWinMmaWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)u.tmem_cols);
  }
}

// 0 = plain convolutions always take the gather kernel; 1 (default) = the window kernel where it applies.
std::atomic<int> g_conv_window_path{1};


// Does the window kernel apply, and with which shape?  (Plain convolution over whole images.)
// Threads of a launch: with tensor copies only the first of the fill warps is needed.
inline int win_threads(int mode) { return parts_of(mode) == 1 ? (kWinFirstFillWarp + 1) * 32 : kWinThreads; }

bool plan_conv_window(const DcnArgs &a, int mode, size_t blob_capacity, ConvWinArgs &u, size_t &smem) {
  if (!g_conv_window_path.load(std::memory_order_relaxed)) return false;
  const bool whole = a.m_first == 0 && a.row_begin == 0 && a.row_end == a.Ho &&
                     a.m_count == (long long)(a.n_end - a.n_begin) * a.Ho * a.Wo;
  if (a.offset != nullptr || !whole || a.bn_scale != nullptr) return false;
  if (a.groups != 1 || a.sh != 1 || a.sw != 1 || a.dh != 1 || a.dw != 1) return false;
  const int chunk_ch = win_chunk_channels(mode), parts = parts_of(mode);
  // a channel group is 8 or 16 chunks of a texel; F32X3 keeps two windows per group and takes the smaller one
  if (a.Cout > (parts == 2 ? 32 : 64) || a.Cin % (8 * chunk_ch) || a.Kh * a.Kw > 49) return false;
  if ((long long)(a.n_end - a.n_begin) * a.H * a.W * a.Cin > 2147483647LL) return false;
  const int K = a.Kh * a.Kw;
  u.n_pad = (a.Cout + 31) / 32 * 32;
  u.win_h = kWinTileH + a.Kh - 1;
  u.win_w = kWinTileW + a.Kw - 1;
  u.win_texels = u.win_h * u.win_w;
  const bool tma = parts == 1;       // WinTraits<mode>::kTma
  if (tma && (u.win_w > 256 || u.win_h > 256)) return false;      // box limits of a tensor copy
  u.chunks = (parts == 1 && a.Cin % (16 * chunk_ch) == 0) ? 16 : 8;
  u.cg_channels = u.chunks * chunk_ch;
  u.cgroups = a.Cin / u.cg_channels;
  u.chunk_stride = (u.win_texels | 1) * 16;
  // TMA layout: one sub-window of 128-byte texel rows per 8 chunks, each starting at a multiple of 1024 bytes
  u.tma_sub_bytes = (unsigned)((128 * u.win_texels + 1023) / 1024 * 1024);
  u.win_part_bytes = tma ? (unsigned)(u.chunks / 8) * u.tma_sub_bytes
                           : (unsigned)(((size_t)u.chunks * u.chunk_stride + 127) / 128 * 128);
  u.win_bytes = (unsigned)parts * u.win_part_bytes;
  u.kp_part_bytes = (unsigned)((size_t)u.chunks * u.n_pad * 16);
  u.kp_bytes = (unsigned)parts * u.kp_part_bytes;
  u.stage_kps = std::max(1, std::min(K, kWinStageBytes / (int)u.kp_bytes));
  u.cg_stages = (K + u.stage_kps - 1) / u.stage_kps;
  u.b_stage_bytes = (unsigned)u.stage_kps * u.kp_bytes;
  if ((size_t)u.cgroups * K * u.kp_bytes > blob_capacity) return false;
  // the un-swizzled descriptor's offsets are 14-bit counts of 16 bytes
  if ((size_t)u.chunk_stride >= (1u << 18) || (size_t)u.n_pad * 16 >= (1u << 18)) return false;
  const size_t fixed = 1024 /*alignment*/ + (2 * kWinMaxBufs + 2 * kWinMaxBStages + 4 + kWinAccs) * 8 + 16 + 64 * sizeof(float);
  const size_t budget = 227 * 1024;
  u.win_bufs = 3;
  while (u.win_bufs > 2 && fixed + (size_t)u.win_bufs * u.win_bytes + 3 * (size_t)u.b_stage_bytes > budget) --u.win_bufs;
  if (fixed + (size_t)u.win_bufs * u.win_bytes + 2 * (size_t)u.b_stage_bytes > budget) return false;
  const size_t left = budget - fixed - (size_t)u.win_bufs * u.win_bytes;
  u.b_stages = (int)std::min<size_t>(kWinMaxBStages, left / u.b_stage_bytes);
  smem = fixed + (size_t)u.win_bufs * u.win_bytes + (size_t)u.b_stages * u.b_stage_bytes;
  u.tiles_x = (a.Wo + kWinTileW - 1) / kWinTileW;
  u.tiles_y = (a.Ho + kWinTileH - 1) / kWinTileH;
  u.tiles_total = (a.n_end - a.n_begin) * u.tiles_x * u.tiles_y;
  int cols = 32;
  while (cols < 2 * parts * kWinAccs * u.n_pad) cols <<= 1;
  u.tmem_cols = cols;      // at most 2 * 4 * 64 = 2 * 2 * 4 * 32 = 512 columns
  return true;
}

template <int MODE>
int launch_conv_window(const DcnArgs &a, ConvWinArgs &u, size_t smem, const void *xt, unsigned char *blob,
                       int32_t *status, cudaStream_t stream, int reuse_flags, int sms, int device) {
  const int K = a.Kh * a.Kw;
  if (!(reuse_flags & GACB_DCN_REUSE_WEIGHTS)) {
    const long long welems = (long long)u.n_pad * a.Cin * K;
    conv_window_pack_weights<MODE><<<(int)((welems + 255) / 256), 256, 0, stream>>>(a.w, blob, a.Cout, a.Cin, K, u.n_pad,
                                                                                  u.cg_channels);
    const int rc = check_cuda(cudaGetLastError(), "conv_window_pack_weights launch");
    if (rc != GACB_OK) return rc;
  }
  u.d = a;
  u.xt = xt;
  u.blob = blob;
  u.status = status;
  u.drop_weight_copies = (reuse_flags & kTestDropWeightCopies) ? 1 : 0;
  CUtensorMap xt_map{};
  if (WinTraits<MODE>::kTma) {
    // X_t as a 4-D tensor (channels, width, height, image), innermost first; a box is one window of one channel group
    TensorMapEncoder fn = nullptr;
    const int rc = tensor_map_encoder(&fn);
    if (rc != GACB_OK) return rc;
    const cuuint64_t es = WinTraits<MODE>::kTf32 ? 4 : 2;
    const cuuint64_t dims[4] = {(cuuint64_t)a.Cin, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)(a.n_end - a.n_begin)};
    const cuuint64_t strides[3] = {(cuuint64_t)a.Cin * es, (cuuint64_t)a.W * a.Cin * es, (cuuint64_t)a.H * a.W * a.Cin * es};
    const cuuint32_t box[4] = {(cuuint32_t)(8 * win_chunk_channels(MODE)), (cuuint32_t)u.win_w, (cuuint32_t)u.win_h, 1u};
    const cuuint32_t unit[4] = {1u, 1u, 1u, 1u};
    const CUresult res = fn(&xt_map, WinTraits<MODE>::kTf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                            const_cast<void *>(xt), dims, strides, box, unit, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GACB_ERR_CUDA, "conv2d: cuTensorMapEncodeTiled failed with %d", (int)res);
  }
  static std::mutex attr_lock;      // one flag set per math mode (this function is a template)
  static bool attr_done[64] = {};
  {
    std::lock_guard<std::mutex> guard(attr_lock);
    if (!attr_done[device]) {
      const int rc = check_cuda(cudaFuncSetAttribute(conv_window_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     227 * 1024),
                                "cudaFuncSetAttribute(conv_window_kernel)");
      if (rc != GACB_OK) return rc;
      attr_done[device] = true;
    }
  }
  const int grid = std::min(u.tiles_total, sms);
  conv_window_kernel<MODE><<<grid, win_threads(MODE), smem, stream>>>(u, xt_map);
  return check_cuda(cudaGetLastError(), "conv_window_kernel launch");
}

// What launch_umma launches for a problem on a GPU with `sms` multiprocessors; fills the tiling fields of `u`.
struct UmmaLaunch {
  bool narrow;
  dim3 grid;
  int threads;
  size_t smem;
};

template <int MODE>
UmmaLaunch shape_umma_launch(const DcnArgs &a, const UmmaPlan &p, int sms, UmmaArgs &u) {
  using T = ModeTraits<MODE>;
  u.tile_n = p.tile_n;
  u.n_tiles = p.n_tiles;
  u.k_blocks = p.k_blocks;
  u.chan_blocks = p.chan_blocks;
  u.m_tiles = p.m_tiles;
  u.m_total = (int)p.m_total;
  u.b_stage_bytes = (unsigned)p.b_stage_bytes;
  // whole images (no row or pixel restriction): 8 x 16 pixel blocks along M
  const bool whole = a.m_first == 0 && a.row_begin == 0 && a.row_end == a.Ho &&
                     a.m_count == (long long)(a.n_end - a.n_begin) * a.Ho * a.Wo;
  u.block_h = whole ? GACB_DCN_BLOCK_H : 0;
  u.block_w = (whole && GACB_DCN_BLOCK_H) ? kTileM / (GACB_DCN_BLOCK_H ? GACB_DCN_BLOCK_H : 1) : 0;
  if (!u.block_w) u.block_h = 0;
  // accumulator columns: tile_n, twice that with the cross-product accumulator; allocations are powers of two >= 32
  const int slab = (p.tile_n + 31) / 32 * 32;
  u.cross_col = slab;
  const int set_cols = T::kParts * slab;      // one issuer's accumulators
  // two issuers when the tile is narrow; each must always meet the same stages of both rings (even ring sizes)
  static_assert(CtaShape<true>::kAStages % 2 == 0 && kBStages % 2 == 0, "two issuers need even rings");
  u.dual = (p.tile_n <= 64 && p.k_blocks >= 2) ? 1 : 0;
  u.acc2_col = set_cols;
  int cols = 32;
  while (cols < (u.dual ? 2 * set_cols : set_cols)) cols <<= 1;
  u.tmem_cols = cols;
  // every (kernel point, deformable group) pair a CTA's channels touch, if the table can hold them
  const int cin_g_ = a.Cin / a.groups, cin_dg_ = a.Cin / a.dgroups;
  // deformable groups the channels of one convolution group can span (groups and deformable groups need not nest)
  int dg_per_cta = 1;
  for (int g = 0; g < a.groups; ++g)
    dg_per_cta = std::max(dg_per_cta, ((g + 1) * cin_g_ - 1) / cin_dg_ - (g * cin_g_) / cin_dg_ + 1);
  const int wanted = a.Kh * a.Kw * dg_per_cta;
  u.precomputed = wanted <= kMaxRecordSlots ? 1 : 0;
  // Two CTAs per SM (CtaShape<true>; at most 256 TMEM columns each) when the tile is narrow and the grid is more
  // than one wave of single CTAs; a grid that fits one wave is faster with the wide shape's four producer groups.
  UmmaLaunch l;
  l.narrow = p.tile_n <= 64 && (long long)p.m_tiles * p.n_tiles * a.groups > sms;
  u.record_slots = u.precomputed ? wanted : (l.narrow ? CtaShape<true>::kGroups : kGroups);
  l.smem = SmemLayout<MODE>::total(p.tile_n, u.record_slots, l.narrow ? CtaShape<true>::kAStages : kAStages,
                                   a.bn_scale ? kEpilogueParams : 0);
  l.grid = dim3(p.m_tiles, p.n_tiles, a.groups);
  l.threads = l.narrow ? CtaShape<true>::kThreads : CtaShape<false>::kThreads;
  return l;
}

template <int MODE>
int launch_umma(const DcnArgs &a, const UmmaPlan &p, void *workspace, int32_t *status, cudaStream_t stream,
                int reuse_flags = 0, size_t workspace_bytes = 0) {
  using T = ModeTraits<MODE>;
  // workspace = [channel-last copy | packed weights], or with GACB_DCN_INPUT_AT_END [packed weights | ... | copy]
  // with the copy in the last xt_bytes of the workspace (so that calls with different weights can share it)
  const bool at_end = (reuse_flags & GACB_DCN_INPUT_AT_END) != 0;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  unsigned char *blob = at_end ? ws : ws + p.xt_bytes;
  const int HW = a.H * a.W;
  using XtT = typename std::conditional<T::kXtBytes == 4, float, __nv_bfloat16>::type;
  XtT *xt = reinterpret_cast<XtT *>(at_end ? ws + (workspace_bytes - p.xt_bytes) : ws);
  const int n_images = a.n_end - a.n_begin;
  const uintptr_t x_addr = reinterpret_cast<uintptr_t>(a.x);
  if (reuse_flags & GACB_DCN_REUSE_INPUT) {
    // the caller vouches that the workspace still holds this X's channel-last copy
  } else if (a.Cin % 32 == 0 && HW % 4 == 0 && x_addr % 16 == 0) {
    dcn_nhwc_vec_kernel<XtT, 4><<<dim3((HW + 127) / 128, a.Cin / 32, n_images), 256, 0, stream>>>(a.x, xt, a.Cin, HW, a.n_begin);
  } else if (a.Cin % 32 == 0 && HW % 2 == 0 && x_addr % 8 == 0) {
    dcn_nhwc_vec_kernel<XtT, 2><<<dim3((HW + 127) / 128, a.Cin / 32, n_images), 256, 0, stream>>>(a.x, xt, a.Cin, HW, a.n_begin);
  } else {
    dcn_nhwc_kernel<XtT><<<dim3((HW + 31) / 32, (a.Cin + 31) / 32, n_images), 256, 0, stream>>>(a.x, xt, a.Cin, HW, a.n_begin);
  }
  int rc = check_cuda(cudaGetLastError(), "dcn_nhwc_kernel launch");
  if (rc != GACB_OK) return rc;
  int sms = 148, device = 0;
  rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != GACB_OK) return rc;
  rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute(SM count)");
  if (rc != GACB_OK) return rc;
  if (device < 0 || device >= 64) return fail(GACB_ERR_UNSUPPORTED, "dcnv2: device ordinal %d is out of range", device);
  {
    // a plain convolution with few output channels reads shifted windows instead of gathering (its own weight layout)
    ConvWinArgs cw{};
    size_t cw_smem = 0;
    if (plan_conv_window(a, MODE, p.blob_bytes, cw, cw_smem))
      return launch_conv_window<MODE>(a, cw, cw_smem, xt, blob, status, stream, reuse_flags, sms, device);
  }
  const int cin_g = a.Cin / a.groups, K = a.Kh * a.Kw;
  const long long welems = (long long)a.groups * p.n_tiles * p.tile_n * cin_g * K;   // padding rows included
  if (!(reuse_flags & GACB_DCN_REUSE_WEIGHTS))
    dcn_pack_weights<<<(int)((welems + 255) / 256), 256, 0, stream>>>(a.w, blob, a.Cout, cin_g, K, a.groups, p.tile_n,
                                                                    p.n_tiles, p.k_blocks, MODE);
  rc = check_cuda(cudaGetLastError(), "dcn_pack_weights launch");
  if (rc != GACB_OK) return rc;

  UmmaArgs u;
  u.d = a;
  u.xt = xt;
  u.blob = blob;
  u.status = status;
  u.drop_weight_copies = (reuse_flags & kTestDropWeightCopies) ? 1 : 0;
  const UmmaLaunch shape = shape_umma_launch<MODE>(a, p, sms, u);
  const bool narrow = shape.narrow;
  const size_t smem = shape.smem;
  const bool plain = a.offset == nullptr;
  auto kernel = narrow ? (plain ? dcn_umma_kernel<MODE, true, true> : dcn_umma_kernel<MODE, false, true>)
                       : (plain ? dcn_umma_kernel<MODE, true, false> : dcn_umma_kernel<MODE, false, false>);
  // Function attributes once per device and kernel variant (calls may come from several host threads): the largest
  // shared-memory size any shape of this variant can ask for, and, for the narrow shape, all of the unified array
  // as shared memory so that two CTAs fit.
  static std::mutex attr_lock;
  static bool attr_done[64][2][2] = {};
  {
    std::lock_guard<std::mutex> guard(attr_lock);
    if (!attr_done[device][narrow][plain]) {
      rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024),
                      "cudaFuncSetAttribute(dcn_umma_kernel)");
      if (rc != GACB_OK) return rc;
      if (narrow) {
        rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared),
                        "cudaFuncSetAttribute(dcn_umma_kernel carve-out)");
        if (rc != GACB_OK) return rc;
      }
      attr_done[device][narrow][plain] = true;
    }
  }
  kernel<<<shape.grid, shape.threads, smem, stream>>>(u);
  return check_cuda(cudaGetLastError(), "dcn_umma_kernel launch");
}

int validate(DcnArgs &a, const float *x, const float *offset, const float *mask, const float *w, const float *bias,
             float *y, int N, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int ph, int pw, int dh,
             int dw, int groups, int dgroups, int n_begin, int n_end, int math_mode, int pb = -1, int pr = -1,
             bool plain = false) {
  // ph/pw pad the top and left; pb/pr the bottom and right (the same as top/left unless given: plain convolution
  // carries four pads, src/gac/core/ops.py:642).  `plain` = no offset/mask operands.
  if (pb < 0) pb = ph;
  if (pr < 0) pr = pw;
  if (N < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0)
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: extents must be positive");
  if (sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0 || groups <= 0 || dgroups <= 0)
    return fail(GACB_ERR_INVALID_ARGUMENT,
                "dcnv2: requires positive stride/dilation/groups and nonnegative padding");
  if (math_mode != MODE_F32X3 && math_mode != MODE_TF32 && math_mode != MODE_BF16)
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: math_mode %d is not a gacb_dcn_math value", math_mode);
  if (Cin % groups || Cin % dgroups || Cout % groups)
    return fail(GACB_ERR_SHAPE_MISMATCH, "dcnv2: channels must be positive and divisible by their groups");
  if (H + ph + pb < dh * (Kh - 1) + 1 || W + pw + pr < dw * (Kw - 1) + 1)
    return fail(GACB_ERR_SHAPE_MISMATCH, "dcnv2: kernel exceeds padded input");
  if (n_begin < 0 || n_end < n_begin || n_end > N)
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: image range [%d,%d) is outside [0,%d)", n_begin, n_end, N);
  a.Ho = (H + ph + pb - dh * (Kh - 1) - 1) / sh + 1;
  a.Wo = (W + pw + pr - dw * (Kw - 1) - 1) / sw + 1;
  const long long lim = 2147483647LL;
  if ((long long)N * Cin * H * W > lim || (long long)N * Cout * a.Ho * a.Wo > lim ||
      (long long)N * 2 * dgroups * Kh * Kw * a.Ho * a.Wo > lim || (long long)Cout * (Cin / groups) * Kh * Kw > lim)
    return fail(GACB_ERR_UNSUPPORTED, "dcnv2: a tensor exceeds the 32-bit indexing range");
  if (n_end > n_begin && (!x || !w || !y || (!plain && (!offset || !mask))))
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: a tensor pointer is NULL");
  a.x = x; a.offset = offset; a.mask = mask; a.w = w; a.bias = bias; a.y = y;
  a.N = N; a.Cin = Cin; a.H = H; a.W = W; a.Cout = Cout; a.Kh = Kh; a.Kw = Kw;
  a.sh = sh; a.sw = sw; a.ph = ph; a.pw = pw; a.dh = dh; a.dw = dw;
  a.groups = groups; a.dgroups = dgroups; a.n_begin = n_begin; a.n_end = n_end;
  a.row_begin = 0; a.row_end = a.Ho;
  a.m_first = 0; a.m_count = (n_end - n_begin) * a.Ho * a.Wo;   // below 2^31 by the check above
  return GACB_OK;
}

}  // namespace
}  // namespace gacb

using namespace gacb;

GACB_API size_t gacb_dcnv2_workspace_bytes(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw,
                                           int ph, int pw, int dh, int dw, int groups, int deform_groups,
                                           int math_mode) {
  DcnArgs a{};
  math_mode &= 0xff;   // reuse flags do not change the size
  if (n <= 0) return 0;
  if (validate(a, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, n, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh,
               dw, groups, deform_groups, 0, 0, math_mode) != GACB_OK)
    return 0;
  a.n_begin = 0;
  a.n_end = n;
  a.m_count = n * a.Ho * a.Wo;
  UmmaPlan p;
  if (!plan_umma(a, math_mode, p)) return 0;
  return p.xt_bytes + p.blob_bytes;
}

struct DcnExtras {
  int mask_is_logits = 0;
  const float *bn_scale = nullptr, *bn_bias = nullptr, *bn_mean = nullptr, *bn_var = nullptr;
  float bn_eps = 1e-5f;
  int relu = 0;
  int row_begin = 0, row_end = -1;   // -1: through the last output row
  int pixel_first = 0, pixel_count = -1;   // run of output pixels counted from pixel 0 of image n_begin; -1: all
  // plain convolution only:
  bool plain = false;
  int pad_bottom = -1, pad_right = -1;
  float *y_split = nullptr;
  int split_at = 0;
};

static int dcnv2_forward_impl(const float *x, const float *offset, const float *mask, const float *w,
                              const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh, int Kw,
                              int sh, int sw, int ph, int pw, int dh, int dw, int groups, int deform_groups,
                              int n_begin, int n_end, int math_mode, void *workspace, size_t workspace_bytes,
                              int32_t *status_word, void *stream_, const DcnExtras &extras) {
  DcnArgs a{};
  const int reuse_flags = math_mode & ~0xff;
  math_mode &= 0xff;
  if (reuse_flags & ~(GACB_DCN_REUSE_WEIGHTS | GACB_DCN_REUSE_INPUT | GACB_DCN_INPUT_AT_END |
                      (GACB_DCN_FAULT_INJECT ? kTestDropWeightCopies : 0)))
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: unknown flag bits 0x%x in math_mode", reuse_flags);
  int rc = validate(a, x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                    deform_groups, n_begin, n_end, math_mode, extras.pad_bottom, extras.pad_right, extras.plain);
  if (rc != GACB_OK) return rc;
  if (extras.y_split != nullptr) {
    if (extras.split_at <= 0 || extras.split_at >= Cout)
      return fail(GACB_ERR_INVALID_ARGUMENT, "conv2d: split_at %d must lie inside (0, %d)", extras.split_at, Cout);
    a.y_split = extras.y_split;
    a.split_at = extras.split_at;
  }
  const bool any_bn = extras.bn_scale || extras.bn_bias || extras.bn_mean || extras.bn_var;
  if (any_bn && !(extras.bn_scale && extras.bn_bias && extras.bn_mean && extras.bn_var))
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: BatchNorm needs scale, bias, mean and variance together");
  if (any_bn && !(extras.bn_eps > 0.0f))
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: BatchNorm epsilon must be finite and positive");
  a.mask_is_logits = extras.mask_is_logits ? 1 : 0;
  a.bn_scale = extras.bn_scale; a.bn_bias = extras.bn_bias; a.bn_mean = extras.bn_mean; a.bn_var = extras.bn_var;
  a.bn_eps = extras.bn_eps;
  a.relu = extras.relu ? 1 : 0;
  if (extras.row_end >= 0) {
    if (extras.row_begin < 0 || extras.row_end < extras.row_begin || extras.row_end > a.Ho)
      return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: output row range [%d,%d) is outside [0,%d)", extras.row_begin,
                  extras.row_end, a.Ho);
    a.row_begin = extras.row_begin;
    a.row_end = extras.row_end;
    a.m_count = (n_end - n_begin) * (a.row_end - a.row_begin) * a.Wo;
  }
  if (extras.pixel_count >= 0) {   // a run of whole-plane pixels starting inside image n_begin
    a.m_first = extras.pixel_first;
    a.m_count = extras.pixel_count;
  }
  if (n_end == n_begin || a.m_count == 0) return GACB_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  UmmaPlan p;
  if (plan_umma(a, math_mode, p)) {
    const size_t need = p.xt_bytes + p.blob_bytes;
    if (!workspace || workspace_bytes < need)
      return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256)
      return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: workspace must be 256-byte aligned");
    if ((reuse_flags & GACB_DCN_INPUT_AT_END) && workspace_bytes % 256)
      return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: with GACB_DCN_INPUT_AT_END workspace_bytes must be a multiple of 256");
    switch (math_mode) {
      case MODE_BF16: return launch_umma<MODE_BF16>(a, p, workspace, status_word, stream, reuse_flags, workspace_bytes);
      case MODE_TF32: return launch_umma<MODE_TF32>(a, p, workspace, status_word, stream, reuse_flags, workspace_bytes);
      default: return launch_umma<MODE_F32X3>(a, p, workspace, status_word, stream, reuse_flags, workspace_bytes);
    }
  }
  const long long total = (long long)Cout * a.m_count;
  dcn_direct_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
  return check_cuda(cudaGetLastError(), "dcn_direct_kernel launch");
}

GACB_API int gacb_dcnv2_forward(const float *x, const float *offset, const float *mask, const float *w,
                                const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh, int Kw,
                                int sh, int sw, int ph, int pw, int dh, int dw, int groups, int deform_groups,
                                int n_begin, int n_end, int math_mode, void *workspace, size_t workspace_bytes,
                                int32_t *status_word, void *stream_) {
  return dcnv2_forward_impl(x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                            deform_groups, n_begin, n_end, math_mode, workspace, workspace_bytes, status_word, stream_,
                            DcnExtras{});
}

GACB_API int gacb_dcnv2_fused_forward(const float *x, const float *offset, const float *mask, int mask_is_logits,
                                      const float *w, const float *bias, const float *bn_scale, const float *bn_bias,
                                      const float *bn_mean, const float *bn_var, float bn_epsilon, int relu, float *y,
                                      int N, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int ph,
                                      int pw, int dh, int dw, int groups, int deform_groups, int n_begin, int n_end,
                                      int math_mode, void *workspace, size_t workspace_bytes, int32_t *status_word,
                                      void *stream_) {
  DcnExtras e;
  e.mask_is_logits = mask_is_logits;
  e.bn_scale = bn_scale; e.bn_bias = bn_bias; e.bn_mean = bn_mean; e.bn_var = bn_var;
  e.bn_eps = bn_epsilon;
  e.relu = relu;
  return dcnv2_forward_impl(x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                            deform_groups, n_begin, n_end, math_mode, workspace, workspace_bytes, status_word, stream_, e);
}

GACB_API size_t gacb_conv2d_workspace_bytes(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw,
                                            int pad_top, int pad_left, int pad_bottom, int pad_right, int dh, int dw,
                                            int groups, int math_mode) {
  DcnArgs a{};
  math_mode &= 0xff;
  if (n <= 0) return 0;
  if (validate(a, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, n, Cin, H, W, Cout, Kh, Kw, sh, sw, pad_top,
               pad_left, dh, dw, groups, 1, 0, 0, math_mode, pad_bottom, pad_right, true) != GACB_OK)
    return 0;
  a.n_begin = 0;
  a.n_end = n;
  a.m_count = n * a.Ho * a.Wo;
  UmmaPlan p;
  if (!plan_umma(a, math_mode, p)) return 0;
  return p.xt_bytes + p.blob_bytes;
}

GACB_API int gacb_conv2d_forward(const float *x, const float *w, const float *bias, int relu, float *y, float *y_split,
                                 int split_at, int N, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw,
                                 int pad_top, int pad_left, int pad_bottom, int pad_right, int dh, int dw, int groups,
                                 int n_begin, int n_end, int math_mode, void *workspace, size_t workspace_bytes,
                                 int32_t *status_word, void *stream_) {
  if (pad_bottom < 0 || pad_right < 0) return fail(GACB_ERR_INVALID_ARGUMENT, "conv2d: pads must be nonnegative");
  DcnExtras e;
  e.plain = true;
  e.pad_bottom = pad_bottom;
  e.pad_right = pad_right;
  e.relu = relu;
  e.y_split = y_split;
  e.split_at = split_at;
  if (y_split == nullptr && split_at != 0)
    return fail(GACB_ERR_INVALID_ARGUMENT, "conv2d: split_at given without a second output");
  return dcnv2_forward_impl(x, nullptr, nullptr, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, pad_top, pad_left, dh,
                            dw, groups, 1, n_begin, n_end, math_mode, workspace, workspace_bytes, status_word, stream_, e);
}

GACB_API int gacb_dcnv2_rows_forward(const float *x, const float *offset, const float *mask, const float *w,
                                     const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                                     int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                                     int deform_groups, int n_begin, int n_end, int row_begin, int row_end,
                                     int math_mode, void *workspace, size_t workspace_bytes, int32_t *status_word,
                                     void *stream_) {
  DcnExtras e;
  e.row_begin = row_begin;
  e.row_end = row_end;
  if (row_end < 0) return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: output row range [%d,%d) is invalid", row_begin, row_end);
  return dcnv2_forward_impl(x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                            deform_groups, n_begin, n_end, math_mode, workspace, workspace_bytes, status_word, stream_, e);
}

GACB_API int gacb_dcnv2_pixels_forward(const float *x, const float *offset, const float *mask, const float *w,
                                       const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                                       int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                                       int deform_groups, long long pixel_begin, long long pixel_end, int math_mode,
                                       void *workspace, size_t workspace_bytes, int32_t *status_word, void *stream_) {
  if (sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || Kh <= 0 || Kw <= 0 || ph < 0 || pw < 0 || H <= 0 || W <= 0 || N < 0)
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: extents must be positive");
  if (H + 2 * ph < dh * (Kh - 1) + 1 || W + 2 * pw < dw * (Kw - 1) + 1)
    return fail(GACB_ERR_SHAPE_MISMATCH, "dcnv2: kernel exceeds padded input");
  const long long plane = (long long)((H + 2 * ph - dh * (Kh - 1) - 1) / sh + 1) * ((W + 2 * pw - dw * (Kw - 1) - 1) / sw + 1);
  if (pixel_begin < 0 || pixel_end < pixel_begin || pixel_end > (long long)N * plane)
    return fail(GACB_ERR_INVALID_ARGUMENT, "dcnv2: pixel range [%lld,%lld) is outside [0,%lld)", pixel_begin, pixel_end,
                (long long)N * plane);
  DcnExtras e;
  const int n_begin = (int)(pixel_begin / plane);
  const int n_end = pixel_end == pixel_begin ? n_begin : (int)((pixel_end + plane - 1) / plane);
  e.pixel_first = (int)(pixel_begin - (long long)n_begin * plane);
  e.pixel_count = (int)(pixel_end - pixel_begin);
  return dcnv2_forward_impl(x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                            deform_groups, n_begin, n_end, math_mode, workspace, workspace_bytes, status_word, stream_, e);
}

GACB_API int gacb_dcnv2_forward_static(const float *x, const float *offset, const float *mask, const float *w,
                                       const float *bias, float *y, int N, int Cin, int H, int W, int Cout, int Kh,
                                       int Kw, int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                                       int deform_groups, int n_begin, int n_end, int math_mode,
                                       int32_t *status_word, void *stream_) {
  DcnArgs a{};
  int rc = validate(a, x, offset, mask, w, bias, y, N, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh, dw, groups,
                    deform_groups, n_begin, n_end, math_mode);
  if (rc != GACB_OK) return rc;
  if (n_end == n_begin) return GACB_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  UmmaPlan p;
  if (!plan_umma(a, math_mode, p)) {
    // shapes outside the tensor-core tiling need no scratch at all
    const long long total = (long long)(n_end - n_begin) * Cout * a.Ho * a.Wo;
    dcn_direct_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
    return check_cuda(cudaGetLastError(), "dcn_direct_kernel launch");
  }
  const size_t need = p.xt_bytes + p.blob_bytes;
  if (need > (size_t)GACB_DCNV2_STATIC_SCRATCH_BYTES)
    return fail(GACB_ERR_UNSUPPORTED,
                "dcnv2_static: this call needs %zu bytes of scratch, the built-in scratch holds %zu; use fewer "
                "images per call (n_begin/n_end) or gacb_dcnv2_forward with a caller workspace",
                need, (size_t)GACB_DCNV2_STATIC_SCRATCH_BYTES);
  // Device address of the scratch array, looked up once per device with that device current.
  static std::mutex lock;
  static void *scratch_of_device[64] = {};
  int device = -1;
  rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != GACB_OK) return rc;
  if (device < 0 || device >= 64) return fail(GACB_ERR_UNSUPPORTED, "dcnv2_static: device ordinal %d is out of range", device);
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(lock);
    if (!scratch_of_device[device]) {
      void *ptr = nullptr;
      rc = check_cuda(cudaGetSymbolAddress(&ptr, g_dcn_static_scratch), "cudaGetSymbolAddress(static scratch)");
      if (rc != GACB_OK) return rc;
      scratch_of_device[device] = ptr;
    }
    scratch = scratch_of_device[device];
  }
  // Nothing in the scratch has to start at zero: the NHWC copy and the packed weights are fully rewritten for the
  // region this call reads, so contents left by an earlier call are never observed.
  switch (math_mode) {
    case MODE_BF16: return launch_umma<MODE_BF16>(a, p, scratch, status_word, stream);
    case MODE_TF32: return launch_umma<MODE_TF32>(a, p, scratch, status_word, stream);
    default: return launch_umma<MODE_F32X3>(a, p, scratch, status_word, stream);
  }
}

namespace gacb {
int dcn_check_record(unsigned int out[2]) {
  out[0] = out[1] = 0;
#if GACB_CHECKED
  return check_cuda(cudaMemcpyFromSymbol(out, g_check_record, 2 * sizeof(unsigned int)), "cudaMemcpyFromSymbol(check record)");
#else
  return GACB_OK;
#endif
}
}  // namespace gacb

GACB_API int gacb_dcnv2_launch_geometry(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int ph,
                                        int pw, int dh, int dw, int groups, int deform_groups, int math_mode, int plain,
                                        int sm_count, gacb_launch_geometry *out) {
  if (!out) return fail(GACB_ERR_INVALID_ARGUMENT, "launch_geometry: out is NULL");
  DcnArgs a{};
  math_mode &= 0xff;
  int rc = validate(a, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, n, Cin, H, W, Cout, Kh, Kw, sh, sw, ph, pw, dh,
                    dw, groups, deform_groups, 0, 0, math_mode, -1, -1, plain != 0);
  if (rc != GACB_OK) return rc;
  a.n_begin = 0;
  a.n_end = n;
  a.m_count = n * a.Ho * a.Wo;
  // only the launch shape is wanted: stand-ins keep "is this a plain convolution" readable from the operands
  static const float kDummy = 0.0f;
  a.offset = plain ? nullptr : &kDummy;
  *out = gacb_launch_geometry{};
  UmmaPlan p;
  if (n <= 0 || !plan_umma(a, math_mode, p)) {
    const long long total = (long long)Cout * a.m_count;
    out->grid[0] = (int)((total + 255) / 256); out->grid[1] = out->grid[2] = 1;
    out->block[0] = 256; out->block[1] = out->block[2] = 1;
    out->units_per_cta = 256;
    snprintf(out->kernel, sizeof(out->kernel), "dcn_direct_kernel");
    return GACB_OK;
  }
  UmmaArgs u{};
  UmmaLaunch l;
  if (sm_count <= 0) sm_count = 148;
  ConvWinArgs cw{};
  size_t cw_smem = 0;
  if (plan_conv_window(a, math_mode, p.blob_bytes, cw, cw_smem)) {
    out->grid[0] = std::min(cw.tiles_total, sm_count); out->grid[1] = out->grid[2] = 1;
    out->block[0] = win_threads(math_mode); out->block[1] = out->block[2] = 1;
    out->dynamic_smem_bytes = cw_smem;
    out->units_per_cta = kTileM;      // per tile; a CTA takes tiles blockIdx.x, blockIdx.x + grid, ...
    snprintf(out->kernel, sizeof(out->kernel), "conv_window_kernel<%s>",
             math_mode == MODE_BF16 ? "bf16" : (math_mode == MODE_TF32 ? "tf32" : "f32x3"));
    return GACB_OK;
  }
  switch (math_mode) {
    case MODE_BF16: l = shape_umma_launch<MODE_BF16>(a, p, sm_count, u); break;
    case MODE_TF32: l = shape_umma_launch<MODE_TF32>(a, p, sm_count, u); break;
    default: l = shape_umma_launch<MODE_F32X3>(a, p, sm_count, u); break;
  }
  out->grid[0] = (int)l.grid.x; out->grid[1] = (int)l.grid.y; out->grid[2] = (int)l.grid.z;
  out->block[0] = l.threads; out->block[1] = out->block[2] = 1;
  out->dynamic_smem_bytes = l.smem;
  out->units_per_cta = kTileM;
  snprintf(out->kernel, sizeof(out->kernel), "dcn_umma_kernel<%s,%s,%s>",
           math_mode == MODE_BF16 ? "bf16" : (math_mode == MODE_TF32 ? "tf32" : "f32x3"), plain ? "plain" : "deform",
           l.narrow ? "narrow" : "wide");
  return GACB_OK;
}

GACB_API int gacb_conv_window_path(int mode) {
  if (mode != 0 && mode != 1) return g_conv_window_path.load();
  return g_conv_window_path.exchange(mode);
}

GACB_API int gacb_dcnv2_workspace_parts(int n, int Cin, int H, int W, int Cout, int Kh, int Kw, int sh, int sw, int pad_top,
                                        int pad_left, int pad_bottom, int pad_right, int dh, int dw, int groups,
                                        int deform_groups, int math_mode, int plain, size_t *input_copy_bytes,
                                        size_t *weights_bytes) {
  if (!input_copy_bytes || !weights_bytes) return fail(GACB_ERR_INVALID_ARGUMENT, "workspace_parts: NULL output");
  *input_copy_bytes = *weights_bytes = 0;
  DcnArgs a{};
  math_mode &= 0xff;
  if (n <= 0) return GACB_OK;
  int rc = validate(a, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, n, Cin, H, W, Cout, Kh, Kw, sh, sw, pad_top,
                    pad_left, dh, dw, groups, deform_groups, 0, 0, math_mode, pad_bottom, pad_right, plain != 0);
  if (rc != GACB_OK) return rc;
  a.n_begin = 0;
  a.n_end = n;
  a.m_count = n * a.Ho * a.Wo;
  UmmaPlan p;
  if (!plan_umma(a, math_mode, p)) return GACB_OK;      // CUDA-core kernel: no workspace at all
  *input_copy_bytes = p.xt_bytes;
  *weights_bytes = p.blob_bytes;
  return GACB_OK;
}
