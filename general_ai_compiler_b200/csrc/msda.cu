// Multi-scale deformable attention (forward) for sm_100a.
//
// Operator semantics: src/gac/core/ops.py:787-851 of the reference (NumPy
// evaluator); the kernels replace the generated CUDA of
// src/gac/targets/cuda/compiler.py:521-557 and the native lowering
// native/lib/DeviceLowering.cpp:755-802 (with its fused-coordinate form
// :763-775).
//
// Work decomposition.  A "row" is one (batch, query, head) triple: it owns
// L*P bilinear samples and D output channels.  Rows are consecutive in
// memory for sampling locations, attention weights and the output, so a CTA
// that takes a block of consecutive rows streams those three tensors fully
// coalesced, exactly once.  The value tensor is the only gathered operand.
//
//   phase A  every thread turns a few (row, sample) pairs into a 20-byte
//            packed tap record in shared memory: the clamped texel index of
//            the (x0,y0) tap with one "x1 is one texel to the right" and one
//            "y1 is one row below" bit, and four factors gx, fx, gy*w, fy*w
//            (a factor is 0 when its column/row lies outside the image: zero
//            padding, align_corners=False; w is the attention weight).
//   phase B  LPR adjacent lanes own one row; each lane keeps CPL channels in
//            registers and walks the row's records four samples at a time:
//            16 independent 16-byte texel loads are issued before the first
//            one is consumed (a row's tap is one 128-byte line for D=32
//            fp32), then accumulated in float32 in level/point/tap order.
//            The L1 data pipe moves one line per cycle, so the record is kept
//            to 20 bytes (5 shared-memory wavefronts per warp-sample next to
//            the 16 of the taps themselves).
//
// The grid runs rows in (batch, query, head) order, so at any moment the
// resident CTAs gather from one batch entry's value slab, which is what keeps
// that slab L2-resident (one BEVFormer-base camera is 31.6 MB in fp32).
#include <atomic>
#include <mutex>

#include "gacb_common.cuh"

namespace gacb {
namespace {

GACB_CHECK_RECORD;
// Sites of the checked build in this file: 1 row table, 2 tap-record table, 3 locations / weights / scores,
// 4 value taps, 5 output rows, 6 compacted row list, 7 normalizer / reference of the fused form.
#if GACB_CHECKED
#define GACB_TAP(o) ((int)(GACB_INDEX((long long)base_off + (o), value_elems - CPL + 1, 4) - base_off))
#else
#define GACB_TAP(o) (o)
#endif

constexpr int kThreads = 256;
constexpr int kMaxLevels = 32;
constexpr int kMaxPoints = 64;
constexpr int kMaxCoordRank = 8;
#ifndef GACB_MSDA_THREADS_F32
#define GACB_MSDA_THREADS_F32 128
#endif
#ifndef GACB_MSDA_THREADS_BF16
#define GACB_MSDA_THREADS_BF16 256
#endif
#ifndef GACB_MSDA_RECORDS_PER_THREAD
#define GACB_MSDA_RECORDS_PER_THREAD 2
#endif
#ifndef GACB_MSDA_RECORDS_PER_THREAD_BF16
#define GACB_MSDA_RECORDS_PER_THREAD_BF16 4
#endif
#ifndef GACB_MSDA_CARVEOUT
#define GACB_MSDA_CARVEOUT 60
#endif
#ifndef GACB_MSDA_FORCE_BATCH
#define GACB_MSDA_FORCE_BATCH 0
#endif
#ifndef GACB_MSDA_UNROLL
#define GACB_MSDA_UNROLL 4
#endif
constexpr int kRecordsPerThread = GACB_MSDA_RECORDS_PER_THREAD;
// Phase-A budget (kRecordsPerThread; RowsCta<VT>::kRecordsPerThreadLongRows for rows longer than that table): 20-byte
// tap records per thread of the CTA.  It sets how many
// samples of a row a CTA takes at a time, and with that the size of the pieces in which it streams the row's
// locations and weights.  Pieces shorter than a 128-byte line cost extra DRAM reads (measured with the spatial
// workload: the rest of the line is read from DRAM again when the next chunk asks for it).  fp32 texels, 2 records per
// thread (64-byte pieces of the weights): 416 MB read, 408 us; 4 per thread (whole rows): 374 MB = every input
// once, but 419 us -- the kernel is not DRAM-bound, so it keeps 2.  bf16 texels, 2 per thread (64- and 32-byte
// pieces): 425 MB, 345 us; 4 per thread: 312 MB, 335 us.
constexpr int kMaxRowsPerGroup = 8;
constexpr int kCarveoutPercent = GACB_MSDA_CARVEOUT;  // shared-memory share of the 256 KB; the rest is L1
constexpr int kUnroll = GACB_MSDA_UNROLL;            // samples whose 4*kUnroll tap loads are in flight together

// Division by a runtime constant as multiply-high + shift (exact for n < 2^31).
struct FastDiv {
  uint32_t mul, shift, div;
  __host__ void set(uint32_t d) {
    div = d;
    if (d <= 1) { mul = 0; shift = 0; return; }
    shift = 0;
    while ((1u << shift) < d) ++shift;                       // ceil(log2 d)
    const uint64_t one = 1;
    mul = (uint32_t)(((one << 32) * ((one << shift) - d)) / d + 1);
  }
  __device__ __forceinline__ uint32_t operator()(uint32_t n) const {
    if (div <= 1) return n;
    const uint32_t t = __umulhi(n, mul);
    return (t + ((n - t) >> 1)) >> (shift - 1);
  }
};

struct MsdaArgs {
  const void *value;
  const float *loc;  // sampling locations, or raw offsets in the fused form
  const float *attn;
  float *out;
  const float *normalizer;
  const float *reference;
  int B, S, H, D, L, P, Q;
  int q_begin, q_count;
  int total_rows;  // B * q_count * H
  int LP;          // L * P samples per row
  int rows_per_group;
  int chunk_len;   // samples per shared-memory chunk
  int chunk_pad;   // chunk_len rounded up to the unroll factor
  FastDiv div_chunk_pad, div_per_b, div_h, div_p, div_q;
  int reference_first;
  const int *row_list;     // optional compacted list of visible (b*Q + q) entries; row_list[-4] holds their count
  const float *row_mask;   // optional [B,Q]: rows of a (b,q) whose entry is 0 are skipped (their output is not written)
  int softmax;     // attn holds raw logits: weights = softmax over the row's L*P logits, formed in the kernel
  int coord_rank;
  int lvl_h[kMaxLevels], lvl_w[kMaxLevels], lvl_start[kMaxLevels];
  int norm_stride[6];  // stride of the normalizer per location axis (0 = broadcast)
  // Reference operand of the fused form, broadcast against coordinate_shape.  The host merges neighbouring axes
  // (both broadcast, or contiguous in the reference) and, when the last axis is the (x, y) pair, takes it out as
  // `ref_comp_stride`; what is left is usually two or three axes, outermost first.
  int coord_dim[kMaxCoordRank];
  int ref_stride[kMaxCoordRank];  // stride of the reference per merged axis (0 = broadcast)
  FastDiv coord_div[kMaxCoordRank];
  int comp_split;                 // the (x, y) axis is handled apart: index with the sample number, not the element
  int ref_comp_stride;
  long long norm_elems, ref_elems;   // element counts of normalizer / reference (bounds of the checked build)
};

struct __align__(16) TapEntry {
  int off[4];   // element offsets of (x0,y0) (x1,y0) (x0,y1) (x1,y1), channel 0 of the row's head
  float c[4];   // bilinear coefficient * attention weight, 0 when the tap is outside the image
};

struct RowId {
  int b, q, h;
  long long grow;  // (b*Q + q)*H + h: row index in the caller's full tensors
};

__device__ __forceinline__ RowId decode_row(const MsdaArgs &a, int r) {
  const int per_b = a.q_count * a.H;
  RowId id;
  id.b = (int)a.div_per_b((uint32_t)r);
  const int rem = r - id.b * per_b;
  const int qq = (int)a.div_h((uint32_t)rem);
  id.h = rem - qq * a.H;
  id.q = a.q_begin + qq;
  id.grow = ((long long)id.b * a.Q + id.q) * a.H + id.h;
  return id;
}

// Index into the reference of the fused form for a flat index over the merged coordinate axes (32-bit arithmetic:
// every tensor has fewer than 2^31 elements).
__device__ __forceinline__ int reference_index(const MsdaArgs &a, uint32_t rest) {
  int ri = 0;
  for (int k = a.coord_rank - 1; k > 0; --k) {
    const uint32_t q = a.coord_div[k](rest);
    ri += (int)(rest - q * (uint32_t)a.coord_dim[k]) * a.ref_stride[k];
    rest = q;
  }
  return ri + (int)rest * a.ref_stride[0];
}

// Both coordinates of a sample in the fused form: offsets[i] / normalizer[...] (+) reference[...],
// divide and add rounded separately (DeviceLowering.cpp:763-775).  `si` = flat (row, sample) index.
__device__ __forceinline__ float2 fused_coordinates(const MsdaArgs &a, const RowId &id, int lvl, int p, int si) {
  const int ni = id.b * a.norm_stride[0] + id.q * a.norm_stride[1] + id.h * a.norm_stride[2] + lvl * a.norm_stride[3] +
                 p * a.norm_stride[4];
  int rx, ry;
  if (a.comp_split) {
    rx = reference_index(a, (uint32_t)si);
    ry = rx + a.ref_comp_stride;
  } else {
    rx = reference_index(a, 2u * (uint32_t)si);
    ry = reference_index(a, 2u * (uint32_t)si + 1u);
  }
  const float2 off = ld_stream_f2(a.loc + 2 * GACB_INDEX(si, (long long)a.B * a.Q * a.H * a.LP, 3));
  const float qx = __fdiv_rn(off.x, a.normalizer[GACB_INDEX(ni, a.norm_elems, 7)]);
  const float qy = __fdiv_rn(off.y, a.normalizer[GACB_INDEX(ni + a.norm_stride[5], a.norm_elems, 7)]);
  const float bx = a.reference[GACB_INDEX(rx, a.ref_elems, 7)], by = a.reference[GACB_INDEX(ry, a.ref_elems, 7)];
  return a.reference_first ? make_float2(__fadd_rn(bx, qx), __fadd_rn(by, qy))
                           : make_float2(__fadd_rn(qx, bx), __fadd_rn(qy, by));
}

// Everything a bilinear sample needs, before packing.
struct SampleGeom {
  int x0, y0, ww, hh, tex;   // floor coordinates, level extent, first texel of the level
  float fx, fy, w;
  bool vx0, vx1, vy0, vy1;
};

// RowId from the global row index alone (used where b, q, h are needed again).
__device__ __forceinline__ RowId row_from_global(const MsdaArgs &a, int grow) {
  RowId id;
  const int bq = (int)a.div_h((uint32_t)grow);
  id.h = grow - bq * a.H;
  id.b = (int)a.div_q((uint32_t)bq);
  id.q = bq - id.b * a.Q;
  id.grow = grow;
  return id;
}

__device__ __forceinline__ SampleGeom geometry_of(float lx, float ly, float w, int4 level);

// `level` = {H_l, W_l, first texel, unused}; `si` = flat (row, sample) index into locations/weights.
template <bool FUSED>
__device__ __forceinline__ SampleGeom sample_geometry(const MsdaArgs &a, int grow, int s, int lvl, int4 level,
                                                      float2 norm) {
  const int si = grow * a.LP + s;
  float lx, ly;
  if (FUSED) {
    const RowId id = row_from_global(a, grow);
    const int p = s - lvl * a.P;
    const float2 v = fused_coordinates(a, id, lvl, p, si);
    lx = v.x;
    ly = v.y;
  } else {
    const float2 v = ld_stream_f2(a.loc + 2 * GACB_INDEX(si, (long long)a.B * a.Q * a.H * a.LP, 3));
    lx = v.x;
    ly = v.y;
  }
  float w = ld_stream_f1(a.attn + GACB_INDEX(si, (long long)a.B * a.Q * a.H * a.LP, 3));
  // softmax as the reference's Softmax op does it: exp(x - max) / sum (src/gac/core/ops.py:1119-1125)
  if (a.softmax) w = __fdiv_rn(expf(__fsub_rn(w, norm.x)), norm.y);
  return geometry_of(lx, ly, w, level);
}

// From normalised coordinates and the (final) attention weight to the sample's texel geometry.
__device__ __forceinline__ SampleGeom geometry_of(float lx, float ly, float w, int4 level) {
  SampleGeom g;
  g.w = w;
  g.hh = level.x;
  g.ww = level.y;
  g.tex = level.z;
  // Pixel coordinates: one rounded multiply then one rounded subtract, as the
  // reference's float32 arithmetic does (ops.py:827-828).
  const float x = __fsub_rn(__fmul_rn(lx, (float)g.ww), 0.5f);
  const float y = __fsub_rn(__fmul_rn(ly, (float)g.hh), 0.5f);
  const float xf = floorf(x), yf = floorf(y);
  g.x0 = (int)xf;  // float->int saturates; NaN -> 0
  g.y0 = (int)yf;
  g.fx = x - xf;
  g.fy = y - yf;
  g.vx0 = (g.x0 >= 0) & (g.x0 < g.ww);
  g.vx1 = (g.x0 >= -1) & (g.x0 < g.ww - 1);
  g.vy0 = (g.y0 >= 0) & (g.y0 < g.hh);
  g.vy1 = (g.y0 >= -1) & (g.y0 < g.hh - 1);
  return g;
}

template <bool FUSED>
__device__ __forceinline__ TapEntry make_entry(const MsdaArgs &a, const RowId &id, int s, float2 norm) {
  const int lvl = (int)a.div_p((uint32_t)s);
  const SampleGeom g = sample_geometry<FUSED>(a, (int)id.grow, s, lvl,
                                              make_int4(a.lvl_h[lvl], a.lvl_w[lvl], a.lvl_start[lvl], 0), norm);
  const float gx = 1.0f - g.fx, gy = 1.0f - g.fy;
  const int cx0 = min(max(g.x0, 0), g.ww - 1);
  const int cx1 = g.vx1 ? g.x0 + 1 : cx0;
  const int cy0 = min(max(g.y0, 0), g.hh - 1);
  const int cy1 = g.vy1 ? g.y0 + 1 : cy0;
  const int tex = id.b * a.S + g.tex;
  const int hd = a.H * a.D;
  const int chan = id.h * a.D;
  TapEntry t;
  t.off[0] = (tex + cy0 * g.ww + cx0) * hd + chan;
  t.off[1] = (tex + cy0 * g.ww + cx1) * hd + chan;
  t.off[2] = (tex + cy1 * g.ww + cx0) * hd + chan;
  t.off[3] = (tex + cy1 * g.ww + cx1) * hd + chan;
  t.c[0] = (g.vx0 & g.vy0) ? __fmul_rn(__fmul_rn(gx, gy), g.w) : 0.0f;
  t.c[1] = (g.vx1 & g.vy0) ? __fmul_rn(__fmul_rn(g.fx, gy), g.w) : 0.0f;
  t.c[2] = (g.vx0 & g.vy1) ? __fmul_rn(__fmul_rn(gx, g.fy), g.w) : 0.0f;
  t.c[3] = (g.vx1 & g.vy1) ? __fmul_rn(__fmul_rn(g.fx, g.fy), g.w) : 0.0f;
  return t;
}

// Packed record of the vector kernel.  `word` = (texel index within batch b of
// the clamped (x0,y0) tap) << 2 | ystep << 1 | xstep; the (x1,*) taps sit xstep
// texels to the right and the (*,y1) taps ystep rows below.  A step is 0 only
// when that neighbour is outside the image, in which case its factor is 0 too.
// factors = {gx, fx, gy*w, fy*w}: tap coefficients are their four products.
__device__ __forceinline__ void pack_geometry(const SampleGeom &g, float4 &factors, uint32_t &word, int &cx0, int &cy0);

template <bool FUSED>
__device__ __forceinline__ void make_packed(const MsdaArgs &a, int grow, int s, int lvl, int4 level, float2 norm,
                                            float4 &factors, uint32_t &word) {
  int cx0, cy0;
  pack_geometry(sample_geometry<FUSED>(a, grow, s, lvl, level, norm), factors, word, cx0, cy0);
}

// (cx0, cy0) = the clamped (x0, y0) tap the word points at.
__device__ __forceinline__ void pack_geometry(const SampleGeom &g, float4 &factors, uint32_t &word, int &cx0, int &cy0) {
  cx0 = min(max(g.x0, 0), g.ww - 1);
  cy0 = min(max(g.y0, 0), g.hh - 1);
  // x1/y1 are reachable by a +1 step only when x0/y0 itself was not clamped.
  const bool xstep = g.vx1 & (g.x0 >= 0);
  const bool ystep = g.vy1 & (g.y0 >= 0);
  // x0 == -1: the only live column is x1 == 0 == cx0, read through the "x0" slot.
  const bool left_edge = g.vx1 & (g.x0 < 0);
  const bool top_edge = g.vy1 & (g.y0 < 0);
  factors.x = g.vx0 ? 1.0f - g.fx : (left_edge ? g.fx : 0.0f);
  factors.y = xstep ? g.fx : 0.0f;
  const float gy = g.vy0 ? 1.0f - g.fy : (top_edge ? g.fy : 0.0f);
  const float fy = ystep ? g.fy : 0.0f;
  factors.z = __fmul_rn(gy, g.w);
  factors.w = __fmul_rn(fy, g.w);
  word = ((uint32_t)(g.tex + cy0 * g.ww + cx0) << 2) | (ystep ? 2u : 0u) | (xstep ? 1u : 0u);
}

// One lane's slice of a texel: CPL channels starting at element `off`.
template <typename VT, int CPL>
struct Tap;

template <>
struct Tap<float, 4> {
  typedef float4 Raw;
  __device__ static __forceinline__ Raw load(const float *value, int off) { return ld_texel_f4(value + off); }
  // Compiler fence on a loaded value: everything that uses it is scheduled after every load that precedes the fence.
  __device__ static __forceinline__ void pin(Raw &v) { asm volatile("" : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w)); }
  __device__ static __forceinline__ void fma(float (&acc)[4], const Raw &v, float c) {
    acc[0] = fmaf(v.x, c, acc[0]);
    acc[1] = fmaf(v.y, c, acc[1]);
    acc[2] = fmaf(v.z, c, acc[2]);
    acc[3] = fmaf(v.w, c, acc[3]);
  }
};

template <>
struct Tap<__nv_bfloat16, 8> {
  typedef uint4 Raw;
  __device__ static __forceinline__ Raw load(const __nv_bfloat16 *value, int off) {
    return ld_texel_u4(value + off);
  }
  __device__ static __forceinline__ void pin(Raw &v) { asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)); }
  __device__ static __forceinline__ void fma(float (&acc)[8], const Raw &v, float c) {
    acc[0] = fmaf(bf16_lo(v.x), c, acc[0]);
    acc[1] = fmaf(bf16_hi(v.x), c, acc[1]);
    acc[2] = fmaf(bf16_lo(v.y), c, acc[2]);
    acc[3] = fmaf(bf16_hi(v.y), c, acc[3]);
    acc[4] = fmaf(bf16_lo(v.z), c, acc[4]);
    acc[5] = fmaf(bf16_hi(v.z), c, acc[5]);
    acc[6] = fmaf(bf16_lo(v.w), c, acc[6]);
    acc[7] = fmaf(bf16_hi(v.w), c, acc[7]);
  }
};

// CTA size of the rows kernel per value type.  Measured on the BEVFormer-base workloads: with fp32 texels (a tap is a
// whole 128-byte line) twelve CTAs of 128 threads per SM interleave record making and gathering better than six of
// 256 (386 against 412 us on the spatial workload); with bf16 texels the larger CTA is the faster one (328 / 337 us).
template <typename VT>
struct RowsCta;
template <>
struct RowsCta<float> {
  static constexpr int kThreads = GACB_MSDA_THREADS_F32;
  static constexpr int kRecordsPerThreadLongRows = GACB_MSDA_RECORDS_PER_THREAD;
};
template <>
struct RowsCta<__nv_bfloat16> {
  static constexpr int kThreads = GACB_MSDA_THREADS_BF16;
  static constexpr int kRecordsPerThreadLongRows = GACB_MSDA_RECORDS_PER_THREAD_BF16;
};

// LPR lanes per row, CPL channels per lane (D == LPR*CPL).
template <typename VT, int CPL, int LPR, bool FUSED>
__global__ void __launch_bounds__(RowsCta<VT>::kThreads) msda_rows_kernel(const __grid_constant__ MsdaArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kThreads = RowsCta<VT>::kThreads;   // shadows the namespace-level CTA size of the other kernels
  static_assert(kThreads % 32 == 0 && kThreads % LPR == 0, "CTA size");
  constexpr int RPI = kThreads / LPR;  // rows gathered side by side
  const int tid = threadIdx.x;
  const int J = a.rows_per_group, CL = a.chunk_len, CLP = a.chunk_pad;
  const int rows_cta = RPI * J;
  const int row0 = blockIdx.x * rows_cta;
  // compacted visibility: rows are (list entry, head); CTAs past the end of the list have nothing to do
  if (a.row_list && row0 >= a.row_list[-4] * a.H) return;
  const int stride = CLP + 1;  // odd record stride: rows never alias the same banks
  // shared memory: level table | tap factors | tap words | global row index per local row
  int4 *levels = reinterpret_cast<int4 *>(smem_raw);
  float4 *factors = reinterpret_cast<float4 *>(levels + kMaxLevels);
  uint32_t *words = reinterpret_cast<uint32_t *>(factors + rows_cta * stride);
  int *row_global = reinterpret_cast<int *>(words + rows_cta * stride);
  float2 *row_norm = reinterpret_cast<float2 *>(row_global + rows_cta);   // (max, sum of exp) per row, softmax form only
  const int grp = tid / LPR, lane = tid - grp * LPR;
  const int hd = a.H * a.D;

  if (tid < a.L) levels[tid] = make_int4(a.lvl_h[tid], a.lvl_w[tid], a.lvl_start[tid], a.lvl_w[tid] * hd);
  for (int rl = tid; rl < rows_cta; rl += kThreads) {
    const int r = row0 + rl;
    int grow = -1;
    if (a.row_list) {
      const int e = (int)a.div_h((uint32_t)r);
      if (e < a.row_list[-4]) grow = a.row_list[GACB_INDEX(e, (long long)a.B * a.Q, 6)] * a.H + (r - e * a.H);
    } else if (r < a.total_rows) {
      const RowId id = decode_row(a, r);
      grow = (int)id.grow;
      if (a.row_mask && a.row_mask[id.b * a.Q + id.q] == 0.0f) grow = -1;   // masked out: no work, no store
    }
    row_global[rl] = grow;
  }
  __syncthreads();
  if (a.softmax) {
    // eight lanes per row, all rows of the CTA side by side: running max, then the sum of exp(x - max), over the
    // row's L*P logits (cached loads: the second pass and the record making read the same lines again)
    const int sub = tid & 7;
    for (int rl = tid >> 3; rl < rows_cta; rl += kThreads / 8) {
      const int grow = row_global[rl];
      const float *logits = a.attn + (long long)(grow < 0 ? 0 : grow) * a.LP;
      const int n = grow < 0 ? 0 : a.LP;       // masked rows take part in the shuffles with nothing to add
      float m = -INFINITY;
      for (int s = sub; s < n; s += 8) m = fmaxf(m, __ldg(logits + s));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      float sum = 0.0f;
      for (int s = sub; s < n; s += 8) sum += expf(__fsub_rn(__ldg(logits + s), m));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (sub == 0 && grow >= 0) row_norm[rl] = make_float2(m, sum);
    }
    __syncthreads();
  }

  float acc[CPL];
  for (int s0 = 0; s0 < a.LP; s0 += CL) {
    const int cl = min(CL, a.LP - s0);
    if (s0 != 0) __syncthreads();  // previous chunk fully consumed
    const int n_records = rows_cta * CLP;
    for (int e = tid; e < n_records; e += kThreads) {
      const int rl = (int)a.div_chunk_pad((uint32_t)e);
      const int s = e - rl * CLP;
      const int grow = row_global[rl];
      float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      uint32_t word = 0;  // padding records read texel 0 with zero factors
      if (grow >= 0 && s < cl) {
        const int lvl = (int)a.div_p((uint32_t)(s0 + s));
        make_packed<FUSED>(a, grow, s0 + s, lvl, levels[lvl], a.softmax ? row_norm[rl] : make_float2(0.0f, 1.0f), f,
                           word);
      }
      factors[GACB_INDEX(rl * stride + s, rows_cta * stride, 2)] = f;
      words[GACB_INDEX(rl * stride + s, rows_cta * stride, 2)] = word;
    }
    __syncthreads();
    for (int j = 0; j < J; ++j) {
      const int rl = j * RPI + grp;
      const int grow = row_global[GACB_INDEX(rl, rows_cta, 1)];
      if (grow < 0) continue;
      if (s0 == 0) {
#pragma unroll
        for (int c = 0; c < CPL; ++c) acc[c] = 0.0f;
      }
      // channel 0 of this lane in texel 0 of batch b, head h
      const RowId id = row_from_global(a, grow);
      const VT *base = static_cast<const VT *>(a.value) + (id.b * a.S * a.H + id.h) * a.D + lane * CPL;
#if GACB_CHECKED
      const long long base_off = (long long)(id.b * a.S * a.H + id.h) * a.D + lane * CPL;
      const long long value_elems = (long long)a.B * a.S * a.H * a.D;
#endif
      const float4 *fr = factors + rl * stride;
      const uint32_t *wr = words + rl * stride;
      for (int s = 0; s < CLP; s += kUnroll) {
        typename Tap<VT, CPL>::Raw v[kUnroll][4];
        float4 f[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          // the level (hence the row pitch) of a sample is the same for the whole CTA
          const int lvl = min((int)a.div_p((uint32_t)(s0 + s + u)), a.L - 1);
          const int pitch = a.lvl_w[lvl] * hd;
          f[u] = fr[GACB_INDEX(s + u, stride, 2)];
          const uint32_t word = wr[GACB_INDEX(s + u, stride, 2)];
          const int o00 = (int)(word >> 2) * hd;
          const int dx = (int)(word & 1u) * hd;
          const int dy = (int)((word >> 1) & 1u) * pitch;
          v[u][0] = Tap<VT, CPL>::load(base, GACB_TAP(o00));
          v[u][1] = Tap<VT, CPL>::load(base, GACB_TAP(o00 + dx));
          v[u][2] = Tap<VT, CPL>::load(base, GACB_TAP(o00 + dy));
          v[u][3] = Tap<VT, CPL>::load(base, GACB_TAP(o00 + dy + dx));
        }
#if GACB_MSDA_FORCE_BATCH
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
          for (int t = 0; t < 4; ++t) Tap<VT, CPL>::pin(v[u][t]);
#endif
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          Tap<VT, CPL>::fma(acc, v[u][0], f[u].x * f[u].z);
          Tap<VT, CPL>::fma(acc, v[u][1], f[u].y * f[u].z);
          Tap<VT, CPL>::fma(acc, v[u][2], f[u].x * f[u].w);
          Tap<VT, CPL>::fma(acc, v[u][3], f[u].y * f[u].w);
        }
      }
      if (s0 + cl == a.LP) {
        float *dst = a.out + GACB_INDEX((long long)grow * a.D + lane * CPL, (long long)a.B * a.Q * a.H * a.D - CPL + 1, 5);
#pragma unroll
        for (int c = 0; c < CPL; c += 4)
          st_stream_f4(dst + c, make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]));
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Tile kernel: one feature level whose queries are that level's own raster (temporal self-attention:
// src/gac/models/bevformer/temporal.py:366-373 samples the previous BEV map around each BEV cell).
//
// Query q = qy*W + qx sits on texel (qx, qy) and its samples fall a few texels around it, so the taps of a 2-D
// block of queries fall in that block of the value map plus a halo.  A CTA takes kTileH x kTileW queries of ONE
// head and one batch entry, brings the (kTileH + 2r + 2) x (kTileW + 2r + 2) window of that head's texels (128
// bytes each, 1 KB apart in `value`) into shared memory with 16-byte asynchronous copies (cp.async: no registers,
// no waiting on a barrier that could fail to complete; one cp.async.bulk per 128-byte texel was measured first and
// took 17 us per CTA -- the copy engine is paced per request, not per byte) and gathers from there: the window is
// read from L2 once instead of once per tap (4 taps x P samples x 256 queries = 4096 tap lines against 784 window
// texels).  Nothing is assumed about where the samples really are: each record says whether all four (clamped)
// taps lie in the window; if not, that sample's taps are fetched from global memory.  Either way the sample enters
// the accumulator through the same fmaf sequence as in msda_rows_kernel, so the two kernels agree bit for bit.
// ----------------------------------------------------------------------------------------------
#ifndef GACB_MSDA_TILE_H
#define GACB_MSDA_TILE_H 16
#endif
#ifndef GACB_MSDA_TILE_W
#define GACB_MSDA_TILE_W 16
#endif
#ifndef GACB_MSDA_TILE_REACH
#define GACB_MSDA_TILE_REACH 5
#endif
#ifndef GACB_MSDA_TILE_CHUNK_RECORDS
#define GACB_MSDA_TILE_CHUNK_RECORDS 512
#endif
constexpr int kTileH = GACB_MSDA_TILE_H, kTileW = GACB_MSDA_TILE_W, kTileReach = GACB_MSDA_TILE_REACH;
// a sample at most r texels from its query's cell touches texels [q - r, q + r + 1]
constexpr int kWinH = kTileH + 2 * kTileReach + 2, kWinW = kTileW + 2 * kTileReach + 2;
#ifndef GACB_MSDA_TILE_THREADS
#define GACB_MSDA_TILE_THREADS 512
#endif
#ifndef GACB_MSDA_TILE_BATCH
#define GACB_MSDA_TILE_BATCH 2
#endif
constexpr int kTileThreads = GACB_MSDA_TILE_THREADS;
constexpr int kTileBatch = GACB_MSDA_TILE_BATCH;     // samples whose four tap loads are in flight together
constexpr int kTileRows = kTileH * kTileW;            // (query, head) rows of a CTA: one head
constexpr int kTileChunkRecords = GACB_MSDA_TILE_CHUNK_RECORDS;   // tap records in shared memory together
constexpr int kTileD = 32, kTileLpr = 8, kTileCpl = 4;
constexpr int kTileMaxSamples = 8;                    // L*P of a row
constexpr int kTileMaxTexels = 1 << 18;               // texel index field of the record word
static_assert(kWinH * kWinW <= 1024, "window index field of the record word");
static_assert(kTileChunkRecords % kTileThreads == 0, "whole records per thread");

// What a tap record is made from, as loaded: kept in registers across a gather so that the loads of the next
// chunk's records are in flight while the current chunk is gathered.
struct TileRaw {
  float2 off;            // sampling location, or raw offset in the fused-coordinate form
  float nx, ny, bx, by;  // fused form: normalizer and reference of both coordinates
  float w;               // attention weight or raw score
};

template <bool FUSED>
__device__ __forceinline__ TileRaw tile_load_raw(const MsdaArgs &a, int grow, int s) {
  TileRaw r;
  const int si = grow * a.LP + s;
  r.off = ld_stream_f2(a.loc + 2 * si);
  r.w = ld_stream_f1(a.attn + si);
  r.nx = r.ny = 1.0f;
  r.bx = r.by = 0.0f;
  if (FUSED) {   // the operands of fused_coordinates() for level 0, point s
    const RowId id = row_from_global(a, grow);
    const int ni = id.b * a.norm_stride[0] + id.q * a.norm_stride[1] + id.h * a.norm_stride[2] + s * a.norm_stride[4];
    int rx, ry;
    if (a.comp_split) {
      rx = reference_index(a, (uint32_t)si);
      ry = rx + a.ref_comp_stride;
    } else {
      rx = reference_index(a, 2u * (uint32_t)si);
      ry = reference_index(a, 2u * (uint32_t)si + 1u);
    }
    r.nx = a.normalizer[ni];
    r.ny = a.normalizer[ni + a.norm_stride[5]];
    r.bx = a.reference[rx];
    r.by = a.reference[ry];
  }
  return r;
}

// The arithmetic of fused_coordinates() on loaded operands.
template <bool FUSED>
__device__ __forceinline__ float2 tile_coordinates(const MsdaArgs &a, const TileRaw &r) {
  if (!FUSED) return r.off;
  const float qx = __fdiv_rn(r.off.x, r.nx), qy = __fdiv_rn(r.off.y, r.ny);
  return a.reference_first ? make_float2(__fadd_rn(r.bx, qx), __fadd_rn(r.by, qy))
                           : make_float2(__fadd_rn(qx, r.bx), __fadd_rn(qy, r.by));
}

// record word of the tile kernel: bit 31 = all taps in the window | window index << 20 | texel << 2 | ystep << 1 | xstep
// CLP = samples of a row rounded up to 4 or 8; the CLP records of a row are made by CLP neighbouring lanes.
template <bool FUSED, int CLP>
__global__ void __launch_bounds__(kTileThreads, 2) msda_tile_kernel(const __grid_constant__ MsdaArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kChunkRows = kTileChunkRecords / CLP;                 // rows whose records are in shared memory together
  constexpr int kPerThread = kTileChunkRecords / kTileThreads;        // records a thread makes per chunk
  constexpr int kStride = CLP + 1;                                    // odd record stride: rows never alias the same banks
  static_assert(kTileRows % kChunkRows == 0 && kChunkRows % (kTileThreads / kTileLpr) == 0, "tile chunking");
  const int tid = threadIdx.x;
  const int W = a.lvl_w[0], Hh = a.lvl_h[0];
  const int LP = a.LP;
  float *window = reinterpret_cast<float *>(smem_raw);                               // [kWinH][kWinW][32]
  float4 *factors = reinterpret_cast<float4 *>(window + kWinH * kWinW * kTileD);      // [kChunkRows][kStride]
  uint32_t *words = reinterpret_cast<uint32_t *>(factors + kChunkRows * kStride);
  int *row_global = reinterpret_cast<int *>(words + kChunkRows * kStride);            // [kTileRows]
  unsigned char *row_fast = reinterpret_cast<unsigned char *>(row_global + kTileRows);   // [kChunkRows]

  const int h = blockIdx.x % a.H, tx = blockIdx.x / a.H, ty = blockIdx.y, b = blockIdx.z;
  const int hd = a.H * a.D;
  const int wx0 = tx * kTileW - kTileReach, wy0 = ty * kTileH - kTileReach;   // window origin in the level
  const int cx0 = max(wx0, 0), cx1 = min(wx0 + kWinW, W), cy0 = max(wy0, 0), cy1 = min(wy0 + kWinH, Hh);
  const int cw = cx1 - cx0, ch = cy1 - cy0;                                   // the part of the window inside the level

  bool any_row = false;
  for (int r = tid; r < kTileRows; r += kTileThreads) {
    const int qy = ty * kTileH + r / kTileW, qx = tx * kTileW + r % kTileW;
    const int q = qy * W + qx;
    const bool live = qy < Hh && qx < W && q >= a.q_begin && q < a.q_begin + a.q_count;
    row_global[r] = live ? (b * a.Q + q) * a.H + h : -1;
    any_row |= live;
  }
  if (__syncthreads_or(any_row) == 0) return;      // a tile above or below this call's query range
  const float *vhead = static_cast<const float *>(a.value) + ((size_t)b * a.S * a.H + h) * a.D;   // texel t at + t*hd
  // window fill: 16-byte asynchronous copies, eight lanes per texel (one 128-byte line), 32 texel columns x
  // (threads / 256) rows per round; they complete while the first records are made
  static_assert(kWinW <= 32 && kTileThreads % 256 == 0, "one group of eight lanes per window column");
  {
    const int xi = (tid >> 3) & 31, piece = tid & 7;
    if (xi < cw) {
      const int x = cx0 + xi;
      for (int y = cy0 + (tid >> 8); y < cy1; y += kTileThreads / 256)
        async_copy_16(smem_u32(window + ((y - wy0) * kWinW + (x - wx0)) * kTileD + piece * 4),
                      vhead + (size_t)(y * W + x) * hd + piece * 4);
    }
    async_copy_commit();
  }
  // padding records (zero factors) point at a texel that is certainly copied: the first one of the clipped window
  const uint32_t pad_word = 0x80000000u | ((uint32_t)((cy0 - wy0) * kWinW + (cx0 - wx0)) << 20);

  const int grp = tid / kTileLpr, lane = tid % kTileLpr;
  const int4 level0 = make_int4(Hh, W, 0, W * hd);
  // record e of a chunk belongs to row e / CLP, sample e % CLP; thread tid makes records tid, tid + 256, ...
  const int my_s = tid % CLP;
  auto load_chunk = [&](int chunk, TileRaw (&raw)[kPerThread], int (&grow)[kPerThread]) {
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      grow[k] = row_global[chunk + (tid + k * kTileThreads) / CLP];
      if (grow[k] >= 0 && my_s < LP) raw[k] = tile_load_raw<FUSED>(a, grow[k], my_s);
      else grow[k] = -1;
    }
  };
  TileRaw raw[kPerThread];
  int raw_row[kPerThread];
  load_chunk(0, raw, raw_row);

  for (int chunk = 0; chunk < kTileRows; chunk += kChunkRows) {
    // ---- tap records of this chunk's rows, from the operands loaded one gather earlier
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      const int e = tid + k * kTileThreads, rl = e / CLP;
      const bool live = raw_row[k] >= 0;
      float w = raw[k].w;
      if (a.softmax) {
        // softmax over the row's scores, held by CLP neighbouring lanes: max, then the sum of exp(x - max) added
        // in the order of the rows kernel's eight-lane butterfly (4, 2, 1), so both kernels form the same sum
        float m = live ? w : -INFINITY;
#pragma unroll
        for (int o = CLP / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float ex = live ? expf(__fsub_rn(w, m)) : 0.0f;
        float sum = ex;
#pragma unroll
        for (int o = CLP / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        w = __fdiv_rn(ex, sum);
      }
      float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      uint32_t word = pad_word;
      bool inside = true;
      if (live) {
        const float2 xy = tile_coordinates<FUSED>(a, raw[k]);
        int px, py;                                                // the clamped (x0, y0) tap
        pack_geometry(geometry_of(xy.x, xy.y, w, level0), f, word, px, py);
        const int ux = px - wx0, uy = py - wy0;
        inside = ux >= 0 && uy >= 0 && ux + (int)(word & 1u) < kWinW && uy + (int)((word >> 1) & 1u) < kWinH;
        if (inside) word |= 0x80000000u | ((uint32_t)(uy * kWinW + ux) << 20);
      }
      factors[rl * kStride + my_s] = f;
      words[rl * kStride + my_s] = word;
      // a row whose samples all lie in the window is gathered with shared-memory loads only
      bool all_in = inside;
#pragma unroll
      for (int o = CLP / 2; o > 0; o >>= 1) all_in &= __shfl_xor_sync(0xffffffffu, (int)all_in, o) != 0;
      if (my_s == 0) row_fast[rl] = all_in ? 1 : 0;
    }
    if (chunk == 0) async_copy_wait_all();   // this thread's share of the window has landed; the barrier publishes it
    __syncthreads();
    if (chunk + kChunkRows < kTileRows) load_chunk(chunk + kChunkRows, raw, raw_row);   // in flight during the gather
    // ---- gather: eight lanes per row, four channels per lane, four samples (sixteen loads) in flight
    for (int j = 0; j < kChunkRows; j += kTileThreads / kTileLpr) {
      const int rl = j + grp;
      const int grow = row_global[chunk + rl];
      // warp-uniform choice: all four rows of this warp gather from the window alone, or the general form
      const bool fast = __all_sync(0xffffffffu, grow < 0 || row_fast[rl] != 0);
      if (grow < 0) continue;
      float acc[kTileCpl] = {0.0f, 0.0f, 0.0f, 0.0f};
      const float4 *fr = factors + rl * kStride;
      const uint32_t *wr = words + rl * kStride;
      if (fast) {
        const float *wbase = window + lane * kTileCpl;
#pragma unroll
        for (int s = 0; s < CLP; s += kTileBatch) {
          float4 v[kTileBatch][4], f[kTileBatch];
#pragma unroll
          for (int u = 0; u < kTileBatch; ++u) {
            f[u] = fr[s + u];
            const uint32_t word = wr[s + u];
            const float *p = wbase + GACB_INDEX((word >> 20) & 0x3ffu, kWinH * kWinW - (word & 1u) - ((word >> 1) & 1u) * kWinW, 4) * kTileD;
            const int dx = (word & 1u) ? kTileD : 0;
            const int dy = (word & 2u) ? kWinW * kTileD : 0;
            v[u][0] = *reinterpret_cast<const float4 *>(p);
            v[u][1] = *reinterpret_cast<const float4 *>(p + dx);
            v[u][2] = *reinterpret_cast<const float4 *>(p + dy);
            v[u][3] = *reinterpret_cast<const float4 *>(p + dy + dx);
          }
#pragma unroll
          for (int u = 0; u < kTileBatch; ++u) {
            Tap<float, 4>::fma(acc, v[u][0], f[u].x * f[u].z);
            Tap<float, 4>::fma(acc, v[u][1], f[u].y * f[u].z);
            Tap<float, 4>::fma(acc, v[u][2], f[u].x * f[u].w);
            Tap<float, 4>::fma(acc, v[u][3], f[u].y * f[u].w);
          }
        }
      } else {
        const float *gbase = vhead + lane * kTileCpl;
        const float *wbase = window + lane * kTileCpl;
#pragma unroll
        for (int s = 0; s < CLP; s += kTileBatch) {
          float4 v[kTileBatch][4], f[kTileBatch];
#pragma unroll
          for (int u = 0; u < kTileBatch; ++u) {
            f[u] = fr[s + u];
            const uint32_t word = wr[s + u];
            const bool in = (word >> 31) != 0u;
            const float *p = in ? wbase + GACB_INDEX((word >> 20) & 0x3ffu, kWinH * kWinW, 4) * kTileD
                                : gbase + (size_t)GACB_INDEX((word >> 2) & 0x3ffffu, a.S - (word & 1u) - ((word >> 1) & 1u) * W, 4) * hd;
            const int dx = (word & 1u) ? (in ? kTileD : hd) : 0;
            const int dy = (word & 2u) ? (in ? kWinW * kTileD : W * hd) : 0;
            v[u][0] = *reinterpret_cast<const float4 *>(p);
            v[u][1] = *reinterpret_cast<const float4 *>(p + dx);
            v[u][2] = *reinterpret_cast<const float4 *>(p + dy);
            v[u][3] = *reinterpret_cast<const float4 *>(p + dy + dx);
          }
#pragma unroll
          for (int u = 0; u < kTileBatch; ++u) {
            Tap<float, 4>::fma(acc, v[u][0], f[u].x * f[u].z);
            Tap<float, 4>::fma(acc, v[u][1], f[u].y * f[u].z);
            Tap<float, 4>::fma(acc, v[u][2], f[u].x * f[u].w);
            Tap<float, 4>::fma(acc, v[u][3], f[u].y * f[u].w);
          }
        }
      }
      st_stream_f4(a.out + GACB_INDEX((long long)grow * a.D + lane * kTileCpl, (long long)a.B * a.Q * a.H * a.D - kTileCpl + 1, 5),
                   make_float4(acc[0], acc[1], acc[2], acc[3]));
    }
    if (chunk + kChunkRows < kTileRows) __syncthreads();   // this chunk's records are consumed
  }
}

// Any H, D, L, P: one thread per output element, the same arithmetic.
template <typename VT, bool FUSED>
__global__ void __launch_bounds__(kThreads) msda_generic_kernel(const __grid_constant__ MsdaArgs a) {
  const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
  if (i >= (long long)a.total_rows * a.D) return;
  const int r = (int)(i / a.D);
  const int ch = (int)(i - (long long)r * a.D);
  const RowId id = decode_row(a, r);
  if (a.row_mask && a.row_mask[id.b * a.Q + id.q] == 0.0f) return;
  const VT *value = static_cast<const VT *>(a.value) + ch;
  float2 norm = make_float2(0.0f, 1.0f);
  if (a.softmax) {
    const float *logits = a.attn + id.grow * a.LP;
    float m = -INFINITY, sum = 0.0f;
    for (int s = 0; s < a.LP; ++s) m = fmaxf(m, logits[s]);
    for (int s = 0; s < a.LP; ++s) sum += expf(__fsub_rn(logits[s], m));
    norm = make_float2(m, sum);
  }
  float acc = 0.0f;
  for (int s = 0; s < a.LP; ++s) {
    const TapEntry t = make_entry<FUSED>(a, id, s, norm);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (t.c[k] != 0.0f)
        acc = fmaf((float)value[GACB_INDEX(t.off[k], (long long)a.B * a.S * a.H * a.D - ch, 4)], t.c[k], acc);
  }
  a.out[GACB_INDEX(id.grow * a.D + ch, (long long)a.B * a.Q * a.H * a.D, 5)] = acc;
}

// Visible (b, q) pairs of the query range, appended to list[] (count in list[-4]); a warp appends with one atomic.
// The order of the list is not fixed between runs, which is harmless: every row's result and destination depend
// on the row alone.
__global__ void __launch_bounds__(256) msda_compact_visible_kernel(const float *__restrict__ vis, int *list, int B, int Q,
                                                                   int q_begin, int q_count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool in_range = i < B * q_count;
  int entry = 0;
  bool visible = false;
  if (in_range) {
    const int b = i / q_count;
    entry = b * Q + q_begin + (i - b * q_count);
    visible = vis[entry] != 0.0f;
  }
  const unsigned ballot = __ballot_sync(0xffffffffu, visible);
  if (ballot == 0) return;
  const int lane = threadIdx.x & 31;
  int base = 0;
  if (lane == 0) base = atomicAdd(list - 4, __popc(ballot));
  base = __shfl_sync(0xffffffffu, base, 0);
  if (visible) list[base + __popc(ballot & ((1u << lane) - 1u))] = entry;
}

// out[g,q,:] = sum_r w[g,r,q] * ctx[g*R+r,q,:] / den, float4 per thread.  mode 1: w = visibility (entries with
// w == 0 are not read: the gather kernel never wrote them), den = max(sum_r w, 1); mode 2: w = 1, den = R.
// The sum runs over r in order, in float32, like the reference's ReduceSum over the camera/queue axis.
__global__ void __launch_bounds__(256) msda_group_reduce_kernel(const float *__restrict__ ctx,
                                                                const float *__restrict__ vis,
                                                                float *__restrict__ out, int G, int R, int Q, int C4,
                                                                int q_begin, int q_count, int mode) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)G * q_count * C4;
  if (i >= total) return;
  const int c4 = (int)(i % C4);
  const long long gq = i / C4;
  const int q = q_begin + (int)(gq % q_count);
  const int g = (int)(gq / q_count);
  float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float count = 0.0f;
  for (int r = 0; r < R; ++r) {
    const long long row = (long long)(g * R + r) * Q + q;
    const float w = mode == 1 ? __ldg(vis + row) : 1.0f;
    count = __fadd_rn(count, w);
    if (w != 0.0f) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(ctx) + row * C4 + c4);
      sum.x = __fadd_rn(sum.x, __fmul_rn(v.x, w));
      sum.y = __fadd_rn(sum.y, __fmul_rn(v.y, w));
      sum.z = __fadd_rn(sum.z, __fmul_rn(v.z, w));
      sum.w = __fadd_rn(sum.w, __fmul_rn(v.w, w));
    }
  }
  const float den = mode == 1 ? fmaxf(count, 1.0f) : (float)R;
  float4 o = make_float4(__fdiv_rn(sum.x, den), __fdiv_rn(sum.y, den), __fdiv_rn(sum.z, den), __fdiv_rn(sum.w, den));
  __stcs(reinterpret_cast<float4 *>(out) + ((long long)g * Q + q) * C4 + c4, o);
}

__global__ void cast_f32_to_bf16_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst,
                                        size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// Launch shape of the rows kernel for one problem: fills the chunking fields of `a`, returns the geometry.
struct RowsGeometry {
  int grid, threads, rows_per_cta;
  size_t smem;
};

template <typename VT, int LPR>
RowsGeometry plan_rows(MsdaArgs &a) {
  constexpr int kThreads = RowsCta<VT>::kThreads;
  constexpr int RPI = kThreads / LPR;
  // rows that do not fit the small table are taken in chunks; those chunks may use the larger table of this texel type
  const int small_cap = kThreads * kRecordsPerThread / RPI;
  const int entries = a.LP <= small_cap ? kThreads * kRecordsPerThread : kThreads * RowsCta<VT>::kRecordsPerThreadLongRows;
  const int cap = entries / RPI > kUnroll ? entries / RPI : kUnroll;
  if (a.LP <= cap) {
    a.chunk_len = a.LP;
    a.chunk_pad = (a.LP + kUnroll - 1) / kUnroll * kUnroll;
    int j = cap / a.chunk_pad;
    a.rows_per_group = j < 1 ? 1 : (j > kMaxRowsPerGroup ? kMaxRowsPerGroup : j);
  } else {
    a.chunk_len = cap / kUnroll * kUnroll;
    a.chunk_pad = a.chunk_len;
    a.rows_per_group = 1;
  }
  a.div_chunk_pad.set((uint32_t)a.chunk_pad);
  RowsGeometry g;
  g.threads = kThreads;
  g.rows_per_cta = RPI * a.rows_per_group;
  g.smem = kMaxLevels * sizeof(int4) +
           (size_t)g.rows_per_cta * ((a.chunk_pad + 1) * (sizeof(float4) + sizeof(uint32_t)) + sizeof(int) + sizeof(float2));
  g.grid = (a.total_rows + g.rows_per_cta - 1) / g.rows_per_cta;
  return g;
}

// Per-device "attributes are set" flags of one kernel instantiation; calls may come from several host threads.
struct OncePerDevice {
  std::mutex lock;
  bool done[64] = {};
};

template <typename VT, int CPL, int LPR, bool FUSED>
int launch_rows(MsdaArgs &a, cudaStream_t stream) {
  const RowsGeometry g = plan_rows<VT, LPR>(a);
  auto kernel = msda_rows_kernel<VT, CPL, LPR, FUSED>;
  // Once per device: allow the largest record table and ask for a shared-memory
  // carve-out that leaves most of the 256 KB to L1, where coarse-level taps hit.
  static OncePerDevice once;
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != GACB_OK) return rc;
  if (device < 0 || device >= 64) return fail(GACB_ERR_UNSUPPORTED, "msda: device ordinal %d is out of range", device);
  {
    std::lock_guard<std::mutex> guard(once.lock);
    if (!once.done[device]) {
      rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024),
                      "cudaFuncSetAttribute(max dynamic shared memory)");
      if (rc != GACB_OK) return rc;
      rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, kCarveoutPercent),
                      "cudaFuncSetAttribute(carve-out)");
      if (rc != GACB_OK) return rc;
      once.done[device] = true;
    }
  }
  kernel<<<g.grid, g.threads, g.smem, stream>>>(a);
  return check_cuda(cudaGetLastError(), "msda_rows_kernel launch");
}

template <typename VT, int CPL, bool FUSED>
int dispatch_lanes(MsdaArgs &a, cudaStream_t stream, bool *handled) {
  *handled = true;
  switch (a.D / CPL) {
    case 1: return launch_rows<VT, CPL, 1, FUSED>(a, stream);
    case 2: return launch_rows<VT, CPL, 2, FUSED>(a, stream);
    case 4: return launch_rows<VT, CPL, 4, FUSED>(a, stream);
    case 8: return launch_rows<VT, CPL, 8, FUSED>(a, stream);
    case 16: return launch_rows<VT, CPL, 16, FUSED>(a, stream);
    case 32: return launch_rows<VT, CPL, 32, FUSED>(a, stream);
    default: *handled = false; return GACB_OK;
  }
}

// 1 = use the tile kernel where it applies, 0 = never (the rows kernel runs those shapes; the default).
// Measured on B200 (BEVFormer-base temporal self-attention, 200 x 200, P = 4): the tile kernel takes 84 us against
// 82 us for the rows kernel.  It cuts the L2 -> L1 traffic 4.6 times (1.3 GB -> 0.28 GB), but a tap read from shared
// memory costs the same 128-byte wavefront of the SM's one data pipe as a tap that hits in L1, and that pipe is
// then the limit: 17.2 M wavefronts per launch (10.2 M of them the taps themselves), 71 % of its peak.
std::atomic<int> g_tile_path{0};

// The tile kernel applies to float32 texels, head dim 32, one level whose texels ARE the query grid, few samples
// per row and no visibility mask.  Whether the samples really stay near their query's cell only decides how fast
// it is, not what it computes.
bool tile_path_applies(const MsdaArgs &a, int value_dtype) {
  return g_tile_path.load() != 0 && value_dtype == GACB_F32 && a.D == kTileD && a.L == 1 && a.LP <= kTileMaxSamples &&
         a.Q == a.lvl_h[0] * a.lvl_w[0] && a.S <= kTileMaxTexels && a.row_list == nullptr && a.row_mask == nullptr &&
         a.lvl_h[0] >= kTileH && a.lvl_w[0] >= kTileW;
}

struct TileGeometry {
  dim3 grid;
  int threads;
  size_t smem;
};

TileGeometry plan_tile(MsdaArgs &a) {
  a.chunk_len = a.LP;
  a.chunk_pad = a.LP <= 4 ? 4 : 8;
  TileGeometry g;
  const int W = a.lvl_w[0];
  const int tiles_x = (W + kTileW - 1) / kTileW;
  // tile rows down to the one holding the last query of [q_begin, q_begin + q_count); tile rows above the first
  // query return at once
  const int qy_last = (a.q_begin + a.q_count - 1) / W;
  g.grid = dim3((unsigned)(a.H * tiles_x), (unsigned)(qy_last / kTileH + 1), (unsigned)a.B);
  g.threads = kTileThreads;
  const int chunk_rows = kTileChunkRecords / a.chunk_pad;
  g.smem = (size_t)kWinH * kWinW * kTileD * 4 + (size_t)chunk_rows * (a.chunk_pad + 1) * (sizeof(float4) + sizeof(uint32_t)) +
           (size_t)kTileRows * sizeof(int) + 16 + (size_t)chunk_rows;
  return g;
}

template <bool FUSED, int CLP>
int launch_tile_clp(MsdaArgs &a, const TileGeometry &g, cudaStream_t stream) {
  auto kernel = msda_tile_kernel<FUSED, CLP>;
  static OncePerDevice once;
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != GACB_OK) return rc;
  if (device < 0 || device >= 64) return fail(GACB_ERR_UNSUPPORTED, "msda: device ordinal %d is out of range", device);
  {
    std::lock_guard<std::mutex> guard(once.lock);
    if (!once.done[device]) {
      rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 113 * 1024),
                      "cudaFuncSetAttribute(tile kernel shared memory)");
      if (rc != GACB_OK) return rc;
      rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared),
                      "cudaFuncSetAttribute(tile kernel carve-out)");
      if (rc != GACB_OK) return rc;
      once.done[device] = true;
    }
  }
  kernel<<<g.grid, g.threads, g.smem, stream>>>(a);
  return check_cuda(cudaGetLastError(), "msda_tile_kernel launch");
}

template <bool FUSED>
int launch_tile(MsdaArgs &a, cudaStream_t stream) {
  const TileGeometry g = plan_tile(a);
  return a.chunk_pad == 4 ? launch_tile_clp<FUSED, 4>(a, g, stream) : launch_tile_clp<FUSED, 8>(a, g, stream);
}

template <bool FUSED>
int launch_msda(MsdaArgs &a, int value_dtype, cudaStream_t stream) {
  if (a.total_rows == 0) return GACB_OK;
  if (tile_path_applies(a, value_dtype)) return launch_tile<FUSED>(a, stream);
  bool handled = false;
  int rc = GACB_OK;
  if (value_dtype == GACB_F32 && a.D % 4 == 0) rc = dispatch_lanes<float, 4, FUSED>(a, stream, &handled);
  if (value_dtype == GACB_BF16 && a.D % 8 == 0)
    rc = dispatch_lanes<__nv_bfloat16, 8, FUSED>(a, stream, &handled);
  if (handled) return rc;
  if (a.row_list) return fail(GACB_ERR_UNSUPPORTED, "msda: compacted visibility needs a head dim of 4*2^k (8*2^k for bf16)");
  const long long elems = (long long)a.total_rows * a.D;
  const int grid = (int)((elems + kThreads - 1) / kThreads);
  if (value_dtype == GACB_F32)
    msda_generic_kernel<float, FUSED><<<grid, kThreads, 0, stream>>>(a);
  else
    msda_generic_kernel<__nv_bfloat16, FUSED><<<grid, kThreads, 0, stream>>>(a);
  return check_cuda(cudaGetLastError(), "msda_generic_kernel launch");
}

int fill_common(MsdaArgs &a, const void *value, int value_dtype, const float *loc, const float *attn,
                float *out, const int32_t *spatial_hw, int L, int B, int S, int Q, int H, int D, int P,
                int q_begin, int q_end) {
  if (!spatial_hw) return fail(GACB_ERR_INVALID_ARGUMENT, "msda: spatial_hw is NULL");
  if (value_dtype != GACB_F32 && value_dtype != GACB_BF16)
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda: value_dtype %d is not GACB_F32/GACB_BF16", value_dtype);
  if (L <= 0 || B < 0 || S <= 0 || Q < 0 || H <= 0 || D <= 0 || P <= 0)
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda: extents must be positive (L=%d B=%d S=%d Q=%d H=%d D=%d P=%d)",
                L, B, S, Q, H, D, P);
  if (L > kMaxLevels) return fail(GACB_ERR_UNSUPPORTED, "msda: at most %d feature levels are supported", kMaxLevels);
  if (P > kMaxPoints)
    return fail(GACB_ERR_UNSUPPORTED, "msda: at most %d sampling points per level are supported", kMaxPoints);
  if (q_begin < 0 || q_end < q_begin || q_end > Q)
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda: query range [%d,%d) is outside [0,%d)", q_begin, q_end, Q);
  long long sum = 0;
  for (int l = 0; l < L; ++l) {
    const int h = spatial_hw[2 * l], w = spatial_hw[2 * l + 1];
    if (h <= 0 || w <= 0)
      return fail(GACB_ERR_SHAPE_MISMATCH, "msda: spatial_shapes[%d] = [%d,%d] must be positive", l, h, w);
    a.lvl_h[l] = h;
    a.lvl_w[l] = w;
    a.lvl_start[l] = (int)sum;
    sum += (long long)h * w;
  }
  if (sum != S)
    return fail(GACB_ERR_SHAPE_MISMATCH, "msda: value spatial dimension %d does not equal sum(H*W)=%lld", S, sum);
  const long long lim = 2147483647LL;
  if ((long long)B * S * H * D > lim || (long long)B * Q * H * L * P * 2 > lim || (long long)B * Q * H * D > lim)
    return fail(GACB_ERR_UNSUPPORTED, "msda: a tensor exceeds the 32-bit indexing range");
  const bool empty = (B == 0) || (q_end == q_begin);
  if (!empty && (!value || !loc || !attn || !out))
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda: a tensor pointer is NULL");
  a.value = value;
  a.loc = loc;
  a.attn = attn;
  a.out = out;
  a.normalizer = nullptr;
  a.reference = nullptr;
  a.B = B; a.S = S; a.H = H; a.D = D; a.L = L; a.P = P; a.Q = Q;
  a.q_begin = q_begin;
  a.q_count = q_end - q_begin;
  a.total_rows = B * a.q_count * H;
  a.LP = L * P;
  a.rows_per_group = 1;
  a.chunk_len = 1;
  a.chunk_pad = 1;
  a.div_chunk_pad.set(1);
  a.div_per_b.set((uint32_t)(a.q_count * H > 0 ? a.q_count * H : 1));
  a.div_h.set((uint32_t)H);
  a.div_p.set((uint32_t)P);
  a.div_q.set((uint32_t)(Q > 0 ? Q : 1));
  a.reference_first = 0;
  a.softmax = 0;
  a.row_mask = nullptr;
  a.row_list = nullptr;
  a.coord_rank = 0;
  return GACB_OK;
}

}  // namespace
}  // namespace gacb

using namespace gacb;

GACB_API int gacb_msda_forward(const void *value, int value_dtype, const float *loc, const float *attn,
                               float *out, const int32_t *spatial_hw, int L, int B, int S, int Q, int H,
                               int D, int P, int q_begin, int q_end, void *stream) {
  MsdaArgs a{};
  int rc = fill_common(a, value, value_dtype, loc, attn, out, spatial_hw, L, B, S, Q, H, D, P, q_begin, q_end);
  if (rc != GACB_OK) return rc;
  return launch_msda<false>(a, value_dtype, static_cast<cudaStream_t>(stream));
}

GACB_API int gacb_msda_logits_forward(const void *value, int value_dtype, const float *loc, const float *logits,
                                      float *out, const int32_t *spatial_hw, int L, int B, int S, int Q, int H,
                                      int D, int P, int q_begin, int q_end, void *stream) {
  MsdaArgs a{};
  int rc = fill_common(a, value, value_dtype, loc, logits, out, spatial_hw, L, B, S, Q, H, D, P, q_begin, q_end);
  if (rc != GACB_OK) return rc;
  a.softmax = 1;
  return launch_msda<false>(a, value_dtype, static_cast<cudaStream_t>(stream));
}

static int msda_offsets_impl(const void *value, int value_dtype, const float *offsets, const float *attn,
                             const float *normalizer, const float *reference, float *out,
                             const int32_t *spatial_hw, int L, int B, int S, int Q, int H, int D, int P,
                             const int32_t *norm_shape, const int32_t *coord_shape, const int32_t *ref_shape,
                             int coord_rank, int reference_first, int q_begin, int q_end, int softmax, void *stream,
                             const float *row_mask = nullptr, const int *row_list = nullptr) {
  MsdaArgs a{};
  int rc = fill_common(a, value, value_dtype, offsets, attn, out, spatial_hw, L, B, S, Q, H, D, P, q_begin, q_end);
  if (rc != GACB_OK) return rc;
  if (!norm_shape || !coord_shape || !ref_shape)
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda_offsets: a shape table is NULL");
  if (coord_rank < 1 || coord_rank > kMaxCoordRank)
    return fail(GACB_ERR_UNSUPPORTED, "msda_offsets: coordinate rank %d is outside [1,%d]", coord_rank, kMaxCoordRank);
  if (a.total_rows > 0 && (!normalizer || !reference))
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda_offsets: normalizer/reference pointer is NULL");
  const int loc_dim[6] = {B, Q, H, L, P, 2};
  long long stride = 1;
  for (int k = 5; k >= 0; --k) {
    if (norm_shape[k] != 1 && norm_shape[k] != loc_dim[k])
      return fail(GACB_ERR_SHAPE_MISMATCH, "msda_offsets: normalizer axis %d has extent %d, want 1 or %d", k,
                  norm_shape[k], loc_dim[k]);
    a.norm_stride[k] = norm_shape[k] == 1 ? 0 : (int)stride;
    stride *= norm_shape[k];
  }
  long long count = 1;
  stride = 1;
  int full_stride[kMaxCoordRank];
  for (int k = coord_rank - 1; k >= 0; --k) {
    if (coord_shape[k] <= 0 || (ref_shape[k] != 1 && ref_shape[k] != coord_shape[k]))
      return fail(GACB_ERR_SHAPE_MISMATCH, "msda_offsets: reference axis %d has extent %d, want 1 or %d", k,
                  ref_shape[k], coord_shape[k]);
    full_stride[k] = ref_shape[k] == 1 ? 0 : (int)stride;
    stride *= ref_shape[k];
    count *= coord_shape[k];
  }
  // The (x, y) axis apart when it is the last one; the other axes merged, innermost first: an outer axis joins the
  // inner one when both are broadcast or when it continues the inner one's run in memory.
  const bool split = coord_shape[coord_rank - 1] == 2;
  int md[kMaxCoordRank], ms[kMaxCoordRank], n = 0;
  for (int k = coord_rank - (split ? 2 : 1); k >= 0; --k) {
    const int d = coord_shape[k], st = full_stride[k];
    if (d == 1) continue;
    if (n > 0 && ((st == 0 && ms[n - 1] == 0) || (ms[n - 1] != 0 && (long long)st == (long long)ms[n - 1] * md[n - 1]))) {
      md[n - 1] *= d;
    } else {
      md[n] = d;
      ms[n] = st;
      ++n;
    }
  }
  if (n == 0) { md[0] = 1; ms[0] = 0; n = 1; }
  for (int k = 0; k < n; ++k) {          // outermost first
    a.coord_dim[k] = md[n - 1 - k];
    a.ref_stride[k] = ms[n - 1 - k];
    a.coord_div[k].set((uint32_t)md[n - 1 - k]);
  }
  a.comp_split = split ? 1 : 0;
  a.ref_comp_stride = split ? full_stride[coord_rank - 1] : 0;
  if (count != (long long)B * Q * H * L * P * 2)
    return fail(GACB_ERR_SHAPE_MISMATCH, "msda_offsets: coordinate_shape has %lld elements, locations have %lld",
                count, (long long)B * Q * H * L * P * 2);
  a.normalizer = normalizer;
  a.reference = reference;
  a.norm_elems = 1;
  for (int k = 0; k < 6; ++k) a.norm_elems *= norm_shape[k];
  a.ref_elems = 1;
  for (int k = 0; k < coord_rank; ++k) a.ref_elems *= ref_shape[k];
  a.coord_rank = n;
  a.reference_first = reference_first ? 1 : 0;
  a.softmax = softmax ? 1 : 0;
  a.row_mask = row_list ? nullptr : row_mask;
  a.row_list = row_list;
  return launch_msda<true>(a, value_dtype, static_cast<cudaStream_t>(stream));
}

GACB_API int gacb_msda_offsets_forward(const void *value, int value_dtype, const float *offsets,
                                       const float *attn, const float *normalizer, const float *reference,
                                       float *out, const int32_t *spatial_hw, int L, int B, int S, int Q,
                                       int H, int D, int P, const int32_t *norm_shape,
                                       const int32_t *coord_shape, const int32_t *ref_shape, int coord_rank,
                                       int reference_first, int q_begin, int q_end, void *stream) {
  return msda_offsets_impl(value, value_dtype, offsets, attn, normalizer, reference, out, spatial_hw, L, B, S, Q, H, D,
                           P, norm_shape, coord_shape, ref_shape, coord_rank, reference_first, q_begin, q_end, 0, stream);
}

GACB_API int gacb_msda_offsets_logits_forward(const void *value, int value_dtype, const float *offsets,
                                              const float *logits, const float *normalizer, const float *reference,
                                              float *out, const int32_t *spatial_hw, int L, int B, int S, int Q,
                                              int H, int D, int P, const int32_t *norm_shape,
                                              const int32_t *coord_shape, const int32_t *ref_shape, int coord_rank,
                                              int reference_first, int q_begin, int q_end, void *stream) {
  return msda_offsets_impl(value, value_dtype, offsets, logits, normalizer, reference, out, spatial_hw, L, B, S, Q, H,
                           D, P, norm_shape, coord_shape, ref_shape, coord_rank, reference_first, q_begin, q_end, 1,
                           stream);
}

GACB_API int gacb_msda_run(const gacb_msda_desc *d, void *stream_) {
  if (!d) return fail(GACB_ERR_INVALID_ARGUMENT, "msda_run: descriptor is NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int R = d->group <= 0 ? 1 : d->group;
  if (d->reduce_mode < 0 || d->reduce_mode > 2)
    return fail(GACB_ERR_INVALID_ARGUMENT, "msda_run: reduce_mode %d is not 0, 1 or 2", d->reduce_mode);
  if (d->reduce_mode != 0) {
    if (R < 1 || d->B % R) return fail(GACB_ERR_SHAPE_MISMATCH, "msda_run: batch %d is not a multiple of group %d", d->B, R);
    if (!d->reduce_out) return fail(GACB_ERR_INVALID_ARGUMENT, "msda_run: reduce_out is NULL");
    if (d->reduce_mode == 1 && !d->visibility)
      return fail(GACB_ERR_INVALID_ARGUMENT, "msda_run: the masked average needs a visibility tensor");
    if ((d->H * d->D) % 4) return fail(GACB_ERR_UNSUPPORTED, "msda_run: the group reduction needs H*D to be a multiple of 4");
    // The gather kernel never writes the rows that `visibility` masks out, and the plain mean reads every row.
    if (d->reduce_mode == 2 && d->visibility)
      return fail(GACB_ERR_INVALID_ARGUMENT,
                  "msda_run: reduce_mode 2 (mean) cannot be combined with a visibility tensor; use reduce_mode 1");
  }
  int rc;
  {
    // the whole descriptor is checked before anything is enqueued
    MsdaArgs probe{};
    rc = fill_common(probe, d->value, d->value_dtype, d->locations, d->attention, d->out, d->spatial_hw, d->L, d->B, d->S,
                     d->Q, d->H, d->D, d->P, d->q_begin, d->q_end);
    if (rc != GACB_OK) return rc;
  }
  const bool fused = d->normalizer || d->reference;
  // With a visibility tensor and scratch for the list, compact first: the gather kernel then runs dense CTAs over
  // the visible rows only.
  const int *row_list = nullptr;
  const int q_count = d->q_end - d->q_begin;
  if (d->visibility && d->compact_scratch && d->B > 0 && q_count > 0 && d->q_begin >= 0 && d->q_end <= d->Q) {
    if (d->compact_scratch_bytes < (size_t)(d->B * (long long)d->Q + 4) * sizeof(int))
      return fail(GACB_ERR_INVALID_ARGUMENT, "msda_run: compact_scratch needs %zu bytes",
                  (size_t)(d->B * (long long)d->Q + 4) * sizeof(int));
    int *list = static_cast<int *>(d->compact_scratch) + 4;
    rc = check_cuda(cudaMemsetAsync(d->compact_scratch, 0, 4 * sizeof(int), stream), "cudaMemsetAsync(compact counter)");
    if (rc != GACB_OK) return rc;
    const int n = d->B * q_count;
    msda_compact_visible_kernel<<<(n + 255) / 256, 256, 0, stream>>>(d->visibility, list, d->B, d->Q, d->q_begin, q_count);
    rc = check_cuda(cudaGetLastError(), "msda_compact_visible_kernel launch");
    if (rc != GACB_OK) return rc;
    row_list = list;
  }
  if (fused) {
    rc = msda_offsets_impl(d->value, d->value_dtype, d->locations, d->attention, d->normalizer, d->reference, d->out,
                           d->spatial_hw, d->L, d->B, d->S, d->Q, d->H, d->D, d->P, d->norm_shape, d->coord_shape,
                           d->ref_shape, d->coord_rank, d->reference_first, d->q_begin, d->q_end, d->attention_is_logits,
                           stream_, d->visibility, row_list);
  } else {
    MsdaArgs a{};
    rc = fill_common(a, d->value, d->value_dtype, d->locations, d->attention, d->out, d->spatial_hw, d->L, d->B, d->S,
                     d->Q, d->H, d->D, d->P, d->q_begin, d->q_end);
    if (rc != GACB_OK) return rc;
    a.softmax = d->attention_is_logits ? 1 : 0;
    a.row_mask = row_list ? nullptr : d->visibility;
    a.row_list = row_list;
    rc = launch_msda<false>(a, d->value_dtype, stream);
  }
  if (rc != GACB_OK || d->reduce_mode == 0) return rc;
  const int G = d->B / R, C4 = d->H * d->D / 4, qc = d->q_end - d->q_begin;
  const long long total = (long long)G * qc * C4;
  if (total == 0) return GACB_OK;
  msda_group_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(d->out, d->visibility, d->reduce_out, G,
                                                                                R, d->Q, C4, d->q_begin, qc,
                                                                                d->reduce_mode);
  return check_cuda(cudaGetLastError(), "msda_group_reduce_kernel launch");
}

GACB_API int gacb_cast_f32_to_bf16(const float *src, void *dst, size_t count, void *stream) {
  if (count == 0) return GACB_OK;
  if (!src || !dst) return fail(GACB_ERR_INVALID_ARGUMENT, "cast_f32_to_bf16: NULL pointer");
  size_t blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cast_f32_to_bf16_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16 *>(dst), count);
  return check_cuda(cudaGetLastError(), "cast_f32_to_bf16 launch");
}

namespace gacb {
int msda_check_record(unsigned int out[2]) {
  out[0] = out[1] = 0;
#if GACB_CHECKED
  return check_cuda(cudaMemcpyFromSymbol(out, g_check_record, 2 * sizeof(unsigned int)), "cudaMemcpyFromSymbol(check record)");
#else
  return GACB_OK;
#endif
}
}  // namespace gacb

GACB_API int gacb_msda_tile_path(int mode) {
  const int previous = g_tile_path.load();
  if (mode == 0 || mode == 1) g_tile_path.store(mode);
  return previous;
}


namespace {
template <typename VT>
bool rows_geometry(MsdaArgs &a, int cpl, gacb_launch_geometry *out) {
  RowsGeometry g;
  switch (a.D / cpl) {
    case 1: g = plan_rows<VT, 1>(a); break;
    case 2: g = plan_rows<VT, 2>(a); break;
    case 4: g = plan_rows<VT, 4>(a); break;
    case 8: g = plan_rows<VT, 8>(a); break;
    case 16: g = plan_rows<VT, 16>(a); break;
    case 32: g = plan_rows<VT, 32>(a); break;
    default: return false;
  }
  out->grid[0] = g.grid; out->grid[1] = out->grid[2] = 1;
  out->block[0] = g.threads; out->block[1] = out->block[2] = 1;
  out->dynamic_smem_bytes = g.smem;
  out->units_per_cta = g.rows_per_cta;
  return true;
}
}  // namespace

GACB_API int gacb_msda_launch_geometry(int value_dtype, const int32_t *spatial_hw, int L, int B, int S, int Q, int H, int D,
                                       int P, int q_begin, int q_end, gacb_launch_geometry *out) {
  if (!out) return fail(GACB_ERR_INVALID_ARGUMENT, "launch_geometry: out is NULL");
  MsdaArgs a{};
  static const float kDummy = 0.0f;     // never dereferenced: only the launch shape is wanted
  float sink = 0.0f;
  int rc = fill_common(a, &kDummy, value_dtype, &kDummy, &kDummy, &sink, spatial_hw, L, B, S, Q, H, D, P, q_begin, q_end);
  if (rc != GACB_OK) return rc;
  *out = gacb_launch_geometry{};
  if (a.total_rows == 0) {
    snprintf(out->kernel, sizeof(out->kernel), "none");
    return GACB_OK;
  }
  if (tile_path_applies(a, value_dtype)) {
    const TileGeometry g = plan_tile(a);
    out->grid[0] = (int)g.grid.x; out->grid[1] = (int)g.grid.y; out->grid[2] = (int)g.grid.z;
    out->block[0] = g.threads; out->block[1] = out->block[2] = 1;
    out->dynamic_smem_bytes = g.smem;
    out->units_per_cta = kTileRows;
    snprintf(out->kernel, sizeof(out->kernel), "msda_tile_kernel<%d>", a.chunk_pad);
    return GACB_OK;
  }
  bool vector = false;
  if (value_dtype == GACB_F32 && D % 4 == 0) vector = rows_geometry<float>(a, 4, out);
  if (value_dtype == GACB_BF16 && D % 8 == 0) vector = rows_geometry<__nv_bfloat16>(a, 8, out);
  if (vector) {
    snprintf(out->kernel, sizeof(out->kernel), "msda_rows_kernel<%s,%d,%d>", value_dtype == GACB_F32 ? "float" : "bf16",
             value_dtype == GACB_F32 ? 4 : 8, D / (value_dtype == GACB_F32 ? 4 : 8));
    return GACB_OK;
  }
  const long long elems = (long long)a.total_rows * a.D;
  out->grid[0] = (int)((elems + kThreads - 1) / kThreads); out->grid[1] = out->grid[2] = 1;
  out->block[0] = kThreads; out->block[1] = out->block[2] = 1;
  out->units_per_cta = kThreads;
  snprintf(out->kernel, sizeof(out->kernel), "msda_generic_kernel");
  return GACB_OK;
}
