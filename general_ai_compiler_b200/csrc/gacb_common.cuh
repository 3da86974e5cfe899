// Shared host/device helpers for the gacb library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/gacb.h"

#define GACB_API extern "C" __attribute__((visibility("default")))

namespace gacb {

// Thread-local error text behind gacb_last_error_string().
void set_error(const char *fmt, ...);
int fail(int status, const char *fmt, ...);

inline int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return GACB_OK;
  return fail(GACB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Streaming (read-once) loads that stay out of L1, and plain cached loads for
// gathered texels.
__device__ __forceinline__ float2 ld_stream_f2(const float *p) {
  float2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream_f1(const float *p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_texel_f4(const float *p) {
  return __ldg(reinterpret_cast<const float4 *>(p));
}
__device__ __forceinline__ uint4 ld_texel_u4(const void *p) {
  return __ldg(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ void st_stream_f4(float *p, float4 v) {
  __stcs(reinterpret_cast<float4 *>(p), v);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }


// Checked build (-DGACB_CHECKED=1): the stand-in for a memory checker on boxes where none can be run.  Every
// gather offset, record-table slot and output index of the kernels goes through GACB_INDEX(index, limit, site):
// an index outside [0, limit) is counted in the translation unit's violation record (count, last site) and
// replaced by 0, so the access is skipped in effect and nothing faults.  gacb_checked_violations() reads the
// records.  In the normal build the macro is the index itself.
#ifndef GACB_CHECKED
#define GACB_CHECKED 0
#endif
#if GACB_CHECKED
#define GACB_CHECK_RECORD static __device__ unsigned int g_check_record[2]
#define GACB_INDEX(index, limit, site) gacb::checked_index((long long)(index), (long long)(limit), (site), g_check_record)
__device__ __forceinline__ long long checked_index(long long index, long long limit, unsigned int site, unsigned int *record) {
  if (index >= 0 && index < limit) return index;
  atomicAdd(&record[0], 1u);
  record[1] = site;
  return 0;
}
#else
#define GACB_CHECK_RECORD static_assert(true, "")
#define GACB_INDEX(index, limit, site) (index)
#endif
// Per translation unit: (violations, last site) of the checked build; both 0 in the normal build.
int msda_check_record(unsigned int out[2]);
int dcn_check_record(unsigned int out[2]);

// cuTensorMapEncodeTiled of the driver, looked up once through the runtime (the library does not link libcuda).
// Declared with plain pointer types so that this header does not need <cuda.h>; cast the arguments at the call.
#ifdef CUDA_VERSION
using TensorMapEncoder = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                      const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int tensor_map_encoder(TensorMapEncoder *fn);
#endif

// mbarrier and bulk-copy wrappers (sm_90+ PTX) shared by the kernels that stage tiles in shared memory.
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, size a multiple of 16);
// completion is counted in bytes on `bar`.  No cluster multicast.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// 16-byte asynchronous copy global -> shared (both 16-byte aligned), bypassing L1; completion is per thread:
// commit the copies issued so far as a group, then wait for all groups.
__device__ __forceinline__ void async_copy_16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void async_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void async_copy_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

}  // namespace gacb
