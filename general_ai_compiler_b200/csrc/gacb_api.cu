// Library-wide entry points: version, error text, device queries.
#include <stdarg.h>

#include <cuda.h>   // CUtensorMap types for tensor_map_encoder (declared in the common header when this comes first)

#include <atomic>

#include "gacb_common.cuh"

namespace gacb {

int tensor_map_encoder(TensorMapEncoder *fn) {
  static std::atomic<TensorMapEncoder> cached{nullptr};
  TensorMapEncoder f = cached.load();
  if (!f) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult found;
    const int rc = check_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &found),
                              "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (rc != GACB_OK) return rc;
    if (found != cudaDriverEntryPointSuccess || !sym)
      return fail(GACB_ERR_UNSUPPORTED, "the driver does not provide cuTensorMapEncodeTiled");
    f = reinterpret_cast<TensorMapEncoder>(sym);
    cached.store(f);
  }
  *fn = f;
  return GACB_OK;
}

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

}  // namespace gacb

GACB_API int gacb_version(void) { return GACB_ABI_VERSION; }

GACB_API const char *gacb_last_error_string(void) { return gacb::g_error; }

GACB_API int gacb_device_count(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return gacb::fail(GACB_ERR_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  return n;
}

GACB_API int gacb_device_capability(int device) {
  int major = 0, minor = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return gacb::fail(GACB_ERR_NO_DEVICE, "device %d: %s", device, cudaGetErrorString(e));
  }
  return major * 10 + minor;
}

GACB_API int gacb_status_from_word(int32_t word) {
  if (word == 0) return GACB_OK;
  return gacb::fail(GACB_ERR_DEVICE_TIMEOUT,
                    "a kernel gave up a bounded wait (device status word = %d); its output is incomplete", (int)word);
}

GACB_API int gacb_read_status_word(const int32_t *status_word, void *stream) {
  if (!status_word) return gacb::fail(GACB_ERR_INVALID_ARGUMENT, "read_status_word: status_word is NULL");
  int32_t word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&word, status_word, sizeof(word), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return gacb::check_cuda(e, "read_status_word");
  return gacb_status_from_word(word);
}

GACB_API int gacb_checked_violations(unsigned int *count, unsigned int *last_site) {
#if GACB_CHECKED
  unsigned int m[2] = {0, 0}, d[2] = {0, 0};
  int rc = gacb::msda_check_record(m);
  if (rc == GACB_OK) rc = gacb::dcn_check_record(d);
  if (rc != GACB_OK) return rc;
  if (count) *count = m[0] + d[0];
  if (last_site) *last_site = d[0] ? d[1] : m[1];
  return GACB_OK;
#else
  (void)count;
  (void)last_site;
  return gacb::fail(GACB_ERR_UNSUPPORTED, "this libgacb.so was not built with -DGACB_CHECKED=1");
#endif
}
