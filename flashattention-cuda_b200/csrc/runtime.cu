// Status plumbing and device queries shared by every entry point of libfa_b200.
#include "common.cuh"

namespace fa {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int device_sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fa

extern "C" const char* fa_last_error(void) { return fa::last_error_buf(); }
extern "C" int fa_version(void) { return 100; }
extern "C" int fa_device_sm_count(int* sm_count) {
  if (!sm_count) return fa::fail(FA_ERR_INVALID, "fa_device_sm_count: null pointer");
  const int n = fa::device_sm_count();
  if (n <= 0) return fa::fail(FA_ERR_CUDA, "cannot query the SM count of the current device");
  *sm_count = n;
  return FA_OK;
}
