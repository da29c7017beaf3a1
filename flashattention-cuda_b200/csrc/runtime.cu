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
extern "C" const char* fa_status_text(int status_word) {
  static thread_local char buf[160];
  if (status_word == 0) return "ok";
  const int code = status_word & 0xffff;
  const char* wait = "";
  switch (code) {
    case 0: break;
    case 21: wait = "dense attention: wait for the Q tiles timed out"; break;
    case 22: wait = "dense attention: wait for a K/V stage to fill timed out"; break;
    case 23: wait = "dense attention: wait for a K/V stage to drain timed out"; break;
    case 24: wait = "dense attention: wait for the scores timed out"; break;
    case 25: wait = "dense attention: wait for P timed out"; break;
    case 26: wait = "dense attention: wait for the last P V timed out"; break;
    case 27: wait = "dense attention: wait for the query buffers to drain timed out"; break;
    case 41: case 42: wait = "MLA pair kernel: wait for the query operand timed out"; break;
    case 43: case 44: wait = "MLA pair kernel: wait on a score-operand tile buffer timed out"; break;
    case 45: case 46: wait = "MLA pair kernel: wait on a value-operand tile buffer timed out"; break;
    case 47: wait = "MLA pair kernel: wait for the scores timed out"; break;
    case 48: wait = "MLA pair kernel: wait for P timed out"; break;
    case 49: wait = "MLA pair kernel: wait for a P V batch timed out"; break;
    case 52: wait = "MLA pair kernel: wait for the token scales timed out"; break;
    case 61: case 62: wait = "FP8 tcgen05 decode: wait on a K/V stage timed out"; break;
    case 63: case 64: wait = "FP8 tcgen05 decode: wait on a score buffer timed out"; break;
    case 65: wait = "FP8 tcgen05 decode: wait for P timed out"; break;
    case 66: wait = "FP8 tcgen05 decode: wait for a P V batch timed out"; break;
    case 67: wait = "FP8 tcgen05 decode: wait for the query operand timed out"; break;
    default: wait = "a bounded device wait timed out"; break;
  }
  snprintf(buf, sizeof buf, "%s%s%s (status 0x%x)", wait, (code && (status_word & FA_STATUS_BAD_BLOCK_TABLE)) ? "; " : "",
           (status_word & FA_STATUS_BAD_BLOCK_TABLE) ? "block-table entry outside [0, num_blocks)" : "", status_word);
  return buf;
}
extern "C" int fa_device_sm_count(int* sm_count) {
  if (!sm_count) return fa::fail(FA_ERR_INVALID, "fa_device_sm_count: null pointer");
  const int n = fa::device_sm_count();
  if (n <= 0) return fa::fail(FA_ERR_CUDA, "cannot query the SM count of the current device");
  *sm_count = n;
  return FA_OK;
}

// ---- tensor maps -------------------------------------------------------------------------------------
#include <cudaTypedefs.h>

#include "sm100.cuh"

namespace fa {

int encode_tensor_map(CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box, int swizzle_128b) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  CUtensorMapDataType dt;
  switch (dtype) {
    case FA_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case FA_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case FA_E4M3: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case FA_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return fail(FA_ERR_INVALID, "encode_tensor_map: unsupported dtype %d", dtype);
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = encode(out, dt, (cuuint32_t)rank, base, gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA_OK;
}

}  // namespace fa
