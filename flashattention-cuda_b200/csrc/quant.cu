// KV-cache data formats: FP8 E4M3 and NVFP4 quantise / dequantise, and the paged-pool scatter / gather.
//
// Bit-exact restatements of the reference's torch functions:
//   quantize_fp8_e4m3 / dequantize_fp8_e4m3   fa_kernels/paged.py:94-118
//   quantize_nvfp4 / dequantize_nvfp4         fa_kernels/paged.py:136-189
//   build_paged_kv (scatter under a block table, zero padded tail page)   fa_kernels/paged.py:48-91
// Rounding semantics that matter: the E4M3 cast is round-to-nearest-even and not saturating
// (>= 480 after rounding is NaN); E2M1 rounding is "number of midpoints strictly below |y|" (ties go
// to the smaller magnitude, NaN takes the largest code); the sign bit is (y < 0), so -0.0 stores +0;
// the low nibble of a packed byte is the even element.  All divisions are IEEE fp32 divisions in the
// order the reference writes them.

#include "common.cuh"

namespace fa {
namespace {

__device__ __forceinline__ uint8_t f32_to_e4m3_rne(float f) {
  uint32_t u = __float_as_uint(f);
  const uint8_t sign = (u >> 24) & 0x80;
  u &= 0x7fffffffu;
  uint32_t r;
  if (u >= 0x43f00000u) {                 // >= 480 (also inf / NaN): no representation
    r = 0x7f;
  } else if (u < 0x3c800000u) {           // below 2^-6: subnormal, quantum 2^-9
    const float q = __fmul_rn(__uint_as_float(u), 512.0f);   // exact scaling
    r = (uint32_t)__float2int_rn(q);      // round-half-even; 8 -> 0x08 = smallest normal
  } else {
    const uint32_t odd = (u >> 20) & 1u;
    u += 0x7ffffu + odd;                  // round to 3 mantissa bits, ties to even
    r = (u >> 20) - ((127u - 7u) << 3);   // rebias exponent 127 -> 7
  }
  return (uint8_t)(r | sign);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  const uint32_t e = (b >> 3) & 0xf, m = b & 7;
  float v;
  if ((b & 0x7f) == 0x7f) v = __uint_as_float(0x7fc00000u);
  else if (e == 0) v = (float)m * 0.001953125f;                    // m * 2^-9
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return (b & 0x80) ? -v : v;
}

__device__ __constant__ float kE2M1Levels[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

__device__ __forceinline__ uint32_t e2m1_code(float y) {
  const float ay = fabsf(y);
  uint32_t idx;
  if (ay != ay) idx = 7;                                            // NaN sorts last
  else idx = (0.25f < ay) + (0.75f < ay) + (1.25f < ay) + (1.75f < ay) + (2.5f < ay) + (3.5f < ay) + (5.0f < ay);
  return ((y < 0.f) ? 8u : 0u) | idx;
}

template <typename T>
__device__ __forceinline__ float load_f32(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_f32<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float load_f32<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float load_f32<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// ---- abs-max: per tensor (one word) or per row of `row` elements ---------------------------------
template <typename T>
__global__ void absmax_tensor_kernel(const T* __restrict__ x, int64_t n, uint32_t* __restrict__ out_bits) {
  float m = 0.f;
  bool nan = false;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fabsf(load_f32(x, i));
    nan |= (v != v);
    m = fmaxf(m, v);
  }
  if (nan) m = __uint_as_float(0x7fc00000u);
  uint32_t bits = __float_as_uint(m);        // non-negative floats order like their bit patterns; NaN on top
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, bits);
}

// ---- FP8 ------------------------------------------------------------------------------------------
// per_row == 0: one scale for the tensor, scale = float(max(amax, 1e-12) / 448) from amax_bits[0]
// per_row  > 0: one scale per row of `per_row` elements (one warp per row), written to scales[row]
template <typename T>
__global__ void quantize_fp8_kernel(const T* __restrict__ x, int64_t n, int per_row, const uint32_t* __restrict__ amax_bits,
                                    uint8_t* __restrict__ out, float* __restrict__ scales) {
  if (per_row == 0) {
    const float amax = fmaxf(__uint_as_float(amax_bits[0]), 1e-12f);
    const float scale = __fdiv_rn(amax, 448.0f);
    if (blockIdx.x == 0 && threadIdx.x == 0) scales[0] = scale;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
      out[i] = f32_to_e4m3_rne(__fdiv_rn(load_f32(x, i), scale));
  } else {
    const int lane = threadIdx.x & 31;
    const int64_t rows = n / per_row;
    for (int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += (int64_t)gridDim.x * (blockDim.x >> 5)) {
      const T* xr = x + row * per_row;
      float m = 0.f;
      for (int i = lane; i < per_row; i += 32) m = fmaxf(m, fabsf(load_f32(xr, i)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float scale = __fdiv_rn(fmaxf(m, 1e-12f), 448.0f);
      if (lane == 0) scales[row] = scale;
      for (int i = lane; i < per_row; i += 32) out[row * per_row + i] = f32_to_e4m3_rne(__fdiv_rn(load_f32(xr, i), scale));
    }
  }
}

__global__ void dequantize_fp8_kernel(const uint8_t* __restrict__ b, int64_t n, float scale, const float* __restrict__ row_scales,
                                      int per_row, float* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float s = row_scales ? row_scales[i / per_row] : scale;
    out[i] = __fmul_rn(e4m3_to_f32(b[i]), s);
  }
}

// ---- NVFP4: one thread per 16-element block -------------------------------------------------------
template <typename T>
__global__ void quantize_nvfp4_kernel(const T* __restrict__ x, int64_t n_blocks, const uint32_t* __restrict__ amax_bits,
                                      uint8_t* __restrict__ packed, uint8_t* __restrict__ micro, float* __restrict__ scale_out) {
  const float gmax = fmaxf(__uint_as_float(amax_bits[0]), 1e-12f);
  const float scale = __fdiv_rn(gmax, 2688.0f);                     // 6 * 448
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_out[0] = scale;
  for (int64_t blk = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; blk < n_blocks; blk += (int64_t)gridDim.x * blockDim.x) {
    float v[16];
    float bmax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = load_f32(x, blk * 16 + i);
      bmax = fmaxf(bmax, fabsf(v[i]));
    }
    bmax = fmaxf(bmax, 1e-12f);
    const uint8_t mb = f32_to_e4m3_rne(__fdiv_rn(__fdiv_rn(bmax, 6.0f), scale));
    micro[blk] = mb;
    const float eff = __fmul_rn(e4m3_to_f32(mb), scale);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo |= e2m1_code(__fdiv_rn(v[i], eff)) << (4 * i);
      hi |= e2m1_code(__fdiv_rn(v[8 + i], eff)) << (4 * i);
    }
    reinterpret_cast<uint2*>(packed)[blk] = make_uint2(lo, hi);
  }
}

__global__ void dequantize_nvfp4_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ micro, int64_t n_blocks,
                                        float scale, float* __restrict__ out) {
  for (int64_t blk = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; blk < n_blocks; blk += (int64_t)gridDim.x * blockDim.x) {
    const uint2 w = reinterpret_cast<const uint2*>(packed)[blk];
    const float m = __fmul_rn(e4m3_to_f32(micro[blk]), scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t code = ((i < 8 ? w.x : w.y) >> (4 * (i & 7))) & 0xf;
      const float mag = kE2M1Levels[code & 7];
      out[blk * 16 + i] = __fmul_rn((code & 8) ? -mag : mag, m);
    }
  }
}

// ---- pager: rows of `row_bytes` bytes ---------------------------------------------------------------
// dense [B, H, N, row] <-> pool [num_blocks, page, H, row] through block_table [B, n_logical].
// One thread moves 16 bytes when row_bytes % 16 == 0 (vec = 16) else 1 byte.
template <int VEC, bool SCATTER>
__global__ void paged_move_kernel(uint8_t* __restrict__ dense, uint8_t* __restrict__ pool, const int32_t* __restrict__ bt,
                                  int B, int H, int N, int row_bytes, int page, int n_logical, int num_blocks) {
  const int vpr = row_bytes / VEC;
  // scatter iterates over the padded pool rows (to zero the tail); gather over the dense rows
  const int64_t n_tok = SCATTER ? (int64_t)n_logical * page : N;
  const int64_t total = (int64_t)B * n_tok * H * vpr;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vpr);
    int64_t r = i / vpr;
    const int h = (int)(r % H);
    r /= H;
    const int tok = (int)(r % n_tok);
    const int b = (int)(r / n_tok);
    const int lp = tok / page, off = tok - lp * page;
    const int pb = bt[(int64_t)b * n_logical + lp];
    if ((unsigned)pb >= (unsigned)num_blocks) continue;
    uint8_t* pp = pool + ((((int64_t)pb * page + off) * H + h) * row_bytes) + (int64_t)v * VEC;
    uint8_t* dp = dense + ((((int64_t)b * H + h) * N + tok) * row_bytes) + (int64_t)v * VEC;
    if constexpr (VEC == 16) {
      if (SCATTER) *reinterpret_cast<uint4*>(pp) = (tok < N) ? *reinterpret_cast<const uint4*>(dp) : make_uint4(0, 0, 0, 0);
      else *reinterpret_cast<uint4*>(dp) = *reinterpret_cast<const uint4*>(pp);
    } else {
      if (SCATTER) *pp = (tok < N) ? *dp : (uint8_t)0;
      else *dp = *pp;
    }
  }
}

// ---- NVFP4 scale-granularity study: quantise-dequantise in fp32 at one scale per tensor, per channel
// (last-dim index) or per token (row) — fa_kernels/nvfp4_recipes.py:42-73 of the reference -------------
// amax[] holds float bit patterns: [1] (tensor), [d] (channel) or [rows] (token)
__global__ void absmax_axis_kernel(const float* __restrict__ x, int64_t rows, int d, int mode, uint32_t* __restrict__ amax) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < rows * d; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fabsf(x[i]);
    const uint32_t bits = (v != v) ? 0x7fc00000u : __float_as_uint(v);
    const int64_t slot = mode == 0 ? 0 : (mode == 1 ? (i % d) : (i / d));
    atomicMax(amax + slot, bits);
  }
}
__global__ void fake_quant_apply_kernel(const float* __restrict__ x, int64_t rows, int d, int mode, int e4m3_scale,
                                        const uint32_t* __restrict__ amax, float* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < rows * d; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t slot = mode == 0 ? 0 : (mode == 1 ? (i % d) : (i / d));
    float scale = fmaxf(__fdiv_rn(__uint_as_float(amax[slot]), 6.0f), 1e-12f);
    if (e4m3_scale) scale = fmaxf(e4m3_to_f32(f32_to_e4m3_rne(scale)), 1e-12f);
    const float y = __fdiv_rn(x[i], scale);
    const uint32_t code = e2m1_code(y);
    const float mag = kE2M1Levels[code & 7];
    // torch.sign: 0 for +-0, NaN stays NaN
    const float sgn = (y != y) ? y : ((y > 0.f) ? 1.f : ((y < 0.f) ? -1.f : 0.f));
    out[i] = __fmul_rn(__fmul_rn(sgn, mag), scale);
  }
}

// ---- KV-cache write path: append T new tokens per sequence to a paged pool, quantising on the way ----------
// x: [B, H, T, d] (f32 / f16 / bf16).  Token t of sequence b goes to logical position pos[b] + t, i.e. to
// pool row (block_table[b][p / page] * page + p % page, h).  One warp per (b, t, h) row.
//   mode 0: store as fp16      mode 1: store as bf16
//   mode 2: FP8 E4M3 with one fp32 scale per row (amax / 448), scale written to scale_pool[row]
//   mode 3: NVFP4 with the caller's tensor scale: E4M3 micro-scale per 16 elements + packed E2M1 codes
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ x, const int32_t* __restrict__ pos, const int32_t* __restrict__ bt,
                                 int B, int H, int Tn, int d, int page, int n_logical, int num_blocks, int mode,
                                 float tensor_scale, uint8_t* __restrict__ pool, float* __restrict__ scale_pool,
                                 uint8_t* __restrict__ micro_pool, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)B * H * Tn;
  for (int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int t = (int)(row % Tn);
    const int h = (int)((row / Tn) % H);
    const int b = (int)(row / ((int64_t)Tn * H));
    const int p = pos[b] + t;
    const int lp = p / page;
    if (p < 0 || lp >= n_logical) { if (status && lane == 0) atomicOr(status, 2); continue; }
    const int pb = bt[(int64_t)b * n_logical + lp];
    if ((unsigned)pb >= (unsigned)num_blocks) { if (status && lane == 0) atomicOr(status, 1); continue; }
    const int64_t prow = ((int64_t)pb * page + (p - lp * page)) * H + h;     // token-head row of the pool
    const T* xr = x + row * d;
    if (mode == 0 || mode == 1) {
      uint16_t* dst = reinterpret_cast<uint16_t*>(pool) + prow * d;
      for (int i = lane; i < d; i += 32) {
        const float v = load_f32(xr, i);
        if (mode == 0) { __half hv = __float2half_rn(v); dst[i] = *reinterpret_cast<uint16_t*>(&hv); }
        else { __nv_bfloat16 bv = __float2bfloat16_rn(v); dst[i] = *reinterpret_cast<uint16_t*>(&bv); }
      }
    } else if (mode == 2) {
      float m = 0.f;
      for (int i = lane; i < d; i += 32) m = fmaxf(m, fabsf(load_f32(xr, i)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float scale = __fdiv_rn(fmaxf(m, 1e-12f), 448.0f);
      if (lane == 0) scale_pool[prow] = scale;
      for (int i = lane; i < d; i += 32) pool[prow * d + i] = f32_to_e4m3_rne(__fdiv_rn(load_f32(xr, i), scale));
    } else {
      for (int blk = lane; blk < d / 16; blk += 32) {
        float v[16];
        float bmax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          v[i] = load_f32(xr, blk * 16 + i);
          bmax = fmaxf(bmax, fabsf(v[i]));
        }
        bmax = fmaxf(bmax, 1e-12f);
        const uint8_t mb = f32_to_e4m3_rne(__fdiv_rn(__fdiv_rn(bmax, 6.0f), tensor_scale));
        micro_pool[prow * (d / 16) + blk] = mb;
        const float eff = __fmul_rn(e4m3_to_f32(mb), tensor_scale);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          lo |= e2m1_code(__fdiv_rn(v[i], eff)) << (4 * i);
          hi |= e2m1_code(__fdiv_rn(v[8 + i], eff)) << (4 * i);
        }
        reinterpret_cast<uint2*>(pool + prow * (d / 2))[blk] = make_uint2(lo, hi);
      }
    }
  }
}

inline int grid_for(int64_t work, int threads, int sms) {
  const int64_t blocks = (work + threads - 1) / threads;
  return (int)std::max<int64_t>(1, std::min<int64_t>(blocks, (int64_t)sms * 8));
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" int fa_quantize_fp8_e4m3(const void* x, int x_dtype, int64_t n, int per_row, uint8_t* out, float* scales,
                                    void* scratch4, void* stream) {
  FA_CHECK_ARG(x && out && scales, "fa_quantize_fp8_e4m3: null pointer");
  FA_CHECK_ARG(n >= 1 && per_row >= 0 && (per_row == 0 || n % per_row == 0), "fa_quantize_fp8_e4m3: bad sizes");
  FA_CHECK_ARG(per_row > 0 || scratch4 != nullptr, "fa_quantize_fp8_e4m3: per-tensor mode needs a 4-byte scratch word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int sms = std::max(device_sm_count(), 1);
  uint32_t* amax = reinterpret_cast<uint32_t*>(scratch4);
  if (per_row == 0) FA_CUDA_OK(cudaMemsetAsync(amax, 0, 4, st));
  const int64_t work = per_row ? (n / per_row) * 32 : n;
#define FA_Q8(T)                                                                                         \
  do {                                                                                                   \
    if (per_row == 0) absmax_tensor_kernel<T><<<grid_for(n, 256, sms), 256, 0, st>>>((const T*)x, n, amax); \
    quantize_fp8_kernel<T><<<grid_for(work, 256, sms), 256, 0, st>>>((const T*)x, n, per_row, amax, out, scales); \
  } while (0)
  if (x_dtype == FA_F32) FA_Q8(float);
  else if (x_dtype == FA_F16) FA_Q8(__half);
  else if (x_dtype == FA_BF16) FA_Q8(__nv_bfloat16);
  else return fail(FA_ERR_INVALID, "fa_quantize_fp8_e4m3: x must be f32/f16/bf16");
#undef FA_Q8
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_dequantize_fp8_e4m3(const uint8_t* bytes, int64_t n, float scale, const float* row_scales, int per_row,
                                      float* out, void* stream) {
  FA_CHECK_ARG(bytes && out && n >= 1, "fa_dequantize_fp8_e4m3: bad arguments");
  FA_CHECK_ARG(row_scales == nullptr || (per_row > 0 && n % per_row == 0), "fa_dequantize_fp8_e4m3: bad per_row");
  const int sms = std::max(device_sm_count(), 1);
  dequantize_fp8_kernel<<<grid_for(n, 256, sms), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      bytes, n, scale, row_scales, per_row > 0 ? per_row : 1, out);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_quantize_nvfp4(const void* x, int x_dtype, int64_t n, uint8_t* packed, uint8_t* micro, float* scale_out,
                                 void* scratch4, void* stream) {
  FA_CHECK_ARG(x && packed && micro && scale_out && scratch4, "fa_quantize_nvfp4: null pointer");
  FA_CHECK_ARG(n >= 16 && n % 16 == 0, "fa_quantize_nvfp4: element count must be a multiple of the NVFP4 block (16)");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int sms = std::max(device_sm_count(), 1);
  uint32_t* amax = reinterpret_cast<uint32_t*>(scratch4);
  FA_CUDA_OK(cudaMemsetAsync(amax, 0, 4, st));
#define FA_Q4(T)                                                                                   \
  do {                                                                                             \
    absmax_tensor_kernel<T><<<grid_for(n, 256, sms), 256, 0, st>>>((const T*)x, n, amax);          \
    quantize_nvfp4_kernel<T><<<grid_for(n / 16, 128, sms), 128, 0, st>>>((const T*)x, n / 16, amax, packed, micro, scale_out); \
  } while (0)
  if (x_dtype == FA_F32) FA_Q4(float);
  else if (x_dtype == FA_F16) FA_Q4(__half);
  else if (x_dtype == FA_BF16) FA_Q4(__nv_bfloat16);
  else return fail(FA_ERR_INVALID, "fa_quantize_nvfp4: x must be f32/f16/bf16");
#undef FA_Q4
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

// ---- quantised MLA latent -> bf16 pool (the operand format of the tensor-core MLA kernels) -----------------
// Only the tokens of the planned key ranges are expanded, each into the same pool row of the bf16 copy.
// One thread per 16 elements (one NVFP4 micro-block, or 16 E4M3 bytes of a token row); grid (items, 8).
__global__ void expand_latent_kernel(const uint8_t* __restrict__ src, const uint8_t* __restrict__ micro,
                                     const float* __restrict__ token_scale, float tensor_scale, int is_nvfp4,
                                     const int32_t* __restrict__ block_table, int n_logical, int num_blocks, int page_size,
                                     int page_shift, const fa_decode_item* __restrict__ items, int dqk,
                                     __nv_bfloat16* __restrict__ out) {
  const fa_decode_item it = items[blockIdx.x];
  const int per_tok = dqk / 16;
  const int64_t n_tok = it.k_end - it.k_begin;
  const int64_t lo = n_tok * blockIdx.y / gridDim.y, hi = n_tok * (blockIdx.y + 1) / gridDim.y;
  const int32_t* bt = block_table + (int64_t)it.b * n_logical;
  for (int64_t w = lo * per_tok + threadIdx.x; w < hi * per_tok; w += blockDim.x) {
    const int key = it.k_begin + (int)(w / per_tok);
    const int c16 = (int)(w % per_tok);
    const int pg = key >> page_shift;
    const int pid = pg < n_logical ? bt[pg] : -1;
    if ((unsigned)pid >= (unsigned)num_blocks) continue;          // the attention kernel flags bad entries
    const int64_t i = ((int64_t)pid * page_size + (key - (pg << page_shift))) * per_tok + c16;   // 16-element chunk in the pool
    float v[16];
    if (is_nvfp4) {
      const uint2 q = *reinterpret_cast<const uint2*>(src + i * 8);
      const float m = __fmul_rn(e4m3_to_f32(micro[i]), tensor_scale);
      uint32_t h[8];                                   // sixteen codes -> eight half2 (exact)
      e2m1x8_to_h2x4(q.x, *reinterpret_cast<uint32_t(*)[4]>(&h[0]));
      e2m1x8_to_h2x4(q.y, *reinterpret_cast<uint32_t(*)[4]>(&h[4]));
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[e]));
        v[2 * e] = __fmul_rn(f.x, m);
        v[2 * e + 1] = __fmul_rn(f.y, m);
      }
    } else {
      const uint4 q = *reinterpret_cast<const uint4*>(src + i * 16);
      const float sc = token_scale ? token_scale[i / per_tok] : tensor_scale;
      const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {                    // four bytes -> two half2 (exact, NaN stays NaN)
        uint32_t lo, hi;
        e4m3x4_to_h2x2(ws[e], lo, hi);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
        const float2 b2 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        v[4 * e] = __fmul_rn(a.x, sc);
        v[4 * e + 1] = __fmul_rn(a.y, sc);
        v[4 * e + 2] = __fmul_rn(b2.x, sc);
        v[4 * e + 3] = __fmul_rn(b2.y, sc);
      }
    }
    uint4 o0, o1;
    o0.x = pack_bf2(v[0], v[1]);   o0.y = pack_bf2(v[2], v[3]);   o0.z = pack_bf2(v[4], v[5]);   o0.w = pack_bf2(v[6], v[7]);
    o1.x = pack_bf2(v[8], v[9]);   o1.y = pack_bf2(v[10], v[11]); o1.z = pack_bf2(v[12], v[13]); o1.w = pack_bf2(v[14], v[15]);
    uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
    dst[0] = o0;
    dst[1] = o1;
  }
}

extern "C" int fa_dequantize_nvfp4(const uint8_t* packed, const uint8_t* micro, int64_t n, float scale, float* out, void* stream) {
  FA_CHECK_ARG(packed && micro && out && n >= 16 && n % 16 == 0, "fa_dequantize_nvfp4: bad arguments");
  const int sms = std::max(device_sm_count(), 1);
  dequantize_nvfp4_kernel<<<grid_for(n / 16, 128, sms), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      packed, micro, n / 16, scale, out);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

static int paged_move(bool scatter, void* dense, void* pool, const int32_t* bt, int B, int H, int N, int row_bytes, int page,
                      int n_logical, int num_blocks, void* stream) {
  FA_CHECK_ARG(dense && pool && bt, "paged scatter/gather: null pointer");
  FA_CHECK_ARG(B >= 1 && H >= 1 && N >= 0 && row_bytes >= 1 && page >= 1 && n_logical >= 1 && num_blocks >= 1,
               "paged scatter/gather: bad sizes");
  FA_CHECK_ARG((int64_t)n_logical * page >= N, "block_table n_logical*page_size must cover N_k logical positions");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int sms = std::max(device_sm_count(), 1);
  const bool vec = (row_bytes % 16 == 0) && (((uintptr_t)dense | (uintptr_t)pool) % 16 == 0);
  const int64_t n_tok = scatter ? (int64_t)n_logical * page : N;
  const int64_t work = (int64_t)B * n_tok * H * (vec ? row_bytes / 16 : row_bytes);
  if (work == 0) return FA_OK;
  uint8_t* d = reinterpret_cast<uint8_t*>(dense);
  uint8_t* p = reinterpret_cast<uint8_t*>(pool);
  const int g = grid_for(work, 256, sms);
  if (vec && scatter) paged_move_kernel<16, true><<<g, 256, 0, st>>>(d, p, bt, B, H, N, row_bytes, page, n_logical, num_blocks);
  else if (vec) paged_move_kernel<16, false><<<g, 256, 0, st>>>(d, p, bt, B, H, N, row_bytes, page, n_logical, num_blocks);
  else if (scatter) paged_move_kernel<1, true><<<g, 256, 0, st>>>(d, p, bt, B, H, N, row_bytes, page, n_logical, num_blocks);
  else paged_move_kernel<1, false><<<g, 256, 0, st>>>(d, p, bt, B, H, N, row_bytes, page, n_logical, num_blocks);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_paged_scatter(const void* dense, void* pool, const int32_t* block_table, int B, int H, int N, int row_bytes,
                                int page_size, int n_logical, int num_blocks, void* stream) {
  return paged_move(true, const_cast<void*>(dense), pool, block_table, B, H, N, row_bytes, page_size, n_logical, num_blocks, stream);
}

extern "C" int fa_paged_gather(const void* pool, void* dense, const int32_t* block_table, int B, int H, int N, int row_bytes,
                               int page_size, int n_logical, int num_blocks, void* stream) {
  return paged_move(false, dense, const_cast<void*>(pool), block_table, B, H, N, row_bytes, page_size, n_logical, num_blocks, stream);
}

extern "C" int fa_fake_quant_e2m1(const float* x, int64_t rows, int d, int granularity, int e4m3_scale, float* out,
                                  void* scratch, size_t scratch_bytes, void* stream) {
  FA_CHECK_ARG(x && out && scratch, "fa_fake_quant_e2m1: null pointer");
  FA_CHECK_ARG(rows >= 1 && d >= 1, "fa_fake_quant_e2m1: bad sizes");
  FA_CHECK_ARG(granularity >= 0 && granularity <= 2, "fa_fake_quant_e2m1: granularity must be 0 (tensor), 1 (channel) or 2 (token)");
  const int64_t n_amax = granularity == 0 ? 1 : (granularity == 1 ? d : rows);
  if (scratch_bytes < (size_t)n_amax * 4) return fail(FA_ERR_WORKSPACE, "fa_fake_quant_e2m1: scratch %zu B < %lld B", scratch_bytes, (long long)n_amax * 4);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int sms = std::max(device_sm_count(), 1);
  uint32_t* amax = reinterpret_cast<uint32_t*>(scratch);
  FA_CUDA_OK(cudaMemsetAsync(amax, 0, (size_t)n_amax * 4, st));
  const int g = grid_for(rows * d, 256, sms);
  absmax_axis_kernel<<<g, 256, 0, st>>>(x, rows, d, granularity, amax);
  fake_quant_apply_kernel<<<g, 256, 0, st>>>(x, rows, d, granularity, e4m3_scale, amax, out);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_kv_append(const void* x, int x_dtype, const int32_t* positions, const int32_t* block_table, int B, int H,
                            int T, int d, int page_size, int n_logical, int num_blocks, int pool_dtype, float tensor_scale,
                            void* pool, float* scale_pool, uint8_t* micro_pool, int* status, void* stream) {
  FA_CHECK_ARG(x && positions && block_table && pool, "fa_kv_append: null pointer");
  FA_CHECK_ARG(B >= 1 && H >= 1 && T >= 1 && d >= 1 && page_size >= 1 && n_logical >= 1 && num_blocks >= 1, "fa_kv_append: bad sizes");
  int mode;
  switch (pool_dtype) {
    case FA_F16: mode = 0; break;
    case FA_BF16: mode = 1; break;
    case FA_E4M3: mode = 2; FA_CHECK_ARG(scale_pool != nullptr, "fa_kv_append: e4m3 pools need the per-token scale pool"); break;
    case FA_NVFP4:
      mode = 3;
      FA_CHECK_ARG(micro_pool != nullptr && d % 16 == 0, "fa_kv_append: nvfp4 pools need the micro-scale pool and d % 16 == 0");
      FA_CHECK_ARG(tensor_scale > 0.f, "fa_kv_append: nvfp4 pools need the positive tensor scale they were quantised with");
      break;
    default: return fail(FA_ERR_INVALID, "fa_kv_append: pool dtype must be f16, bf16, e4m3 or nvfp4");
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int sms = std::max(device_sm_count(), 1);
  const int g = grid_for((int64_t)B * H * T * 32, 256, sms);
#define FA_APP(TT) kv_append_kernel<TT><<<g, 256, 0, st>>>((const TT*)x, positions, block_table, B, H, T, d, page_size, n_logical, \
                                                      num_blocks, mode, tensor_scale, (uint8_t*)pool, scale_pool, micro_pool, status)
  if (x_dtype == FA_F32) FA_APP(float);
  else if (x_dtype == FA_F16) FA_APP(__half);
  else if (x_dtype == FA_BF16) FA_APP(__nv_bfloat16);
  else return fail(FA_ERR_INVALID, "fa_kv_append: x must be f32/f16/bf16");
#undef FA_APP
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_mla_expand_latent(const void* l_pool, int latent_dtype, const uint8_t* l_micro, const float* token_scale,
                                    float tensor_scale, const int32_t* block_table, int n_logical, int num_blocks, int page_size,
                                    const fa_decode_item* items, int n_items, int dqk, void* out_bf16, void* stream) {
  FA_CHECK_ARG(l_pool && out_bf16 && block_table && items, "fa_mla_expand_latent: null pointer");
  FA_CHECK_ARG(n_items >= 1 && n_logical >= 1 && num_blocks >= 1 && dqk >= 16 && dqk % 16 == 0, "fa_mla_expand_latent: bad sizes");
  FA_CHECK_ARG(page_size >= 1 && (page_size & (page_size - 1)) == 0, "fa_mla_expand_latent: page_size must be a power of two");
  FA_CHECK_ARG(latent_dtype == FA_E4M3 || latent_dtype == FA_NVFP4, "fa_mla_expand_latent: latent must be E4M3 or NVFP4");
  FA_CHECK_ARG(latent_dtype != FA_NVFP4 || l_micro != nullptr, "fa_mla_expand_latent: NVFP4 needs micro-scales");
  dim3 grid((unsigned)n_items, 8u, 1u);
  expand_latent_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(l_pool), l_micro, token_scale, tensor_scale, latent_dtype == FA_NVFP4 ? 1 : 0, block_table,
      n_logical, num_blocks, page_size, __builtin_ctz((unsigned)page_size), items, dqk, reinterpret_cast<__nv_bfloat16*>(out_bf16));
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}
