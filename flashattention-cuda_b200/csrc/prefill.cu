// Dense (causal) attention forward on tcgen05 tensor cores with TMEM accumulators, fed by TMA.
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value tiles of 128 keys.
// Warp roles (6 warps):
//   warp 0      TMA producer: Q once, then K/V tiles into a 2-stage ring (3-D tensor maps over
//               [B*H, N, d], 128-byte swizzle, out-of-range rows zero filled)
//   warp 1      allocates TMEM, issues every tcgen05.mma (one elected lane):
//               S_j = Q K_j^T (K-major operands from shared memory) into one of two S buffers in TMEM,
//               O  += P_j V_j  (P from shared memory, V as an MN-major operand) into the O columns
//   warps 2..5  softmax: thread r owns query row r — reads its S row from TMEM (tcgen05.ld), scales,
//               masks, keeps the running max / sum, rescales its O row in TMEM when the max moved,
//               writes P (fp16 / bf16) into swizzled shared memory for the second MMA, and at the end
//               normalises and stores its O row
// TMEM columns: O [0,128)  S0 [128,256)  S1 [256,384).
// Behaviour follows the reference's dense entry point (fa_kernels/__init__.py:26-42 ->
// kernels/v5_wmma/wmma_attention.cu:229-263): inputs in half precision, fp32 accumulation, optional
// top-left causal mask (key j masked when j > i, wmma_attention.cu:159), default output fp32.

#include <cstdlib>

#include "sm100.cuh"

namespace fa {
namespace {

using namespace sm100;

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 128;          // keys per tile
constexpr int kStages = 2;
constexpr int kPrefillThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2eF = 1.4426950408889634f;

struct PrefillParams {
  void* out;
  float* lse;
  int* status;
  int B, H, N_q, N_k;
  int causal, out_dtype;
  float scale_log2;
};

enum PrefillErr { ERR_Q = 11, ERR_KV_FULL = 12, ERR_KV_EMPTY = 13, ERR_S_FULL = 14, ERR_S_EMPTY = 15, ERR_P_FULL = 16,
                  ERR_PV_DONE = 17 };

template <int D, bool BF16>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
  constexpr int KB = D / 64;                     // 64-element (128-byte) blocks along d
  constexpr int TILE_BYTES = 128 * D * 2;        // one 128-row tile of Q, K or V
  constexpr int BLK_BYTES = 128 * 128;           // one [128 rows][64 elements] block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;                 // [stage]
  uint8_t* sV = sK + kStages * TILE_BYTES;       // [stage]
  uint8_t* sP = sV + kStages * TILE_BYTES;       // [2 key blocks][128 rows][64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * BLK_BYTES);
  // barrier indices
  enum { Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 3, S_FULL = 5, S_EMPTY = 7, P_FULL = 9, PV_DONE = 10, NBARS = 11 };
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.N_q + kBM - 1) / kBM;
  const int qt = n_qt - 1 - (int)blockIdx.x;     // heaviest (last) causal tiles first
  const int bh = blockIdx.y;
  const int q0 = qt * kBM;
  int n_tiles = (p.N_k + kBN - 1) / kBN;
  if (p.causal) n_tiles = min(n_tiles, (q0 + kBM - 1) / kBN + 1);

  if (threadIdx.x == 0) {
    *s_abort = 0;
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(KV_FULL + s), 1);
      mbar_init(bar(KV_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(S_EMPTY + s), 128);
    }
    mbar_init(bar(P_FULL), 128);
    mbar_init(bar(PV_DONE), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tm_o = tmem, tm_s0 = tmem + 128;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
      for (int kb = 0; kb < KB; ++kb) tma_load_3d(smem_u32(sQ + kb * BLK_BYTES), &tm_q, kb * 64, q0, bh, bar(Q_FULL));
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        if (j >= kStages && !mbar_wait(bar(KV_EMPTY + s), ((j / kStages) - 1) & 1, s_abort, p.status, ERR_KV_EMPTY)) break;
        mbar_expect_tx(bar(KV_FULL + s), 2 * TILE_BYTES);
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_3d(smem_u32(sK + s * TILE_BYTES + kb * BLK_BYTES), &tm_k, kb * 64, j * kBN, bh, bar(KV_FULL + s));
          tma_load_3d(smem_u32(sV + s * TILE_BYTES + kb * BLK_BYTES), &tm_v, kb * 64, j * kBN, bh, bar(KV_FULL + s));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_f16(kBM, kBN, BF16, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(kBM, D, BF16, false, true);
      auto issue_qk = [&](int j) {
        const int s = j % kStages;
        const uint32_t d_tmem = tm_s0 + (uint32_t)(j & 1) * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * BLK_BYTES + (k & 3) * 32;
          mma_f16_ss(d_tmem, smem_desc_sw128(smem_u32(sQ) + off, 16, 1024),
                     smem_desc_sw128(smem_u32(sK + s * TILE_BYTES) + off, 16, 1024), idesc_qk, k > 0);
        }
        mma_commit(bar(S_FULL + (j & 1)));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, s_abort, p.status, ERR_Q) &&
                mbar_wait(bar(KV_FULL + 0), 0, s_abort, p.status, ERR_KV_FULL);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) {
          const int s = (j + 1) % kStages;
          ok = mbar_wait(bar(KV_FULL + s), ((j + 1) / kStages) & 1, s_abort, p.status, ERR_KV_FULL);
          if (ok && j + 1 >= 2) ok = mbar_wait(bar(S_EMPTY + ((j + 1) & 1)), (((j + 1) >> 1) - 1) & 1, s_abort, p.status, ERR_S_EMPTY);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        ok = mbar_wait(bar(P_FULL), j & 1, s_abort, p.status, ERR_P_FULL);
        if (!ok) break;
        tc_fence_after();
        const int s = j % kStages;
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          // A = P [128 rows][128 keys], K-major: key block k/4, 32 bytes per 16 keys inside the atom
          const uint64_t a_desc = smem_desc_sw128(smem_u32(sP) + (k >> 2) * BLK_BYTES + (k & 3) * 32, 16, 1024);
          // B = V [128 keys][D], MN-major: 16 keys = 2 atoms of 8 rows; d blocks of 64 are BLK_BYTES apart
          const uint64_t b_desc = smem_desc_sw128(smem_u32(sV + s * TILE_BYTES) + k * 2048, BLK_BYTES, 1024);
          mma_f16_ss(tm_o, a_desc, b_desc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(bar(PV_DONE));
        mma_commit(bar(KV_EMPTY + s));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;                // query row inside the tile
    const int gi = q0 + row;                         // query index
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, s_abort, p.status, ERR_S_FULL);
      if (!ok) break;
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tm_s0 + (uint32_t)(j & 1) * 128 + lane_base + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(S_EMPTY + (j & 1)));

      const int k0 = j * kBN;
      const bool need_mask = (k0 + kBN > p.N_k) || (p.causal && k0 + kBN - 1 > q0);
      float mx = -INFINITY;
      if (need_mask) {
        const int limit = p.causal ? min(gi, p.N_k - 1) : p.N_k - 1;   // largest key this row may see
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          s[c] = (k0 + c <= limit) ? s[c] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          s[c] *= p.scale_log2;
          mx = fmaxf(mx, s[c]);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m_run - m_use);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        s[c] = fast_exp2(s[c] - m_use);
        sum += s[c];
      }
      l_run = l_run * alpha + sum;
      const bool moved = (m_new != m_run);
      m_run = m_new;

      if (j > 0) {
        ok = mbar_wait(bar(PV_DONE), (j - 1) & 1, s_abort, p.status, ERR_PV_DONE);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            float o[32];
            tmem_ld32(tm_o + lane_base + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(tm_o + lane_base + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // P row -> shared memory, K-major, 128-byte swizzle: chunk of 8 keys = 16 bytes
      {
        uint8_t* prow = sP + row * 128;
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          uint4 v;
          if constexpr (BF16) {
            v.x = pack_bf2(s[ch * 8 + 0], s[ch * 8 + 1]); v.y = pack_bf2(s[ch * 8 + 2], s[ch * 8 + 3]);
            v.z = pack_bf2(s[ch * 8 + 4], s[ch * 8 + 5]); v.w = pack_bf2(s[ch * 8 + 6], s[ch * 8 + 7]);
          } else {
            v.x = pack_h2(s[ch * 8 + 0], s[ch * 8 + 1]); v.y = pack_h2(s[ch * 8 + 2], s[ch * 8 + 3]);
            v.z = pack_h2(s[ch * 8 + 4], s[ch * 8 + 5]); v.w = pack_h2(s[ch * 8 + 6], s[ch * 8 + 7]);
          }
          const int kb = ch >> 3, cc = ch & 7;
          *reinterpret_cast<uint4*>(prow + kb * BLK_BYTES + ((cc ^ (row & 7)) << 4)) = v;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar(P_FULL));
    }
    // epilogue: wait for the last P V, normalise, store
    if (ok) ok = mbar_wait(bar(PV_DONE), (n_tiles - 1) & 1, s_abort, p.status, ERR_PV_DONE);
    if (ok) {
      tc_fence_after();
      const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
      const bool valid = gi < p.N_q;
      const int64_t orow = (int64_t)bh * p.N_q + gi;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld32(tm_o + lane_base + c * 32, o);
        tmem_wait_ld();
        if (valid) {
          if (p.out_dtype == FA_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + orow * D + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
          } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + orow * D + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              if (p.out_dtype == FA_BF16) {
                v.x = pack_bf2(o[8 * i] * inv, o[8 * i + 1] * inv); v.y = pack_bf2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
                v.z = pack_bf2(o[8 * i + 4] * inv, o[8 * i + 5] * inv); v.w = pack_bf2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
              } else {
                v.x = pack_h2(o[8 * i] * inv, o[8 * i + 1] * inv); v.y = pack_h2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
                v.z = pack_h2(o[8 * i + 4] * inv, o[8 * i + 5] * inv); v.w = pack_h2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
              }
              dst[i] = v;
            }
          }
        }
      }
      if (valid && p.lse) p.lse[orow] = (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }

  // ---- teardown: all roles meet, TMEM is released by the warp that allocated it --------------------
  tc_fence_before();
  __syncthreads();
  if (*s_abort) __nanosleep(200000);   // after a timed-out wait: give copies still in flight time to land
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, bool BF16>
int launch_prefill(const fa_dense_args* a, const PrefillParams& p, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  const int dt = BF16 ? FA_BF16 : FA_F16;
  const uint64_t BH = (uint64_t)a->B * a->H;
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->N_q, BH};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->N_q * D * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = encode_tensor_map(&tq, dt, 3, const_cast<void*>(a->q), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->N_k, BH};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->N_k * D * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = encode_tensor_map(&tk, dt, 3, const_cast<void*>(a->k), dims, strides, box, 1);
    if (rc) return rc;
    rc = encode_tensor_map(&tv, dt, 3, const_cast<void*>(a->v), dims, strides, box, 1);
    if (rc) return rc;
  }
  constexpr int TILE = 128 * D * 2;
  constexpr int SMEM = TILE * (1 + 2 * kStages) + 2 * 128 * 128 + 256 + 1024;
  auto kern = prefill_kernel<D, BF16>;
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured_device = dev;
  }
  dim3 grid((unsigned)((a->N_q + kBM - 1) / kBM), (unsigned)BH);
  kern<<<grid, kPrefillThreads, SMEM, st>>>(tq, tk, tv, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace
}  // namespace fa

namespace fa {
int launch_prefill2(const fa_dense_args* a, float scale_log2, cudaStream_t st);   // prefill2.cu
}

using namespace fa;

extern "C" int fa_dense_fwd(const fa_dense_args* a) {
  FA_CHECK_ARG(a != nullptr, "fa_dense_fwd: null args");
  FA_CHECK_ARG(a->q && a->k && a->v && a->out, "fa_dense_fwd: q, k, v, out must be non-null");
  FA_CHECK_ARG(a->B >= 1 && a->H >= 1 && a->N_q >= 1 && a->N_k >= 1, "fa_dense_fwd: bad B/H/N");
  FA_CHECK_ARG((int64_t)a->B * a->H <= 65535, "B*H must be <= 65535 (grid.y); got %lld", (long long)a->B * a->H);
  FA_CHECK_ARG(a->dtype == FA_F16 || a->dtype == FA_BF16, "fa_dense_fwd: q/k/v must be f16 or bf16");
  FA_CHECK_ARG(a->out_dtype == FA_F32 || a->out_dtype == FA_F16 || a->out_dtype == FA_BF16, "out_dtype must be f32/f16/bf16");
  FA_CHECK_ARG((((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15) == 0,
               "fa_dense_fwd: q, k, v, out must be 16-byte aligned");
  if (a->D != 64 && a->D != 128) return fail(FA_ERR_UNSUPPORTED, "dense attention supports head_dim 64 or 128 (got %d)", a->D);
  PrefillParams p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = a->status;
  p.B = a->B; p.H = a->H; p.N_q = a->N_q; p.N_k = a->N_k;
  p.causal = a->causal; p.out_dtype = a->out_dtype;
  p.scale_log2 = a->softmax_scale * kLog2eF;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  // Two generations of the kernel exist; the second (two query tiles per CTA, P through tensor memory)
  // is the default, FA_B200_PREFILL_GEN=1 selects the first.
  static const int gen = [] { const char* e = getenv("FA_B200_PREFILL_GEN"); return (e && e[0] == '1') ? 1 : 2; }();
  if (gen == 2) return launch_prefill2(a, p.scale_log2, st);
  if (a->D == 128) return a->dtype == FA_BF16 ? launch_prefill<128, true>(a, p, st) : launch_prefill<128, false>(a, p, st);
  return a->dtype == FA_BF16 ? launch_prefill<64, true>(a, p, st) : launch_prefill<64, false>(a, p, st);
}
