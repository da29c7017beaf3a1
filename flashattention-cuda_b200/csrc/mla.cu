// MLA latent-KV decode: MQA of h_q query heads over ONE shared latent per token.  Scores span the
// full latent width DQK (kv_lora_rank + rope), values are the first DV = kv_lora_rank dims of the same
// latent row, so every latent byte is read once and serves as both K and V.
//
// One CTA (8 warps) serves one (sequence, key range, 32 packed query rows).  64-key latent tiles are
// staged with 16-byte cp.async through a 2-stage ring; FP8 E4M3 and NVFP4 tiles are expanded once per
// tile into a 16-bit shared-memory tile (the reference expands to fp16 in shared memory as well,
// kernels/v11_mla/mla_attention.cu:170-183), bf16 tiles are used as they land.  Per tile:
//   phase 1  warp (m-tile, key group): S = Q L^T for 16 rows x 16 keys over DQK (mma.sync, Q fragments
//            from shared memory), row maxima exchanged through shared memory, P written to shared memory
//   phase 2  warp (m-tile, value quarter): O += P L[:, quarter] for 16 rows x DV/4 dims (registers)
// Splits of a sequence are merged by the last CTA to finish, as in the GQA decode kernel.
//
// Reference behaviour: kernels/v11_mla/mla_attention.cu:104-258 (row m -> head, i_q; mask key j when
// j > i_q + q_offset; output O_latent [B,h_q,N_q,DV] fp32) and :320-409 (argument checks).

#include <algorithm>
#include <climits>
#include <cstdlib>

#include "common.cuh"

namespace fa {
namespace {

constexpr int kMlaThreads = 256;
constexpr int kMlaTN = 64;        // keys per tile
constexpr int kMlaRows = 32;      // packed query rows per CTA
constexpr int kMlaMaxPages = 2048;
constexpr float kLog2eM = 1.4426950408889634f;
constexpr float kLn2M = 0.6931471805599453f;

enum MlaFmt { MLA_BF16 = 0, MLA_E4M3 = 1, MLA_NVFP4 = 2 };

struct MlaParams {
  const uint16_t* q;
  const uint8_t* pool;
  const uint8_t* micro;
  const float* tok_scale;
  const int32_t* block_table;
  const int32_t* q_offsets;
  const fa_decode_item* items;
  void* out;
  float* lse;
  float* part_o;
  float* part_lse;
  int32_t* counters;
  int32_t* status;
  float scale_l, softmax_scale;
  int n_logical, num_blocks, page_size, page_shift;
  int B, H_q, N_q, M;
  int causal, q_offset, out_dtype, bt_cap;
};

template <int DQK, int DV, int FMT>
struct MlaGeo {
  static constexpr int STRIDE = DQK * 2 + 16;                 // bytes per key row of the 16-bit tile (odd # of chunks)
  static constexpr int TILE16 = kMlaTN * STRIDE;
  static constexpr int RAW_ROW = FMT == MLA_E4M3 ? DQK : (FMT == MLA_NVFP4 ? DQK / 2 : 0);
  static constexpr int MICRO = FMT == MLA_NVFP4 ? DQK / 16 : 0;
  static constexpr int MICRO_STRIDE = (MICRO + 3) / 4 * 4;
  static constexpr int AUX = FMT == MLA_E4M3 ? kMlaTN * 4 : kMlaTN * MICRO_STRIDE;
  static constexpr int RAW_STAGE = (kMlaTN * RAW_ROW + AUX + 15) / 16 * 16;
  static constexpr int STAGE = FMT == MLA_BF16 ? TILE16 : RAW_STAGE;
  static constexpr int P_STRIDE = kMlaTN * 2 + 16;
  static constexpr int Q_BYTES = kMlaRows * STRIDE;
  static constexpr int SMEM = Q_BYTES + 2 * STAGE + (FMT == MLA_BF16 ? 0 : TILE16) + kMlaRows * P_STRIDE +
                              2 * 4 * kMlaRows * 4 /* s_max, s_l */;
};

template <int DQK, int DV, int FMT>
__global__ void __launch_bounds__(kMlaThreads, 1) mla_decode_kernel(const MlaParams p) {
  using G_ = MlaGeo<DQK, DV, FMT>;
  constexpr int STRIDE = G_::STRIDE;
  constexpr bool BF = (FMT == MLA_BF16);
  constexpr int NKS = DQK / 16;
  constexpr int DVQ = DV / 4;          // value dims per warp in phase 2
  constexpr int NOT = DVQ / 8;         // 8-wide output tiles per warp

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sStage = sQ + G_::Q_BYTES;
  uint8_t* sTile16 = sStage + 2 * G_::STAGE;                       // only used for the quantised formats
  uint8_t* sP = sTile16 + (BF ? 0 : G_::TILE16);
  float* s_max = reinterpret_cast<float*>(sP + kMlaRows * G_::P_STRIDE);   // [4 key groups][32 rows]
  float* s_l = s_max + 4 * kMlaRows;                                       // [4][32]
  int32_t* s_bt = reinterpret_cast<int32_t*>(s_l + 4 * kMlaRows);
  __shared__ int s_ticket;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g4 = lane >> 2, c = lane & 3;
  const int mt = warp & 1, kg = warp >> 1;

  const fa_decode_item it = p.items[blockIdx.x];
  const int b = it.b;
  const int qoff = p.q_offsets ? p.q_offsets[b] : p.q_offset;
  const int m0 = blockIdx.y * kMlaRows;
  const int rows_valid = min(kMlaRows, p.M - m0);

  // rows are m = i_q * H_q + head; the largest key row m may attend is i_q + q_offset
  int lim[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = mt * 16 + g4 + 8 * r;
    lim[r] = (p.causal && row < rows_valid) ? ((m0 + row) / p.H_q) + qoff : INT_MAX;
  }
  const int k_begin = it.k_begin;
  int k_end = it.k_end;
  int tile_min_lim = INT_MAX;
  if (p.causal) {
    k_end = min(k_end, max((m0 + rows_valid - 1) / p.H_q + qoff, -1) + 1);
    tile_min_lim = m0 / p.H_q + qoff;
  }
  const int n_keys = max(k_end - k_begin, 0);
  const int n_tiles = (n_keys + kMlaTN - 1) / kMlaTN;
  const int mask_lim = min(tile_min_lim, k_end - 1);
  lim[0] = min(lim[0], k_end - 1);
  lim[1] = min(lim[1], k_end - 1);

  // ---- block-table slice and the query rows ------------------------------------------------------
  const int pg0 = (p.page_shift >= 0) ? (k_begin >> p.page_shift) : (k_begin / p.page_size);
  if (n_keys > 0) {
    const int pg1 = (p.page_shift >= 0) ? ((k_end - 1) >> p.page_shift) : ((k_end - 1) / p.page_size);
    const int32_t* bt = p.block_table + (int64_t)b * p.n_logical;
    for (int i = tid; i <= pg1 - pg0 && i < p.bt_cap; i += kMlaThreads) {
      int pid = (pg0 + i < p.n_logical) ? bt[pg0 + i] : -2;
      if ((unsigned)pid >= (unsigned)p.num_blocks) {
        if (p.status) atomicOr(p.status, FA_STATUS_BAD_BLOCK_TABLE);
        pid = -1;
      }
      s_bt[i] = pid;
    }
  }
  {
    constexpr int CPR = DQK / 8;   // 16-byte chunks per query row
    for (int idx = tid; idx < kMlaRows * CPR; idx += kMlaThreads) {
      const int row = idx / CPR, ch = idx - row * CPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < rows_valid) {
        const int m = m0 + row;
        const int iq = m / p.H_q, h = m - iq * p.H_q;
        v = *reinterpret_cast<const uint4*>(p.q + (((int64_t)b * p.H_q + h) * p.N_q + iq) * DQK + ch * 8);
      }
      *reinterpret_cast<uint4*>(sQ + row * STRIDE + ch * 16) = v;
    }
  }
  __syncthreads();

  auto tok_row = [&](int key, bool& valid) -> int64_t {
    valid = key < k_end;
    if (!valid) return 0;
    const int pg = (p.page_shift >= 0) ? (key >> p.page_shift) : (key / p.page_size);
    const int pid = s_bt[pg - pg0];
    valid = pid >= 0;
    return valid ? (int64_t)pid * p.page_size + (key - pg * p.page_size) : 0;
  };

  // ---- producer -------------------------------------------------------------------------------------
  auto issue = [&](int stage, int kt) {
    uint8_t* dst = sStage + stage * G_::STAGE;
    if constexpr (FMT == MLA_BF16) {
      constexpr int CPR = DQK / 8;
      for (int idx = tid; idx < kMlaTN * CPR; idx += kMlaThreads) {
        const int r = idx / CPR, ch = idx - r * CPR;
        bool valid;
        const int64_t tr = tok_row(kt + r, valid);
        cp_async16(smem_u32(dst + r * STRIDE + ch * 16), p.pool + tr * (DQK * 2) + ch * 16, valid ? 16 : 0);
      }
    } else {
      constexpr int RAW = G_::RAW_ROW;
      constexpr int CPR = RAW / 16;
      for (int idx = tid; idx < kMlaTN * CPR; idx += kMlaThreads) {
        const int r = idx / CPR, ch = idx - r * CPR;
        bool valid;
        const int64_t tr = tok_row(kt + r, valid);
        cp_async16(smem_u32(dst + r * RAW + ch * 16), p.pool + tr * RAW + ch * 16, valid ? 16 : 0);
      }
      uint8_t* aux = dst + kMlaTN * RAW;
      if constexpr (FMT == MLA_E4M3) {
        if (p.tok_scale != nullptr && tid < kMlaTN) {
          bool valid;
          const int64_t tr = tok_row(kt + tid, valid);
          cp_async4(smem_u32(aux + tid * 4), p.tok_scale + tr, valid ? 4 : 0);
        }
      } else if constexpr (G_::MICRO % 4 == 0) {
        constexpr int WPR = G_::MICRO / 4;
        for (int idx = tid; idx < kMlaTN * WPR; idx += kMlaThreads) {
          const int r = idx / WPR, w = idx - r * WPR;
          bool valid;
          const int64_t tr = tok_row(kt + r, valid);
          cp_async4(smem_u32(aux + r * G_::MICRO_STRIDE + w * 4), p.micro + tr * G_::MICRO + w * 4, valid ? 4 : 0);
        }
      }
    }
  };

  // ---- expansion of a quantised tile into the 16-bit tile --------------------------------------------
  auto expand = [&](int stage, int kt) {
    if constexpr (FMT == MLA_E4M3) {
      const uint8_t* raw = sStage + stage * G_::STAGE;
      constexpr int CPR = DQK / 16;
      for (int idx = tid; idx < kMlaTN * CPR; idx += kMlaThreads) {
        const int r = idx / CPR, ch = idx - r * CPR;
        const uint4 w = *reinterpret_cast<const uint4*>(raw + r * DQK + ch * 16);
        uint4 lo, hi;
        lo.x = e4m3x2_to_h2(w.x); lo.y = e4m3x2_to_h2(w.x >> 16); lo.z = e4m3x2_to_h2(w.y); lo.w = e4m3x2_to_h2(w.y >> 16);
        hi.x = e4m3x2_to_h2(w.z); hi.y = e4m3x2_to_h2(w.z >> 16); hi.z = e4m3x2_to_h2(w.w); hi.w = e4m3x2_to_h2(w.w >> 16);
        uint4* d = reinterpret_cast<uint4*>(sTile16 + r * STRIDE + ch * 32);
        d[0] = lo;
        d[1] = hi;
      }
    } else if constexpr (FMT == MLA_NVFP4) {
      const uint8_t* raw = sStage + stage * G_::STAGE;
      const uint8_t* aux = raw + kMlaTN * G_::RAW_ROW;
      constexpr int CPR = DQK / 32;
      for (int idx = tid; idx < kMlaTN * CPR; idx += kMlaThreads) {
        const int r = idx / CPR, ch = idx - r * CPR;
        const uint4 w = *reinterpret_cast<const uint4*>(raw + r * G_::RAW_ROW + ch * 16);
        uint32_t m0b, m1b;
        if constexpr (G_::MICRO % 4 == 0) {
          m0b = aux[r * G_::MICRO_STRIDE + 2 * ch];
          m1b = aux[r * G_::MICRO_STRIDE + 2 * ch + 1];
        } else {   // narrow latents: micro-scale rows are not 4-byte aligned, read them straight from the pool
          bool valid;
          const int64_t tr = tok_row(kt + r, valid);
          m0b = valid ? p.micro[tr * G_::MICRO + 2 * ch] : 0;
          m1b = valid ? p.micro[tr * G_::MICRO + 2 * ch + 1] : 0;
        }
        const uint32_t mh0 = e4m3x2_to_h2(m0b | (m0b << 8)), mh1 = e4m3x2_to_h2(m1b | (m1b << 8));
        uint32_t h[4];
        uint4 o0, o1, o2, o3;
        e2m1x8_to_h2x4(w.x, h);
        o0 = make_uint4(hmul2_u32(h[0], mh0), hmul2_u32(h[1], mh0), hmul2_u32(h[2], mh0), hmul2_u32(h[3], mh0));
        e2m1x8_to_h2x4(w.y, h);
        o1 = make_uint4(hmul2_u32(h[0], mh0), hmul2_u32(h[1], mh0), hmul2_u32(h[2], mh0), hmul2_u32(h[3], mh0));
        e2m1x8_to_h2x4(w.z, h);
        o2 = make_uint4(hmul2_u32(h[0], mh1), hmul2_u32(h[1], mh1), hmul2_u32(h[2], mh1), hmul2_u32(h[3], mh1));
        e2m1x8_to_h2x4(w.w, h);
        o3 = make_uint4(hmul2_u32(h[0], mh1), hmul2_u32(h[1], mh1), hmul2_u32(h[2], mh1), hmul2_u32(h[3], mh1));
        uint4* d = reinterpret_cast<uint4*>(sTile16 + r * STRIDE + ch * 64);
        d[0] = o0; d[1] = o1; d[2] = o2; d[3] = o3;
      }
    }
  };

  // ---- running state ------------------------------------------------------------------------------
  float o[NOT][4];
#pragma unroll
  for (int t = 0; t < NOT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_part[2] = {0.f, 0.f};          // sums over this warp's key group only
  const float sc_log2 = p.softmax_scale * kLog2eM * p.scale_l;
  const bool tok_scales = (FMT == MLA_E4M3) && (p.tok_scale != nullptr);

  if (n_tiles > 0) issue(0, k_begin);
  cp_async_commit();

  for (int t = 0; t < n_tiles; ++t) {
    if (t + 1 < n_tiles) issue((t + 1) & 1, k_begin + (t + 1) * kMlaTN);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int kt = k_begin + t * kMlaTN;
    const uint8_t* tile;
    if constexpr (BF) {
      tile = sStage + (t & 1) * G_::STAGE;
    } else {
      expand(t & 1, kt);
      __syncthreads();
      tile = sTile16;
    }

    // ---------------- phase 1: S for (m-tile mt) x (16 keys of group kg) ---------------------------
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    {
      const int qrow = mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const uint32_t qbase = smem_u32(sQ + qrow * STRIDE) + ((lane >> 4) << 4);
      const int krow = kg * 16 + (lane & 7) + ((lane >> 4) << 3);
      const uint32_t kbase = smem_u32(tile + krow * STRIDE) + (((lane >> 3) & 1) << 4);
#pragma unroll 4
      for (int ks = 0; ks < NKS; ++ks) {
        uint32_t a[4], r[4];
        ldmatrix_x4(a, qbase + ks * 32);
        ldmatrix_x4(r, kbase + ks * 32);
        mma16816<BF>(s[0], a, r[0], r[1]);
        mma16816<BF>(s[1], a, r[2], r[3]);
      }
    }
    float vsc[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if constexpr (FMT == MLA_E4M3) {
      if (tok_scales) {
        const float* ts = reinterpret_cast<const float*>(sStage + (t & 1) * G_::STAGE + kMlaTN * G_::RAW_ROW);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float2 kk = *reinterpret_cast<const float2*>(ts + kg * 16 + 8 * n + 2 * c);
          s[n][0] *= kk.x; s[n][1] *= kk.y; s[n][2] *= kk.x; s[n][3] *= kk.y;
          vsc[n][0] = kk.x; vsc[n][1] = kk.y;
        }
      }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] *= sc_log2;
    if (kt + kMlaTN - 1 > mask_lim) {
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt + kg * 16 + 8 * n + 2 * c + (e & 1);
          if (key > lim[e >> 1]) s[n][e] = -INFINITY;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      if (c == 0) s_max[kg * kMlaRows + mt * 16 + g4 + 8 * r] = mx;
    }
    __syncthreads();
    float alpha[2];
    bool changed = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = mt * 16 + g4 + 8 * r;
      const float mx = fmaxf(fmaxf(s_max[row], s_max[kMlaRows + row]), fmaxf(s_max[2 * kMlaRows + row], s_max[3 * kMlaRows + row]));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_use);
      changed |= (m_new != m_run[r]);
      m_run[r] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        s[n][2 * r] = fast_exp2(s[n][2 * r] - m_use);
        s[n][2 * r + 1] = fast_exp2(s[n][2 * r + 1] - m_use);
        sum += s[n][2 * r] + s[n][2 * r + 1];
      }
      l_part[r] = l_part[r] * alpha[r] + sum;
      // P (times the per-token value scale) -> shared memory [row][key]
      uint8_t* prow = sP + row * G_::P_STRIDE + (kg * 16 + 2 * c) * 2;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = s[n][2 * r] * vsc[n][0], p1 = s[n][2 * r + 1] * vsc[n][1];
        *reinterpret_cast<uint32_t*>(prow + n * 16) = BF ? pack_bf2(p0, p1) : pack_h2(p0, p1);
      }
    }
    __syncthreads();

    // ---------------- phase 2: O[16 rows][quarter kg of DV] += P[16 x 64] L[64 x quarter] ---------------
    if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
      for (int tt = 0; tt < NOT; ++tt) {
        o[tt][0] *= alpha[0]; o[tt][1] *= alpha[0];
        o[tt][2] *= alpha[1]; o[tt][3] *= alpha[1];
      }
    }
    {
      const int prow = mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const uint32_t pbase = smem_u32(sP + prow * G_::P_STRIDE) + ((lane >> 4) << 4);
      const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
      const uint32_t vbase = smem_u32(tile + vrow * STRIDE) + kg * (DVQ * 2) + ((lane >> 4) << 4);
#pragma unroll
      for (int ks = 0; ks < kMlaTN / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, pbase + ks * 32);
#pragma unroll
        for (int jp = 0; jp < NOT / 2; ++jp) {
          uint32_t r[4];
          ldmatrix_x4_trans(r, vbase + ks * 16 * STRIDE + jp * 32);
          mma16816<BF>(o[2 * jp], a, r[0], r[1]);
          mma16816<BF>(o[2 * jp + 1], a, r[2], r[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- row sums across the four key groups ---------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 1);
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 2);
    if (c == 0) s_l[kg * kMlaRows + mt * 16 + g4 + 8 * r] = l_part[r];
  }
  __syncthreads();

  const bool single = (it.n_split == 1);
  const int slot = it.slot_base + it.split;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = mt * 16 + g4 + 8 * r;
    if (row >= rows_valid) continue;
    const float l = s_l[row] + s_l[kMlaRows + row] + s_l[2 * kMlaRows + row] + s_l[3 * kMlaRows + row];
    const float inv = (l > 0.f) ? p.scale_l / l : 0.f;
    const float m_use = (m_run[r] == -INFINITY) ? 0.f : m_run[r];
    const float lse = (l > 0.f) ? (m_use + log2f(l)) * kLn2M : -INFINITY;
    const int m = m0 + row;
    const int iq = m / p.H_q, h = m - iq * p.H_q;
    const int64_t hrow = (int64_t)h * p.N_q + iq;
    const int64_t orow = (int64_t)b * p.H_q * p.N_q + hrow;
    const int64_t prow = (int64_t)slot * p.H_q * p.N_q + hrow;
#pragma unroll
    for (int tt = 0; tt < NOT; ++tt) {
      const int dd = kg * DVQ + 8 * tt + 2 * c;
      const float v0 = o[tt][2 * r] * inv, v1 = o[tt][2 * r + 1] * inv;
      if (single) {
        store_out_dyn(p.out, p.out_dtype, orow * DV + dd, v0);
        store_out_dyn(p.out, p.out_dtype, orow * DV + dd + 1, v1);
      } else {
        *reinterpret_cast<float2*>(p.part_o + prow * DV + dd) = make_float2(v0, v1);
      }
    }
    if (kg == 0 && c == 0) {
      if (single) { if (p.lse) p.lse[orow] = lse; }
      else p.part_lse[prow] = lse;
    }
  }
  if (single) return;

  // ---- the last CTA of this (sequence, row tile) merges all key ranges --------------------------------
  __threadfence();
  __syncthreads();
  const int cidx = b * gridDim.y + blockIdx.y;
  if (tid == 0) s_ticket = atomicAdd(p.counters + cidx, 1);
  __syncthreads();
  if (s_ticket != it.n_split - 1) return;
  __threadfence();
  if (tid == 0) p.counters[cidx] = 0;
  const int64_t slot_stride = (int64_t)p.H_q * p.N_q;
  for (int idx = tid; idx < rows_valid * DV; idx += kMlaThreads) {
    const int row = idx / DV, dd = idx - row * DV;
    const int m = m0 + row;
    const int iq = m / p.H_q, h = m - iq * p.H_q;
    const int64_t hrow = (int64_t)h * p.N_q + iq;
    float mstar = -INFINITY;
    for (int sidx = 0; sidx < it.n_split; ++sidx)
      mstar = fmaxf(mstar, __ldcg(p.part_lse + (it.slot_base + sidx) * slot_stride + hrow));
    const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
    float acc = 0.f, l = 0.f;
    for (int sidx = 0; sidx < it.n_split; ++sidx) {
      const int64_t prow = (it.slot_base + sidx) * slot_stride + hrow;
      const float wgt = __expf(__ldcg(p.part_lse + prow) - m_use);
      acc += wgt * __ldcg(p.part_o + prow * DV + dd);
      l += wgt;
    }
    const int64_t orow = (int64_t)b * p.H_q * p.N_q + hrow;
    store_out_dyn(p.out, p.out_dtype, orow * DV + dd, (l > 0.f) ? acc / l : 0.f);
    if (p.lse && dd == 0) p.lse[orow] = (l > 0.f) ? m_use + __logf(l) : -INFINITY;
  }
}

template <int DQK, int DV, int FMT>
int launch_mla(const MlaParams& p, int n_items, int row_tiles, cudaStream_t st) {
  using G_ = MlaGeo<DQK, DV, FMT>;
  const int smem = G_::SMEM + p.bt_cap * 4;
  constexpr int SMEM_MAX = G_::SMEM + kMlaMaxPages * 4;
  static_assert(SMEM_MAX <= 227 * 1024, "MLA tile does not fit shared memory");
  auto kern = mla_decode_kernel<DQK, DV, FMT>;
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX));
    configured_device = dev;
  }
  dim3 grid((unsigned)n_items, (unsigned)row_tiles);
  kern<<<grid, kMlaThreads, smem, st>>>(p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace
}  // namespace fa

namespace fa {
// CTA-pair tensor-core path (mla_pair.cu, mla_pair_f8.cu)
bool mla_pair_applicable(const fa_mla_args* a);
int mla_pair_max_pages();
size_t mla_pair_workspace_bytes(int n_slots, int M);
size_t mla_pair_counters_len(int B, int M);
int launch_mla_pair(const fa_mla_args* a, cudaStream_t st);
}  // namespace fa

using namespace fa;

extern "C" size_t fa_mla_counters_len(int B, int H_q, int N_q) {
  const int row_tiles = (H_q * N_q + kMlaRows - 1) / kMlaRows;
  return std::max((size_t)B * row_tiles + 1, mla_pair_counters_len(B, H_q * N_q));
}

extern "C" size_t fa_mla_workspace_bytes(int n_slots, int H_q, int N_q, int DV) {
  return std::max((size_t)n_slots * H_q * N_q * (DV + 1) * 4, mla_pair_workspace_bytes(n_slots, H_q * N_q));
}

// Largest key range (in keys, a multiple of 128) one CTA pair of the tensor-core kernel can take at this page size.
extern "C" int fa_mla_pair_max_range(int page_size) {
  const long long keys = (long long)(mla_pair_max_pages() - 2) * page_size / 128 * 128;
  return (int)std::min<long long>(keys, 1 << 30);
}

extern "C" int fa_mla_decode_fwd(const fa_mla_args* a) {
  FA_CHECK_ARG(a != nullptr, "fa_mla_decode_fwd: null args");
  FA_CHECK_ARG(a->q && a->l_pool && a->block_table && a->items && a->out,
               "fa_mla_decode_fwd: q, l_pool, block_table, items, out must be non-null");
  FA_CHECK_ARG(a->B >= 1 && a->H_q >= 1 && a->N_q >= 1, "fa_mla_decode_fwd: bad B/H_q/N_q");
  FA_CHECK_ARG(a->DQK % 16 == 0, "DQK (latent width) must be a multiple of the NVFP4 block (16); got %d", a->DQK);
  FA_CHECK_ARG(a->DV >= 1 && a->DV <= a->DQK && a->DV % 32 == 0,
               "kv_lora_rank (DV) must be in [1,DQK], a multiple of 32; got %d DQK=%d", a->DV, a->DQK);
  FA_CHECK_ARG(a->page_size >= 1 && a->n_logical >= 1 && a->num_blocks >= 1, "bad page_size / n_logical / num_blocks");
  FA_CHECK_ARG(a->n_items >= 1, "empty plan");
  FA_CHECK_ARG(a->out_dtype == FA_F32 || a->out_dtype == FA_F16 || a->out_dtype == FA_BF16, "out_dtype must be f32/f16/bf16");
  int fmt;
  switch (a->latent_dtype) {
    case FA_BF16: fmt = MLA_BF16; FA_CHECK_ARG(a->q_dtype == FA_BF16, "a bf16 latent needs bf16 q"); break;
    case FA_E4M3: fmt = MLA_E4M3; FA_CHECK_ARG(a->q_dtype == FA_F16, "an e4m3 latent needs f16 q"); break;
    case FA_NVFP4:
      fmt = MLA_NVFP4;
      FA_CHECK_ARG(a->q_dtype == FA_F16, "an nvfp4 latent needs f16 q");
      FA_CHECK_ARG(a->l_micro != nullptr, "an nvfp4 latent needs the micro-scale pool");
      break;
    default: return fail(FA_ERR_INVALID, "latent dtype must be bf16, e4m3 or nvfp4 (got %d)", a->latent_dtype);
  }
  FA_CHECK_ARG(a->l_token_scale == nullptr || fmt == MLA_E4M3, "per-token scales are only defined for an e4m3 latent");
  const int M = a->H_q * a->N_q;
  const int row_tiles = (M + kMlaRows - 1) / kMlaRows;
  FA_CHECK_ARG(row_tiles <= 65535, "too many query rows (%d)", M);
  FA_CHECK_ARG(a->n_slots == 0 || a->n_slots == a->n_items, "n_slots must be 0 (no sequence is split) or n_items");
  const size_t need = (size_t)a->n_slots * a->H_q * a->N_q * (a->DV + 1) * 4;
  FA_CHECK_ARG(need == 0 || a->workspace != nullptr, "workspace must be non-null when a sequence is split");
  if (a->workspace_bytes < need) return fail(FA_ERR_WORKSPACE, "workspace %zu B < %zu B", a->workspace_bytes, need);
  const size_t n_counters = fa_mla_counters_len(a->B, a->H_q, a->N_q);
  FA_CHECK_ARG(a->counters != nullptr, "counters must be non-null");
  if (a->counters_len < n_counters) return fail(FA_ERR_WORKSPACE, "counters hold %zu ints < %zu", a->counters_len, n_counters);

  // bf16 and E4M3 (576, 512) latents on power-of-two pages >= 64 run on the CTA-pair tcgen05 kernels unless the
  // caller asks for the fused mma.sync kernel (engine_hint 2) or a key range is too long for them
  if (a->engine_hint != 2 && mla_pair_applicable(a)) {
    if (a->workspace_bytes < mla_pair_workspace_bytes(a->n_slots, M))
      return fail(FA_ERR_WORKSPACE, "workspace %zu B < %zu B", a->workspace_bytes, mla_pair_workspace_bytes(a->n_slots, M));
    return launch_mla_pair(a, reinterpret_cast<cudaStream_t>(a->stream));
  }

  MlaParams p{};
  p.q = reinterpret_cast<const uint16_t*>(a->q);
  p.pool = reinterpret_cast<const uint8_t*>(a->l_pool);
  p.micro = reinterpret_cast<const uint8_t*>(a->l_micro);
  p.tok_scale = a->l_token_scale;
  p.block_table = a->block_table;
  p.q_offsets = a->q_offsets;
  p.items = a->items;
  p.out = a->out;
  p.lse = a->lse;
  p.part_o = reinterpret_cast<float*>(a->workspace);
  p.part_lse = p.part_o + (size_t)a->n_slots * a->H_q * a->N_q * a->DV;
  p.status = a->counters;          // word 0: sticky error flags; the arrival counters follow
  p.counters = a->counters + 1;
  p.scale_l = a->l_scale;
  p.softmax_scale = a->softmax_scale;
  p.n_logical = a->n_logical;
  p.num_blocks = a->num_blocks;
  p.page_size = a->page_size;
  p.page_shift = ((a->page_size & (a->page_size - 1)) == 0) ? __builtin_ctz((unsigned)a->page_size) : -1;
  p.B = a->B; p.H_q = a->H_q; p.N_q = a->N_q; p.M = M;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  p.bt_cap = a->max_range_keys / a->page_size + 2;
  if (p.bt_cap > kMlaMaxPages) return fail(FA_ERR_INVALID, "key range of %d keys spans more than %d pages", a->max_range_keys, kMlaMaxPages);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);

#define FA_MLA(DQK_, DV_)                                                                  \
  if (a->DQK == DQK_ && a->DV == DV_) {                                                    \
    if (fmt == MLA_BF16) return launch_mla<DQK_, DV_, MLA_BF16>(p, a->n_items, row_tiles, st); \
    if (fmt == MLA_E4M3) return launch_mla<DQK_, DV_, MLA_E4M3>(p, a->n_items, row_tiles, st); \
    return launch_mla<DQK_, DV_, MLA_NVFP4>(p, a->n_items, row_tiles, st);                 \
  }
  FA_MLA(576, 512)
  FA_MLA(160, 128)
  FA_MLA(96, 64)
#undef FA_MLA
  return fail(FA_ERR_UNSUPPORTED, "mla: unsupported (DQK,DV)=(%d,%d); supported: (96,64) (160,128) (576,512)", a->DQK, a->DV);
}
