// Paged GQA split-KV decode for sm_100a.
//
// One CTA (4 warps) serves one (sequence, KV head, key range, 16-row tile of packed query rows).
// The G query heads that share a KV head are packed into the M dimension of the score product
// (row m = i_q * G + g), so the KV bytes of a head are read once for the whole group.  Keys stream
// through a multi-stage cp.async pipeline of 64-key tiles (16-byte coalesced loads of the page rows,
// XOR-swizzled in shared memory so ldmatrix is conflict free); each warp owns 16 keys of a tile,
// keeps its scores in registers (mma.sync m16n8k16, fp32 accumulate), runs an online softmax per
// tile and accumulates P.V in registers.  FP8 E4M3 and NVFP4 pages are dequantised in registers
// after ldmatrix (cvt.rn.f16x2.e4m3x2 / cvt.rn.f16x2.e2m1x2); the head-dim order of the contraction
// is permuted per format so that no byte shuffling is needed on the K side.  The per-warp results
// are combined in shared memory; the last CTA to finish a (sequence, head, row tile) merges the
// partial results of all key ranges (arrival counter), so there is no second launch.
//
// Reference behaviour reproduced: kernels/v8_gqa_ss/gqa_ss_attention.cu:66-231 (M-packing
// h_q = h_kv*G + g, block-table gather, q_offset causal mask, split + LSE merge),
// kernels/v9_fp8/fp8_attention.cu:46-48,132-144 (E4M3 dequant x per-tensor scale),
// kernels/v10_nvfp4/nvfp4_attention.cu:52-60,158-174 (E2M1 nibble x E4M3 micro-scale x tensor scale).

#include <algorithm>
#include <climits>
#include <vector>

#include "common.cuh"

namespace fa {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTN = 16 * kWarps;     // keys per pipeline stage
constexpr int kRowTile = 16;         // packed query rows per CTA
constexpr int kMaxPages = 2048;      // block-table entries staged in shared memory per CTA
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

enum KvFmt { KV_F16 = 0, KV_BF16 = 1, KV_E4M3 = 2, KV_NVFP4 = 3 };

struct DecodeParams {
  const uint16_t* q;
  const uint8_t* k_pool;
  const uint8_t* v_pool;
  const uint8_t* k_micro;
  const uint8_t* v_micro;
  const float* k_tok;
  const float* v_tok;
  const int32_t* block_table;
  const int32_t* q_offsets;
  const fa_decode_item* items;
  void* out;
  float* lse;
  float* part_o;
  float* part_lse;
  int32_t* counters;
  int32_t* status;
  float k_scale, v_scale, softmax_scale;
  int n_logical, num_blocks, page_size, page_shift;
  int B, H_q, H_kv, N_q, G, M;
  int causal, q_offset, out_dtype, bt_cap;
  int n_items, head_major;
};

template <int D, int FMT>
struct Geo {
  static constexpr int KROW = (FMT == KV_NVFP4) ? D / 2 : (FMT == KV_E4M3 ? D : D * 2);  // bytes per key row
  static constexpr int CPR = KROW / 16;                                                   // 16B chunks per row
  static constexpr int MR = (FMT == KV_NVFP4) ? D / 16 : 0;                               // micro bytes per key
  static constexpr int AUX = (FMT == KV_NVFP4) ? 2 * kTN * MR : (FMT == KV_E4M3 ? 2 * kTN * 4 : 0);
  static constexpr int TILE = kTN * KROW;
  static constexpr int STAGE = 2 * TILE + AUX;
  static constexpr int MERGE = kWarps * kRowTile * (D + 2) * 4;
};

template <int KROW>
__device__ __forceinline__ int swz(int row, int chunk) {
  if constexpr (KROW >= 128) return chunk ^ (row & 7);
  else if constexpr (KROW == 64) return chunk ^ ((row >> 1) & 3);
  else return chunk ^ ((row >> 2) & 1);
}

// head-dim index of accumulator column e (0/1) of output tile t for lane-in-quad c
template <int FMT>
__device__ __forceinline__ int out_dim(int t, int c, int e) {
  if constexpr (FMT == KV_E4M3) return 16 * (t >> 1) + 4 * c + 2 * e + (t & 1);
  else if constexpr (FMT == KV_NVFP4) return 32 * (t >> 2) + 8 * c + 4 * e + (t & 3);
  else return 8 * t + 2 * c + e;
}
// head-dim index of the first element of the A-fragment pair `sel` (0: a0/a1, 1: a2/a3) of k-step ks
template <int FMT>
__device__ __forceinline__ int q_dim(int ks, int c, int sel) {
  if constexpr (FMT == KV_E4M3) return 16 * ks + 4 * c + 2 * sel;
  else if constexpr (FMT == KV_NVFP4) return 32 * (ks >> 1) + 8 * c + 4 * (ks & 1) + 2 * sel;
  else return 16 * ks + 2 * c + 8 * sel;
}

template <int D, int FMT, int NSTAGE, int MINB, bool R8>
__global__ void __launch_bounds__(kThreads, MINB) paged_decode_kernel(const DecodeParams p) {
  // R8: at most 8 packed query rows (decode with G <= 8): rows 8..15 of the 16-row MMA tile are padding,
  // their A-fragment registers are constant zero and their accumulators are never kept, which halves
  // the register footprint of S and O.
  constexpr int NR = R8 ? 1 : 2;
  using G_ = Geo<D, FMT>;
  constexpr int KROW = G_::KROW;
  constexpr int CPR = G_::CPR;
  constexpr int TILE = G_::TILE;
  constexpr int STAGE = G_::STAGE;
  constexpr int MR = G_::MR;
  constexpr bool BF = (FMT == KV_BF16);
  constexpr int NKS = D / 16;   // k-steps of the score product
  constexpr int NOT = D / 8;    // 8-wide output tiles

  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int PIPE_BYTES = (NSTAGE * STAGE > G_::MERGE) ? NSTAGE * STAGE : G_::MERGE;
  int32_t* s_bt = reinterpret_cast<int32_t*>(smem + PIPE_BYTES);
  __shared__ int s_ticket;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g4 = lane >> 2, c = lane & 3;

  // consecutive CTAs serve the KV heads of one key range, so that the 8 x 256-byte head rows of a
  // token (one contiguous 2 KB line of the pool) are fetched by CTAs that run at the same time
  const int item_idx = p.head_major ? (int)(blockIdx.x % p.n_items) : (int)(blockIdx.x / p.H_kv);
  const int h_kv = p.head_major ? (int)(blockIdx.x / p.n_items) : (int)(blockIdx.x - item_idx * p.H_kv);
  const int m0 = blockIdx.y * kRowTile;
  const fa_decode_item it = p.items[item_idx];
  const int b = it.b;
  const int qoff = p.q_offsets ? p.q_offsets[b] : p.q_offset;

  // ---- per-row limits (largest key index a row may attend) -------------------------------------
  const int rows_valid = min(kRowTile, p.M - m0);
  int lim[2] = {INT_MAX, INT_MAX};
  int tile_max_lim = p.causal ? INT_MIN : INT_MAX, tile_min_lim = INT_MAX;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int row = g4 + 8 * r;
    lim[r] = INT_MAX;
    if (p.causal && row < rows_valid) {
      lim[r] = ((m0 + row) / p.G) + qoff;
      tile_max_lim = max(tile_max_lim, lim[r]);
      tile_min_lim = min(tile_min_lim, lim[r]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    tile_max_lim = max(tile_max_lim, __shfl_xor_sync(0xffffffffu, tile_max_lim, o));
    tile_min_lim = min(tile_min_lim, __shfl_xor_sync(0xffffffffu, tile_min_lim, o));
  }
  const int k_begin = it.k_begin;
  int k_end = it.k_end;
  if (p.causal) k_end = min(k_end, max(tile_max_lim, -1) + 1);
  const int n_keys = max(k_end - k_begin, 0);
  const int n_tiles = (n_keys + kTN - 1) / kTN;
  const int mask_lim = min(tile_min_lim, k_end - 1);   // tiles reaching past this need masking
  lim[0] = min(lim[0], k_end - 1);
  lim[1] = min(lim[1], k_end - 1);

  // ---- stage the block-table slice of this key range -------------------------------------------
  const int pg0 = (p.page_shift >= 0) ? (k_begin >> p.page_shift) : (k_begin / p.page_size);
  if (n_keys > 0) {
    const int pg1 = (p.page_shift >= 0) ? ((k_end - 1) >> p.page_shift) : ((k_end - 1) / p.page_size);
    const int32_t* bt = p.block_table + (int64_t)b * p.n_logical;
    for (int i = tid; i <= pg1 - pg0 && i < p.bt_cap; i += kThreads) {
      int pid = (pg0 + i < p.n_logical) ? bt[pg0 + i] : -2;
      if ((unsigned)pid >= (unsigned)p.num_blocks) {   // never follow a bad table entry
        if (p.status) atomicOr(p.status, FA_STATUS_BAD_BLOCK_TABLE);
        pid = -1;
      }
      s_bt[i] = pid;
    }
  }

  // ---- query fragments (registers, whole kernel) -----------------------------------------------
  uint32_t qf[NKS][4] = {};
  {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int row = g4 + 8 * r;
      const int m = m0 + row;
      const bool ok = row < rows_valid;
      const int iq = ok ? m / p.G : 0;
      const int g = ok ? m - iq * p.G : 0;
      const uint16_t* qrow = p.q + (((int64_t)b * p.H_q + (h_kv * p.G + g)) * p.N_q + iq) * D;
#pragma unroll
      for (int ks = 0; ks < NKS; ++ks) {
#pragma unroll
        for (int sel = 0; sel < 2; ++sel) {
          uint32_t v = 0;
          if (ok) v = *reinterpret_cast<const uint32_t*>(qrow + q_dim<FMT>(ks, c, sel));
          qf[ks][r + 2 * sel] = v;
        }
      }
    }
  }
  __syncthreads();

  // ---- producer: one 64-key tile of K and V (+ scales) into a stage ----------------------------
  const int64_t row_stride_tok = (int64_t)p.H_kv;   // token rows are [page][tok][H_kv]
  auto issue = [&](int stage, int kt) {
    uint8_t* sk = smem + stage * STAGE;
    uint8_t* sv = sk + TILE;
    constexpr int RPP = kThreads / CPR;
    constexpr int PASSES = (kTN + RPP - 1) / RPP;
    const int chunk = tid % CPR;
    const int r0 = tid / CPR;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const int r = r0 + i * RPP;
      if (RPP > kTN && r >= kTN) break;
      const int key = kt + r;
      bool valid = key < k_end;
      int64_t tokrow = 0;
      if (valid) {
        const int pg = (p.page_shift >= 0) ? (key >> p.page_shift) : (key / p.page_size);
        const int pid = s_bt[pg - pg0];
        const int off = key - pg * p.page_size;
        valid = pid >= 0;
        tokrow = ((int64_t)pid * p.page_size + off) * row_stride_tok + h_kv;
      }
      if (!valid) tokrow = 0;
      const int sw = swz<KROW>(r, chunk) * 16;
      cp_async16(smem_u32(sk + r * KROW + sw), p.k_pool + tokrow * KROW + chunk * 16, valid ? 16 : 0);
      cp_async16(smem_u32(sv + r * KROW + sw), p.v_pool + tokrow * KROW + chunk * 16, valid ? 16 : 0);
    }
    if constexpr (FMT == KV_NVFP4 || FMT == KV_E4M3) {
      if (FMT == KV_NVFP4 || p.k_tok != nullptr) {
        // threads 0..63: K-side scale of key tid; threads 64..127: V-side scale of key tid-64
        const int r = tid & (kTN - 1);
        const bool is_v = tid >= kTN;
        const int key = kt + r;
        bool valid = key < k_end;
        int64_t tokrow = 0;
        if (valid) {
          const int pg = (p.page_shift >= 0) ? (key >> p.page_shift) : (key / p.page_size);
          const int pid = s_bt[pg - pg0];
          const int off = key - pg * p.page_size;
          valid = pid >= 0;
          tokrow = ((int64_t)pid * p.page_size + off) * row_stride_tok + h_kv;
        }
        if (!valid) tokrow = 0;
        uint8_t* aux = sv + TILE;
        if constexpr (FMT == KV_NVFP4) {
          const uint8_t* src = (is_v ? p.v_micro : p.k_micro) + tokrow * MR;
          const uint32_t dst = smem_u32(aux + (is_v ? kTN * MR : 0) + r * MR);
          if constexpr (MR == 8) cp_async8(dst, src, valid ? 8 : 0);
          else cp_async4(dst, src, valid ? 4 : 0);
        } else {
          const float* src = (is_v ? p.v_tok : p.k_tok) + tokrow;
          cp_async4(smem_u32(aux + (is_v ? kTN * 4 : 0) + r * 4), src, valid ? 4 : 0);
        }
      }
    }
  };

  // ---- running state ----------------------------------------------------------------------------
  float o[NOT][4];
#pragma unroll
  for (int t = 0; t < NOT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float sc_log2 = p.softmax_scale * kLog2e * p.k_scale;
  const bool tok_scales = (FMT == KV_E4M3) && (p.k_tok != nullptr);

#pragma unroll
  for (int s = 0; s < NSTAGE - 1; ++s) {
    if (s < n_tiles) issue(s, k_begin + s * kTN);
    cp_async_commit();
  }

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<NSTAGE - 2>();
    __syncthreads();
    {
      const int nt = t + NSTAGE - 1;
      if (nt < n_tiles) issue(nt % NSTAGE, k_begin + nt * kTN);
      cp_async_commit();
    }
    const int stage = t % NSTAGE;
    const uint8_t* sk = smem + stage * STAGE;
    const uint8_t* sv = sk + TILE;
    const uint8_t* aux = sv + TILE;
    const int kt = k_begin + t * kTN;
    const int kw = 16 * warp;   // this warp's first key within the tile

    // ---------------- S = Q K^T for 16 keys -----------------------------------------------------
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    {
      const int krow = kw + (lane & 7) + ((lane >> 4) << 3);
      const int csel = (lane >> 3) & 1;
      const uint32_t kbase = smem_u32(sk + krow * KROW);
      if constexpr (FMT == KV_F16 || FMT == KV_BF16) {
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks) {
          uint32_t r[4];
          ldmatrix_x4(r, kbase + swz<KROW>(krow, 2 * ks + csel) * 16);
          mma_rows<BF, R8>(s[0], qf[ks], r[0], r[1]);
          mma_rows<BF, R8>(s[1], qf[ks], r[2], r[3]);
        }
      } else if constexpr (FMT == KV_E4M3) {
#pragma unroll
        for (int kp = 0; kp < NKS / 2; ++kp) {
          uint32_t r[4];
          ldmatrix_x4(r, kbase + swz<KROW>(krow, 2 * kp + csel) * 16);
          uint32_t lo, hi;
          e4m3x4_to_h2x2(r[0], lo, hi);
          mma_rows<false, R8>(s[0], qf[2 * kp], lo, hi);
          e4m3x4_to_h2x2(r[1], lo, hi);
          mma_rows<false, R8>(s[0], qf[2 * kp + 1], lo, hi);
          e4m3x4_to_h2x2(r[2], lo, hi);
          mma_rows<false, R8>(s[1], qf[2 * kp], lo, hi);
          e4m3x4_to_h2x2(r[3], lo, hi);
          mma_rows<false, R8>(s[1], qf[2 * kp + 1], lo, hi);
        }
      } else {
        // NVFP4: one 16-byte chunk = 32 head dims = 2 k-steps; lane-in-quad c owns dims 8c..8c+7 of
        // the chunk, which lie inside micro block 2*chunk + (c >> 1).
        const uint8_t* kmic = aux;
        uint32_t mic[2];   // per n-tile: the D/32 micro bytes this lane needs, one per chunk
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const uint8_t* mrow = kmic + (kw + 8 * n + g4) * MR;
          if constexpr (MR == 8) {
            const uint2 w = *reinterpret_cast<const uint2*>(mrow);
            mic[n] = prmt(w.x, w.y, (c >> 1) ? 0x7531u : 0x6420u);
          } else {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(mrow);
            mic[n] = prmt(w, 0u, (c >> 1) ? 0x4431u : 0x4420u);
          }
        }
#pragma unroll
        for (int kp = 0; kp < (D / 64 > 0 ? D / 64 : 1); ++kp) {
          uint32_t r[4];
          ldmatrix_x4(r, kbase + swz<KROW>(krow, 2 * kp + csel) * 16);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = j >> 1;              // r0,r1 -> keys 0-7 ; r2,r3 -> keys 8-15
            const int ch = 2 * kp + (j & 1);   // chunk index
            uint32_t h[4];
            e2m1x8_to_h2x4(r[j], h);
            const uint32_t mb = (mic[n] >> (8 * ch)) & 0xffu;
            const uint32_t mh = e4m3x2_to_h2(mb | (mb << 8));
            mma_rows<false, R8>(s[n], qf[2 * ch], hmul2_u32(h[0], mh), hmul2_u32(h[1], mh));
            mma_rows<false, R8>(s[n], qf[2 * ch + 1], hmul2_u32(h[2], mh), hmul2_u32(h[3], mh));
          }
        }
      }
    }

    // ---------------- scale, mask, online softmax ------------------------------------------------
    float vsc[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if constexpr (FMT == KV_E4M3) {
      if (tok_scales) {
        const float* ks_s = reinterpret_cast<const float*>(aux);
        const float* vs_s = ks_s + kTN;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float2 kk = *reinterpret_cast<const float2*>(ks_s + kw + 8 * n + 2 * c);
          const float2 vv = *reinterpret_cast<const float2*>(vs_s + kw + 8 * n + 2 * c);
          s[n][0] *= kk.x; s[n][1] *= kk.y; s[n][2] *= kk.x; s[n][3] *= kk.y;
          vsc[n][0] = vv.x; vsc[n][1] = vv.y;
        }
      }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] *= sc_log2;
    if (kt + kTN - 1 > mask_lim) {
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt + kw + 8 * n + 2 * c + (e & 1);
          if ((!R8 || e < 2) && key > lim[e >> 1]) s[n][e] = -INFINITY;
        }
    }
    float alpha[2] = {1.f, 1.f};
    bool changed = false;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
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
      l_run[r] = l_run[r] * alpha[r] + sum;
    }
    if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
      for (int tt = 0; tt < NOT; ++tt) {
        o[tt][0] *= alpha[0]; o[tt][1] *= alpha[0];
        if constexpr (!R8) { o[tt][2] *= alpha[1]; o[tt][3] *= alpha[1]; }
      }
    }

    // ---------------- O += P V --------------------------------------------------------------------
    uint32_t pa[4];
    if constexpr (BF) {
      pa[0] = pack_bf2(s[0][0], s[0][1]); pa[1] = pack_bf2(s[0][2], s[0][3]);
      pa[2] = pack_bf2(s[1][0], s[1][1]); pa[3] = pack_bf2(s[1][2], s[1][3]);
    } else {
      pa[0] = pack_h2(s[0][0] * vsc[0][0], s[0][1] * vsc[0][1]);
      pa[1] = pack_h2(s[0][2] * vsc[0][0], s[0][3] * vsc[0][1]);
      pa[2] = pack_h2(s[1][0] * vsc[1][0], s[1][1] * vsc[1][1]);
      pa[3] = pack_h2(s[1][2] * vsc[1][0], s[1][3] * vsc[1][1]);
    }
    {
      const int vrow = kw + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int csel = lane >> 4;
      const uint32_t vbase = smem_u32(sv + vrow * KROW);
      if constexpr (FMT == KV_F16 || FMT == KV_BF16) {
#pragma unroll
        for (int jp = 0; jp < D / 16; ++jp) {
          uint32_t r[4];
          ldmatrix_x4_trans(r, vbase + swz<KROW>(vrow, 2 * jp + csel) * 16);
          mma_rows<BF, R8>(o[2 * jp], pa, r[0], r[1]);
          mma_rows<BF, R8>(o[2 * jp + 1], pa, r[2], r[3]);
        }
      } else if constexpr (FMT == KV_E4M3) {
        // after the 16-bit transpose a register holds (k0,d0)(k0,d1)(k1,d0)(k1,d1); regroup to
        // (k0,d0)(k1,d0) | (k0,d1)(k1,d1): even head dims feed tile 2j, odd head dims tile 2j+1.
#pragma unroll
        for (int jp = 0; jp < D / 32; ++jp) {
          uint32_t r[4];
          ldmatrix_x4_trans(r, vbase + swz<KROW>(vrow, 2 * jp + csel) * 16);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint32_t e0, o0, e1, o1;      // even / odd head dims of keys 0-7 and of keys 8-15
            e4m3x4_to_h2x2(prmt(r[2 * u], 0u, 0x3120u), e0, o0);
            e4m3x4_to_h2x2(prmt(r[2 * u + 1], 0u, 0x3120u), e1, o1);
            const int j = 2 * jp + u;
            mma_rows<false, R8>(o[2 * j], pa, e0, e1);
            mma_rows<false, R8>(o[2 * j + 1], pa, o0, o1);
          }
        }
      } else {
        // NVFP4 V: a 16-bit unit holds 4 head dims of one key.  Lane g4 owns unit g4 of the chunk
        // (dims 4*g4..4*g4+3, micro block 2*chunk + (g4 >> 2)) for keys 2c, 2c+1 (and +8).
        const uint8_t* vmic = aux + kTN * MR;
        uint32_t mlo[2], mhi[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint8_t* r0p = vmic + (kw + 8 * u + 2 * c) * MR;
          uint32_t a, bq;
          if constexpr (MR == 8) {
            const uint2 w0 = *reinterpret_cast<const uint2*>(r0p);
            const uint2 w1 = *reinterpret_cast<const uint2*>(r0p + MR);
            const uint32_t sel = (g4 >> 2) ? 0x7531u : 0x6420u;
            a = prmt(w0.x, w0.y, sel);
            bq = prmt(w1.x, w1.y, sel);
          } else {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(r0p);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(r0p + MR);
            const uint32_t sel = (g4 >> 2) ? 0x4431u : 0x4420u;
            a = prmt(w0, 0u, sel);
            bq = prmt(w1, 0u, sel);
          }
          // interleave: chunk ch -> bytes (a[ch], b[ch])
          mlo[u] = prmt(a, bq, 0x5140u);   // chunks 0,1
          mhi[u] = prmt(a, bq, 0x7362u);   // chunks 2,3
        }
#pragma unroll
        for (int jp = 0; jp < (D / 64 > 0 ? D / 64 : 1); ++jp) {
          uint32_t r[4];
          ldmatrix_x4_trans(r, vbase + swz<KROW>(vrow, 2 * jp + csel) * 16);
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int ch = 2 * jp + cc;
            uint32_t bfrag[2][4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              uint32_t h[4];
              e2m1x8_to_h2x4(r[2 * cc + u], h);
              const uint32_t mw = (ch < 2) ? mlo[u] : mhi[u];
              const uint32_t mm = e4m3x2_to_h2(mw >> (16 * (ch & 1)));
              bfrag[u][0] = hmul2_u32(prmt(h[0], h[2], 0x5410u), mm);
              bfrag[u][1] = hmul2_u32(prmt(h[0], h[2], 0x7632u), mm);
              bfrag[u][2] = hmul2_u32(prmt(h[1], h[3], 0x5410u), mm);
              bfrag[u][3] = hmul2_u32(prmt(h[1], h[3], 0x7632u), mm);
            }
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) mma_rows<false, R8>(o[4 * ch + qd], pa, bfrag[0][qd], bfrag[1][qd]);
          }
        }
      }
    }
  }

  // ---- combine the four warps ---------------------------------------------------------------------
  cp_async_wait<0>();
  __syncthreads();
  float* s_o = reinterpret_cast<float*>(smem);                 // [warp][16][D]
  float* s_m = s_o + kWarps * kRowTile * D;                    // [warp][16]
  float* s_l = s_m + kWarps * kRowTile;                        // [warp][16]
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  {
    const float out_scale = p.v_scale;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int row = g4 + 8 * r;
      if (row < rows_valid) {
        float* dst = s_o + (warp * kRowTile + row) * D;
#pragma unroll
        for (int t = 0; t < NOT; ++t) {
          dst[out_dim<FMT>(t, c, 0)] = o[t][2 * r] * out_scale;
          dst[out_dim<FMT>(t, c, 1)] = o[t][2 * r + 1] * out_scale;
        }
        if (c == 0) {
          s_m[warp * kRowTile + row] = m_run[r];
          s_l[warp * kRowTile + row] = l_run[r];
        }
      }
    }
  }
  __syncthreads();

  const bool single = (it.n_split == 1);
  const int slot = it.slot_base + it.split;
  for (int idx = tid; idx < rows_valid * D; idx += kThreads) {
    const int row = idx / D, dd = idx - row * D;
    float mw[kWarps];
    float mstar = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      mw[w] = s_m[w * kRowTile + row];
      mstar = fmaxf(mstar, mw[w]);
    }
    const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float wgt = fast_exp2(mw[w] - m_use);
      acc += wgt * s_o[(w * kRowTile + row) * D + dd];
      l += wgt * s_l[w * kRowTile + row];
    }
    const float val = (l > 0.f) ? acc / l : 0.f;
    const float lse = (l > 0.f) ? (m_use + log2f(l)) * kLn2 : -INFINITY;
    const int m = m0 + row;
    const int iq = m / p.G, g = m - iq * p.G;
    const int64_t orow = ((int64_t)b * p.H_q + (h_kv * p.G + g)) * p.N_q + iq;
    if (single) {
      store_out_dyn(p.out, p.out_dtype, orow * D + dd, val);
      if (p.lse && dd == 0) p.lse[orow] = lse;
    } else {
      const int64_t prow = ((int64_t)slot * p.H_q + (h_kv * p.G + g)) * p.N_q + iq;
      p.part_o[prow * D + dd] = val;
      if (dd == 0) p.part_lse[prow] = lse;
    }
  }
  if (single) return;

  // ---- last CTA of this (sequence, head, row tile) merges all key ranges -------------------------
  __threadfence();
  __syncthreads();
  const int cidx = (b * p.H_kv + h_kv) * gridDim.y + blockIdx.y;
  if (tid == 0) s_ticket = atomicAdd(p.counters + cidx, 1);
  __syncthreads();
  if (s_ticket != it.n_split - 1) return;
  __threadfence();
  if (tid == 0) p.counters[cidx] = 0;   // self-reset for the next launch
  // A thread owns (row, four output columns) and, when there are fewer such columns than threads, one of
  // `groups` interleaved subsets of the ranges; the partials of kU ranges are fetched before any is used,
  // so a merge over n ranges costs about n / (kU * groups) L2 round trips, with a running maximum.  The
  // groups meet in shared memory (the K/V pipeline is drained by now).
  constexpr int D4 = D / 4;
  constexpr int kU = 8;
  const int64_t slot_stride = (int64_t)p.H_q * p.N_q;
  const int n_cols = rows_valid * D4;
  int groups = 1;
  while (groups * 2 * n_cols <= kThreads && groups * 2 <= it.n_split) groups *= 2;
  float* s_part = reinterpret_cast<float*>(smem);          // [groups][n_cols][6]: m, l, acc.xyzw
  static_assert(PIPE_BYTES >= kThreads * 6 * 4, "merge scratch does not fit the pipeline buffers");
  const int n_work = groups > 1 ? groups * n_cols : n_cols;
  for (int idx0 = 0; idx0 < n_work; idx0 += kThreads) {
    const int idx = idx0 + tid;
    const bool active = idx < n_work;
    const int grp = groups > 1 ? idx / n_cols : 0;
    const int col = groups > 1 ? idx - grp * n_cols : idx;
    const int row = active ? col / D4 : 0, d4 = col - row * D4;
    const int m = m0 + row;
    const int iq = m / p.G, g = m - iq * p.G;
    const int64_t hrow = (int64_t)(h_kv * p.G + g) * p.N_q + iq;
    float m_run = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
      const float* lse_base = p.part_lse + it.slot_base * slot_stride + hrow;
      const float4* o_base = reinterpret_cast<const float4*>(p.part_o + (it.slot_base * slot_stride + hrow) * D) + d4;
      const int n_mine = (it.n_split - grp + groups - 1) / groups;       // ranges grp, grp + groups, ...
      for (int s0 = 0; s0 < n_mine; s0 += kU) {
        float ls[kU];
        float4 ov[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int sidx = grp + groups * min(s0 + u, n_mine - 1);
          ls[u] = __ldcg(lse_base + sidx * slot_stride);
          ov[u] = __ldcg(o_base + sidx * slot_stride * D4);
          if (s0 + u >= n_mine) ls[u] = -INFINITY;
        }
        float mb = m_run;
#pragma unroll
        for (int u = 0; u < kU; ++u) mb = fmaxf(mb, ls[u]);
        if (mb == -INFINITY) continue;
        const float resc = __expf(m_run - mb);
        acc.x *= resc, acc.y *= resc, acc.z *= resc, acc.w *= resc, l *= resc;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const float wgt = __expf(ls[u] - mb);
          acc.x += wgt * ov[u].x, acc.y += wgt * ov[u].y, acc.z += wgt * ov[u].z, acc.w += wgt * ov[u].w;
          l += wgt;
        }
        m_run = mb;
      }
    }
    if (groups > 1) {            // n_work <= kThreads: a single pass, every thread reaches the barriers
      float* mine = s_part + (size_t)idx * 6;
      if (active) {
        mine[0] = m_run, mine[1] = l, mine[2] = acc.x, mine[3] = acc.y, mine[4] = acc.z, mine[5] = acc.w;
      }
      __syncthreads();
      if (!active || grp != 0) continue;
      for (int g2 = 1; g2 < groups; ++g2) {
        const float* o = s_part + ((size_t)g2 * n_cols + col) * 6;
        const float mb = fmaxf(m_run, o[0]);
        if (mb == -INFINITY) continue;
        const float ra = __expf(m_run - mb), rb = __expf(o[0] - mb);
        acc.x = acc.x * ra + o[2] * rb, acc.y = acc.y * ra + o[3] * rb;
        acc.z = acc.z * ra + o[4] * rb, acc.w = acc.w * ra + o[5] * rb;
        l = l * ra + o[1] * rb;
        m_run = mb;
      }
    } else if (!active) {
      continue;
    }
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    const int64_t orow = (int64_t)b * p.H_q * p.N_q + hrow;
    const int64_t o0 = orow * D + d4 * 4;
    store_out_dyn(p.out, p.out_dtype, o0 + 0, acc.x * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 1, acc.y * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 2, acc.z * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 3, acc.w * inv);
    if (p.lse && d4 == 0) p.lse[orow] = (l > 0.f) ? m_run + __logf(l) : -INFINITY;
  }
}

template <int D, int FMT, int NSTAGE, int MINB, bool R8>
int launch_decode(const DecodeParams& p, int n_items, int row_tiles, cudaStream_t stream) {
  using G_ = Geo<D, FMT>;
  constexpr int PIPE = (NSTAGE * G_::STAGE > G_::MERGE) ? NSTAGE * G_::STAGE : G_::MERGE;
  const int SMEM = PIPE + p.bt_cap * 4;
  constexpr int SMEM_MAX = PIPE + kMaxPages * 4;
  auto kern = paged_decode_kernel<D, FMT, NSTAGE, MINB, R8>;
  static int configured_device = -1;   // attribute is per device
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX));
    configured_device = dev;
  }
  dim3 grid((unsigned)(n_items * p.H_kv), (unsigned)row_tiles);
  kern<<<grid, kThreads, SMEM, stream>>>(p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace

// ---- merge of rank-major partials --------------------------------------------------------------
__global__ void merge_partials_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                                      int n_parts, int64_t rows, int D, int64_t o_stride, int64_t lse_stride,
                                      void* out, int out_dtype, float* lse_out) {
  const int64_t row = blockIdx.x;
  float mstar = -INFINITY;
  for (int s = 0; s < n_parts; ++s) mstar = fmaxf(mstar, lse_parts[s * lse_stride + row]);
  const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
  float l = 0.f;
  for (int s = 0; s < n_parts; ++s) l += __expf(lse_parts[s * lse_stride + row] - m_use);
  for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_parts; ++s)
      acc += __expf(lse_parts[s * lse_stride + row] - m_use) * o_parts[s * o_stride + row * D + dd];
    store_out_dyn(out, out_dtype, row * D + dd, (l > 0.f) ? acc / l : 0.f);
  }
  if (lse_out && threadIdx.x == 0) lse_out[row] = (l > 0.f) ? m_use + __logf(l) : -INFINITY;
}

}  // namespace fa

using namespace fa;

extern "C" int fa_decode_plan_max_items(const int32_t* seq_lens_host, int n_k, int B, int page_size) {
  (void)page_size;
  int64_t total = 0;
  for (int b = 0; b < B; ++b) total += (seq_lens_host ? std::max(seq_lens_host[b], 0) : std::max(n_k, 0)) / kTN + 2;
  return (int)std::min<int64_t>(total, INT_MAX);
}

extern "C" int fa_decode_plan(const int32_t* seq_lens_host, int n_k, int B, int H_kv, int rows, int page_size,
                              int num_sms, int chunk_hint, fa_decode_item* items, int max_items,
                              int* n_items, int* max_range_keys) {
  FA_CHECK_ARG(B >= 1 && H_kv >= 1 && rows >= 1 && page_size >= 1, "fa_decode_plan: B, H_kv, rows, page_size must be >= 1");
  FA_CHECK_ARG(items && n_items && max_range_keys, "fa_decode_plan: null output pointer");
  if (num_sms == 0) num_sms = 148;
  const int row_tiles = (rows + kRowTile - 1) / kRowTile;
  int64_t total = 0;
  for (int b = 0; b < B; ++b) {
    const int len = seq_lens_host ? seq_lens_host[b] : n_k;
    FA_CHECK_ARG(len >= 0, "fa_decode_plan: negative sequence length at b=%d", b);
    total += len;
  }
  // Every range pays a fixed start-up (metadata, block table, pipeline fill; worth 300-500 keys), and a
  // launch ends with its last wave.  Candidates: whole sequences (longest first); two or three equal
  // ranges per sequence; shrinking ranges (guided scheduling): with `share` = keys per slot under perfect
  // balance, each sequence gives half of what is left of it to ranges of `share` keys, half of the rest to
  // ranges of share/2, ... down to a floor of 1024 keys, so that the short ranges fill the tail and every
  // level holds about slots/2 ranges.  The candidate with the shortest list-scheduling estimate is taken;
  // with many waves of whole sequences (>= 6 per slot) nothing is cut.
  // (Measured on B200: FP8 KV, B=4, 8 KV heads, 1 Mi-key contexts 1810 -> 1691 us against eight equal
  // waves; fp16, 8 KV heads, 8192-key contexts: 55 sequences 330 -> 294 us, 80 sequences 477 -> 457 us.)
  // A range of n keys that starts anywhere inside a page touches at most n / page_size + 2 pages, and that
  // is the number of block-table entries the kernel stages (at most kMaxPages).
  const int64_t max_chunk = (int64_t)(kMaxPages - 2) * page_size / kTN * kTN;
  FA_CHECK_ARG(max_chunk >= kTN, "fa_decode_plan: page_size too small");
  const int64_t slots = num_sms > 0 ? (int64_t)num_sms * 3 : -(int64_t)num_sms;   // negative: the slot count itself
  const int64_t units = (int64_t)B * H_kv * row_tiles;
  const int64_t work = total * H_kv * row_tiles;      // keys x heads x row tiles
  auto round_tile = [](int64_t x) { return std::max<int64_t>((x + kTN - 1) / kTN * kTN, kTN); };
  int64_t chunk = max_chunk;
  if (chunk_hint > 0) chunk = chunk_hint;
  chunk = std::min(round_tile(chunk), max_chunk);

  constexpr int64_t floor_keys = 1024;     // shortest range of the shrinking schedule
  constexpr double level_frac = 0.5;       // share of what is left of a sequence that each level takes
  const int64_t share = std::max<int64_t>(work / slots, 1);
  // small jobs: let the floor fall to 256 keys so that there are still ranges for every slot
  const int64_t floor_chunk = std::min(std::min(round_tile(floor_keys), std::max<int64_t>(round_tile(share / 2), 256)), max_chunk);

  // one candidate plan: whole sequences (cut only at `chunk`) or shrinking ranges
  auto build = [&](bool guided, int parts, std::vector<fa_decode_item>& v, int& max_range) {
  std::vector<int64_t> cuts;
  int slot = 0;
  max_range = 0;
  v.clear();
  for (int b = 0; b < B; ++b) {
    const int len = seq_lens_host ? seq_lens_host[b] : n_k;
    cuts.clear();                                       // range boundaries after 0
    if (!guided) {
      int ns = (int)std::max<int64_t>((len + chunk - 1) / chunk, 1);
      if (parts > 1 && len >= (int64_t)parts * 512) ns = std::max(ns, parts);   // `parts` equal ranges per sequence
      const int64_t cb = round_tile((len + ns - 1) / ns);
      ns = (int)std::max<int64_t>((len + cb - 1) / cb, 1);
      for (int s2 = 1; s2 <= ns; ++s2) cuts.push_back(std::min<int64_t>((int64_t)s2 * cb, len));
    } else {
      int64_t pos = 0;
      int64_t c = std::min(std::max(round_tile(share), floor_chunk), max_chunk);
      while (pos < len) {
        const int64_t rem = len - pos;
        if (c <= floor_chunk || rem <= floor_chunk) {   // the rest in equal ranges of about the floor
          const int64_t n = std::max<int64_t>((rem + floor_chunk - 1) / floor_chunk, 1);
          const int64_t cb = round_tile((rem + n - 1) / n);
          while (pos < len) { pos = std::min<int64_t>(pos + cb, len); cuts.push_back(pos); }
          break;
        }
        const int64_t n = (int64_t)(rem * level_frac) / c;
        for (int64_t i = 0; i < n; ++i) { pos += c; cuts.push_back(pos); }
        c = std::max(round_tile(c / 2), floor_chunk);
      }
      if (cuts.empty()) cuts.push_back(len);
    }
    const int ns = (int)cuts.size();
    int64_t begin = 0;
    for (int s2 = 0; s2 < ns; ++s2) {
      fa_decode_item it{};
      it.b = b;
      it.k_begin = (int)begin;
      it.k_end = (int)cuts[s2];
      it.slot_base = slot;
      it.n_split = ns;
      it.split = s2;
      begin = cuts[s2];
      max_range = std::max(max_range, it.k_end - it.k_begin);
      v.push_back(it);
    }
    slot += ns;
  }
  };
  // Estimated length of the launch, in units of the time one CTA needs for one key when every slot is busy.
  // A fluid model fitted to measurements on B200 (fp16 KV, 8 KV heads, 8 / 16 / 32 sequences of 1024-8192 keys
  // cut into ranges of 256 ... 8192 keys: 30 launches of 41 ... 190 us, rms error 2 %; FP8 KV, 4 sequences of
  // 131072 / 524288 keys, ranges of 2048 ... 131072 keys: 17 launches, rms error 6 %): CTAs take the slots in
  // launch order (longest range first); a CTA first spends a start-up (4 us for the fp16 kernel with two
  // CTAs per SM, 2 us for the kernels with three: metadata, block table, first tiles in flight), then streams
  // its keys; all streaming CTAs progress at the same rate, which falls linearly from 1.4 with one CTA per SM
  // (a lone CTA is latency bound) to 1 with every slot streaming (the HBM or issue bound).  The H_kv x row-tile
  // CTAs of a range are equal and adjacent in launch order, so they are scheduled as one job on
  // slots / (H_kv x row tiles) groups of slots, which keeps this pass at a few microseconds.
  const double kCtasPerSm = num_sms > 0 ? 3.0 : 2.0;
  const double kStartUp = num_sms > 0 ? 90.0 : 160.0;
  constexpr double kSoloRate = 1.4;
  auto estimate = [&](std::vector<fa_decode_item>& v) -> int64_t {
    std::stable_sort(v.begin(), v.end(), [](const fa_decode_item& a, const fa_decode_item& b2) {
      return (a.k_end - a.k_begin) > (b2.k_end - b2.k_begin);
    });
    const int64_t per_item = (int64_t)H_kv * row_tiles;
    const int64_t groups = slots / per_item;
    if (groups <= 1) {
      int64_t sum = 0;
      for (const fa_decode_item& it : v) sum += (it.k_end - it.k_begin) + (int64_t)kStartUp;
      return sum * per_item / std::max<int64_t>(slots, 1);
    }
    // min-heaps: CTAs still starting up (by the time they begin to stream), streaming CTAs (by the value of
    // the common progress counter at which they finish)
    std::vector<std::pair<double, int>> starting;
    std::vector<double> streaming;
    auto later_s = [](const std::pair<double, int>& x, const std::pair<double, int>& y) { return x.first > y.first; };
    auto later_d = [](double x, double y) { return x > y; };
    size_t next = 0;
    double t = 0.0, progress = 0.0;
    auto dispatch = [&]() {
      while (next < v.size() && (int64_t)(starting.size() + streaming.size()) < groups) {
        starting.emplace_back(t + kStartUp, v[next].k_end - v[next].k_begin);
        std::push_heap(starting.begin(), starting.end(), later_s);
        ++next;
      }
    };
    dispatch();
    while (!starting.empty() || !streaming.empty()) {
      const double per_sm = kCtasPerSm * (double)streaming.size() / (double)groups;      // streaming CTAs per SM
      const double rate = streaming.empty() ? 0.0
                          : std::max(1.0, std::min(kSoloRate, kSoloRate - (kSoloRate - 1.0) * (per_sm - 1.0) / (kCtasPerSm - 1.0)));
      const double t_start = starting.empty() ? 1e300 : starting.front().first;
      const double t_finish = streaming.empty() ? 1e300 : t + (streaming.front() - progress) / rate;
      if (t_start <= t_finish) {
        progress += rate * (t_start - t);
        t = t_start;
        const int keys = starting.front().second;
        std::pop_heap(starting.begin(), starting.end(), later_s);
        starting.pop_back();
        streaming.push_back(progress + keys);
        std::push_heap(streaming.begin(), streaming.end(), later_d);
      } else {
        progress = streaming.front();
        t = t_finish;
        std::pop_heap(streaming.begin(), streaming.end(), later_d);
        streaming.pop_back();
        dispatch();
      }
    }
    return (int64_t)t;
  };
  std::vector<fa_decode_item> v;
  int max_range = 0;
  if (chunk_hint > 0 || units >= 6 * slots) {
    build(false, 1, v, max_range);                       // as asked, or enough whole sequences for many waves
  } else {
    // few waves: whole sequences leave the last wave partly empty; two or three equal ranges per sequence,
    // or shrinking ranges, fill it at the price of a start-up per range.  Take the candidate
    // with the shortest estimated launch.
    build(false, 1, v, max_range);
    int64_t best = estimate(v);
    // no plan beats (all work + one start-up per unit) / slots: stop when whole sequences are within 6 % of it
    const int64_t lower = (work + (int64_t)kStartUp * units) / std::max<int64_t>(slots, 1);
    std::vector<fa_decode_item> alt;
    int alt_range = 0;
    // shrinking ranges only pay when there are fewer units than slots; with more they are not tried
    for (int cand = (units >= slots ? 1 : 0); cand < 3 && best * 100 > lower * 106; ++cand) {
      if (cand == 0) build(true, 1, alt, alt_range);
      else build(false, cand + 1, alt, alt_range);
      const int64_t t = estimate(alt);
      if (t < best) {
        best = t;
        v = alt;
        max_range = alt_range;
      }
    }
    // Full waves of equal ranges: the shortest common range length whose CTAs still fit w waves of slots,
    // every sequence cut into equal parts no longer than that.  A launch that is one (or two, three) full
    // waves has no partly empty last wave, and for small jobs -- what one GPU of several sees of a sharded
    // batch -- it beats the shrinking ranges (measured on 8 sequences of ~5000 keys, 8 KV heads: 41 us for
    // one wave of 288 CTAs against 47 us for 488 CTAs of shrinking ranges).
    const int64_t per_item = (int64_t)H_kv * row_tiles;
    auto ctas_at = [&](int64_t len_cap) {
      int64_t n = 0;
      for (int b = 0; b < B; ++b) {
        const int64_t len = seq_lens_host ? seq_lens_host[b] : n_k;
        n += std::max<int64_t>((len + len_cap - 1) / len_cap, 1) * per_item;
      }
      return n;
    };
    const int64_t saved_chunk = chunk;
    for (int waves = 1; waves <= 3 && best * 100 > lower * 106; ++waves) {
      if (ctas_at(max_chunk) > waves * slots) continue;               // not even the longest ranges fit
      int64_t lo = 1, hi = max_chunk / kTN;                            // in tiles: smallest cap that fits
      while (lo < hi) {
        const int64_t mid = (lo + hi) / 2;
        if (ctas_at(mid * kTN) <= waves * slots) hi = mid; else lo = mid + 1;
      }
      chunk = lo * kTN;
      if (chunk < 256) break;                                          // ranges this short are all start-up
      build(false, 1, alt, alt_range);
      const int64_t t = estimate(alt);
      if (t < best) {
        best = t;
        v = alt;
        max_range = alt_range;
      }
    }
    chunk = saved_chunk;
  }
  std::stable_sort(v.begin(), v.end(), [](const fa_decode_item& a, const fa_decode_item& b2) {
    return (a.k_end - a.k_begin) > (b2.k_end - b2.k_begin);
  });
  if ((int)v.size() > max_items) return fail(FA_ERR_INVALID, "fa_decode_plan: %zu items exceed capacity %d", v.size(), max_items);
  std::copy(v.begin(), v.end(), items);
  *n_items = (int)v.size();
  *max_range_keys = max_range;
  return FA_OK;
}

extern "C" size_t fa_decode_workspace_bytes(int n_slots, int H_q, int N_q, int D) {
  return (size_t)n_slots * H_q * N_q * (D + 1) * 4;
}

extern "C" size_t fa_decode_counters_len(int B, int H_q, int H_kv, int N_q) {
  const int G = H_kv > 0 ? H_q / H_kv : 1;
  const int row_tiles = (G * N_q + kRowTile - 1) / kRowTile;
  return (size_t)B * H_kv * row_tiles + 1;   // word 0 is the status word
}

// Every argument check of the decode entry points; nothing is enqueued before this has passed.
static int decode_check(const fa_decode_args* a) {
  FA_CHECK_ARG(a != nullptr, "fa_paged_decode_fwd: null args");
  FA_CHECK_ARG(a->q && a->k_pool && a->v_pool && a->block_table && a->items && a->out,
               "fa_paged_decode_fwd: q, k_pool, v_pool, block_table, items, out must be non-null");
  FA_CHECK_ARG(a->B >= 1 && a->H_q >= 1 && a->H_kv >= 1 && a->N_q >= 1, "fa_paged_decode_fwd: bad B/H/N_q");
  FA_CHECK_ARG(a->H_q % a->H_kv == 0,
               "H_q must be a positive multiple of H_kv (GQA group factor G = H_q/H_kv); got H_q=%d H_kv=%d",
               a->H_q, a->H_kv);
  if (a->D != 64 && a->D != 128) return fail(FA_ERR_UNSUPPORTED, "paged decode supports head_dim 64 or 128 (got %d)", a->D);
  FA_CHECK_ARG(a->page_size >= 1 && a->n_logical >= 1 && a->num_blocks >= 1, "bad page_size / n_logical / num_blocks");
  FA_CHECK_ARG(a->n_items >= 1, "empty plan");
  FA_CHECK_ARG(a->out_dtype == FA_F32 || a->out_dtype == FA_F16 || a->out_dtype == FA_BF16, "out_dtype must be f32/f16/bf16");
  int fmt;
  switch (a->kv_dtype) {
    case FA_F16: fmt = KV_F16; FA_CHECK_ARG(a->q_dtype == FA_F16, "f16 pools need f16 q"); break;
    case FA_BF16: fmt = KV_BF16; FA_CHECK_ARG(a->q_dtype == FA_BF16, "bf16 pools need bf16 q"); break;
    case FA_E4M3: fmt = KV_E4M3; FA_CHECK_ARG(a->q_dtype == FA_F16, "e4m3 pools need f16 q"); break;
    case FA_NVFP4:
      fmt = KV_NVFP4;
      FA_CHECK_ARG(a->q_dtype == FA_F16, "nvfp4 pools need f16 q");
      FA_CHECK_ARG(a->k_micro && a->v_micro, "nvfp4 pools need micro-scale pools");
      break;
    default: return fail(FA_ERR_INVALID, "unknown kv_dtype %d", a->kv_dtype);
  }
  FA_CHECK_ARG((a->k_token_scale == nullptr) == (a->v_token_scale == nullptr), "k/v token scales must both be set or both null");
  FA_CHECK_ARG(a->k_token_scale == nullptr || fmt == KV_E4M3, "per-token scales are only defined for e4m3 pools");

  const int G = a->H_q / a->H_kv;
  const int M = G * a->N_q;
  const int row_tiles = (M + kRowTile - 1) / kRowTile;
  FA_CHECK_ARG(row_tiles <= 65535, "too many query rows per KV head (%d)", M);

  FA_CHECK_ARG(a->n_slots == 0 || a->n_slots == a->n_items, "n_slots must be 0 (no sequence is split) or n_items");
  FA_CHECK_ARG(a->max_range_keys >= 0, "max_range_keys must be >= 0");
  const size_t need = fa_decode_workspace_bytes(a->n_slots, a->H_q, a->N_q, a->D);
  FA_CHECK_ARG(need == 0 || a->workspace != nullptr, "workspace must be non-null when a sequence is split");
  if (a->workspace_bytes < need) return fail(FA_ERR_WORKSPACE, "workspace %zu B < %zu B", a->workspace_bytes, need);
  const size_t n_counters = fa_decode_counters_len(a->B, a->H_q, a->H_kv, a->N_q);
  FA_CHECK_ARG(a->counters != nullptr, "counters must be non-null");
  if (a->counters_len < n_counters) return fail(FA_ERR_WORKSPACE, "counters hold %zu ints < %zu", a->counters_len, n_counters);

  if (a->max_range_keys / a->page_size + 2 > kMaxPages)
    return fail(FA_ERR_INVALID, "key range of %d keys spans more than %d pages", a->max_range_keys, kMaxPages);
  (void)fmt;
  return FA_OK;
}

namespace fa {
// tcgen05 path for E4M3 pools (decode_tc.cu)
bool decode_tc_applicable(const fa_decode_args* a);
int launch_decode_tc(const fa_decode_args* a, cudaStream_t st);
}  // namespace fa

extern "C" int fa_paged_decode_fwd(const fa_decode_args* a) {
  const int rc_check = decode_check(a);
  if (rc_check != FA_OK) return rc_check;
  // E4M3 pools on pages of 64 or more tokens, one query position, at most 8 heads per KV head: the keys become
  // the M dimension of tcgen05 MMAs on the stored bytes (variant 9 keeps the mma.sync kernel)
  if (a->variant != 9 && a->variant != 2 && fa::decode_tc_applicable(a))
    return fa::launch_decode_tc(a, reinterpret_cast<cudaStream_t>(a->stream));
  const int fmt = a->kv_dtype == FA_F16 ? KV_F16 : a->kv_dtype == FA_BF16 ? KV_BF16 : a->kv_dtype == FA_E4M3 ? KV_E4M3 : KV_NVFP4;
  const int G = a->H_q / a->H_kv;
  const int M = G * a->N_q;
  const int row_tiles = (M + kRowTile - 1) / kRowTile;
  DecodeParams p{};
  p.q = reinterpret_cast<const uint16_t*>(a->q);
  p.k_pool = reinterpret_cast<const uint8_t*>(a->k_pool);
  p.v_pool = reinterpret_cast<const uint8_t*>(a->v_pool);
  p.k_micro = reinterpret_cast<const uint8_t*>(a->k_micro);
  p.v_micro = reinterpret_cast<const uint8_t*>(a->v_micro);
  p.k_tok = a->k_token_scale;
  p.v_tok = a->v_token_scale;
  p.block_table = a->block_table;
  p.q_offsets = a->q_offsets;
  p.items = a->items;
  p.out = a->out;
  p.lse = a->lse;
  p.status = a->counters;          // word 0: sticky error flags; the arrival counters follow
  p.counters = a->counters + 1;
  p.part_o = reinterpret_cast<float*>(a->workspace);
  p.part_lse = p.part_o + (size_t)a->n_slots * a->H_q * a->N_q * a->D;
  p.bt_cap = a->max_range_keys / a->page_size + 2;
  p.k_scale = a->k_scale;
  p.v_scale = a->v_scale;
  p.softmax_scale = a->softmax_scale;
  p.n_logical = a->n_logical;
  p.num_blocks = a->num_blocks;
  p.page_size = a->page_size;
  p.page_shift = ((a->page_size & (a->page_size - 1)) == 0) ? __builtin_ctz((unsigned)a->page_size) : -1;
  p.B = a->B; p.H_q = a->H_q; p.H_kv = a->H_kv; p.N_q = a->N_q; p.G = G; p.M = M;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  p.n_items = a->n_items; p.head_major = (a->variant == 2);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);

#define FA_LAUNCH(D_, F_, NS_, MB_, R8_) return launch_decode<D_, F_, NS_, MB_, R8_>(p, a->n_items, row_tiles, st)
  // R8 kernels: at most 8 packed rows (decode with G <= 8), rows 8..15 of the MMA tile are never kept.
  const bool r8 = (M <= 8);
  if (a->D == 128) {
    switch (fmt) {
      case KV_F16:
        if (r8) { if (a->variant == 1) FA_LAUNCH(128, KV_F16, 2, 3, true); FA_LAUNCH(128, KV_F16, 3, 2, true); }
        FA_LAUNCH(128, KV_F16, 3, 2, false);
      case KV_BF16:
        if (r8) FA_LAUNCH(128, KV_BF16, 3, 2, true);
        FA_LAUNCH(128, KV_BF16, 3, 2, false);
      case KV_E4M3:
        if (r8) FA_LAUNCH(128, KV_E4M3, 4, 3, true);
        FA_LAUNCH(128, KV_E4M3, 4, 3, false);
      default:
        if (r8) FA_LAUNCH(128, KV_NVFP4, 6, 3, true);
        FA_LAUNCH(128, KV_NVFP4, 6, 3, false);
    }
  } else {
    switch (fmt) {
      case KV_F16: if (r8) FA_LAUNCH(64, KV_F16, 4, 3, true); FA_LAUNCH(64, KV_F16, 4, 3, false);
      case KV_BF16: if (r8) FA_LAUNCH(64, KV_BF16, 4, 3, true); FA_LAUNCH(64, KV_BF16, 4, 3, false);
      case KV_E4M3: if (r8) FA_LAUNCH(64, KV_E4M3, 4, 3, true); FA_LAUNCH(64, KV_E4M3, 4, 3, false);
      default: if (r8) FA_LAUNCH(64, KV_NVFP4, 6, 3, true); FA_LAUNCH(64, KV_NVFP4, 6, 3, false);
    }
  }
#undef FA_LAUNCH
}

// ---- decode without any caller-supplied or allocated scratch ---------------------------------------
// Scratch of fa_paged_decode_fwd_static: word 0 is the status word (kept across calls until it is read with
// fa_paged_decode_static_status), the next kStaticUnits int32 words are the arrival counters, and the
// partial results of split sequences start at kStaticHeaderBytes.  The array lives in the library's device
// image, so every GPU that loads the library carries these bytes until the process exits.
namespace {
constexpr size_t kStaticUnits = 16384;                                  // (sequence, KV head, row tile) units per call
constexpr size_t kStaticHeaderBytes = (kStaticUnits + 64) * sizeof(int32_t);
constexpr size_t kStaticScratchBytes = FA_DECODE_STATIC_SCRATCH_BYTES;
static_assert(kStaticHeaderBytes % 256 == 0 && kStaticHeaderBytes < kStaticScratchBytes, "static scratch layout");
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
unsigned char* g_static_scratch_ptr[kMaxDevices] = {nullptr};   // device address per device ordinal

// Device address of the array on the current device: in host code the array's name is only a handle, the
// address has to be asked for, once per device, with that device current.
int static_scratch(unsigned char** out) {
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  FA_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    FA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
    g_static_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_static_scratch_ptr[dev];
  return FA_OK;
}
}  // namespace

extern "C" int fa_paged_decode_fwd_static(const fa_decode_args* a) {
  FA_CHECK_ARG(a != nullptr, "fa_paged_decode_fwd_static: null args");
  // the cheap shape checks come first, so that a rejected call has touched nothing on the device
  FA_CHECK_ARG(a->B >= 1 && a->H_q >= 1 && a->H_kv >= 1 && a->N_q >= 1, "fa_paged_decode_fwd_static: bad B/H/N_q");
  FA_CHECK_ARG(a->H_q % a->H_kv == 0, "H_q must be a positive multiple of H_kv; got H_q=%d H_kv=%d", a->H_q, a->H_kv);
  if (a->D != 64 && a->D != 128) return fail(FA_ERR_UNSUPPORTED, "paged decode supports head_dim 64 or 128 (got %d)", a->D);
  FA_CHECK_ARG(a->n_items >= 1 && (a->n_slots == 0 || a->n_slots == a->n_items), "n_slots must be 0 or n_items >= 1");
  const size_t n_units = fa_decode_counters_len(a->B, a->H_q, a->H_kv, a->N_q) - 1;
  if (n_units > kStaticUnits)
    return fail(FA_ERR_WORKSPACE,
                "fa_paged_decode_fwd_static: %zu (sequence, head, row tile) units exceed the built-in %zu; "
                "use fa_paged_decode_fwd with caller scratch", n_units, kStaticUnits);
  const size_t part_cap = kStaticScratchBytes - kStaticHeaderBytes;
  const size_t part_need = fa_decode_workspace_bytes(a->n_slots, a->H_q, a->N_q, a->D);
  if (part_need > part_cap)
    return fail(FA_ERR_WORKSPACE,
                "fa_paged_decode_fwd_static: partial results need %zu B, the built-in scratch holds %zu B; "
                "use fa_paged_decode_fwd with caller scratch", part_need, part_cap);
  unsigned char* base = nullptr;
  const int rc = static_scratch(&base);
  if (rc != FA_OK) return rc;
  fa_decode_args b = *a;
  b.counters = reinterpret_cast<int32_t*>(base);
  b.counters_len = kStaticUnits + 1;
  b.workspace = base + kStaticHeaderBytes;
  b.workspace_bytes = part_cap;
  const int rc_check = decode_check(&b);
  if (rc_check != FA_OK) return rc_check;
  // The array keeps whatever the previous call left; the arrival counters have to start at zero (an earlier
  // call that ended in an error may have left some behind).  The status word is not cleared here.
  FA_CUDA_OK(cudaMemsetAsync(b.counters + 1, 0, n_units * sizeof(int32_t), reinterpret_cast<cudaStream_t>(a->stream)));
  return fa_paged_decode_fwd(&b);
}

extern "C" int fa_paged_decode_static_status(int32_t* status_host, int clear, void* stream) {
  FA_CHECK_ARG(status_host != nullptr, "fa_paged_decode_static_status: null pointer");
  unsigned char* base = nullptr;
  const int rc = static_scratch(&base);
  if (rc != FA_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FA_CUDA_OK(cudaMemcpyAsync(status_host, base, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  if (clear) FA_CUDA_OK(cudaMemsetAsync(base, 0, sizeof(int32_t), st));
  FA_CUDA_OK(cudaStreamSynchronize(st));
  return FA_OK;
}

extern "C" int fa_merge_partials(const float* o_parts, const float* lse_parts, int n_parts, int64_t rows, int D,
                                 int64_t o_part_stride, int64_t lse_part_stride, void* out, int out_dtype,
                                 float* lse_out, void* stream) {
  FA_CHECK_ARG(o_parts && lse_parts && out, "fa_merge_partials: null pointer");
  FA_CHECK_ARG(n_parts >= 1 && rows >= 1 && D >= 1, "fa_merge_partials: bad sizes");
  FA_CHECK_ARG(rows <= INT_MAX, "fa_merge_partials: too many rows");
  FA_CHECK_ARG(out_dtype == FA_F32 || out_dtype == FA_F16 || out_dtype == FA_BF16, "out_dtype must be f32/f16/bf16");
  if (o_part_stride <= 0) o_part_stride = rows * D;
  if (lse_part_stride <= 0) lse_part_stride = rows;
  const int threads = D >= 256 ? 256 : (D >= 128 ? 128 : 64);
  merge_partials_kernel<<<(unsigned)rows, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      o_parts, lse_parts, n_parts, rows, D, o_part_stride, lse_part_stride, out, out_dtype, lse_out);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_paged_decode_host(const fa_decode_host_args* h) {
  FA_CHECK_ARG(h != nullptr, "fa_paged_decode_host: null args");
  FA_CHECK_ARG(h->q_host && h->block_table_host && h->out_host && h->items_host, "fa_paged_decode_host: null host buffer");
  FA_CHECK_ARG(h->dev.q && h->dev.block_table && h->dev.items && h->dev.out, "fa_paged_decode_host: null device staging buffer");
  FA_CHECK_ARG(h->max_items >= 1, "fa_paged_decode_host: max_items must be >= 1");
  fa_decode_args a = h->dev;
  FA_CHECK_ARG(a.B >= 1 && a.H_kv >= 1 && a.H_q >= 1 && a.N_q >= 1 && a.H_q % a.H_kv == 0, "fa_paged_decode_host: bad B/H/N_q");
  FA_CHECK_ARG(a.page_size >= 1 && a.n_logical >= 1 && a.num_blocks >= 1, "fa_paged_decode_host: bad page_size / n_logical / num_blocks");
  FA_CHECK_ARG(h->block_table_bytes >= (size_t)a.B * a.n_logical * sizeof(int32_t), "fa_paged_decode_host: block_table_host smaller than [B, n_logical]");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a.stream);
  FA_CUDA_OK(cudaMemcpyAsync(const_cast<void*>(a.q), h->q_host, h->q_bytes, cudaMemcpyHostToDevice, st));
  FA_CUDA_OK(cudaMemcpyAsync(const_cast<int32_t*>(a.block_table), h->block_table_host, h->block_table_bytes, cudaMemcpyHostToDevice, st));
  // The table is in host memory here, so a bad entry is refused before any kernel is launched (the kernel
  // would mask the page and raise its status flag; the reference's host checks are of the same kind,
  // kernels/v8_gqa_ss/gqa_ss_attention.cu:267-291).  The scan runs while the two copies above are in flight; a
  // refused call leaves the staging buffers overwritten and nothing else.
  for (int b = 0; b < a.B; ++b) {
    const int len = h->seq_lens_host ? h->seq_lens_host[b] : h->n_k;
    FA_CHECK_ARG(len >= 0, "fa_paged_decode_host: negative sequence length at b=%d", b);
    const int64_t pages = ((int64_t)len + a.page_size - 1) / a.page_size;
    FA_CHECK_ARG(pages <= a.n_logical, "fa_paged_decode_host: sequence %d needs %lld pages, the table has %d columns", b, (long long)pages, a.n_logical);
    const int32_t* row = h->block_table_host + (size_t)b * a.n_logical;
    for (int64_t j = 0; j < pages; ++j)
      FA_CHECK_ARG((uint32_t)row[j] < (uint32_t)a.num_blocks, "fa_paged_decode_host: block_table[%d][%lld] = %d is outside [0, %d)", b, (long long)j, row[j], a.num_blocks);
  }
  int n_items = 0, max_range = 0;
  // as the Python host does: the fp16 / bf16 kernel at d = 128 runs two CTAs per SM, the planner counts three
  const int sms = device_sm_count();
  int plan_sms = ((a.kv_dtype == FA_F16 || a.kv_dtype == FA_BF16) && a.D == 128) ? -2 * sms : sms;
  {
    fa_decode_args probe = a;        // the tcgen05 kernel for E4M3 pools keeps one CTA per SM
    probe.max_range_keys = 0;
    if (a.variant != 9 && a.variant != 2 && fa::decode_tc_applicable(&probe)) plan_sms = -sms;
  }
  const int rc = fa_decode_plan(h->seq_lens_host, h->n_k, a.B, a.H_kv, (a.H_q / a.H_kv) * a.N_q, a.page_size, plan_sms,
                                h->chunk_hint, h->items_host, h->max_items, &n_items, &max_range);
  if (rc != FA_OK) return rc;
  FA_CUDA_OK(cudaMemcpyAsync(const_cast<fa_decode_item*>(a.items), h->items_host, (size_t)n_items * sizeof(fa_decode_item),
                             cudaMemcpyHostToDevice, st));
  a.n_items = n_items;
  a.n_slots = n_items > a.B ? n_items : 0;
  a.max_range_keys = max_range;
  const int rc2 = fa_paged_decode_fwd(&a);
  if (rc2 != FA_OK) return rc2;
  FA_CUDA_OK(cudaMemcpyAsync(h->out_host, a.out, h->out_bytes, cudaMemcpyDeviceToHost, st));
  return FA_OK;
}
