// MLA latent decode over an FP8 E4M3 latent on a pair of CTAs: tcgen05.mma kind::f8f6f4 straight on the stored
// bytes.  DQK = 576, DV = 512, fp16 queries, page_size a power of two >= 64, one fp32 scale per token or one
// for the tensor.
//
// The latent never exists in 16 bits anywhere: TMA brings the E4M3 bytes of a tile into 128-byte-swizzled
// operand blocks (64 keys x 128 one-byte dims) and the tensor core multiplies them as they are.  Its other
// operand must then be 8 bits wide as well, and a single E4M3 number (4 significant bits) is far too coarse
// for a query or a probability, so each is written as the sum of two E4M3 numbers, x = x1 + x2 with
// x1 = e4m3(x) and x2 = e4m3(x - x1): eight significant bits, what bf16 carries.  Every product is issued
// twice, once per piece, into the same fp32 accumulator; at the doubled rate of 8-bit operands that costs
// the tensor core what the fp16 product would, and HBM, L2 and shared memory see 576 bytes per token.
//
//   queries      row r of the pair's 128 rows is scaled by a power of two 2^e_r so that its largest element
//                lies in [128, 256), then split; the softmax undoes 2^e_r together with the softmax scale
//   scales       the same bytes serve as key and as value, so the scale s_k of token k multiplies column k of
//                the scores and the weight of row k in P V (the dequantisation of the reference,
//                kernels/v11_mla/mla_attention.cu:170-183, factored out of the element loop).  The V side is
//                folded into the exponent: with t_k = score_k + log2 s_k and the running maximum taken over t,
//                w_k = 2^(t_k - m) <= 1 is what goes to the tensor core (times 16, split in two pieces), and
//                the denominator adds w_k / s_k = 2^(score_k - m).  A rise of the maximum by less than 2^4 is
//                not followed (lazy rescale), so 16 w_k <= 256 stays inside E4M3.
//   geometry     as for the bf16 latent (mla_pair.cu): M = 128 rows over the two CTAs, scores N = 128 keys
//                (CTA r supplies keys [64 r, 64 r + 64)), output N = 256 per value segment s (CTA r supplies
//                columns [256 s + 128 r, +128) of the 64 keys of half h).  A tile of 64 keys is five blocks:
//                dims [0,128) [128,256) [256,384) [384,512) and [448,576) (the last box overlaps the fourth
//                so that every box is 128 bytes wide; its upper 64 bytes are the rope dims).  Block d < 4 is
//                also the value operand: its own keys' columns of segment d >> 1 when d & 1 == r, and after
//                the scores of the tile it is overwritten with this CTA's columns of the peer's keys when
//                d & 1 != r, so block parity = key half in both CTAs and one descriptor serves the pair.
//
//   memory       per CTA, shared: three tile buffers (3 x 40 KB), two P buffers (two pieces of 64 rows x 128 keys,
//                32 KB), the second query pieces (40 KB) and the first pieces of the rope dims (8 KB).  Tensor
//                memory: O (256 columns), two score buffers (2 x 64), and the first query pieces of dims
//                [0, 512) as the A operand (128 columns, four dims per column), which takes their reads off
//                shared memory -- the resource the N = 128 score products are short of.
//
// Warps: 0 = TMA producer (own keys), 1 = TMEM owner + score MMA issuer, 2 = TMA producer (peer keys) and
// token scales, 3 = P V MMA issuer, 4..11 = query split, softmax, epilogue (two warpgroups: the exponentials and
// the E4M3 conversions of a tile share the special-function pipe, 2.5 operations per score, and two warps per
// scheduler hide the shared-memory latency next to the tensor core's operand reads).  Every wait is bounded
// (sm100.cuh).
//
// Reference behaviour: kernels/v11_mla/mla_attention.cu:104-258 (what is computed) with the FP8 latent of
// kernels/v11_mla/mla_attention.cu:170-183; intended tensor-core backend kernels/v12_mla_tc/mla_tc_attention.cu:35-45.

#include "mla_pair.cuh"

namespace fa {
namespace {

using namespace sm100;
using namespace pair;


constexpr int kFBlocks = 5;                   // operand blocks of a 64-key tile / of the 64 query rows
constexpr float kFThreshold = 4.f;            // the running maximum is followed once it is 2^4 behind
constexpr float kFPre = 4.f;                  // weights go to the tensor core times 2^4
constexpr int kFThreads = 384;                // 4 producer / issuer warps + 8 softmax warps
constexpr int kFSoft = 256;                   // softmax threads
constexpr int kFTiles = 3;                    // tile buffers (score and P buffers: two)

// kind::f8f6f4 MMAs over the pair, descriptors as words (see mla_pair.cuh: one low word per operand buffer, a
// constant added per step)
__device__ __forceinline__ void mma2_f8_w(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
               " tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %4, p;\n}\n"
               ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma2_f8_ts_w(uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n .reg .b64 db;\n setp.ne.b32 p, %5, 0;\n mov.b64 db, {%2, %3};\n"
               " tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], [%1], db, %4, p;\n}\n"
               ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void softmax_bar256() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }
// two floats -> two E4M3 bytes (lo in bits 0..7), round to nearest, saturating
__device__ __forceinline__ uint32_t f2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f2(uint32_t v) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"((uint16_t)v));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// x = x1 + x2 in E4M3 for two numbers at once
__device__ __forceinline__ void split2(float a, float b, uint32_t& p1, uint32_t& p2) {
  p1 = f2_to_e4m3x2(a, b);
  const float2 f = e4m3x2_to_f2(p1);
  p2 = f2_to_e4m3x2(a - f.x, b - f.y);
}
// sixteen numbers -> their first and second pieces, sixteen bytes each
__device__ __forceinline__ void split16(const float* x, uint4& q1, uint4& q2) {
  uint32_t a[8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) split2(x[2 * i], x[2 * i + 1], a[i], b[i]);
  q1 = make_uint4(a[0] | (a[1] << 16), a[2] | (a[3] << 16), a[4] | (a[5] << 16), a[6] | (a[7] << 16));
  q2 = make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16));
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFThreads, 1)
mla_pair_f8_kernel(const __grid_constant__ CUtensorMap map_l, const MlaPairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // second pieces: [5 blocks][64 rows][128 dims]
  uint8_t* sQr = sQ + kFBlocks * kPBlk;        // first pieces of the rope dims: one block laid out like block 4
  uint8_t* sP = sQr + kPBlk;                   // [2 tiles][2 pieces][64 rows][128 keys]
  uint8_t* sT = sP + 4 * kPBlk;                // [3 tiles][5 blocks][64 keys][128 dims]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sT + kFTiles * kFBlocks * kPBlk);
  // tile buffers and their barriers (X_FULL, X_FULLB, R_FULL, T_FREEA, T_FREE) are indexed by j % 3, score and P
  // buffers (S_FULL, P_READY) by j & 1, scale buffers by j & 3
  enum { QT_READY = 0, X_FULL = 1, X_FULLB = 4, R_FULL = 7, T_FREEA = 10, T_FREE = 13, S_FULL = 16, P_READY = 18, SC_READY = 20,
         Z_GO = 24, NBARS = 25 };
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 26);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ticket = const_cast<int*>(reinterpret_cast<volatile int*>(s_tmem + 2));
  float* s_red = reinterpret_cast<float*>(s_tmem + 4);             // [2][256]
  float* s_sc = s_red + 512;                                       // [4 tiles][scale, log2 scale, 1 / scale][128 keys]
  int32_t* s_bt = reinterpret_cast<int32_t*>(s_sc + 4 * 3 * 128);  // [kPMaxPages]
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0 = even CTA (issues the MMAs), 1 = its peer
  const fa_decode_item it = p.items[blockIdx.x >> 1];
  const int b = it.b;
  const int rt = blockIdx.y;
  const int tile_m0 = rt * 128;                            // first row of the pair's 128-row tile
  const int tile_rows = min(128, p.M - tile_m0);
  const int m0 = tile_m0 + 64 * (int)rank;                 // first row of this CTA
  const int rows_valid = max(0, min(64, p.M - m0));
  const int qoff = p.q_offsets ? p.q_offsets[b] : p.q_offset;
  const int k_begin = it.k_begin;
  int k_end = it.k_end;
  // rows are m = h * N_q + i_q; a row may attend keys <= i_q + q_offset.  Both CTAs must agree on the
  // number of tiles, so the bound is taken over the pair's rows.
  int iq_max = 0, iq_min = 0;
  if (p.causal) {
    const int last = tile_m0 + tile_rows - 1;
    iq_max = (last / p.N_q > tile_m0 / p.N_q) ? p.N_q - 1 : last % p.N_q;
    iq_min = (last / p.N_q > tile_m0 / p.N_q) ? 0 : tile_m0 % p.N_q;
    k_end = min(k_end, max(iq_max + qoff, -1) + 1);
  }
  const int n_keys = max(k_end - k_begin, 0);
  const int n_tiles = (n_keys + 127) / 128;
  const bool ragged_end = (n_keys & 127) != 0;             // the last tile has value rows past the sequence

  if (threadIdx.x == 0) {
    *s_abort = 0;
    mbar_init(bar(QT_READY), 2 * kFSoft);
    for (int i = 0; i < kFTiles; ++i) {
      mbar_init(bar(X_FULL + i), 1);
      mbar_init(bar(X_FULLB + i), 1);
      mbar_init(bar(R_FULL + i), 1);
      mbar_init(bar(T_FREEA + i), 1);
      mbar_init(bar(T_FREE + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(P_READY + i), 2 * kFSoft);
    }
    for (int i = 0; i < 4; ++i) mbar_init(bar(SC_READY + i), 32);     // this CTA's scale loader warp
    mbar_init(bar(Z_GO), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_l);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(s_tmem)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  // block-table slice of this key range (every 64-key half lies inside one page)
  const int pg0 = k_begin >> p.page_shift;
  if (n_keys > 0) {
    const int pg1 = (k_end - 1) >> p.page_shift;
    const int32_t* bt = p.block_table + (int64_t)b * p.n_logical;
    for (int i = threadIdx.x; i <= pg1 - pg0 && i < kPMaxPages; i += kFThreads) {
      int pid = (pg0 + i < p.n_logical) ? bt[pg0 + i] : -2;
      if ((unsigned)pid >= (unsigned)p.num_blocks) {
        if (p.status) atomicOr(p.status, FA_STATUS_BAD_BLOCK_TABLE);
        pid = 0;                     // never follow a bad entry: read block 0 instead and flag it
      }
      s_bt[i] = pid;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // barriers of both CTAs are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tm_o = tmem, tm_s = tmem + 256, tm_q = tmem + 384;     // S of tile j at tm_s + 64 (j & 1)
  const int64_t qrow0 = (int64_t)b * p.M + m0;           // first query row of this CTA in the [B*M, 576] view
  // token row of a key in the pool view; keys past the range read the zero fill beyond the tensor
  auto token_of = [&](int key) {
    if (key >= k_end) return p.total_tokens;
    const int pg = key >> p.page_shift;
    return s_bt[pg - pg0] * p.page_size + (key - (pg << p.page_shift));
  };
  // box x of the five blocks of a tile
  auto block_x = [](int d) { return d < 4 ? 128 * d : kPDQK - 128; };

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      // ------------------------------------------------- TMA producer of the score operand (both CTAs)
      // tile j -> buffer j % 3.  Blocks 0, 1 are released by the first half of the P V of the tile that used
      // the buffer, the others by the second half; the scores start on blocks 0, 1.
      for (int j = 0; j < n_tiles; ++j) {
        const int bf = j % kFTiles, use = j / kFTiles;           // tile buffer and how often it has been used
        const int tok_own = token_of(k_begin + j * 128 + 64 * (int)rank);
        if (j >= kFTiles && !mbar_wait(bar(T_FREEA + bf), (use - 1) & 1, s_abort, p.status, P2_ERR_X_EMPTY)) break;
        const uint32_t xa_full0 = map_to_cta(bar(X_FULL + bf), 0), xb_full0 = map_to_cta(bar(X_FULLB + bf), 0);
        if (rank == 0) mbar_expect_tx(bar(X_FULL + bf), 2 * 2 * kPBlk);
        for (int d = 0; d < 2; ++d) tma_pair_2d(smem_u32(sT + (bf * kFBlocks + d) * kPBlk), &map_l, block_x(d), tok_own, xa_full0);
        if (j >= kFTiles && !mbar_wait(bar(T_FREE + bf), (use - 1) & 1, s_abort, p.status, P2_ERR_X_EMPTY)) break;
        if (rank == 0) mbar_expect_tx(bar(X_FULLB + bf), 2 * 3 * kPBlk);
        for (int d = 2; d < kFBlocks; ++d) tma_pair_2d(smem_u32(sT + (bf * kFBlocks + d) * kPBlk), &map_l, block_x(d), tok_own, xb_full0);
        // pull the first tile that has no buffer yet into L2
        if (j + kFTiles < n_tiles) {
          const int tok_pf = token_of(k_begin + (j + kFTiles) * 128 + 64 * (int)rank);
          if (tok_pf < p.total_tokens)
            for (int d = 0; d < kFBlocks; ++d) tma_prefetch_l2_2d(&map_l, block_x(d), tok_pf);
        }
      }
    }
  } else if (warp == 2) {
    if (n_tiles > 0) {
      // ------------------------------------------------- TMA producer of the peer's keys, token scales
      // Once the scores of tile j are done, the two blocks of the other CTA's value columns are dead here:
      // they are overwritten by this CTA's value columns of the peer's 64 keys, which puts the value
      // operand of key half h at the same offsets in both CTAs (lane 0).
      // The whole warp then leaves the scales of tile j + 1 in shared memory: for each of its 128 keys (both
      // CTAs' keys: a softmax thread works on one key half of the whole tile) the scale, its logarithm and
      // its reciprocal, in buffer (j + 1) & 3, whose last reader (tile j - 3) finished before the scores of
      // tile j - 1 could start.  A tile's scales are requested from global memory two steps before they are
      // written and nothing touches the registers in between (`odd` / `even`: the tiles of that parity).
      auto fetch_scales = [&](int j, float (&raw)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = k_begin + j * 128 + lane + 32 * i;
          const int tok = (j < n_tiles && key < k_end) ? token_of(key) : 0;
          raw[i] = p.tok_scale ? __ldg(p.tok_scale + tok) : 1.f;
        }
      };
      // A zero scale (an all-zero token) keeps a finite logarithm; its weight still counts in the denominator.
      auto put_scales = [&](int j, const float (&raw)[4]) {
        float* dst = s_sc + (j & 3) * 3 * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool in = k_begin + j * 128 + lane + 32 * i < k_end;
          const float sc = raw[i] * p.tensor_scale;
          const float s_eff = fmaxf(sc, 1e-30f);
          dst[lane + 32 * i] = in ? sc : 0.f;
          dst[128 + lane + 32 * i] = in ? __log2f(s_eff) : 0.f;
          dst[256 + lane + 32 * i] = in ? __frcp_rn(s_eff) : 0.f;
        }
        mbar_arrive(bar(SC_READY + (j & 3)));
      };
      auto tile_step = [&](int j, float (&nxt)[4]) -> bool {        // nxt: the scales of tile j + 1
        const int bf = j % kFTiles;
        bool ok = true;
        if (lane == 0) {
          ok = mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, s_abort, p.status, P2_ERR_S_FULL);
          if (ok) {
            const uint32_t r_full0 = map_to_cta(bar(R_FULL + bf), 0);
            if (rank == 0) mbar_expect_tx(bar(R_FULL + bf), 2 * 2 * kPBlk);
            const int tok_peer = token_of(k_begin + j * 128 + 64 * (1 - (int)rank));
            for (int s = 0; s < 2; ++s)
              tma_pair_2d(smem_u32(sT + (bf * kFBlocks + 2 * s + (1 - (int)rank)) * kPBlk), &map_l, 256 * s + 128 * (int)rank, tok_peer, r_full0);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        if (j + 1 < n_tiles) {
          put_scales(j + 1, nxt);
          fetch_scales(j + 3, nxt);
        }
        return true;
      };
      float even[4], odd[4];
      fetch_scales(0, even);
      fetch_scales(1, odd);
      put_scales(0, even);
      fetch_scales(2, even);
      for (int j = 0; j < n_tiles; j += 2) {
        if (!tile_step(j, odd)) break;
        if (j + 1 < n_tiles && !tile_step(j + 1, even)) break;
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && n_tiles > 0) {
      // the whole warp walks the control flow (uniform arithmetic); one elected lane executes the tcgen05 instructions
      const bool lead = elect_one();
      // ------------------------------------------------- score MMA issuer (even CTA, for the pair)
      // Two issuing threads (this one and warp 3) keep the tensor pipe fed across batch boundaries.  Scores
      // run at most two tiles ahead of the P V: tile j reuses the score buffer of tile j - 2, free once P of
      // j - 2 is out.  The 18 steps of 32 dims: step t < 16 in block t / 4 at byte 32 (t % 4); the rope dims
      // (steps 16, 17) in the upper half of block 4.
      constexpr uint32_t idesc_qk = idesc_f16(128, 128, false, false, false);    // format 0 of kind::f8f6f4 = E4M3
      bool ok = mbar_wait(bar(QT_READY), 0, s_abort, p.status, P2_ERR_QT);
      auto step_off = [](int t) { return t < 16 ? (t >> 2) * kPBlk + (t & 3) * 32 : 4 * kPBlk + 64 + (t - 16) * 32; };
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16);
      const uint32_t qr_lo = desc_lo(smem_u32(sQr), 16) - ((4 * kPBlk) >> 4);   // so that step_off(16), step_off(17) land in sQr
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int sb = j & 1, tb = j % kFTiles, use = j / kFTiles;   // score buffer; tile buffer and its use count
        if (j >= 2) ok = mbar_wait(bar(P_READY + sb), ((j >> 1) - 1) & 1, s_abort, p.status, P2_ERR_P_READY);
        if (ok) ok = mbar_wait(bar(X_FULL + tb), use & 1, s_abort, p.status, P2_ERR_X_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_lo = desc_lo(smem_u32(sT + tb * kFBlocks * kPBlk), 16), d_s = tm_s + 64 * sb;
        if (lead) {
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            mma2_f8_ts_w(d_s, tm_q + 8 * t, t_lo + (step_off(t) >> 4), idesc_qk, t > 0 ? 1u : 0u);
            mma2_f8_w(d_s, q_lo + (step_off(t) >> 4), t_lo + (step_off(t) >> 4), idesc_qk, 1u);
          }
        }
        ok = mbar_wait(bar(X_FULLB + tb), use & 1, s_abort, p.status, P2_ERR_X_FULL);
        if (!ok) break;
        tc_fence_after();
        if (lead) {
#pragma unroll
          for (int t = 8; t < 18; ++t) {
            if (t < 16)
              mma2_f8_ts_w(d_s, tm_q + 8 * t, t_lo + (step_off(t) >> 4), idesc_qk, 1u);
            else
              mma2_f8_w(d_s, qr_lo + (step_off(t) >> 4), t_lo + (step_off(t) >> 4), idesc_qk, 1u);
            mma2_f8_w(d_s, q_lo + (step_off(t) >> 4), t_lo + (step_off(t) >> 4), idesc_qk, 1u);
          }
          mma2_commit_both(bar(S_FULL + sb));
        }
      }
    }
  } else if (warp == 3) {
    if (rank == 0 && n_tiles > 0) {
      // the whole warp walks the control flow (uniform arithmetic); one elected lane executes the tcgen05 instructions
      const bool lead = elect_one();
      // ------------------------------------------------- P V MMA issuer (even CTA, for the pair)
      // Per value segment s: key half h, 32-key step kk, piece pc.  A = P piece (row-major over the 128 keys of
      // the tile), B = value block 2 s + h (keys down, 128 columns across: the transposed, MN-major form).
      constexpr uint32_t idesc_pv = idesc_f16(128, 256, false, false, true);
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int sb = j & 1, tb = j % kFTiles, use = j / kFTiles;
        ok = mbar_wait(bar(R_FULL + tb), use & 1, s_abort, p.status, P2_ERR_Y_FULL);
        if (!ok) break;
        if (lead && ragged_end && j + 1 == n_tiles) {
          // everything of the last tile has landed in both CTAs: let the softmax threads clear the value
          // rows past the end of the sequence
          mbar_arrive(bar(Z_GO));
          mbar_arrive_cluster(map_to_cta(bar(Z_GO), 1));
        }
        ok = mbar_wait(bar(P_READY + sb), (j >> 1) & 1, s_abort, p.status, P2_ERR_P_READY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_lo = desc_lo(smem_u32(sT + tb * kFBlocks * kPBlk), kPBlk), p_lo = desc_lo(smem_u32(sP + sb * 2 * kPBlk), 16);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (lead) {
#pragma unroll
            for (int hk = 0; hk < 4; ++hk) {
              const int h = hk >> 1, kk = hk & 1;
#pragma unroll
              for (int pc = 0; pc < 2; ++pc)
                mma2_f8_w(tm_o + 128 * s, p_lo + ((pc * kPBlk + hk * 32) >> 4), v_lo + (((2 * s + h) * kPBlk + kk * 4096) >> 4), idesc_pv,
                          (j > 0 || hk > 0 || pc > 0) ? 1u : 0u);
            }
            mma2_commit_both(bar((s == 0 ? T_FREEA : T_FREE) + tb));
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ query split / softmax / epilogue
    // Two warpgroups: a warp reaches the TMEM lanes 32 (warp % 4) .. + 31, so warps 4..7 and 8..11 each see
    // all 128 lanes, and warpgroup hh takes the score columns [32 hh, 32 hh + 32) of its lane.  Four threads
    // share a row: (key half g = lane half, hh); they meet through shared memory for the row maximum.
    const int quad = warp & 3;
    const int hh = (warp - 4) >> 2;                   // warpgroup: which 32 of the lane's 64 score columns
    const int L = quad * 32 + lane;                   // TMEM lane of this thread
    const int row = L & 63;                           // row of this CTA
    const int g = L >> 6;                             // key half (scores) / column half (output)
    const int part = 2 * g + hh;                      // which 32 keys of a tile's 128: [32 part, 32 part + 32)
    const int tid_sm = hh * 128 + L;                  // index among the 256 softmax threads
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const bool row_ok = row < rows_valid;
    const int m = m0 + row;
    const int iq = m % p.N_q;
    const int limit = min(p.causal ? iq + qoff : INT_MAX, k_end - 1);    // largest key this row may attend
    const int tile_limit = min(p.causal ? iq_min + qoff : INT_MAX, k_end - 1);
    float m_ref = -INFINITY, l_run = 0.f;
    float c_row = 0.f;                                // softmax scale (log2 units) over the row's power of two
    bool ok = true;
    // the values of the row's four threads, in a fixed order so that all four compute the same result
    auto row_max4 = [&](const float* red) {
      return fmaxf(fmaxf(red[row], red[64 + row]), fmaxf(red[128 + row], red[192 + row]));
    };
    if (n_tiles > 0) {
      // This thread's quarter of its query row (dims [144 part, + 144), fp16 in global memory): the row's
      // largest magnitude, then the two E4M3 pieces of every element times 2^e, written as 16-byte chunks of
      // the swizzled operand blocks.  Padding rows are zeros.
      const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + (qrow0 + row) * kPDQK + 144 * part);
      float amax = 0.f;
      if (row_ok) {
#pragma unroll 6
        for (int i = 0; i < 18; ++i) {
          const uint4 v = __ldg(qsrc + i);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
        }
      }
      s_red[64 * part + row] = amax;
      softmax_bar256();
      amax = row_max4(s_red);
      // 2^e with amax * 2^e in [128, 256); rows of zeros (and anything not a normal number) keep e = 0
      int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
      if (!(amax >= 1e-30f && amax <= 65504.f)) ex = 7;
      const float up = __uint_as_float((uint32_t)(7 - ex + 127) << 23);
      c_row = p.scale_log2 * __uint_as_float((uint32_t)(ex - 7 + 127) << 23);
#pragma unroll 3
      for (int c = 0; c < 9; ++c) {
        float x[16];
        const uint4 v0 = row_ok ? __ldg(qsrc + 2 * c) : make_uint4(0, 0, 0, 0);
        const uint4 v1 = row_ok ? __ldg(qsrc + 2 * c + 1) : make_uint4(0, 0, 0, 0);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
          x[2 * e] = f.x * up, x[2 * e + 1] = f.y * up;
        }
        uint4 q1, q2;
        split16(x, q1, q2);
        const int d0 = 144 * part + 16 * c;           // first dim of the chunk
        const int blk = d0 < 512 ? d0 >> 7 : 4, ch = d0 < 512 ? (d0 & 127) >> 4 : 4 + ((d0 - 512) >> 4);
        const int off = row * 128 + ((ch ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(sQ + blk * kPBlk + off) = q2;
        if (blk == 4) *reinterpret_cast<uint4*>(sQr + off) = q1;       // the other first pieces go to tensor memory
      }
      // The first pieces of dims [0, 512) are read by the tensor core from tensor memory (half the shared-memory
      // traffic of those steps): four dims per 32-bit column, the 64 rows in both lane halves.  This thread
      // fills columns [64 hh, 64 hh + 64) of its lane with dims [256 hh, 256 hh + 256) of its row; the bytes
      // are the ones the loop above computed for shared memory (same inputs, same operations).
      {
        const uint4* qrow = reinterpret_cast<const uint4*>(p.q + (qrow0 + row) * kPDQK + 256 * hh);
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint4 v = row_ok ? __ldg(qrow + 16 * c2 + i) : make_uint4(0, 0, 0, 0);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
              e[k] = f2_to_e4m3x2(f2.x * up, f2.y * up);
            }
            r[2 * i] = e[0] | (e[1] << 16), r[2 * i + 1] = e[2] | (e[3] << 16);
          }
          tmem_st32u(tm_q + lane_base + 64 * hh + 32 * c2, r);
        }
        tmem_wait_st();
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_peer(map_to_cta(bar(QT_READY), 0));
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int bf = j & 1;
      // the scales of this thread's 32 keys were left in shared memory while the previous tile's scores ran:
      // they are in registers (times the row's constant) before the scores arrive
      ok = mbar_wait(bar(SC_READY + (j & 3)), (j >> 2) & 1, s_abort, p.status, P2_ERR_SCALES);
      if (!ok) break;
      const float* tsc = s_sc + (j & 3) * 3 * 128 + 32 * part;
      float ka[32], lg[32];
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(tsc + c);
        const float4 l4 = *reinterpret_cast<const float4*>(tsc + 128 + c);
        ka[c] = a4.x * c_row, ka[c + 1] = a4.y * c_row, ka[c + 2] = a4.z * c_row, ka[c + 3] = a4.w * c_row;
        lg[c] = l4.x, lg[c + 1] = l4.y, lg[c + 2] = l4.z, lg[c + 3] = l4.w;
      }
      ok = mbar_wait(bar(S_FULL + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_S_FULL);
      if (!ok) break;
      tc_fence_after();
      float s[32];
      tmem_ld32(tm_s + 64 * bf + lane_base + 32 * hh, s);
      tmem_wait_ld();
      // t_k = score_k (log2 units) + log2 s_k
#pragma unroll
      for (int c = 0; c < 32; ++c) s[c] = fmaf(s[c], ka[c], lg[c]);
      const int k0 = k_begin + j * 128;
      const int k0p = k0 + 32 * part;
      if (k0 + 127 > tile_limit) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (k0p + c > limit) s[c] = -INFINITY;
      }
      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        mxa = fmaxf(mxa, s[c]);
        mxb = fmaxf(mxb, s[c + 1]);
      }
      float* red = s_red + (j & 1) * 256;
      red[64 * part + row] = fmaxf(mxa, mxb);
      softmax_bar256();
      const float mx = row_max4(red);
      const bool raise = (mx > m_ref + kFThreshold) || (m_ref == -INFINITY && mx > -INFINITY);
      float alpha = 1.f;
      if (raise) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = ((m_ref == -INFINITY) ? 0.f : m_ref) - kFPre;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const float4 iv = *reinterpret_cast<const float4*>(tsc + 256 + c);
        s[c] = fast_exp2(s[c] - m_use), s[c + 1] = fast_exp2(s[c + 1] - m_use);
        s[c + 2] = fast_exp2(s[c + 2] - m_use), s[c + 3] = fast_exp2(s[c + 3] - m_use);
        sum0 = fmaf(s[c], iv.x, sum0), sum1 = fmaf(s[c + 1], iv.y, sum1);
        sum0 = fmaf(s[c + 2], iv.z, sum0), sum1 = fmaf(s[c + 3], iv.w, sum1);
      }
      l_run = l_run * alpha + (sum0 + sum1);
      // O may only be rescaled between two P V: this tile's is not issued before P arrives, the previous
      // one has to be waited for (rare after the first tiles).  Each warpgroup rescales half of the columns.
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        ok = mbar_wait(bar(T_FREE + ((j - 1) % kFTiles)), ((j - 1) / kFTiles) & 1, s_abort, p.status, P2_ERR_PV_DONE);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float o[32];
          tmem_ld32(tm_o + lane_base + (4 * hh + c) * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st32(tm_o + lane_base + (4 * hh + c) * 32, o);
        }
        tmem_wait_st();
      }
      // the P buffer of tile j - 2 has been read once its P V is done (with three tile buffers the scores of
      // tile j no longer wait for that)
      if (j >= 2) {
        ok = mbar_wait(bar(T_FREE + ((j - 2) % kFTiles)), ((j - 2) / kFTiles) & 1, s_abort, p.status, P2_ERR_PV_DONE);
        if (!ok) break;
      }
      // this thread's 32 weights -> bytes [32 part, + 32) of row `row` of the two P pieces (16-byte chunks
      // swizzled by the row)
      {
        uint8_t* prow = sP + bf * 2 * kPBlk + row * 128;
#pragma unroll
        for (int c16 = 0; c16 < 2; ++c16) {
          uint4 q1, q2;
          split16(&s[16 * c16], q1, q2);
          const int off = ((2 * part + c16) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(prow + off) = q1;
          *reinterpret_cast<uint4*>(prow + kPBlk + off) = q2;
        }
      }
      // value rows past the end of the sequence may hold anything (E4M3 has NaN bytes): zero them so that
      // 0 * x stays 0.  Value block d holds keys of half d & 1 in both CTAs once the peer's keys are in.
      if (ragged_end && j + 1 == n_tiles) {
        ok = mbar_wait(bar(Z_GO), 0, s_abort, p.status, P2_ERR_Y_FULL);
        if (!ok) break;
        const int blk = tid_sm >> 6;                   // 4 value blocks, 64 threads each
        const int kr = tid_sm & 63;
        if (k0 + 64 * (blk & 1) + kr >= k_end) {
          uint4* d = reinterpret_cast<uint4*>(sT + ((j % kFTiles) * kFBlocks + blk) * kPBlk + kr * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] = make_uint4(0, 0, 0, 0);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_peer(map_to_cta(bar(P_READY + bf), 0));
    }
    if (ok && n_tiles > 0)
      ok = mbar_wait(bar(T_FREE + ((n_tiles - 1) % kFTiles)), ((n_tiles - 1) / kFTiles) & 1, s_abort, p.status, P2_ERR_PV_DONE);
    // the four threads of a row add up their sums (the tile loop's last use of this half of s_red is two tiles back)
    float* red = s_red + (n_tiles & 1) * 256;
    red[64 * part + row] = l_run;
    softmax_bar256();
    const float l_tot = (red[row] + red[64 + row]) + (red[128 + row] + red[192 + row]);
    if (ok) {
      tc_fence_after();
      const bool single = (it.n_split == 1);
      // numerator and denominator both carry the factor 2^kFPre
      const float inv = (l_tot > 0.f) ? p.scale_l / l_tot : 0.f;
      const float lse = (l_tot > 0.f) ? (m_ref - kFPre + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      const int h = m / p.N_q;
      const int64_t orow = ((int64_t)b * p.H_q + h) * p.N_q + iq;      // output is [B, H_q, N_q, DV]
      const int64_t prow = (int64_t)(it.slot_base + it.split) * p.M + m;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const int c = 4 * hh + c4;                                     // this warpgroup's half of the columns
        float o[32];
        if (n_tiles > 0) {
          tmem_ld32(tm_o + lane_base + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0.f;
        }
        if (!row_ok) continue;
        const int dd = 256 * (c >> 2) + 128 * g + 32 * (c & 3);       // value column of TMEM column 32 c in lane half g
        if (single) {
#pragma unroll
          for (int e = 0; e < 32; ++e) store_out_dyn(p.out, p.out_dtype, orow * kPDV + dd + e, o[e] * inv);
        } else {
          float4* dst = reinterpret_cast<float4*>(p.part_o + prow * kPDV + dd);
#pragma unroll
          for (int e = 0; e < 8; ++e) dst[e] = make_float4(o[4 * e] * inv, o[4 * e + 1] * inv, o[4 * e + 2] * inv, o[4 * e + 3] * inv);
        }
      }
      if (row_ok && part == 0) {
        if (single) { if (p.lse) p.lse[orow] = lse; }
        else p.part_lse[prow] = lse;
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // nothing of the pair touches the other CTA's barriers or TMEM after this
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
  }
  if (it.n_split == 1) return;
  merge_ranges(p, it, b, rt, (int)rank, m0, rows_valid, s_ticket, *s_abort != 0);
}

}  // namespace

// Host side: launched by launch_mla_pair (mla_pair.cu) for an E4M3 latent.
int launch_mla_pair_f8(const fa_mla_args* a, cudaStream_t st) {
  const int M = a->H_q * a->N_q;
  const int row_tiles = (M + 127) / 128;
  CUtensorMap tl;
  {
    // the pool as bytes: boxes of 64 tokens x 128 dims, 128-byte swizzle
    const uint64_t dims[2] = {(uint64_t)kPDQK, (uint64_t)a->num_blocks * a->page_size};
    const uint64_t strides[1] = {(uint64_t)kPDQK};
    const uint32_t box[2] = {128, 64};
    int rc = encode_tensor_map(&tl, FA_E4M3, 2, const_cast<void*>(a->l_pool), dims, strides, box, 1);
    if (rc) return rc;
  }
  MlaPairParams p{};
  p.q = reinterpret_cast<const uint16_t*>(a->q);
  p.block_table = a->block_table;
  p.q_offsets = a->q_offsets;
  p.items = a->items;
  p.out = a->out;
  p.lse = a->lse;
  p.part_o = reinterpret_cast<float*>(a->workspace);
  p.part_lse = p.part_o + (size_t)a->n_slots * M * kPDV;
  p.status = a->counters;          // word 0: sticky error flags; the arrival counters follow
  p.counters = a->counters + 1;
  // the scales of the latent (per token, or the tensor's) are applied key by key in the softmax threads
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.scale_l = 1.f;
  p.n_logical = a->n_logical;
  p.num_blocks = a->num_blocks;
  p.page_size = a->page_size;
  p.page_shift = __builtin_ctz((unsigned)a->page_size);
  p.total_tokens = a->num_blocks * a->page_size;
  p.B = a->B; p.H_q = a->H_q; p.N_q = a->N_q; p.M = M; p.n_slots = a->n_slots;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  p.tok_scale = a->l_token_scale;
  p.tensor_scale = a->l_scale;
  constexpr int SMEM = (kFBlocks + 1 + 4 + kFTiles * kFBlocks) * kPBlk + 12288 + 1024;
  static_assert(SMEM <= 227 * 1024, "MLA FP8 pair tile does not fit shared memory");
  static_assert(26 * 8 + 16 + 2048 + 4 * 3 * 128 * 4 + kPMaxPages * 4 <= 12288, "barriers, scratch, token scales and block table exceed their 12 KB");
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(mla_pair_f8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured_device = dev;
  }
  dim3 grid(2u * (unsigned)a->n_items, (unsigned)row_tiles, 1u);
  mla_pair_f8_kernel<<<grid, kFThreads, SMEM, st>>>(tl, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa
