// MLA latent decode on a pair of CTAs (thread-block cluster of two, tcgen05 cta_group::2).
// bf16 latent, DQK = 576, DV = 512, page_size a power of two >= 64.
//
// One CTA cannot hold the 128 x 512 fp32 output of 128 heads next to a score tile (it is all of tensor
// memory), and cutting the value dimension over two independent CTAs makes both compute the scores.  A
// CTA pair avoids both: with cta_group::2 an M = 128 MMA gives each CTA 64 of the 128 rows, and its
// accumulator of N columns occupies N/2 TMEM columns (rows in lanes 0..63 hold columns [0, N/2), lanes
// 64..127 hold [N/2, N)).  Per CTA: O[64 x 512] = 256 columns, two S[64 x 128] of 64 columns, and 256 of
// the 576 query dims as the A operand in TMEM (128 columns, the 64 rows written to both lane halves).
//
// Per 128-key tile (both CTAs, one thread of the even CTA issues every MMA for the pair):
//   S = Q L^T    N = 128 keys: CTA r supplies the latent rows of keys [64 r, 64 r + 64) (nine 64-dim blocks)
//   softmax      thread (row, key half) = TMEM lane; the two halves of a row meet through shared memory;
//                lazy-rescaled running maximum; P (bf16) goes to shared memory as the next A operand
//   O += P L_v   per key half h and value segment s one N = 256 MMA group; CTA r supplies the value
//                columns [256 s + 128 r, +128) of the 64 keys of half h
// The descriptors of an MMA are the same numbers in both CTAs.  For its own keys a CTA finds its value
// columns inside the score operand; for the peer's keys it must hold them at the offsets where the peer
// holds its own -- which is where this CTA keeps the peer's value columns of its own keys, dead once the
// scores are done.  So after S of a tile those four blocks are overwritten (a second TMA producer) with
// this CTA's value columns of the peer's keys: 72 KB of shared memory and 104 KB of loads per tile,
// two tile buffers, two score buffers, two P buffers.  The MMA thread issues whatever is ready (P V
// first): scores run up to two tiles ahead of the oldest unfinished P V, so softmax overlaps the MMAs.
//
// Warps: 0 = TMA producer (own keys), 1 = TMEM owner (+ MMA issuer in the even CTA), 2..5 = softmax /
// epilogue, 6 = TMA producer (peer keys), 7 = second MMA issuer (P V) in the even CTA.
// Every wait is bounded (sm100.cuh); the only unbounded synchronisation is the cluster barrier, which
// both CTAs always reach.
//
// Reference behaviour: kernels/v11_mla/mla_attention.cu:104-258 (what is computed), and the intended
// tensor-core backend kernels/v12_mla_tc/mla_tc_attention.cu:94-139.

#include "mla_pair.cuh"

namespace fa {
namespace {

using namespace sm100;
using namespace pair;

constexpr int kPQT = 256;                     // query dims held in tensor memory
constexpr int kPQB = (kPDQK - kPQT) / 64;     // query blocks in shared memory

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
mla_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_l, const MlaPairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // [5 blocks][64 rows][64 cols]: query dims 256..575 of this CTA's rows
  uint8_t* sP = sQ + kPQB * kPBlk;             // [2 tiles][2 key halves][64 rows][64 keys]
  uint8_t* sT = sP + 4 * kPBlk;                // [2 tiles][9 dim blocks][64 keys][64 dims]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sT + 18 * kPBlk);
  enum { Q_FULL = 0, QT_READY = 1, X_FULL = 2, R_FULL = 4, S_FULL = 6, T_FREE = 8, P_READY = 10, Z_GO = 12, X_FULLB = 13, T_FREEA = 15, NBARS = 17 };
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ticket = const_cast<int*>(reinterpret_cast<volatile int*>(s_tmem + 2));
  float* s_red = reinterpret_cast<float*>(s_tmem + 4);             // [2][128]
  int32_t* s_bt = reinterpret_cast<int32_t*>(s_red + 256);         // [kPMaxPages]
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
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(QT_READY), 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(X_FULL + i), 1);
      mbar_init(bar(X_FULLB + i), 1);
      mbar_init(bar(T_FREEA + i), 1);
      mbar_init(bar(R_FULL + i), 1);
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(T_FREE + i), 1);
      mbar_init(bar(P_READY + i), 256);
    }
    mbar_init(bar(Z_GO), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
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
    for (int i = threadIdx.x; i <= pg1 - pg0 && i < kPMaxPages; i += kPThreads) {
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
  const uint32_t tm_o = tmem, tm_q = tmem + 256, tm_s = tmem + 384;     // S of tile j at tm_s + 64 (j & 1)
  const int64_t qrow0 = (int64_t)b * p.M + m0;          // first query row of this CTA in the [B*M, 576] view
  // token row of a key in the pool view; keys past the range read the zero fill beyond the tensor
  auto token_of = [&](int key) {
    if (key >= k_end) return p.total_tokens;
    const int pg = key >> p.page_shift;
    return s_bt[pg - pg0] * p.page_size + (key - (pg << p.page_shift));
  };

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      // ------------------------------------------------- TMA producer of the score operand (both CTAs)
      // tile j -> buffer j & 1: the nine 64-dim blocks of this CTA's own 64 keys
      const uint32_t q_full0 = map_to_cta(bar(Q_FULL), 0);
      if (rank == 0) mbar_expect_tx(bar(Q_FULL), 2 * kPQB * kPBlk);
      for (int kb = 0; kb < kPQB; ++kb) tma_pair_2d(smem_u32(sQ + kb * kPBlk), &map_q, kPQT + kb * 64, (int)qrow0, q_full0);
      for (int j = 0; j < n_tiles; ++j) {
        const int bf = j & 1;
        // blocks 0..3 are released by the first half of the P V of the tile that used this buffer, the rest
        // by the second half; the scores start on blocks 0..3
        const int tok_own = token_of(k_begin + j * 128 + 64 * (int)rank);
        if (j >= 2 && !mbar_wait(bar(T_FREEA + bf), ((j >> 1) - 1) & 1, s_abort, p.status, P2_ERR_X_EMPTY)) break;
        const uint32_t xa_full0 = map_to_cta(bar(X_FULL + bf), 0), xb_full0 = map_to_cta(bar(X_FULLB + bf), 0);
        if (rank == 0) mbar_expect_tx(bar(X_FULL + bf), 2 * 4 * kPBlk);
        for (int d = 0; d < 4; ++d) tma_pair_2d(smem_u32(sT + (bf * 9 + d) * kPBlk), &map_l, d * 64, tok_own, xa_full0);
        if (j >= 2 && !mbar_wait(bar(T_FREE + bf), ((j >> 1) - 1) & 1, s_abort, p.status, P2_ERR_X_EMPTY)) break;
        if (rank == 0) mbar_expect_tx(bar(X_FULLB + bf), 2 * 5 * kPBlk);
        for (int d = 4; d < 9; ++d) tma_pair_2d(smem_u32(sT + (bf * 9 + d) * kPBlk), &map_l, d * 64, tok_own, xb_full0);
        // pull the tile after the next one into L2 while there is no buffer for it yet
        if (j + 2 < n_tiles) {
          const int tok_pf = token_of(k_begin + (j + 2) * 128 + 64 * (int)rank);
          if (tok_pf < p.total_tokens)
            for (int d = 0; d < 9; ++d) tma_prefetch_l2_2d(&map_l, d * 64, tok_pf);
        }
      }
    }
  } else if (warp == 6) {
    if (lane == 0 && n_tiles > 0) {
      // ------------------------------------------------- TMA producer of the peer's keys (both CTAs)
      // Once the scores of tile j are done, the four blocks of the other CTA's value columns are dead
      // here: they are overwritten by this CTA's value columns of the peer's 64 keys, which puts the value
      // operand of key half h at the same offsets in both CTAs.
      for (int j = 0; j < n_tiles; ++j) {
        const int bf = j & 1;
        if (!mbar_wait(bar(S_FULL + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_S_FULL)) break;
        const uint32_t r_full0 = map_to_cta(bar(R_FULL + bf), 0);
        if (rank == 0) mbar_expect_tx(bar(R_FULL + bf), 2 * 4 * kPBlk);
        const int tok_peer = token_of(k_begin + j * 128 + 64 * (1 - (int)rank));
        for (int s = 0; s < 2; ++s)
          for (int i = 0; i < 2; ++i)
            tma_pair_2d(smem_u32(sT + (bf * 9 + 4 * s + 2 * (1 - (int)rank) + i) * kPBlk), &map_l, 64 * (4 * s + 2 * (int)rank + i), tok_peer,
                        r_full0);
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && n_tiles > 0) {
      // the whole warp walks the control flow (uniform arithmetic); one elected lane executes the tcgen05 instructions
      const bool lead = elect_one();
      // ------------------------------------------------- score MMA issuer (even CTA, for the pair)
      // Two issuing threads (this one and warp 7) keep the tensor pipe fed across batch boundaries: while
      // one is blocked behind its own batch the other has the next one queued.  Scores run at most two
      // tiles ahead of the P V: tile j reuses the score buffer of tile j - 2, free once P of j - 2 is out.
      constexpr uint32_t idesc_qk = idesc_f16(128, 128, true, false, false);
      bool ok = mbar_wait(bar(Q_FULL), 0, s_abort, p.status, P2_ERR_Q) && mbar_wait(bar(QT_READY), 0, s_abort, p.status, P2_ERR_QT);
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int bf = j & 1;
        if (j >= 2) ok = mbar_wait(bar(P_READY + bf), ((j >> 1) - 1) & 1, s_abort, p.status, P2_ERR_P_READY);
        if (ok) ok = mbar_wait(bar(X_FULL + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_X_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_lo = desc_lo(smem_u32(sT + bf * 9 * kPBlk), 16), d_s = tm_s + 64 * bf;
        if (lead) {
#pragma unroll
          for (int k = 0; k < kPQT / 16; ++k)          // leading query dims from tensor memory
            mma2_ts_w(d_s, tm_q + k * 8, t_lo + (((k >> 2) * kPBlk + (k & 3) * 32) >> 4), idesc_qk, k > 0);
        }
        ok = mbar_wait(bar(X_FULLB + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_X_FULL);
        if (!ok) break;
        tc_fence_after();
        if (lead) {
#pragma unroll
          for (int k = kPQT / 16; k < kPDQK / 16; ++k) {   // the other query dims from shared memory
            const int kq = k - kPQT / 16;
            mma2_ss_w(d_s, q_lo + (((kq >> 2) * kPBlk + (kq & 3) * 32) >> 4), t_lo + (((k >> 2) * kPBlk + (k & 3) * 32) >> 4), idesc_qk, 1u);
          }
          mma2_commit_both(bar(S_FULL + bf));
        }
      }
    }
  } else if (warp == 7) {
    if (rank == 0 && n_tiles > 0) {
      // the whole warp walks the control flow (uniform arithmetic); one elected lane executes the tcgen05 instructions
      const bool lead = elect_one();
      // ------------------------------------------------- P V MMA issuer (even CTA, for the pair)
      constexpr uint32_t idesc_pv = idesc_f16(128, 256, true, false, true);
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int bf = j & 1;
        ok = mbar_wait(bar(R_FULL + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_Y_FULL);
        if (!ok) break;
        if (lead && ragged_end && j + 1 == n_tiles) {
          // everything of the last tile has landed in both CTAs: let the softmax threads clear the value
          // rows past the end of the sequence
          mbar_arrive(bar(Z_GO));
          mbar_arrive_cluster(map_to_cta(bar(Z_GO), 1));
        }
        ok = mbar_wait(bar(P_READY + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_P_READY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_lo = desc_lo(smem_u32(sT + bf * 9 * kPBlk), kPBlk), p_lo = desc_lo(smem_u32(sP + bf * 2 * kPBlk), 16);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (lead) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const int h = ks >> 2;
              mma2_ss_w(tm_o + 128 * s, p_lo + ((h * kPBlk + (ks & 3) * 32) >> 4),
                        v_lo + (((4 * s + 2 * h) * kPBlk + (ks & 3) * 2048) >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            }
            mma2_commit_both(bar((s == 0 ? T_FREEA : T_FREE) + bf));
          }
        }
      }
    }
  }
  else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quad = warp & 3;
    const int L = quad * 32 + lane;                   // TMEM lane of this thread
    const int row = L & 63;                           // row of this CTA
    const int g = L >> 6;                             // key half (scores) / column half (output)
    const int tid_sm = L;                             // index among the 128 softmax threads
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const bool row_ok = row < rows_valid;
    const int m = m0 + row;
    const int iq = m % p.N_q;
    const int limit = min(p.causal ? iq + qoff : INT_MAX, k_end - 1);    // largest key this row may attend
    const int tile_limit = min(p.causal ? iq_min + qoff : INT_MAX, k_end - 1);
    const uint32_t qt_ready0 = map_to_cta(bar(QT_READY), 0);
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    if (n_tiles > 0) {
      // leading query dims of this row -> tensor memory, two bf16 per column, the same row in both lane
      // halves (zero for padding rows)
      const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + (qrow0 + row) * kPDQK);
#pragma unroll
      for (int c = 0; c < kPQT / 64; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = row_ok ? qsrc[c * 8 + i] : make_uint4(0, 0, 0, 0);
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        tmem_st32u(tm_q + lane_base + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_peer(qt_ready0);
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int bf = j & 1;
      ok = mbar_wait(bar(S_FULL + bf), (j >> 1) & 1, s_abort, p.status, P2_ERR_S_FULL);
      if (!ok) break;
      tc_fence_after();
      float s[64];
      tmem_ld32(tm_s + 64 * bf + lane_base, *reinterpret_cast<float(*)[32]>(&s[0]));
      tmem_ld32(tm_s + 64 * bf + lane_base + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
      tmem_wait_ld();
      const int k0 = k_begin + j * 128;
      const int k0h = k0 + 64 * g;
      if (k0 + 127 > tile_limit) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (k0h + c > limit) s[c] = -INFINITY;
      }
      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        mxa = fmaxf(mxa, s[c]);
        mxb = fmaxf(mxb, s[c + 1]);
      }
      float* red = s_red + (j & 1) * 128;
      red[tid_sm] = fmaxf(mxa, mxb);
      softmax_bar();
      const float mx = fmaxf(red[tid_sm], red[tid_sm ^ 64]) * p.scale_log2;
      const bool raise = (mx > m_ref + kPThreshold) || (m_ref == -INFINITY && mx > -INFINITY);
      float alpha = 1.f;
      if (raise) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        s[c] = fast_exp2(fmaf(s[c], p.scale_log2, -m_use));
        s[c + 1] = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_use));
        sum0 += s[c];
        sum1 += s[c + 1];
      }
      l_run = l_run * alpha + (sum0 + sum1);
      // O may only be rescaled between two P V: this tile's is not issued before P arrives, the previous
      // one has to be waited for (rare: the maximum seldom rises by 2^8 after the first tiles)
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        ok = mbar_wait(bar(T_FREE + ((j - 1) & 1)), ((j - 1) >> 1) & 1, s_abort, p.status, P2_ERR_PV_DONE);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float o[32];
          tmem_ld32(tm_o + lane_base + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st32(tm_o + lane_base + c * 32, o);
        }
        tmem_wait_st();
      }
      // this thread's 64 probabilities -> row `row` of P block g (128 bytes, 16-byte chunks swizzled by row)
      {
        uint8_t* prow = sP + (bf * 2 + g) * kPBlk + row * 128;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          uint4 v;
          v.x = pack_bf2(s[8 * c16 + 0], s[8 * c16 + 1]);
          v.y = pack_bf2(s[8 * c16 + 2], s[8 * c16 + 3]);
          v.z = pack_bf2(s[8 * c16 + 4], s[8 * c16 + 5]);
          v.w = pack_bf2(s[8 * c16 + 6], s[8 * c16 + 7]);
          *reinterpret_cast<uint4*>(prow + ((c16 ^ (row & 7)) << 4)) = v;
        }
      }
      // value rows past the end of the sequence may hold anything: zero them so that 0 * x stays 0.
      // Block d of the tile holds keys of half (d >> 1) & 1 in both CTAs once the peer's keys are in.
      if (ragged_end && j + 1 == n_tiles) {
        ok = mbar_wait(bar(Z_GO), 0, s_abort, p.status, P2_ERR_Y_FULL);
        if (!ok) break;
        const int blk = tid_sm >> 4;                   // 8 value blocks, 16 threads each
        const int h = (blk >> 1) & 1;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int kr = (tid_sm & 15) + 16 * q4;
          if (k0 + 64 * h + kr >= k_end) {
            uint4* d = reinterpret_cast<uint4*>(sT + (bf * 9 + blk) * kPBlk + kr * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) d[i] = make_uint4(0, 0, 0, 0);
          }
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_peer(map_to_cta(bar(P_READY + bf), 0));
    }
    if (ok && n_tiles > 0)
      ok = mbar_wait(bar(T_FREE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, s_abort, p.status, P2_ERR_PV_DONE);
    // the two key halves of a row add up their sums
    s_red[tid_sm] = l_run;
    softmax_bar();
    const float l_tot = l_run + s_red[tid_sm ^ 64];
    if (ok) {
      tc_fence_after();
      const bool single = (it.n_split == 1);
      const float inv = (l_tot > 0.f) ? p.scale_l / l_tot : 0.f;
      const float lse = (l_tot > 0.f) ? (m_ref + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      const int h = m / p.N_q;
      const int64_t orow = ((int64_t)b * p.H_q + h) * p.N_q + iq;      // output is [B, H_q, N_q, DV]
      const int64_t prow = (int64_t)(it.slot_base + it.split) * p.M + m;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
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
      if (row_ok && g == 0) {
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

// Host side; called by fa_mla_decode_fwd (mla.cu) after validation when the tensor-core path applies.
int mla_pair_max_pages() { return kPMaxPages; }

int launch_mla_pair_f8(const fa_mla_args* a, cudaStream_t st);   // mla_pair_f8.cu

bool mla_pair_applicable(const fa_mla_args* a) {
  if ((a->latent_dtype != FA_BF16 && a->latent_dtype != FA_E4M3) || a->DQK != kPDQK || a->DV != kPDV) return false;
  // the E4M3 pool is read by TMA as rows of 576 bytes; with fewer than 64 head rows the MMA tile would be mostly
  // padding and the mma.sync kernel, which reads the bytes in place as well, is the better one
  if (a->latent_dtype == FA_E4M3 &&
      (a->q_dtype != FA_F16 || reinterpret_cast<uintptr_t>(a->l_pool) % 16 != 0 || a->H_q * a->N_q < 64)) return false;
  if (a->page_size % 64 != 0 || (a->page_size & (a->page_size - 1)) != 0) return false;
  if (a->max_range_keys / a->page_size + 2 > kPMaxPages) return false;
  if ((int64_t)a->B * a->H_q * a->N_q > INT_MAX || (int64_t)a->num_blocks * a->page_size > INT_MAX) return false;
  return true;
}

size_t mla_pair_workspace_bytes(int n_slots, int M) { return (size_t)n_slots * M * (kPDV + 2) * 4; }
size_t mla_pair_counters_len(int B, int M) { return (size_t)B * ((M + 127) / 128) * 2 + 1; }   // word 0: status

int launch_mla_pair(const fa_mla_args* a, cudaStream_t st) {
  if (a->latent_dtype == FA_E4M3) return launch_mla_pair_f8(a, st);
  const int M = a->H_q * a->N_q;
  const int row_tiles = (M + 127) / 128;
  CUtensorMap tq, tl;
  {
    const uint64_t dims[2] = {(uint64_t)kPDQK, (uint64_t)a->B * M};
    const uint64_t strides[1] = {(uint64_t)kPDQK * 2};
    const uint32_t box[2] = {64, 64};
    int rc = encode_tensor_map(&tq, FA_BF16, 2, const_cast<void*>(a->q), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)kPDQK, (uint64_t)a->num_blocks * a->page_size};
    const uint64_t strides[1] = {(uint64_t)kPDQK * 2};
    const uint32_t box[2] = {64, 64};
    int rc = encode_tensor_map(&tl, FA_BF16, 2, const_cast<void*>(a->l_pool), dims, strides, box, 1);
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
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f * a->l_scale;
  p.scale_l = a->l_scale;
  p.n_logical = a->n_logical;
  p.num_blocks = a->num_blocks;
  p.page_size = a->page_size;
  p.page_shift = __builtin_ctz((unsigned)a->page_size);
  p.total_tokens = a->num_blocks * a->page_size;
  p.B = a->B; p.H_q = a->H_q; p.N_q = a->N_q; p.M = M; p.n_slots = a->n_slots;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  constexpr int SMEM = (kPQB + 4 + 18) * kPBlk + 128 + 16 + 1024 + kPMaxPages * 4 + 1024;
  static_assert(SMEM <= 227 * 1024, "MLA pair tile does not fit shared memory");
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(mla_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured_device = dev;
  }
  dim3 grid(2u * (unsigned)a->n_items, (unsigned)row_tiles, 1u);
  mla_pair_kernel<<<grid, kPThreads, SMEM, st>>>(tq, tl, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa
