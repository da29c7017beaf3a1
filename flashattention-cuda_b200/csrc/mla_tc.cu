// MLA latent decode on tcgen05 tensor cores (bf16 latent, DQK = 576, DV = 512, page_size % 64 == 0).
//
// The 128 x 512 fp32 output of 128 heads would fill all 512 TMEM columns, so the value dimension is cut
// in two: CTA (range, dvh) accumulates O[:, dvh*256 : dvh*256+256] and both halves compute the scores.
// Per CTA, per 32-key latent tile (TMA, nine 64-column blocks, 128-byte swizzle, 4-stage ring: with one
// CTA per SM the loads of three tiles have to be in flight to cover the TMA latency):
//   S = Q L^T   M=128 heads, N=32 keys, K=576: the first 384 query dims live in tensor memory (A operand
//               from TMEM, so they cost no shared-memory bandwidth), the other 192 in shared memory
//   softmax     thread r owns head r: tcgen05.ld of its 32 scores, lazy-rescaled running maximum, P written
//               as packed bf16 over the S columns
//   O += P L_v  A = P from TMEM, B = the tile's value columns as an MN-major operand, N = 256
// TMEM columns: O [0,256)  S0 [256,288)  S1 [288,320)  Q [320,512).
// Warps: 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2..5 = softmax / epilogue (lane quadrant = warp % 4).
// Rows pack m = h * N_q + i_q so that a sequence's query rows are contiguous for the Q tensor map.
// Splits of a sequence are merged by the last CTA to arrive, per value half.
//
// Measured anatomy of one 32-key tile (clock64 trace of one CTA, 128 heads, 8000-key sequences): period
// 3040 cycles, of which the softmax warps spend 2340 waiting for the scores, 30 in tcgen05.ld, 520 computing
// and 40 in tcgen05.st; the MMA thread waits 145 cycles for P.  The tensor pipe sets the pace: the 36
// k-steps of Q L^T cost ~64 cycles each whatever N is (the 128 x 16 A operand is fetched per instruction),
// so time per key falls with wider key tiles, which shared memory (query + latent ring) does not allow
// in one CTA.  Moving query dims between TMEM and shared memory (FA_B200_MLA_QT) changes nothing.
//
// Reference behaviour: kernels/v11_mla/mla_attention.cu:104-258 (what is computed), and the intended
// tensor-core backend kernels/v12_mla_tc/mla_tc_attention.cu:94-139, which validates and then raises.

#include <climits>
#include <cstdlib>

#include "sm100.cuh"

namespace fa {
namespace {

using namespace sm100;

constexpr int kTcThreads = 192;
constexpr int kTcDQK = 576, kTcDV = 512, kTcDVH = 256;
constexpr int kTcKB = kTcDQK / 64;            // 9 column blocks per latent tile
constexpr int kTcQBlk = 128 * 128;            // bytes of one [128 rows][64 cols] block
constexpr int kTcMaxPages = 128;          // block-table entries staged per CTA (shared memory is nearly full)
constexpr float kTcThreshold = 8.f;

struct MlaTcParams {
  const uint16_t* q;
  const int32_t* block_table;
  const int32_t* q_offsets;
  const fa_decode_item* items;
  void* out;
  float* lse;
  float* part_o;     // [n_slots][rows][DV]
  float* part_lse;   // [2][n_slots][rows]
  int32_t* counters; // [B][row_tiles][2]
  int32_t* status;
  float scale_log2, scale_l;
  int n_logical, num_blocks, page_size, page_shift;
  int B, H_q, N_q, M, n_slots;
  int causal, q_offset, out_dtype;
};

enum { TC_ERR_Q = 31, TC_ERR_QT = 32, TC_ERR_KV_FULL = 33, TC_ERR_KV_EMPTY = 34, TC_ERR_S_FULL = 35, TC_ERR_P_READY = 36,
       TC_ERR_O_DONE = 37 };

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_st32r(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16r(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// QT: query dims held in tensor memory (0, 128, 256 or 384); the rest sits in shared memory, and what
// shared memory is left decides the depth of the latent ring.
template <int kTcQT, int kTcBN>
__global__ void __launch_bounds__(kTcThreads, 1)
mla_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_l, const MlaTcParams p) {
  constexpr int kTcQB = (kTcDQK - kTcQT) / 64;                              // query column blocks in shared memory
  constexpr int kTcLBlk = kTcBN * 128;                                      // bytes of one [BN keys][64 cols] block
  constexpr int kTcStage = kTcKB * kTcLBlk;
  // BN = 32: two score buffers, Q L^T of the next tile is issued before P V of the current one.
  // BN = 64: one score buffer and a strictly serial tile (Q L^T -> softmax -> P V); only two tiles fit in
  //          shared memory, and releasing a tile's stage before the next Q L^T starts is what lets the
  //          load of the tile after that overlap a whole tile of work.
  constexpr bool kSerial = (kTcBN == 64);
  constexpr int kTcStages = (226 * 1024 - kTcQB * kTcQBlk) / kTcStage > 4 ? 4 : (226 * 1024 - kTcQB * kTcQBlk) / kTcStage;
  static_assert(kTcStages >= 2, "latent ring needs two stages");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // [kTcQB blocks][128 rows][64 cols]: query dims 384..575
  uint8_t* sL = sQ + kTcQB * kTcQBlk;          // [4 stages][9 blocks][32 keys][64 cols]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sL + kTcStages * kTcStage);
  enum { Q_FULL = 0, QT_READY = 1, KV_FULL = 2, KV_EMPTY = 6, S_FULL = 10, P_READY = 12, O_DONE = 13, NBARS = 14 };   // room for 4 stages
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ticket = const_cast<int*>(reinterpret_cast<volatile int*>(s_tmem + 2));
  int32_t* s_bt = reinterpret_cast<int32_t*>(s_tmem + 4);          // [kTcMaxPages]
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const fa_decode_item it = p.items[blockIdx.x];
  const int b = it.b;
  const int dvh = blockIdx.y;
  const int rt = blockIdx.z;
  const int m0 = rt * 128;
  const int rows_valid = min(128, p.M - m0);
  const int qoff = p.q_offsets ? p.q_offsets[b] : p.q_offset;
  const int k_begin = it.k_begin;
  int k_end = it.k_end;
  // rows are m = h * N_q + i_q; a row may attend keys <= i_q + q_offset
  int iq_max = 0, iq_min = 0;
  if (p.causal) {
    const int last = m0 + rows_valid - 1;
    iq_max = (last / p.N_q > m0 / p.N_q) ? p.N_q - 1 : last % p.N_q;      // tile spans whole heads -> all i_q
    iq_min = (last / p.N_q > m0 / p.N_q) ? 0 : m0 % p.N_q;
    k_end = min(k_end, max(iq_max + qoff, -1) + 1);
  }
  const int n_keys = max(k_end - k_begin, 0);
  const int n_tiles = (n_keys + kTcBN - 1) / kTcBN;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(QT_READY), 128);
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(bar(KV_FULL + s), 1);
      mbar_init(bar(KV_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) mbar_init(bar(S_FULL + s), 1);
    mbar_init(bar(P_READY), 128);
    mbar_init(bar(O_DONE), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_l);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), 512);
    tmem_relinquish();
  }
  // block-table slice of this key range (every tile lies inside one page: page_size % 64 == 0, ranges start
  // on multiples of 64)
  const int pg0 = k_begin >> p.page_shift;
  if (n_keys > 0) {
    const int pg1 = (k_end - 1) >> p.page_shift;
    const int32_t* bt = p.block_table + (int64_t)b * p.n_logical;
    for (int i = threadIdx.x; i <= pg1 - pg0 && i < kTcMaxPages; i += kTcThreads) {
      int pid = (pg0 + i < p.n_logical) ? bt[pg0 + i] : -2;
      if ((unsigned)pid >= (unsigned)p.num_blocks) {
        if (p.status) atomicOr(p.status, 1);
        pid = 0;                     // never follow a bad entry: read block 0 instead and flag it
      }
      s_bt[i] = pid;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tm_o = tmem, tm_s = tmem + 256, tm_q = tmem + 320;
  (void)tm_q;
  const int64_t qrow0 = (int64_t)b * p.M + m0;          // first query row of this tile in the [B*M, 576] view

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      // ---------------------------------------------------------------- TMA producer
      if (kTcQB > 0) mbar_expect_tx(bar(Q_FULL), kTcQB * kTcQBlk);
      for (int kb = 0; kb < kTcQB; ++kb)
        tma_load_2d(smem_u32(sQ + kb * kTcQBlk), &map_q, kTcQT + kb * 64, (int)qrow0, bar(Q_FULL));
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kTcStages;
        if (j >= kTcStages && !mbar_wait(bar(KV_EMPTY + s), ((j / kTcStages) - 1) & 1, s_abort, p.status, TC_ERR_KV_EMPTY)) break;
        const int key = k_begin + j * kTcBN;
        const int pg = key >> p.page_shift;
        const int tok = s_bt[pg - pg0] * p.page_size + (key - (pg << p.page_shift));
        mbar_expect_tx(bar(KV_FULL + s), kTcStage);
        for (int kb = 0; kb < kTcKB; ++kb)
          tma_load_2d(smem_u32(sL + s * kTcStage + kb * kTcLBlk), &map_l, kb * 64, tok, bar(KV_FULL + s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = idesc_f16(128, kTcBN, true, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(128, kTcDVH, true, false, true);
      auto issue_qk = [&](int j) {
        const uint32_t l_base = smem_u32(sL + (j % kTcStages) * kTcStage);
        const uint32_t d = tm_s + (kSerial ? 0u : (uint32_t)(j & 1) * kTcBN);
#pragma unroll
        for (int k = 0; k < kTcQT / 16; ++k)         // query dims 0..383 from tensor memory
          mma_f16_ts(d, tm_q + k * 8, smem_desc_sw128(l_base + (k >> 2) * kTcLBlk + (k & 3) * 32, 16, 1024), idesc_qk, k > 0);
#pragma unroll
        for (int k = kTcQT / 16; k < kTcDQK / 16; ++k) {   // query dims 384..575 from shared memory
          const int kq = k - kTcQT / 16;
          mma_f16_ss(d, smem_desc_sw128(smem_u32(sQ) + (kq >> 2) * kTcQBlk + (kq & 3) * 32, 16, 1024),
                     smem_desc_sw128(l_base + (k >> 2) * kTcLBlk + (k & 3) * 32, 16, 1024), idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(S_FULL + (kSerial ? 0 : (j & 1))));
      };
      bool ok = (kTcQB == 0 || mbar_wait(bar(Q_FULL), 0, s_abort, p.status, TC_ERR_Q)) &&
                (kTcQT == 0 || mbar_wait(bar(QT_READY), 0, s_abort, p.status, TC_ERR_QT)) &&
                mbar_wait(bar(KV_FULL + 0), 0, s_abort, p.status, TC_ERR_KV_FULL);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        auto next_qk = [&]() {
          if (j + 1 < n_tiles) {
            ok = mbar_wait(bar(KV_FULL + ((j + 1) % kTcStages)), ((j + 1) / kTcStages) & 1, s_abort, p.status, TC_ERR_KV_FULL);
            if (!ok) return;
            tc_fence_after();
            issue_qk(j + 1);      // the score buffer last held P of an earlier tile whose P V was issued before: in order
          }
        };
        if (!kSerial) next_qk();
        if (!ok) break;
        ok = mbar_wait(bar(P_READY), j & 1, s_abort, p.status, TC_ERR_P_READY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sL + (j % kTcStages) * kTcStage) + (uint32_t)dvh * 4 * kTcLBlk;
        const uint32_t p_tmem = tm_s + (kSerial ? 0u : (uint32_t)(j & 1) * kTcBN);
#pragma unroll
        for (int k = 0; k < kTcBN / 16; ++k)
          mma_f16_ts(tm_o, p_tmem + k * 8, smem_desc_sw128(v_base + k * 2048, kTcLBlk, 1024), idesc_pv,
                     (j > 0 || k > 0) ? 1u : 0u);
        mma_commit(bar(KV_EMPTY + (j % kTcStages)));
        if (j + 1 == n_tiles) mma_commit(bar(O_DONE));
        if (kSerial) next_qk();
      }
    }
  }
  else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                 // head-row inside the tile
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const bool row_ok = row < rows_valid;
    const int m = m0 + row;
    const int iq = m % p.N_q;
    const int limit = min(p.causal ? iq + qoff : INT_MAX, k_end - 1);    // largest key this row may attend
    const int tile_limit = min(p.causal ? iq_min + qoff : INT_MAX, k_end - 1);
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    if (n_tiles > 0 && kTcQT > 0) {
      // leading query dims of this row -> tensor memory, two bf16 per column (zero for padding rows)
      const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + (qrow0 + row) * kTcDQK);
#pragma unroll
      for (int c = 0; c < kTcQT / 64; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = row_ok ? qsrc[c * 8 + i] : make_uint4(0, 0, 0, 0);
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        tmem_st32r(tm_q + lane_base + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(QT_READY));
    }
    for (int j = 0; j < n_tiles; ++j) {
      ok = kSerial ? mbar_wait(bar(S_FULL), j & 1, s_abort, p.status, TC_ERR_S_FULL)
                   : mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, s_abort, p.status, TC_ERR_S_FULL);
      if (!ok) break;
      tc_fence_after();
      float s[kTcBN];
      const uint32_t ts = tm_s + (kSerial ? 0u : (uint32_t)(j & 1) * kTcBN) + lane_base;
#pragma unroll
      for (int c = 0; c < kTcBN / 32; ++c) tmem_ld32(ts + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
      tmem_wait_ld();
      const int k0 = k_begin + j * kTcBN;
      if (k0 + kTcBN - 1 > tile_limit) {
#pragma unroll
        for (int c = 0; c < kTcBN; ++c)
          if (k0 + c > limit) s[c] = -INFINITY;
        // value rows past the end of the sequence may hold anything: zero them so that 0 * x stays 0
        if (k0 + kTcBN > k_end && row < kTcBN && k0 + row >= k_end) {
          uint8_t* base = sL + (j % kTcStages) * kTcStage + row * 128;
#pragma unroll
          for (int kb = 0; kb < kTcKB; ++kb) {
            uint4* d = reinterpret_cast<uint4*>(base + kb * kTcLBlk);
#pragma unroll
            for (int i = 0; i < 8; ++i) d[i] = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async();
        }
      }
      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int c = 0; c < kTcBN; c += 2) {
        mxa = fmaxf(mxa, s[c]);
        mxb = fmaxf(mxb, s[c + 1]);
      }
      const float mx = fmaxf(mxa, mxb) * p.scale_log2;
      const bool raise = (mx > m_ref + kTcThreshold) || (m_ref == -INFINITY && mx > -INFINITY);
      float alpha = 1.f;
      if (raise) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < kTcBN; c += 2) {
        s[c] = fast_exp2(fmaf(s[c], p.scale_log2, -m_use));
        s[c + 1] = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_use));
        sum0 += s[c];
        sum1 += s[c + 1];
      }
      l_run = l_run * alpha + (sum0 + sum1);
      // S_FULL of tile j was committed after the P V of tile j-1 was issued by the same thread, so O is quiet
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll
        for (int c = 0; c < kTcDVH / 32; ++c) {
          float o[32];
          tmem_ld32(tm_o + lane_base + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st32(tm_o + lane_base + c * 32, o);
        }
      }
      uint32_t pk[kTcBN / 2];
#pragma unroll
      for (int c = 0; c < kTcBN / 2; ++c) pk[c] = pack_bf2(s[2 * c], s[2 * c + 1]);
      if constexpr (kTcBN == 32) tmem_st16r(ts, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
      else tmem_st32r(ts, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
    }
    if (ok && n_tiles > 0) ok = mbar_wait(bar(O_DONE), 0, s_abort, p.status, TC_ERR_O_DONE);
    if (ok) {
      tc_fence_after();
      const bool single = (it.n_split == 1);
      const float inv = (l_run > 0.f) ? p.scale_l / l_run : 0.f;
      const float lse = (l_run > 0.f) ? (m_ref + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      const int h = m / p.N_q;
      const int64_t orow = ((int64_t)b * p.H_q + h) * p.N_q + iq;      // output is [B, H_q, N_q, DV]
      const int64_t prow = (int64_t)(it.slot_base + it.split) * p.M + m;
#pragma unroll
      for (int c = 0; c < kTcDVH / 32; ++c) {
        float o[32];
        if (n_tiles > 0) {
          tmem_ld32(tm_o + lane_base + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0.f;
        }
        if (!row_ok) continue;
        const int dd = dvh * kTcDVH + c * 32;
        if (single) {
#pragma unroll
          for (int e = 0; e < 32; ++e) store_out_dyn(p.out, p.out_dtype, orow * kTcDV + dd + e, o[e] * inv);
        } else {
          float4* dst = reinterpret_cast<float4*>(p.part_o + prow * kTcDV + dd);
#pragma unroll
          for (int e = 0; e < 8; ++e) dst[e] = make_float4(o[4 * e] * inv, o[4 * e + 1] * inv, o[4 * e + 2] * inv, o[4 * e + 3] * inv);
        }
      }
      if (row_ok) {
        if (single) { if (p.lse && dvh == 0) p.lse[orow] = lse; }
        else p.part_lse[((int64_t)dvh * p.n_slots + it.slot_base + it.split) * p.M + m] = lse;
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*s_abort) __nanosleep(200000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (it.n_split == 1 || *s_abort) return;

  // ---- the last CTA of this (sequence, row tile, value half) merges all key ranges ---------------------
  __threadfence();
  __syncthreads();
  const int cidx = (b * gridDim.z + rt) * 2 + dvh;
  if (threadIdx.x == 0) *s_ticket = atomicAdd(p.counters + cidx, 1);
  __syncthreads();
  if (*s_ticket != it.n_split - 1) return;
  __threadfence();
  if (threadIdx.x == 0) p.counters[cidx] = 0;
  const float* lse_base = p.part_lse + (int64_t)dvh * p.n_slots * p.M;
  for (int idx = threadIdx.x; idx < rows_valid * kTcDVH; idx += kTcThreads) {
    const int row = idx / kTcDVH, dd = dvh * kTcDVH + (idx - row * kTcDVH);
    const int m = m0 + row;
    float mstar = -INFINITY;
    for (int sidx = 0; sidx < it.n_split; ++sidx) mstar = fmaxf(mstar, __ldcg(lse_base + (int64_t)(it.slot_base + sidx) * p.M + m));
    const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
    float acc = 0.f, l = 0.f;
    for (int sidx = 0; sidx < it.n_split; ++sidx) {
      const int64_t prow = (int64_t)(it.slot_base + sidx) * p.M + m;
      const float wgt = __expf(__ldcg(lse_base + prow) - m_use);
      acc += wgt * __ldcg(p.part_o + prow * kTcDV + dd);
      l += wgt;
    }
    const int h = m / p.N_q, iq = m - h * p.N_q;
    const int64_t orow = ((int64_t)b * p.H_q + h) * p.N_q + iq;
    store_out_dyn(p.out, p.out_dtype, orow * kTcDV + dd, (l > 0.f) ? acc / l : 0.f);
    if (p.lse && dvh == 0 && dd == 0) p.lse[orow] = (l > 0.f) ? m_use + __logf(l) : -INFINITY;
  }
}

}  // namespace

// Host side; called by fa_mla_decode_fwd (mla.cu) after validation when the tensor-core path applies.
// `max_pages`: block-table entries the chosen kernel stages per CTA (0 = this file's kernel)
bool mla_tc_applicable(const fa_mla_args* a, int max_pages) {
  if (max_pages <= 0) max_pages = kTcMaxPages;
  if (a->latent_dtype != FA_BF16 || a->DQK != kTcDQK || a->DV != kTcDV) return false;
  if (a->page_size % 64 != 0 || (a->page_size & (a->page_size - 1)) != 0) return false;
  if (a->max_range_keys / a->page_size + 2 > max_pages) return false;
  if ((int64_t)a->B * a->H_q * a->N_q > INT_MAX || (int64_t)a->num_blocks * a->page_size > INT_MAX) return false;
  return true;
}

size_t mla_tc_workspace_bytes(int n_slots, int M) { return (size_t)n_slots * M * (kTcDV + 2) * 4; }
size_t mla_tc_counters_len(int B, int M) { return (size_t)B * ((M + 127) / 128) * 2 + 1; }

template <int QT, int BN>
static int launch_qt(const CUtensorMap& tq, const CUtensorMap& tl, const MlaTcParams& p, dim3 grid, cudaStream_t st) {
  constexpr int QB = (kTcDQK - QT) / 64;
  constexpr int STAGE = kTcKB * BN * 128;
  constexpr int ST = (226 * 1024 - QB * kTcQBlk) / STAGE > 4 ? 4 : (226 * 1024 - QB * kTcQBlk) / STAGE;
  constexpr int SMEM = QB * kTcQBlk + ST * STAGE + 1024 + 160 + kTcMaxPages * 4;
  static_assert(SMEM <= 227 * 1024, "MLA tensor-core tile does not fit shared memory");
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(mla_tc_kernel<QT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured_device = dev;
  }
  mla_tc_kernel<QT, BN><<<grid, kTcThreads, SMEM, st>>>(tq, tl, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

int launch_mla_tc(const fa_mla_args* a, cudaStream_t st) {
  // FA_B200_MLA_BN = 32 (two score buffers, 4-stage ring) or 64 (serial tile, 2-stage ring)
  static const int bn = [] { const char* e = getenv("FA_B200_MLA_BN"); return (e && atoi(e) == 32) ? 32 : 64; }();
  const int M = a->H_q * a->N_q;
  const int row_tiles = (M + 127) / 128;
  CUtensorMap tq, tl;
  {
    const uint64_t dims[2] = {(uint64_t)kTcDQK, (uint64_t)a->B * M};
    const uint64_t strides[1] = {(uint64_t)kTcDQK * 2};
    const uint32_t box[2] = {64, 128};
    int rc = encode_tensor_map(&tq, FA_BF16, 2, const_cast<void*>(a->q), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)kTcDQK, (uint64_t)a->num_blocks * a->page_size};
    const uint64_t strides[1] = {(uint64_t)kTcDQK * 2};
    const uint32_t box[2] = {64, (uint32_t)bn};
    int rc = encode_tensor_map(&tl, FA_BF16, 2, const_cast<void*>(a->l_pool), dims, strides, box, 1);
    if (rc) return rc;
  }
  MlaTcParams p{};
  p.q = reinterpret_cast<const uint16_t*>(a->q);
  p.block_table = a->block_table;
  p.q_offsets = a->q_offsets;
  p.items = a->items;
  p.out = a->out;
  p.lse = a->lse;
  p.part_o = reinterpret_cast<float*>(a->workspace);
  p.part_lse = p.part_o + (size_t)a->n_slots * M * kTcDV;
  p.counters = a->counters;
  p.status = a->counters + (mla_tc_counters_len(a->B, M) - 1);
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f * a->l_scale;
  p.scale_l = a->l_scale;
  p.n_logical = a->n_logical;
  p.num_blocks = a->num_blocks;
  p.page_size = a->page_size;
  p.page_shift = __builtin_ctz((unsigned)a->page_size);
  p.B = a->B; p.H_q = a->H_q; p.N_q = a->N_q; p.M = M; p.n_slots = a->n_slots;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  // FA_B200_MLA_QT = 0 / 256 / 384 query dims in tensor memory for the 32-key kernel (default 384)
  static const int qt = [] { const char* e = getenv("FA_B200_MLA_QT"); return e ? atoi(e) : 384; }();
  dim3 grid((unsigned)a->n_items, 2u, (unsigned)row_tiles);
  if (bn == 64) return launch_qt<384, 64>(tq, tl, p, grid, st);
  switch (qt) {
    case 0: return launch_qt<0, 32>(tq, tl, p, grid, st);
    case 256: return launch_qt<256, 32>(tq, tl, p, grid, st);
    default: return launch_qt<384, 32>(tq, tl, p, grid, st);
  }
}

}  // namespace fa
