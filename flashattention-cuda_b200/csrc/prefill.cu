// Dense (causal) attention forward: two 128-row query tiles per CTA that take turns on the tensor core
// ("ping-pong"), probabilities handed to the second MMA through tensor memory.  TMA (3-D tensor maps over
// [B*H, N, d], 64 x 128 boxes, 128-byte swizzle, zero fill past N) -> shared memory -> tcgen05.mma.kind::f16
// with fp32 accumulators in TMEM.
//
// One CTA per SM walks a fixed share of the work items (an item = two 128-row query tiles of one head): the next
// item's queries are loaded as soon as the last score MMAs of the current one have run, its first scores are
// computed while the softmax threads still write the previous output, and tensor memory is allocated once.
//
// Warp roles (12 warps, three warpgroups):
//   warpgroup 0   warp 0: TMA producer (both Q tiles per item, K/V tiles into a 2-stage ring that runs on across
//                 items); warp 1: TMEM allocation + every tcgen05.mma; warps 2, 3 idle; registers released
//   warpgroup 1   softmax / correction / epilogue of query tile 0 (thread r owns row r)
//   warpgroup 2   the same for query tile 1
// TMEM (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).  P_i (fp16 / bf16, two keys
// per 32-bit column) overwrites the first 64 columns of S_i and is read from there as the A operand
// of O_i += P_i V (tcgen05.mma with A in tensor memory), so it never touches shared memory.
// MMA order per key tile j:  PV_j(0)  QK_{j+1}(0)  PV_j(1)  QK_{j+1}(1): while one tile's softmax runs on the
// CUDA cores, the tensor core works for the other tile.  MMAs of one thread execute in issue order,
// which is what makes reusing S_i for P_i and then for S_i of the next key tile (or item) safe.
// The running maximum is only raised (and O rescaled) when it grew by more than 2^8, which keeps
// P <= 256 in half precision and makes TMEM round trips of O rare.
// The output leaves through shared memory and TMA stores (32 rows x 128 bytes per warp and pass).
//
// Measured on B = 4, H = 32, N = 4096, d = 128 fp16 (CUDA events, A/B on one GPU each):
//   one CTA per item, row-by-row output stores, 64-bit descriptors assembled per MMA by a single issuing lane  0.651 ms
//   persistent CTAs + TMA-store epilogue                                                                       0.589 ms
//   MMAs issued from precomputed 32-bit descriptor words (0.587 ->)                                            0.547 ms
//   barrier waits that try the barrier before reading the abort flag (0.545 ->)                                0.535 ms
//   issuing warp walks the control flow whole, one elected lane executes the tcgen05 instructions (0.512 ->)  0.482 ms
// (0.50-0.51 ms = 65-66 % of the measured dense bf16 peak in the benchmark runs).  A clock64 trace of the item boundary
// showed why the stores mattered: row-by-row stores (each warp instruction touching 32 lines) kept the SM's memory path
// busy for ~4000 cycles per warpgroup, the next item's Q load finished only after them (8000-9000 cycles after it was
// issued) and the first score MMAs ran at a tenth of their speed meanwhile.  The other three steps all shorten the
// issuing thread's own instruction stream, which sets the pace between MMA batches: in isolation an M = 128, N = 128,
// K = 16 MMA takes 64 cycles; with descriptors assembled per MMA by one lane of a diverged warp the kernel saw 80-98.
// Measured and not kept: two exponentials per instruction (ex2.approx.f16x2) +0.6 %; two threads per query row
// (four softmax warpgroups) +7 %; two 64-key score buffers per query tile +30 %; the exponentials of a tile taken
// against the reference maximum as it stands while the tile's own maximum is found alongside (so that no pass
// over the scores precedes them) +3 to +8 %; score MMAs with the Q operand in tensor memory instead of shared
// memory (timing probe, wrong data) -1.6 %, so the shared-memory operand traffic is not what bounds the MMAs;
// L2 prefetch of the next item's first boxes: no change.
//
// Behaviour: the reference's dense entry point (fa_kernels/__init__.py:26-42,
// kernels/v5_wmma/wmma_attention.cu:229-263).

#include <algorithm>
#include <cstdlib>

#include "sm100.cuh"

namespace fa {
namespace {

using namespace sm100;

constexpr int kP2Threads = 384;
constexpr uint32_t kP2TmemCols = 512;
constexpr float kRescaleThreshold = 8.f;     // log2 units

struct PrefillParams {
  void* out;
  float* lse;
  int* status;
  int B, H, N_q, N_k;
  int causal, out_dtype;
  float scale_log2;
  int n_qt;        // 256-row query tile pairs per (batch, head)
  int n_units;     // work units of the launch
  int paired;      // 1: a unit is the heaviest remaining and the lightest remaining causal tile pair of a head
};

// The launch is a fixed number of CTAs that each walk their share of the work units (unit u, u + gridDim.x, ...)
// so that loading the next queries and keys overlaps the previous item's last steps and its epilogue.  Units
// are numbered head-major, which keeps the CTAs that run at the same time on the same few heads' keys (L2).
// Causal launches with enough work pair the k-th heaviest with the k-th lightest query tile pair of a head in one
// unit: every unit then costs the same and the static deal is even.
struct ItemWalk {
  int u, half;   // everything else is read from the kernel parameters at each step (registers are short)
  __device__ ItemWalk() : u((int)blockIdx.x), half(0) {}
  // next item of this CTA: (batch*head, query tile pair); false when the walk is over
  __device__ __forceinline__ bool next(const PrefillParams& p, int& bh, int& qt) {
    const int per_head = p.paired ? (p.n_qt + 1) / 2 : p.n_qt;
    while (u < p.n_units) {
      bh = u / per_head;
      const int k = u - bh * per_head;
      if (!p.paired) {
        qt = p.n_qt - 1 - k;               // heaviest causal tiles first
        u += (int)gridDim.x;
        return true;
      }
      if (half == 0) {
        qt = p.n_qt - 1 - k;
        half = 1;
        return true;
      }
      half = 0;
      u += (int)gridDim.x;
      if (k != p.n_qt - 1 - k) {
        qt = k;
        return true;
      }
    }
    return false;
  }
};

enum { P2_ERR_Q = 21, P2_ERR_KV_FULL = 22, P2_ERR_KV_EMPTY = 23, P2_ERR_S_FULL = 24, P2_ERR_P_READY = 25, P2_ERR_O_DONE = 26, P2_ERR_Q_EMPTY = 27 };

// 32 packed columns (64 half-precision values) of this thread's TMEM lane
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&r)[32]) {
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

// ---- packed fp32 pairs (two fp32 lanes in one 64-bit register: fma / add issue once for two values) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// MMA with the two 32-bit words of each shared-memory descriptor given separately: the issuing thread keeps one low
// word per operand buffer and adds a constant per k step, instead of assembling 64-bit descriptors per MMA.
template <bool ACC>
__device__ __forceinline__ void mma_ss_words(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
  asm volatile(
      "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
__device__ __forceinline__ void mma_ts_words(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n .reg .b64 db;\n setp.ne.b32 p, %5, 0;\n mov.b64 db, {%2, %3};\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
template <int D, bool BF16>
__global__ void __launch_bounds__(kP2Threads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_out,
               const PrefillParams p) {
  constexpr int KB = D / 64;
  constexpr int TILE_BYTES = 128 * D * 2;
  constexpr int BLK_BYTES = 128 * 128;
  constexpr int STAGES = 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                  // [2 query tiles]
  uint8_t* sK = sQ + 2 * TILE_BYTES;                   // [stage]
  uint8_t* sV = sK + STAGES * TILE_BYTES;              // [stage]
  uint8_t* sO = sV + STAGES * TILE_BYTES;              // [8 softmax warps] 32 output rows x 128 bytes each
  uint64_t* bars = reinterpret_cast<uint64_t*>(sO + 8 * 4096);
  enum { Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 3, S_FULL = 5, P_READY = 7, O_DONE = 9, Q_EMPTY = 11, NBARS = 12 };
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  const int n_all = (p.N_k + 127) / 128;
  // key tiles the two query tiles of an item need (causal: up to the tile holding the last row)
  auto tiles_of = [&](int q0, int (&n_t)[2]) {
    n_t[0] = p.causal ? min(n_all, (q0 + 127) / 128 + 1) : n_all;
    n_t[1] = p.causal ? min(n_all, (q0 + 255) / 128 + 1) : n_all;
    if (q0 + 128 >= p.N_q) n_t[1] = 0;                 // second query tile entirely out of range
  };

  if (threadIdx.x == 0) {
    *s_abort = 0;
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(Q_EMPTY), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(KV_FULL + s), 1);
      mbar_init(bar(KV_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_READY + s), 128);
      mbar_init(bar(O_DONE + s), 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), kP2TmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (wg == 0) {
    setmaxnreg_dec<56>();   // 128 x 56 + 256 x 224 = 384 x 168, the register total the CTA was launched with
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      ItemWalk walk;
      int bh, qt, n_t[2];
      int g = 0;                                       // key tiles loaded so far (ring position), over all items
      bool ok = true;
      for (int it = 0; ok && walk.next(p, bh, qt); ++it) {
        const int q0 = qt * 256;
        tiles_of(q0, n_t);
        const int n_max = max(n_t[0], n_t[1]);
        // the query buffers are free once the previous item's last score MMAs have run
        if (it > 0 && !mbar_wait(bar(Q_EMPTY), (it - 1) & 1, s_abort, p.status, P2_ERR_Q_EMPTY)) break;
        mbar_expect_tx(bar(Q_FULL), 2 * TILE_BYTES);
        for (int i = 0; i < 2; ++i)
          for (int kb = 0; kb < KB; ++kb)
            tma_load_3d(smem_u32(sQ + i * TILE_BYTES + kb * BLK_BYTES), &tm_q, kb * 64, q0 + i * 128, bh, bar(Q_FULL));
        for (int j = 0; j < n_max; ++j, ++g) {
          const int s = g % STAGES;
          if (g >= STAGES && !mbar_wait(bar(KV_EMPTY + s), ((g / STAGES) - 1) & 1, s_abort, p.status, P2_ERR_KV_EMPTY)) { ok = false; break; }
          mbar_expect_tx(bar(KV_FULL + s), 2 * TILE_BYTES);
          for (int kb = 0; kb < KB; ++kb) {
            tma_load_3d(smem_u32(sK + s * TILE_BYTES + kb * BLK_BYTES), &tm_k, kb * 64, j * 128, bh, bar(KV_FULL + s));
            tma_load_3d(smem_u32(sV + s * TILE_BYTES + kb * BLK_BYTES), &tm_v, kb * 64, j * 128, bh, bar(KV_FULL + s));
          }
        }
      }
    } else if (warp == 1) {
      // The whole warp walks the issuer's control flow (waits, counters, descriptor words), so that this arithmetic is
      // warp-uniform; one elected lane executes the tcgen05 instructions.
      const bool lead = elect_one();
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = idesc_f16(128, 128, BF16, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(128, D, BF16, false, true);
      auto wait = [&](int b, int parity, int code) { return mbar_wait(bar(b), parity, s_abort, p.status, code); };
      // low descriptor words of the operand buffers (address >> 4 in bits 0-13, leading byte offset >> 4 in bits
      // 16-29) and the high word all of them share (stride 1024 >> 4, descriptor version, 128-byte swizzle)
      const uint32_t hi_w = (1024u >> 4) | (1u << 14) | (2u << 29);
      uint32_t q_lo[2], k_lo[STAGES], v_lo[STAGES];
#pragma unroll
      for (int i = 0; i < 2; ++i) q_lo[i] = ((smem_u32(sQ + i * TILE_BYTES) & 0x3ffffu) >> 4) | ((16u >> 4) << 16);
#pragma unroll
      for (int st = 0; st < STAGES; ++st) {
        k_lo[st] = ((smem_u32(sK + st * TILE_BYTES) & 0x3ffffu) >> 4) | ((16u >> 4) << 16);
        v_lo[st] = ((smem_u32(sV + st * TILE_BYTES) & 0x3ffffu) >> 4) | (((uint32_t)BLK_BYTES >> 4) << 16);
      }
      auto issue_qk = [&](int i, int gt) {              // gt: ring position of the key tile
        const uint32_t a0 = q_lo[i], b0 = k_lo[gt % STAGES], d = tmem + i * 128;
        if (lead) {
          mma_ss_words<false>(d, a0, b0, hi_w, idesc_qk);
#pragma unroll
          for (int k = 1; k < D / 16; ++k) {
            const uint32_t off = ((k >> 2) * BLK_BYTES + (k & 3) * 32) >> 4;
            mma_ss_words<true>(d, a0 + off, b0 + off, hi_w, idesc_qk);
          }
          mma_commit(bar(S_FULL + i));
        }
      };
      auto issue_pv = [&](int i, int gt, bool first) {
        // A = P_i in tensor memory: 16 keys = 8 packed columns; B = V [128 keys][D], MN-major
        const uint32_t b0 = v_lo[gt % STAGES], d = tmem + 256 + i * 128, a = tmem + i * 128;
        if (lead) {
          mma_ts_words(d, a, b0, hi_w, idesc_pv, first ? 0u : 1u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ts_words(d, a + k * 8, b0 + (k * 2048 >> 4), hi_w, idesc_pv, 1u);
        }
      };
      ItemWalk walk;
      int bh, qt, n_t[2];
      int g = 0;                                       // ring position of the item's first key tile
      int n_p[2] = {0, 0};                             // P_READY phases consumed per query tile
      bool ok = true;
      for (int it = 0; ok && walk.next(p, bh, qt); ++it) {
        tiles_of(qt * 256, n_t);
        const int n_max = max(n_t[0], n_t[1]);
        ok = wait(Q_FULL, it & 1, P2_ERR_Q) &&
             wait(KV_FULL + (g % STAGES), (g / STAGES) & 1, P2_ERR_KV_FULL);
        if (!ok) break;
        tc_fence_after();
        // S_i is free: the P V of the previous item's last key tile was issued before this by the same thread.
        // O_i is overwritten by the first P V below, which waits for this item's first P_READY; the softmax
        // threads arrive there only after they have read the previous item's O_i.
        if (n_t[0] > 0) issue_qk(0, g);
        if (n_t[1] > 0) issue_qk(1, g);
        if (lead && n_max == 1) mma_commit(bar(Q_EMPTY));
        for (int j = 0; ok && j < n_max; ++j) {
          const int gt = g + j;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            if (j < n_t[i]) {
              ok = wait(P_READY + i, n_p[i] & 1, P2_ERR_P_READY);
              if (!ok) break;
              ++n_p[i];
              tc_fence_after();
              issue_pv(i, gt, j == 0);
              if (lead && j + 1 == n_t[i]) mma_commit(bar(O_DONE + i));
            }
            if (lead && i == 1) mma_commit(bar(KV_EMPTY + (gt % STAGES)));
            if (i == 0 && j + 1 < n_max) {   // the next key tile is only needed from here on
              ok = wait(KV_FULL + ((gt + 1) % STAGES), ((gt + 1) / STAGES) & 1, P2_ERR_KV_FULL);
              if (!ok) break;
              tc_fence_after();
            }
            if (j + 1 < n_t[i]) issue_qk(i, gt + 1);
          }
          if (lead && ok && j + 2 == n_max) mma_commit(bar(Q_EMPTY));   // the item's last score MMAs are in the queue
        }
        g += n_max;
      }
    }
  } else {
    setmaxnreg_inc<224>();
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int i = wg - 1;                              // query tile of this warpgroup
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const uint32_t tm_s = tmem + i * 128 + lane_base;
    const uint32_t tm_o = tmem + 256 + i * 128 + lane_base;
    ItemWalk walk;
    int bh, qt, n_t[2];
    int n_s = 0, n_o = 0;                              // S_FULL / O_DONE phases consumed so far
    bool ok = true;
    while (ok && walk.next(p, bh, qt)) {
    const int q0 = qt * 256;
    tiles_of(q0, n_t);
    const int gi = q0 + i * 128 + row;
    const int nt = n_t[i];
    float m_ref = -INFINITY, l_run = 0.f;              // m_ref: the maximum P and O are currently scaled by
    for (int j = 0; j < nt; ++j) {
      ok = mbar_wait(bar(S_FULL + i), n_s & 1, s_abort, p.status, P2_ERR_S_FULL);
      if (!ok) break;
      ++n_s;
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
      tmem_wait_ld();

      const int k0 = j * 128;
      const bool need_mask = (k0 + 128 > p.N_k) || (p.causal && k0 + 127 > q0 + i * 128);
      // scores stay unscaled until the exponent: max commutes with the (positive) scale, and
      // scale * s - m is one fused multiply-add per pair
      if (need_mask) {
        const int limit = p.causal ? min(gi, p.N_k - 1) : p.N_k - 1;
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (k0 + c > limit) s[c] = -INFINITY;
      }
      // four independent chains each for the maximum and the sum: one warp per scheduler per query
      // tile is all the parallelism there is, so dependent chains of 64 operations would set the pace
      float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
      for (int c = 0; c < 128; c += 8) {
        mxa = max3(mxa, s[c], s[c + 1]);
        mxb = max3(mxb, s[c + 2], s[c + 3]);
        mxc = max3(mxc, s[c + 4], s[c + 5]);
        mxd = max3(mxd, s[c + 6], s[c + 7]);
      }
      float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd)) * p.scale_log2;
      // raise the reference maximum only when it is more than 2^8 behind
      const bool raise = (mx > m_ref + kRescaleThreshold) || (m_ref == -INFINITY && mx > -INFINITY);
      float alpha = 1.f;
      if (raise) {
        alpha = fast_exp2(m_ref - mx);                 // m_ref = -inf -> 0
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(-m_use, -m_use);
      // P as packed half-precision pairs: register c holds keys 2c, 2c+1
      uint32_t pk[64];
      uint64_t sums[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float x0, x1;
        unpack2(fma2(pack2(s[2 * c], s[2 * c + 1]), sc2, nm2), x0, x1);
        const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
        sums[c & 3] = add2(sums[c & 3], pack2(e0, e1));
        pk[c] = BF16 ? pack_bf2(e0, e1) : pack_h2(e0, e1);
      }
      float sum_lo, sum_hi;
      unpack2(add2(add2(sums[0], sums[1]), add2(sums[2], sums[3])), sum_lo, sum_hi);
      const float sum = sum_lo + sum_hi;
      l_run = l_run * alpha + sum;
      // S_FULL of key tile j implies P V of key tile j-1 has finished (same issuing thread, in order),
      // so O may be rescaled here
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tmem_ld32(tm_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st32(tm_o + c * 32, o);
        }
      }
      // P -> tensor memory over the first 64 columns of S_i: column c holds keys 2c, 2c+1
      tmem_st32u(tm_s, *reinterpret_cast<const uint32_t(*)[32]>(&pk[0]));
      tmem_st32u(tm_s + 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[32]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_READY + i));
    }
    if (ok && nt > 0) ok = mbar_wait(bar(O_DONE + i), (n_o++) & 1, s_abort, p.status, P2_ERR_O_DONE);
    if (ok && nt > 0) {
      tc_fence_after();
      const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
      const bool valid = gi < p.N_q;
      const int64_t orow = (int64_t)bh * p.N_q + gi;
      // O_i leaves through shared memory: each warp stages 128 bytes of its 32 rows (128-byte swizzle, so the
      // 16-byte stores of a warp spread over all banks) and one lane hands the box to TMA, which writes whole rows
      // and drops the rows past N_q.  Row-by-row stores from the owning threads touch 32 lines per instruction and
      // hold up the SM's next loads for thousands of cycles.
      const uint32_t so = smem_u32(sO + ((wg - 1) * 4 + quad) * 4096);
      const uint32_t so_row = so + lane * 128;
      const int row_w = q0 + i * 128 + quad * 32;      // first row of this warp
      const int passes = (p.out_dtype == FA_F32) ? D / 32 : D / 64;
      for (int c = 0; c < passes; ++c) {
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        if (p.out_dtype == FA_F32) {
          float o[32];
          tmem_ld32(tm_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            st_shared_v4(so_row + ((e ^ (lane & 7)) << 4), __float_as_uint(o[4 * e] * inv), __float_as_uint(o[4 * e + 1] * inv),
                         __float_as_uint(o[4 * e + 2] * inv), __float_as_uint(o[4 * e + 3] * inv));
        } else {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            float o[32];
            tmem_ld32(tm_o + c * 64 + hh * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint32_t v[4];
#pragma unroll
              for (int w = 0; w < 4; ++w)
                v[w] = (p.out_dtype == FA_BF16) ? pack_bf2(o[8 * e + 2 * w] * inv, o[8 * e + 2 * w + 1] * inv)
                                                : pack_h2(o[8 * e + 2 * w] * inv, o[8 * e + 2 * w + 1] * inv);
              st_shared_v4(so_row + (((hh * 4 + e) ^ (lane & 7)) << 4), v[0], v[1], v[2], v[3]);
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && row_w < p.N_q) {
          tma_store_3d(&tm_out, so, c * ((p.out_dtype == FA_F32) ? 32 : 64), row_w, bh);
          tma_store_commit();
        }
      }
      if (valid && p.lse) p.lse[orow] = (l_run > 0.f) ? (m_ref + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      // the next item's first P_READY, which lets the tensor core overwrite O_i, follows these reads in program order
      tc_fence_before();
    }
    }   // items
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) __nanosleep(200000);   // after a timed-out wait: give copies still in flight time to land
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kP2TmemCols);
  }
}

}  // namespace

template <int D, bool BF16>
static int launch_prefill(const fa_dense_args* a, float scale_log2, cudaStream_t st) {
  CUtensorMap tq, tk, tv, to;
  const int dt = BF16 ? FA_BF16 : FA_F16;
  const uint64_t BH = (uint64_t)a->B * a->H;
  const uint32_t box[3] = {64, 128, 1};
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->N_q, BH};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->N_q * D * 2};
    int rc = encode_tensor_map(&tq, dt, 3, const_cast<void*>(a->q), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->N_k, BH};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->N_k * D * 2};
    int rc = encode_tensor_map(&tk, dt, 3, const_cast<void*>(a->k), dims, strides, box, 1);
    if (rc) return rc;
    rc = encode_tensor_map(&tv, dt, 3, const_cast<void*>(a->v), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t es = (a->out_dtype == FA_F32) ? 4 : 2;
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->N_q, BH};
    const uint64_t strides[2] = {(uint64_t)D * es, (uint64_t)a->N_q * D * es};
    const uint32_t obox[3] = {(uint32_t)(128 / es), 32, 1};
    int rc = encode_tensor_map(&to, a->out_dtype, 3, a->out, dims, strides, obox, 1);
    if (rc) return rc;
  }
  PrefillParams p{};
  p.out = a->out; p.lse = a->lse; p.status = a->status;
  p.B = a->B; p.H = a->H; p.N_q = a->N_q; p.N_k = a->N_k;
  p.causal = a->causal; p.out_dtype = a->out_dtype; p.scale_log2 = scale_log2;
  const int sms = std::max(device_sm_count(), 1);
  p.n_qt = (a->N_q + 255) / 256;
  const int64_t items = (int64_t)BH * p.n_qt, pairs = (int64_t)BH * ((p.n_qt + 1) / 2);
  p.paired = (a->causal && p.n_qt > 1 && pairs >= sms) ? 1 : 0;
  p.n_units = (int)(p.paired ? pairs : items);
  constexpr int TILE = 128 * D * 2;
  constexpr int SMEM = TILE * 6 + 8 * 4096 + 256 + 1024;
  auto kern = prefill_kernel<D, BF16>;
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured_device = dev;
  }
  const unsigned grid = (unsigned)std::min<int64_t>(p.n_units, sms);
  kern<<<grid, kP2Threads, SMEM, st>>>(tq, tk, tv, to, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa

using namespace fa;

extern "C" int fa_dense_fwd(const fa_dense_args* a) {
  FA_CHECK_ARG(a != nullptr, "fa_dense_fwd: null args");
  FA_CHECK_ARG(a->q && a->k && a->v && a->out, "fa_dense_fwd: q, k, v, out must be non-null");
  FA_CHECK_ARG(a->B >= 1 && a->H >= 1 && a->N_q >= 1 && a->N_k >= 1, "fa_dense_fwd: bad B/H/N");
  FA_CHECK_ARG((int64_t)a->B * a->H * ((a->N_q + 255) / 256) <= 0x7fffffffLL, "fa_dense_fwd: B * H * ceil(N_q / 256) must fit 31 bits");
  FA_CHECK_ARG(a->dtype == FA_F16 || a->dtype == FA_BF16, "fa_dense_fwd: q/k/v must be f16 or bf16");
  FA_CHECK_ARG(a->out_dtype == FA_F32 || a->out_dtype == FA_F16 || a->out_dtype == FA_BF16, "out_dtype must be f32/f16/bf16");
  FA_CHECK_ARG((((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15) == 0,
               "fa_dense_fwd: q, k, v, out must be 16-byte aligned");
  if (a->D != 64 && a->D != 128) return fail(FA_ERR_UNSUPPORTED, "dense attention supports head_dim 64 or 128 (got %d)", a->D);
  const float scale_log2 = a->softmax_scale * 1.4426950408889634f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  if (a->D == 128) return a->dtype == FA_BF16 ? launch_prefill<128, true>(a, scale_log2, st) : launch_prefill<128, false>(a, scale_log2, st);
  return a->dtype == FA_BF16 ? launch_prefill<64, true>(a, scale_log2, st) : launch_prefill<64, false>(a, scale_log2, st);
}
