// Paged GQA decode over an FP8 E4M3 KV cache on the tensor core, with the keys as the M dimension.
// d = 128, one query position per sequence, at most 8 query heads per KV head, page_size a power of two >= 64,
// per-tensor scales or one fp32 scale per token and head for K and for V.
//
// A decode step has G <= 8 query rows per KV head, so as rows of an MMA they would fill a sixteenth of the tile
// and the softmax of those few rows would run on G lanes.  Here the products are transposed:
//   S^T[key, head] = K[key, :] . Q[head, :]       M = 128 keys, N = 16 (G heads + padding), K = 128 dims
//   O^T[dim, head] += V^T[dim, key] . P^T[key, head]   M = 128 dims, N = 16, K = 128 keys
// The K tile is the A operand as TMA leaves it (row = key, 128 one-byte dims, 128-byte swizzle); the V tile is
// the A operand of the second product in its transposed (MN-major) form, again as TMA leaves it.  tcgen05
// kind::f8f6f4 multiplies the stored bytes: nothing is dequantised, HBM, L2 and shared memory see one byte per
// element.  The small operands (Q^T, P^T) are written as the sum of two E4M3 numbers, x = x1 + x2 with
// x1 = e4m3(x), x2 = e4m3(x - x1) (eight significant bits); the first pieces of the G heads are rows 0..7 of the
// 16-row operand and the second pieces rows 8..15, so one MMA yields both partial products side by side
// (columns h and 8 + h of the accumulator) and the thread that reads them adds the two.
// Softmax runs with one thread per key (TMEM lane): G scores each, the tile maximum per head by warp shuffles
// and one exchange through shared memory.  Scales: the K scale of a key multiplies its scores; the V scale is
// folded into the exponent, t = score + log2 s_v, w = 2^(t - m) goes to the tensor core (times 16; the running
// maximum is followed from 2^4 on, so 16 w <= 256 stays inside E4M3) and the denominator adds w / s_v.
//
// One thread per key keeps a softmax warpgroup busy for longer than HBM needs to deliver a tile, so a CTA runs
// two streams: tiles of even index belong to warpgroup 0, tiles of odd index to warpgroup 1, each with its own
// running maximum, denominator and O^T accumulator; the two are merged at the end like two key ranges.
//
// Warps: 0 = TMA producer (a ring of 128-key K / V tiles, 32 KB per stage), 1 = MMA issuer and TMEM owner,
// 2..5 = softmax of the even tiles (+ query split, epilogue), 6..9 = softmax of the odd tiles.  Every wait is
// bounded (sm100.cuh).
//
// Reference behaviour: kernels/v9_fp8/fp8_attention.cu:275-350 (what is computed), split merge
// kernels/v8_gqa_ss/gqa_ss_attention.cu:209-231.

#include <climits>

#include "sm100.cuh"

namespace fa {
namespace {

using namespace sm100;

constexpr int kTThreads = 320;                 // producer, issuer, two softmax warpgroups
constexpr int kTStages = 5;
constexpr int kTTile = 128;                   // keys per tile
constexpr int kTBlk = kTTile * 128;           // bytes of a K or V tile
constexpr int kTSmall = 16 * 128;             // bytes of one piece of Q^T or P^T: 16 rows x 128 bytes
constexpr int kTMaxPages = 2048;              // block-table entries staged per CTA
constexpr int kTD = 128;
constexpr float kTThreshold = 4.f, kTPre = 4.f;
constexpr float kLog2eT = 1.4426950408889634f, kLn2T = 0.6931471805599453f;

enum { DT_ERR_FULL = 61, DT_ERR_EMPTY = 62, DT_ERR_S_FULL = 63, DT_ERR_S_FREE = 64, DT_ERR_P_READY = 65, DT_ERR_PV_DONE = 66,
       DT_ERR_Q = 67 };

struct DecodeTcParams {
  const uint16_t* q;
  const float* k_tok;        // [tokens][H_kv] or null
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
  int n_logical, num_blocks, page_size, page_shift, total_tokens;
  int B, H_q, H_kv, G;
  int causal, q_offset, out_dtype, bt_cap;
};

__device__ __forceinline__ void mma_f8_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
               " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar) : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float (&v)[N]) {
  static_assert(N == 4 || N == 8, "4 or 8 columns");
  uint32_t* u = reinterpret_cast<uint32_t*>(v);
  if constexpr (N == 4)
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]) : "r"(taddr) : "memory");
  else
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]) : "r"(taddr) : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const float (&v)[N]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(v);
  if constexpr (N == 4)
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n"
                 ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]) : "memory");
  else
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]) : "memory");
}
// two floats -> two E4M3 bytes (lo in bits 0..7), round to nearest, saturating; and back
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
__device__ __forceinline__ void stream_bar(int z) {      // the 128 threads of one softmax warpgroup
  if (z == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
  else asm volatile("bar.sync 2, 128;\n" ::: "memory");
}
// The same barrier, which also tells every thread whether any of them has seen a wait give up: the threads of a
// stream leave its tile loop only here, all together (a thread that left alone would let the others wait at
// the barrier for ever).
__device__ __forceinline__ bool stream_vote(int z, bool bad) {
  uint32_t any;
  if (z == 0)
    asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 1, 128, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(any) : "r"((uint32_t)bad) : "memory");
  else
    asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 2, 128, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(any) : "r"((uint32_t)bad) : "memory");
  return any != 0;
}
__device__ __forceinline__ void softmax_bar256() { asm volatile("bar.sync 3, 256;\n" ::: "memory"); }

template <int NR>
__global__ void __launch_bounds__(kTThreads, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const DecodeTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;                               // [stages][128 keys][128 dims]
  uint8_t* sV = sK + kTStages * kTBlk;              // [stages][128 keys][128 dims]
  uint8_t* sQ = sV + kTStages * kTBlk;              // [16 rows: first pieces 0..7, second pieces 8..15][128 dims]
  uint8_t* sP = sQ + kTSmall;                       // [4 tiles][16 rows, the same split][128 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 4 * kTSmall);
  // score / weight buffers and their barriers are indexed by j & 3 (two per stream)
  enum { FULL = 0, EMPTY = kTStages, S_FULL = 2 * kTStages, S_FREE = S_FULL + 4, P_READY = S_FREE + 4, PV_DONE = P_READY + 4,
         Q_READY = PV_DONE + 4, NBARS = Q_READY + 1 };
  static_assert(NBARS <= 32, "barrier block");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 32);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ticket = const_cast<int*>(reinterpret_cast<volatile int*>(s_tmem + 2));
  float* s_c = reinterpret_cast<float*>(s_tmem + 4);               // [16]: score scale per row (log2 units)
  float* s_red = s_c + 16;                                         // [2 streams][2][4 warps][8]
  float* s_ml = s_red + 128;                                       // [2 streams][m, l][8]
  float* s_merge = s_ml + 32;                                      // [kTThreads][6]; also O^T of stream 1: [128][8]
  int32_t* s_bt = reinterpret_cast<int32_t*>(s_merge + kTThreads * 6);   // [kTMaxPages]
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // consecutive CTAs serve the KV heads of one key range: the head rows of a token are adjacent in the pool
  const int item_idx = (int)(blockIdx.x / p.H_kv), h_kv = (int)(blockIdx.x - item_idx * p.H_kv);
  const fa_decode_item it = p.items[item_idx];
  const int b = it.b;
  const int qoff = p.q_offsets ? p.q_offsets[b] : p.q_offset;
  const int k_begin = it.k_begin;
  int k_end = it.k_end;
  if (p.causal) k_end = min(k_end, max(qoff, -1) + 1);      // one query position: keys <= q_offset
  const int n_keys = max(k_end - k_begin, 0);
  const int n_tiles = (n_keys + kTTile - 1) / kTTile;
  const int rows_valid = p.G;                                 // <= NR

  if (tid == 0) {
    *s_abort = 0;
    for (int i = 0; i < kTStages; ++i) {
      mbar_init(bar(FULL + i), 1);
      mbar_init(bar(EMPTY + i), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_FREE + i), 128);
      mbar_init(bar(P_READY + i), 128);
      mbar_init(bar(PV_DONE + i), 1);
    }
    mbar_init(bar(Q_READY), 128);
    fence_barrier_init();
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), 128);
    tmem_relinquish();
  }
  // block-table slice of this key range (every 64-key box lies inside one page)
  const int pg0 = k_begin >> p.page_shift;
  if (n_keys > 0) {
    const int pg1 = (k_end - 1) >> p.page_shift;
    const int32_t* bt = p.block_table + (int64_t)b * p.n_logical;
    for (int i = tid; i <= pg1 - pg0 && i < p.bt_cap; i += kTThreads) {
      int pid = (pg0 + i < p.n_logical) ? bt[pg0 + i] : -2;
      if ((unsigned)pid >= (unsigned)p.num_blocks) {
        if (p.status) atomicOr(p.status, FA_STATUS_BAD_BLOCK_TABLE);
        pid = 0;                     // never follow a bad entry: read block 0 instead and flag it
      }
      s_bt[i] = pid;
    }
  }
  // the padding rows of P^T stay zero for the whole kernel
  for (int i = tid; i < 4 * kTSmall / 16; i += kTThreads) reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tm_s = tmem, tm_o = tmem + 64;          // S^T of tile j at tm_s + 16 (j & 3), O^T of stream z at tm_o + 16 z
  // token row of a key in the pool view; keys past the range read the zero fill beyond the tensor
  auto token_of = [&](int key) {
    if (key >= k_end) return p.total_tokens;
    const int pg = key >> p.page_shift;
    return s_bt[pg - pg0] * p.page_size + (key - (pg << p.page_shift));
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------- TMA producer: tile j -> stage j % kTStages
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kTStages;
        if (j >= kTStages && !mbar_wait(bar(EMPTY + st), ((j / kTStages) - 1) & 1, s_abort, p.status, DT_ERR_EMPTY)) break;
        mbar_expect_tx(bar(FULL + st), 2 * kTBlk);
        const int k0 = k_begin + j * kTTile;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int tok = token_of(k0 + 64 * h);
          tma_load_2d(smem_u32(sK + st * kTBlk + h * (kTBlk / 2)), &map_k, h_kv * kTD, tok, bar(FULL + st));
          tma_load_2d(smem_u32(sV + st * kTBlk + h * (kTBlk / 2)), &map_v, h_kv * kTD, tok, bar(FULL + st));
        }
      }
    }
  } else if (warp == 1) {
    if (n_tiles > 0) {
      // ------------------------------------------------- MMA issuer
      // the whole warp walks the control flow (uniform arithmetic); one elected lane executes the tcgen05 instructions
      const bool lead = elect_one();
      // The scores of tile j are issued before the weights of tile j - 2 (the previous tile of the same stream)
      // are waited for, so that the tensor core works on S^T(j) while both warpgroups are busy.
      constexpr uint32_t idesc_qk = idesc_f16(128, 16, false, false, false);   // format 0 of kind::f8f6f4 = E4M3
      constexpr uint32_t idesc_pv = idesc_f16(128, 16, false, true, false);    // A = V^T: the M dimension is contiguous
      bool ok = mbar_wait(bar(Q_READY), 0, s_abort, p.status, DT_ERR_Q);
      for (int j = 0; ok && j < n_tiles + 2; ++j) {
        if (j < n_tiles) {
          const int st = j % kTStages, sb = j & 3;
          ok = mbar_wait(bar(FULL + st), (j / kTStages) & 1, s_abort, p.status, DT_ERR_FULL);
          if (ok && j >= 4) ok = mbar_wait(bar(S_FREE + sb), ((j >> 2) - 1) & 1, s_abort, p.status, DT_ERR_S_FREE);
          if (!ok) break;
          tc_fence_after();
          const uint32_t k_base = smem_u32(sK + st * kTBlk), q_base = smem_u32(sQ);
          if (lead) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_f8_ss(tm_s + 16 * sb, smem_desc_sw128(k_base + ks * 32, 16, 1024), smem_desc_sw128(q_base + ks * 32, 16, 1024),
                        idesc_qk, ks > 0 ? 1u : 0u);
            mma_commit(bar(S_FULL + sb));
          }
        }
        if (j >= 2) {
          const int jj = j - 2, st = jj % kTStages, sb = jj & 3;
          ok = mbar_wait(bar(P_READY + sb), (jj >> 2) & 1, s_abort, p.status, DT_ERR_P_READY);
          if (!ok) break;
          tc_fence_after();
          const uint32_t v_base = smem_u32(sV + st * kTBlk), p_base = smem_u32(sP + sb * kTSmall);
          if (lead) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_f8_ss(tm_o + 16 * (jj & 1), smem_desc_sw128(v_base + ks * 4096, kTBlk, 1024), smem_desc_sw128(p_base + ks * 32, 16, 1024),
                        idesc_pv, (jj >= 2 || ks > 0) ? 1u : 0u);
            mma_commit(bar(EMPTY + st));
            mma_commit(bar(PV_DONE + sb));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ query split / softmax / epilogue
    const int z = (warp - 2) >> 2;                    // stream: tiles j = z, z + 2, ...
    const int L = (warp & 3) * 32 + lane;             // TMEM lane: key of the tile (scores), head dim (output)
    const int wq = warp & 3;
    const uint32_t tm_oz = tm_o + 16 * z;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    float m_ref[NR], l_run[NR], c_row[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) m_ref[h] = -INFINITY, l_run[h] = 0.f;
    if (z == 0) {
      // Q^T: thread (head = L / 8 mod 8, 16-dim chunk = L % 8); threads 0..63 write the first pieces (rows 0..7),
      // threads 64..127 the second pieces (rows 8..15).  A row is scaled by a power of two so that its largest
      // magnitude lies in [128, 256), then split; rows past the group are zeros.
      const int row = (L >> 3) & 7, ch = L & 7, second = L >> 6;
      float x[16];
      float amax = 0.f;
      if (row < rows_valid) {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + ((int64_t)b * p.H_q + h_kv * p.G + row) * kTD + 16 * ch);
        const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
          x[2 * e] = f.x, x[2 * e + 1] = f.y;
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] = 0.f;
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
      if (!(amax >= 1e-30f && amax <= 65504.f)) ex = 7;
      const float up = __uint_as_float((uint32_t)(7 - ex + 127) << 23);
      if (ch == 0 && !second) s_c[row] = p.softmax_scale * kLog2eT * p.k_scale * __uint_as_float((uint32_t)(ex - 7 + 127) << 23);
      uint32_t a[8], bq[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) split2(x[2 * i] * up, x[2 * i + 1] * up, a[i], bq[i]);
      const int orow = row + 8 * second;               // row & 7 is the same for both pieces
      const int off = orow * 128 + ((ch ^ (row & 7)) << 4);
      *reinterpret_cast<uint4*>(sQ + off) = second
          ? make_uint4(bq[0] | (bq[1] << 16), bq[2] | (bq[3] << 16), bq[4] | (bq[5] << 16), bq[6] | (bq[7] << 16))
          : make_uint4(a[0] | (a[1] << 16), a[2] | (a[3] << 16), a[4] | (a[5] << 16), a[6] | (a[7] << 16));
      fence_proxy_async();
      mbar_arrive(bar(Q_READY));
    }
    softmax_bar256();
#pragma unroll
    for (int h = 0; h < NR; ++h) c_row[h] = s_c[h];
    // the scales of this thread's key of a tile, requested one tile ahead
    const bool tok_scales = p.k_tok != nullptr;
    // (volatile loads: issued where they stand, two tiles before their use; keys past the range read token 0)
    auto fetch_scales = [&](int j, float& ks, float& vs) {
      ks = 1.f, vs = 1.f;
      if (tok_scales) {
        const int key = k_begin + j * kTTile + L;
        const int64_t t = (int64_t)((j < n_tiles && key < k_end) ? token_of(key) : 0) * p.H_kv + h_kv;
        asm volatile("ld.global.nc.f32 %0, [%1];\n" : "=f"(ks) : "l"(p.k_tok + t));
        asm volatile("ld.global.nc.f32 %0, [%1];\n" : "=f"(vs) : "l"(p.v_tok + t));
      }
    };
    float ks_a, vs_a, ks_b, vs_b;                     // alternate tiles of this stream
    fetch_scales(z, ks_a, vs_a);
    fetch_scales(z + 2, ks_b, vs_b);
    int j_last = -1;
    bool bad = false;                                 // a wait of this thread gave up (carried to the next vote)
    for (int j = z; j < n_tiles; j += 2) {
      const int sb = j & 3, st = j % kTStages;
      j_last = j;
      float ks_c, vs_c;
      if ((j & 2) == 0) { ks_c = ks_a, vs_c = vs_a; fetch_scales(j + 4, ks_a, vs_a); }
      else { ks_c = ks_b, vs_c = vs_b; fetch_scales(j + 4, ks_b, vs_b); }
      bad |= !mbar_wait(bar(S_FULL + sb), (j >> 2) & 1, s_abort, p.status, DT_ERR_S_FULL);
      tc_fence_after();
      float s[NR], s2[NR];
      tmem_ld_cols<NR>(tm_s + 16 * sb + lane_base, s);
      tmem_ld_cols<NR>(tm_s + 16 * sb + 8 + lane_base, s2);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(S_FREE + sb));
#pragma unroll
      for (int h = 0; h < NR; ++h) s[h] += s2[h];
      const int key = k_begin + j * kTTile + L;
      const bool valid = key < k_end;
      const float vs_eff = fmaxf(vs_c, 1e-30f);
      const float lg = tok_scales ? __log2f(vs_eff) : 0.f, inv = tok_scales ? __frcp_rn(vs_eff) : 1.f;
      float mt[NR];
#pragma unroll
      for (int h = 0; h < NR; ++h) {
        s[h] = valid ? fmaf(s[h] * ks_c, c_row[h], lg) : -INFINITY;
        mt[h] = s[h];
      }
      // warp maximum with the integer reduction instruction (floats compare like sign-magnitude integers)
#pragma unroll
      for (int h = 0; h < NR; ++h) {
        int i = __float_as_int(mt[h]);
        i ^= (i >> 31) & 0x7fffffff;
        i = __reduce_max_sync(0xffffffffu, i);
        i ^= (i >> 31) & 0x7fffffff;
        mt[h] = __int_as_float(i);
      }
      float* red = s_red + (z * 2 + ((j >> 1) & 1)) * 32;
      if (lane == 0)
#pragma unroll
        for (int h = 0; h < NR; ++h) red[wq * 8 + h] = mt[h];
      if (stream_vote(z, bad)) {
        ok = false;
        break;
      }
      bool raise_any = false;
      float alpha[NR];
#pragma unroll
      for (int h = 0; h < NR; ++h) {
        const float mx = fmaxf(fmaxf(red[h], red[8 + h]), fmaxf(red[16 + h], red[24 + h]));
        const bool raise = (mx > m_ref[h] + kTThreshold) || (m_ref[h] == -INFINITY && mx > -INFINITY);
        alpha[h] = 1.f;
        if (raise) {
          alpha[h] = fast_exp2(m_ref[h] - mx);
          m_ref[h] = mx;
          raise_any = true;
        }
        const float m_use = ((m_ref[h] == -INFINITY) ? 0.f : m_ref[h]) - kTPre;
        s[h] = fast_exp2(s[h] - m_use);
        l_run[h] = l_run[h] * alpha[h] + s[h] * inv;
      }
      // O^T may only be rescaled between two P V: this tile's is not issued before P^T arrives, the previous one
      // has to be waited for.  Lane = head dim here: every thread rescales its own row of O^T.
      if (j >= 2 && raise_any) {
        bad |= !mbar_wait(bar(PV_DONE + ((j - 2) & 3)), ((j - 2) >> 2) & 1, s_abort, p.status, DT_ERR_PV_DONE);
        tc_fence_after();
        float o[NR], o2[NR];
        tmem_ld_cols<NR>(tm_oz + lane_base, o);
        tmem_ld_cols<NR>(tm_oz + 8 + lane_base, o2);
        tmem_wait_ld();
#pragma unroll
        for (int h = 0; h < NR; ++h) o[h] *= alpha[h], o2[h] *= alpha[h];
        tmem_st_cols<NR>(tm_oz + lane_base, o);
        tmem_st_cols<NR>(tm_oz + 8 + lane_base, o2);
        tmem_wait_st();
      }
      // the P^T buffer of tile j - 4 has been read once its P V is done
      if (j >= 4) bad |= !mbar_wait(bar(PV_DONE + sb), ((j >> 2) - 1) & 1, s_abort, p.status, DT_ERR_PV_DONE);
      {
        uint8_t* pb = sP + sb * kTSmall + (L & 15);      // sb = j & 3
#pragma unroll
        for (int h = 0; h < NR; h += 2) {
          uint32_t p1, p2;
          split2(s[h], s[h + 1], p1, p2);
          const int o0 = h * 128 + (((L >> 4) ^ (h & 7)) << 4), o1 = (h + 1) * 128 + (((L >> 4) ^ ((h + 1) & 7)) << 4);
          pb[o0] = (uint8_t)(p1 & 0xffu), pb[o1] = (uint8_t)(p1 >> 8);
          pb[8 * 128 + o0] = (uint8_t)(p2 & 0xffu), pb[8 * 128 + o1] = (uint8_t)(p2 >> 8);      // rows 8 + h: the same swizzle
        }
      }
      // value rows past the end of the sequence may hold anything (E4M3 has NaN bytes): zero them so that
      // 0 * x stays 0 (this thread's key row of the V tile; the tile has landed, its scores are done)
      if (!valid) {
        uint4* d = reinterpret_cast<uint4*>(sV + st * kTBlk + L * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar(P_READY + sb));
    }
    ok = ok && !bad;
    if (ok && j_last >= 0)
      ok = mbar_wait(bar(PV_DONE + (j_last & 3)), (j_last >> 2) & 1, s_abort, p.status, DT_ERR_PV_DONE);
    // denominators: the 128 keys of every tile were spread over the threads of the stream
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int h = 0; h < NR; ++h) l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], o);
    float* red = s_red + (z * 2 + (((j_last + 2) >> 1) & 1)) * 32;
    if (lane == 0)
#pragma unroll
      for (int h = 0; h < NR; ++h) red[wq * 8 + h] = l_run[h];
    stream_bar(z);
    float o[NR], l_z[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) l_z[h] = (red[h] + red[8 + h]) + (red[16 + h] + red[24 + h]);
    if (ok && j_last >= 0) {
      tc_fence_after();
      float o2[NR];
      tmem_ld_cols<NR>(tm_oz + lane_base, o);
      tmem_ld_cols<NR>(tm_oz + 8 + lane_base, o2);
      tmem_wait_ld();
#pragma unroll
      for (int h = 0; h < NR; ++h) o[h] += o2[h];
    } else {
#pragma unroll
      for (int h = 0; h < NR; ++h) o[h] = 0.f, l_z[h] = 0.f, m_ref[h] = -INFINITY;
    }
    // the odd stream hands (m, l, O^T) to the even one, which merges the two like two key ranges
    if (z == 1) {
#pragma unroll
      for (int h = 0; h < NR; ++h) s_merge[L * 8 + h] = o[h];
      if (L == 0)
#pragma unroll
        for (int h = 0; h < NR; ++h) s_ml[16 + h] = m_ref[h], s_ml[24 + h] = l_z[h];
    }
    softmax_bar256();
    if (z == 0 && !*s_abort) {
      const bool single = (it.n_split == 1);
#pragma unroll
      for (int h = 0; h < NR; ++h) {
        if (h >= rows_valid) continue;
        const float m1 = s_ml[16 + h], l1 = s_ml[24 + h], o1 = s_merge[L * 8 + h];
        const float mm = fmaxf(m_ref[h], m1);
        const float w0 = (m_ref[h] == -INFINITY) ? 0.f : fast_exp2(m_ref[h] - mm), w1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mm);
        const float l_tot = l_z[h] * w0 + l1 * w1;
        // numerator and denominator both carry the factor 2^kTPre
        const float val = (l_tot > 0.f) ? (o[h] * w0 + o1 * w1) * p.v_scale / l_tot : 0.f;
        const float lse = (l_tot > 0.f) ? (mm - kTPre + log2f(l_tot)) * kLn2T : -INFINITY;
        const int64_t hrow = (int64_t)(h_kv * p.G + h);            // N_q = 1
        if (single) {
          const int64_t orow = (int64_t)b * p.H_q + hrow;
          store_out_dyn(p.out, p.out_dtype, orow * kTD + L, val);
          if (p.lse && L == 0) p.lse[orow] = lse;
        } else {
          const int64_t prow = (int64_t)(it.slot_base + it.split) * p.H_q + hrow;
          p.part_o[prow * kTD + L] = val;
          if (L == 0) p.part_lse[prow] = lse;
        }
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
  if (it.n_split == 1) return;

  // ---- the last CTA of this (sequence, KV head) merges all key ranges -----------------------------------
  __threadfence();
  __syncthreads();
  const int cidx = b * p.H_kv + h_kv;
  if (tid == 0) *s_ticket = atomicAdd(p.counters + cidx, 1);
  __syncthreads();
  if (*s_ticket != it.n_split - 1) return;
  __threadfence();
  if (tid == 0) p.counters[cidx] = 0;   // self-reset for the next launch
  // after a wait that gave up the ticket is still taken, but there is nothing valid to merge
  if (*s_abort) return;
  // A thread owns (row, four output columns) and, when there are fewer such columns than threads, one of
  // `groups` interleaved subsets of the ranges; the partials of kU ranges are fetched before any is used.
  constexpr int D4 = kTD / 4;
  constexpr int kU = 8;
  const int64_t slot_stride = (int64_t)p.H_q;
  const int n_cols = rows_valid * D4;
  int groups = 1;
  while (groups * 2 * n_cols <= kTThreads && groups * 2 <= it.n_split) groups *= 2;
  const int n_work = groups > 1 ? groups * n_cols : n_cols;
  for (int idx0 = 0; idx0 < n_work; idx0 += kTThreads) {
    const int idx = idx0 + tid;
    const bool active = idx < n_work;
    const int grp = groups > 1 ? idx / n_cols : 0;
    const int col = groups > 1 ? idx - grp * n_cols : idx;
    const int row = active ? col / D4 : 0, d4 = col - row * D4;
    const int64_t hrow = (int64_t)(h_kv * p.G + row);
    float m_run = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
      const float* lse_base = p.part_lse + it.slot_base * slot_stride + hrow;
      const float4* o_base = reinterpret_cast<const float4*>(p.part_o + (it.slot_base * slot_stride + hrow) * kTD) + d4;
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
    if (groups > 1) {            // n_work <= kTThreads: a single pass, every thread reaches the barrier
      float* mine = s_merge + (size_t)idx * 6;
      if (active) {
        mine[0] = m_run, mine[1] = l, mine[2] = acc.x, mine[3] = acc.y, mine[4] = acc.z, mine[5] = acc.w;
      }
      __syncthreads();
      if (!active || grp != 0) continue;
      for (int g2 = 1; g2 < groups; ++g2) {
        const float* o = s_merge + ((size_t)g2 * n_cols + col) * 6;
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
    const int64_t orow = (int64_t)b * p.H_q + hrow;
    const int64_t o0 = orow * kTD + d4 * 4;
    store_out_dyn(p.out, p.out_dtype, o0 + 0, acc.x * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 1, acc.y * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 2, acc.z * inv);
    store_out_dyn(p.out, p.out_dtype, o0 + 3, acc.w * inv);
    if (p.lse && d4 == 0) p.lse[orow] = (l > 0.f) ? m_run + __logf(l) : -INFINITY;
  }
}

constexpr int kTSmem = 2 * kTStages * kTBlk + 5 * kTSmall + 32 * 8 + 16 + (16 + 128 + 32 + kTThreads * 6) * 4 + kTMaxPages * 4 + 1024;
static_assert(kTSmem <= 227 * 1024, "decode_tc tile ring does not fit shared memory");

}  // namespace

// Host side; called by fa_paged_decode_fwd (decode.cu) after validation.
int decode_tc_max_pages() { return kTMaxPages; }

bool decode_tc_applicable(const fa_decode_args* a) {
  if (a->kv_dtype != FA_E4M3 || a->q_dtype != FA_F16 || a->D != kTD || a->N_q != 1) return false;
  if (a->H_q / a->H_kv > 8) return false;
  if (a->page_size < 64 || (a->page_size & (a->page_size - 1)) != 0) return false;
  if (a->max_range_keys / a->page_size + 2 > kTMaxPages) return false;
  if (reinterpret_cast<uintptr_t>(a->k_pool) % 16 != 0 || reinterpret_cast<uintptr_t>(a->v_pool) % 16 != 0) return false;
  if (((int64_t)a->H_kv * kTD) % 16 != 0 || (int64_t)a->num_blocks * a->page_size > INT_MAX) return false;
  return true;
}

int launch_decode_tc(const fa_decode_args* a, cudaStream_t st) {
  CUtensorMap tk, tv;
  const uint64_t dims[2] = {(uint64_t)a->H_kv * kTD, (uint64_t)a->num_blocks * a->page_size};
  const uint64_t strides[1] = {(uint64_t)a->H_kv * kTD};
  const uint32_t box[2] = {128, 64};
  int rc = encode_tensor_map(&tk, FA_E4M3, 2, const_cast<void*>(a->k_pool), dims, strides, box, 1);
  if (rc) return rc;
  rc = encode_tensor_map(&tv, FA_E4M3, 2, const_cast<void*>(a->v_pool), dims, strides, box, 1);
  if (rc) return rc;
  DecodeTcParams p{};
  p.q = reinterpret_cast<const uint16_t*>(a->q);
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
  p.page_shift = __builtin_ctz((unsigned)a->page_size);
  p.total_tokens = a->num_blocks * a->page_size;
  p.B = a->B; p.H_q = a->H_q; p.H_kv = a->H_kv; p.G = a->H_q / a->H_kv;
  p.causal = a->causal; p.q_offset = a->q_offset; p.out_dtype = a->out_dtype;
  static int configured_device = -1;
  int dev = 0;
  FA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    FA_CUDA_OK(cudaFuncSetAttribute(decode_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
    FA_CUDA_OK(cudaFuncSetAttribute(decode_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
    configured_device = dev;
  }
  dim3 grid((unsigned)a->n_items * (unsigned)a->H_kv, 1u, 1u);
  if (p.G <= 4) decode_tc_kernel<4><<<grid, kTThreads, kTSmem, st>>>(tk, tv, p);
  else decode_tc_kernel<8><<<grid, kTThreads, kTSmem, st>>>(tk, tv, p);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa
