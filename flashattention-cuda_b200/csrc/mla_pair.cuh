// Pieces shared by the CTA-pair MLA decode kernels (mla_pair.cu: bf16 latent, mla_pair_f8.cu: E4M3 latent):
// launch parameters, wait codes, the cluster / cta_group::2 PTX wrappers, and the merge of key ranges that
// the last CTA of a (sequence, row tile, row half) runs.
#pragma once

#include <climits>

#include "sm100.cuh"

namespace fa {
namespace pair {

using namespace sm100;

constexpr int kPThreads = 256;
constexpr int kPDQK = 576, kPDV = 512;
constexpr int kPBlk = 64 * 128;          // bytes of one operand block: 64 rows of 128 bytes
constexpr int kPMaxPages = 512;          // block-table entries staged per CTA
constexpr float kPThreshold = 8.f;

struct MlaPairParams {
  const uint16_t* q;
  const int32_t* block_table;
  const int32_t* q_offsets;
  const fa_decode_item* items;
  void* out;
  float* lse;
  float* part_o;     // [n_slots][rows][DV]
  float* part_lse;   // [n_slots][rows]
  int32_t* counters; // [B][row_tiles][2]
  int32_t* status;
  float scale_log2, scale_l;
  int n_logical, num_blocks, page_size, page_shift, total_tokens;
  int B, H_q, N_q, M, n_slots;
  int causal, q_offset, out_dtype;
  // FP8 latent only
  const float* tok_scale;    // [num_blocks * page_size] or null
  float tensor_scale;        // multiplies every token's scale (alone when tok_scale is null)
};

enum { P2_ERR_Q = 41, P2_ERR_QT = 42, P2_ERR_X_FULL = 43, P2_ERR_X_EMPTY = 44, P2_ERR_Y_FULL = 45, P2_ERR_Y_EMPTY = 46,
       P2_ERR_S_FULL = 47, P2_ERR_P_READY = 48, P2_ERR_PV_DONE = 49, P2_ERR_SCALES = 52 };

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// Arrival on a barrier of the even CTA that orders nothing across CTAs by itself: what the waiting MMA
// thread then starts reads this CTA's own shared / tensor memory, which the fences before the arrival
// have already published to this SM's tensor core.
__device__ __forceinline__ void mbar_arrive_peer(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y) : "memory");
}
// TMA tile into this CTA's shared memory; the bytes are counted on a barrier of the even CTA.
__device__ __forceinline__ void tma_pair_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
               " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma2_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
               " tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// The same MMAs with the two 32-bit words of each shared-memory descriptor given separately: an issuing thread keeps
// one low word per operand buffer (address >> 4 in bits 0-13, leading byte offset >> 4 in bits 16-29) and adds a
// constant per k step; every descriptor here shares the high word (stride 1024 >> 4, descriptor version, 128-byte
// swizzle).  Assembling 64-bit descriptors per MMA made the issuing thread, not the tensor pipe, set the pace.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3ffffu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ void mma2_ss_w(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
               " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n}\n"
               ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma2_ts_w(uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n .reg .b64 db;\n setp.ne.b32 p, %5, 0;\n mov.b64 db, {%2, %3};\n"
               " tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n}\n"
               ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(acc) : "memory");
}
// arrive on the barrier at this offset in both CTAs once every MMA issued so far has completed
__device__ __forceinline__ void mma2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
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
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

// The last CTA of a (sequence, row tile, row half) to finish merges all key ranges of its 64 rows; every
// CTA of a split sequence calls this after its partial result is in global memory.  `s_ticket` is a word
// of shared memory, `aborted` whether a wait of this CTA gave up.
__device__ __forceinline__ void merge_ranges(const MlaPairParams& p, const fa_decode_item& it, int b, int rt, int rank, int m0,
                                             int rows_valid, int* s_ticket, bool aborted) {
  __threadfence();
  __syncthreads();
  const int cidx = (b * gridDim.y + rt) * 2 + (int)rank;
  if (threadIdx.x == 0) *s_ticket = atomicAdd(p.counters + cidx, 1);
  __syncthreads();
  if (*s_ticket != it.n_split - 1) return;
  __threadfence();
  if (threadIdx.x == 0) p.counters[cidx] = 0;
  // after a wait that gave up the ticket is still taken, so that the counters are zero again for the next
  // launch, but there is nothing valid to merge (the status word tells the host)
  if (aborted) return;
  // A thread owns (row, four output columns) quads; the partials of kU ranges of kI quads are fetched before
  // any is used, so that a merge over n ranges of the 64 x 512 outputs of this CTA costs about
  // (8192 / 256 / kI) * ceil(n / kU) L2 round trips instead of one per quad.
  constexpr int kU = 4, kI = 4;
  const int n_quads = rows_valid * (kPDV / 4);
  const int nthr = (int)blockDim.x;
  for (int idx0 = threadIdx.x; idx0 < n_quads; idx0 += nthr * kI) {
    const float* lse_base[kI];
    const float4* o_base[kI];
    float m_run[kI], l[kI];
    float4 acc[kI];
    bool live[kI];
#pragma unroll
    for (int q = 0; q < kI; ++q) {
      const int idx = idx0 + q * nthr;
      live[q] = idx < n_quads;
      const int row = live[q] ? idx / (kPDV / 4) : 0, d4 = live[q] ? idx - row * (kPDV / 4) : 0;
      const int m = m0 + row;
      lse_base[q] = p.part_lse + (int64_t)it.slot_base * p.M + m;
      o_base[q] = reinterpret_cast<const float4*>(p.part_o + ((int64_t)it.slot_base * p.M + m) * kPDV) + d4;
      m_run[q] = -INFINITY, l[q] = 0.f, acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s0 = 0; s0 < it.n_split; s0 += kU) {
      float ls[kI][kU];
      float4 ov[kI][kU];
#pragma unroll
      for (int q = 0; q < kI; ++q)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int sidx = min(s0 + u, it.n_split - 1);
          ls[q][u] = __ldcg(lse_base[q] + (int64_t)sidx * p.M);
          ov[q][u] = __ldcg(o_base[q] + (int64_t)sidx * p.M * (kPDV / 4));
          if (s0 + u >= it.n_split) ls[q][u] = -INFINITY;
        }
#pragma unroll
      for (int q = 0; q < kI; ++q) {
        float mb = m_run[q];
#pragma unroll
        for (int u = 0; u < kU; ++u) mb = fmaxf(mb, ls[q][u]);
        if (mb == -INFINITY) continue;
        const float resc = __expf(m_run[q] - mb);
        acc[q].x *= resc, acc[q].y *= resc, acc[q].z *= resc, acc[q].w *= resc, l[q] *= resc;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const float wgt = __expf(ls[q][u] - mb);
          acc[q].x += wgt * ov[q][u].x, acc[q].y += wgt * ov[q][u].y, acc[q].z += wgt * ov[q][u].z, acc[q].w += wgt * ov[q][u].w;
          l[q] += wgt;
        }
        m_run[q] = mb;
      }
    }
#pragma unroll
    for (int q = 0; q < kI; ++q) {
      if (!live[q]) continue;
      const int idx = idx0 + q * nthr;
      const int row = idx / (kPDV / 4), d4 = idx - row * (kPDV / 4);
      const int m = m0 + row;
      const float inv = (l[q] > 0.f) ? 1.f / l[q] : 0.f;
      const int h = m / p.N_q, iq = m - h * p.N_q;
      const int64_t orow = ((int64_t)b * p.H_q + h) * p.N_q + iq;
      const int64_t o0 = orow * kPDV + d4 * 4;
      store_out_dyn(p.out, p.out_dtype, o0 + 0, acc[q].x * inv);
      store_out_dyn(p.out, p.out_dtype, o0 + 1, acc[q].y * inv);
      store_out_dyn(p.out, p.out_dtype, o0 + 2, acc[q].z * inv);
      store_out_dyn(p.out, p.out_dtype, o0 + 3, acc[q].w * inv);
      if (p.lse && d4 == 0) p.lse[orow] = (l[q] > 0.f) ? m_run[q] + __logf(l[q]) : -INFINITY;
    }
  }
}

}  // namespace pair
}  // namespace fa
