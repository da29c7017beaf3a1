/*
 * fa_b200 — C ABI of the B200 (sm_100a) attention library.
 *
 * One shared library, `libfa_b200.so`, replaces the per-kernel JIT modules that the reference
 * project loads through bindings/load.py:107-131 (`build_kernel(name)` -> pybind module with a
 * `.forward(...)`).  Each entry point below names the reference `forward` it stands in for.
 *
 * Conventions
 *   - every function returns an int status (FA_OK == 0); `fa_last_error()` gives the text of the last
 *     failure on the calling thread.  Nothing throws, nothing calls exit.
 *   - pointers marked "device" are CUDA device pointers on the current device; "host" are ordinary
 *     host pointers.  Tensors are contiguous row-major in the layouts stated.
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); no entry point synchronises and
 *     none allocates device memory: scratch ("workspace") is supplied by the caller, sized by the
 *     matching *_workspace_bytes query.
 */
#ifndef FA_B200_H
#define FA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FA_API __attribute__((visibility("default")))
#else
#define FA_API
#endif

enum fa_status {
  FA_OK = 0,
  FA_ERR_INVALID = 1,      /* bad argument (shape, dtype, null pointer) */
  FA_ERR_UNSUPPORTED = 2,  /* valid request this build has no kernel for (e.g. head_dim) */
  FA_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed */
  FA_ERR_WORKSPACE = 4     /* workspace too small */
};

enum fa_dtype {
  FA_F16 = 0,
  FA_BF16 = 1,
  FA_F32 = 2,
  FA_E4M3 = 3,   /* uint8 FP8 E4M3 bytes (fa_kernels/paged.py:94-109) */
  FA_NVFP4 = 4   /* packed E2M1 nibbles + one E4M3 micro-scale per 16 elements (paged.py:136-170) */
};

FA_API const char* fa_last_error(void);
FA_API int fa_version(void);

/* Device status word.  Kernels never follow a bad block-table entry and never wait without a bound; what
 * they met instead is recorded in one int32 in device memory that the host reads after the step: word 0
 * of the `counters` buffer of the decode / MLA entry points, `fa_dense_args.status` for dense attention.
 * The word is sticky: kernels only OR / compare-and-swap into it and the caller clears it after reading.
 *   bit 16 (FA_STATUS_BAD_BLOCK_TABLE): a block-table entry outside [0, num_blocks) was met; the page was
 *           treated as masked (decode) or read from block 0 (MLA tensor-core kernel), the output is wrong
 *   bits 0..15: code of the first pipeline wait that gave up after its cycle bound (21..27 dense attention,
 *           41..52 MLA CTA-pair kernels, 61..67 FP8 tcgen05 decode); the kernel ended early and the output is invalid
 * A non-zero word after a launch also means the arrival counters behind it may not be zero again: zero
 * the whole counters buffer before the next launch.  (The reference has no counterpart: its kernels read
 * whatever the table holds, kernels/v8_gqa_ss/gqa_ss_attention.cu:124-136.) */
#define FA_STATUS_BAD_BLOCK_TABLE 0x10000
/* Text for a status word (static storage, valid until the next call on the same thread). */
FA_API const char* fa_status_text(int status_word);
/* Self-test of the bounded waits (no counterpart in the reference, whose kernels have no waits): one warp
 * waits on an mbarrier that nothing arrives on, gives up after `max_cycles` SM clock cycles, records `code`
 * in `*status` (device int32, as above) and sets `*gave_up` (device int32, optional) to 1.  Lets a host
 * check its handling of a timed-out kernel without disturbing a real pipeline. */
FA_API int fa_selftest_bounded_wait(int32_t* status, long long max_cycles, int code, int32_t* gave_up, void* stream);
/* Number of SMs of the current device (cached per device). */
FA_API int fa_device_sm_count(int* sm_count);

/* ------------------------------------------------------------------------------------------------
 * Paged GQA decode (split-KV, M-packed query heads, fused LSE merge).
 * Replaces `forward` of kernels/v7_paged/binding.cpp, kernels/v8_gqa_ss/binding.cpp:9-20,
 * kernels/v9_fp8/binding.cpp:9-23 and kernels/v10_nvfp4/binding.cpp — i.e. the calls made at
 * fa_kernels/paged.py:232-234, 258-260, 282-284, 400-402.
 * ---------------------------------------------------------------------------------------------- */

/* One unit of work: keys [k_begin, k_end) of sequence b.  Produced by fa_decode_plan on the host and
 * consumed by the kernel from device memory (the caller copies it). 8 x int32. */
typedef struct fa_decode_item {
  int32_t b;
  int32_t k_begin;
  int32_t k_end;
  int32_t slot_base;  /* first partial-result slot of sequence b */
  int32_t n_split;    /* number of key ranges sequence b was cut into */
  int32_t split;      /* index of this range within the sequence */
  int32_t pad0;
  int32_t pad1;
} fa_decode_item;

/* Host-side split planner (no CUDA calls).  The reference picks ONE split count for the whole batch
 * from a single n_k (choose_splits, kernels/v8_gqa_ss/gqa_ss_attention.cu:248-259); this planner
 * cuts each sequence by its own length so that the grid is a multiple of the SM count's worth of
 * similar-sized ranges, longest first.
 *   seq_lens_host : host int32[B] per-sequence key counts, or NULL to use n_k for every sequence
 *   rows          : packed query rows per KV head = (H_q / H_kv) * N_q
 *   num_sms       : SMs of the device, three CTA slots each; 0 = 148; a negative value is minus the number
 *                   of CTA slots itself (a kernel configuration that fits two CTAs per SM: -2 * SMs)
 *   chunk_hint    : 0 = choose (the cheaper of whole sequences and shrinking ranges under a list-scheduling
 *                   estimate); otherwise the target keys per range (rounded to a multiple of 64)
 *   items         : host output, capacity max_items
 *   n_items       : output, number of ranges (each range owns one partial-result slot)
 *   max_range_keys: output, the longest range in keys */
FA_API int fa_decode_plan(const int32_t* seq_lens_host, int n_k, int B, int H_kv, int rows, int page_size,
                   int num_sms, int chunk_hint, fa_decode_item* items, int max_items,
                   int* n_items, int* max_range_keys);
/* Upper bound on the number of items fa_decode_plan can emit for these arguments. */
FA_API int fa_decode_plan_max_items(const int32_t* seq_lens_host, int n_k, int B, int page_size);

typedef struct fa_decode_args {
  /* queries: device, [B, H_q, N_q, D], dtype FA_F16 or FA_BF16 (FA_BF16 only with FA_BF16 pools) */
  const void* q;
  int q_dtype;
  /* pools: device, [num_blocks, page_size, H_kv, DX].  DX = D (f16/bf16/e4m3) or D/2 (nvfp4). */
  const void* k_pool;
  const void* v_pool;
  int kv_dtype;
  /* NVFP4 only: device uint8 [num_blocks, page_size, H_kv, D/16] E4M3 micro-scales */
  const void* k_micro;
  const void* v_micro;
  /* per-tensor dequant scales (1.0 for f16/bf16) — `scale_k`, `scale_v` of paged.py:237,263 */
  float k_scale;
  float v_scale;
  /* E4M3 only, optional: device float32 [num_blocks, page_size, H_kv] per-token-per-head scales that
   * multiply k_scale / v_scale.  NULL = per-tensor only (the reference layout). */
  const float* k_token_scale;
  const float* v_token_scale;
  /* device int32 [B, n_logical] */
  const int32_t* block_table;
  int n_logical;
  int num_blocks;
  int page_size;
  int B, H_q, H_kv, N_q, D;
  float softmax_scale;
  int causal;          /* key j is masked when j > i_q + q_offset (v7_paged/paged_attention.cu:138) */
  int q_offset;
  /* optional device int32[B]: per-sequence q_offset overriding the scalar */
  const int32_t* q_offsets;
  /* plan */
  const fa_decode_item* items;  /* device copy of the planner output */
  int n_items;
  int n_slots;         /* n_items, or 0 when no sequence is split (no partial storage is used) */
  int max_range_keys;  /* from fa_decode_plan */
  /* outputs: device, [B, H_q, N_q, D] in out_dtype (FA_F32 is the reference behaviour, FA_F16/FA_BF16
   * are accepted); lse optional float32 [B, H_q, N_q] (natural log), may be NULL */
  void* out;
  int out_dtype;
  float* lse;
  /* scratch: partial results of split sequences (fa_decode_workspace_bytes; contents need no
   * initialisation) and fa_decode_counters_len int32 words, zero before the first call: word 0 is the
   * device status word (see above), the others are arrival counters, which the kernel leaves zero
   * again.  Neither may be shared by decode calls that overlap in time. */
  void* workspace;
  size_t workspace_bytes;
  int32_t* counters;
  size_t counters_len;
  void* stream;
  int variant;         /* 0 = the library chooses: E4M3 pools with D = 128 on power-of-two pages >= 64, N_q = 1 and
                          H_q / H_kv <= 8 run on the tcgen05 kernel (keys as the M dimension, one CTA per SM: plan
                          with num_sms = -SMs), everything else on the mma.sync kernel; 9 = always the mma.sync
                          kernel; 1, 2 = tuning variants of the mma.sync kernel */
} fa_decode_args;

FA_API size_t fa_decode_workspace_bytes(int n_slots, int H_q, int N_q, int D);
FA_API size_t fa_decode_counters_len(int B, int H_q, int H_kv, int N_q);
FA_API int fa_paged_decode_fwd(const fa_decode_args* args);

/* One decode step from HOST buffers: what a serving loop does around fa_paged_decode_fwd, in one call and
 * without Python or allocator work between the launches.  On `dev.stream` it enqueues
 *   q_host -> dev.q, block_table_host -> dev.block_table        (cudaMemcpyAsync, host to device)
 *   fa_decode_plan(seq_lens_host / n_k) into items_host, items_host -> dev.items
 *   the decode kernel (as fa_paged_decode_fwd; dev.n_items / n_slots / max_range_keys are filled in here)
 *   dev.out -> out_host                                         (device to host)
 * and returns without synchronising; the result is in out_host once the stream has drained.  `dev` holds
 * the resident KV pools and DEVICE staging buffers for q, block table, items (capacity max_items) and out,
 * plus workspace and counters as for fa_paged_decode_fwd.  Host buffers should be pinned (the copies are
 * asynchronous only then); items_host must be pinned and must not be reused before its copy has finished.
 * The reference has no such entry point: its wrappers take CUDA tensors (fa_kernels/paged.py:379-402) and
 * leave the copies to the caller. */
typedef struct fa_decode_host_args {
  fa_decode_args dev;
  const void* q_host;
  size_t q_bytes;
  const int32_t* block_table_host;
  size_t block_table_bytes;
  const int32_t* seq_lens_host;   /* int32[B] or NULL (then n_k for every sequence) */
  int n_k;
  void* out_host;
  size_t out_bytes;
  fa_decode_item* items_host;     /* pinned staging for the plan */
  int max_items;                  /* capacity of items_host and of dev.items */
  int chunk_hint;                 /* as fa_decode_plan */
} fa_decode_host_args;
FA_API int fa_paged_decode_host(const fa_decode_host_args* args);

/* Same computation as fa_paged_decode_fwd for callers that have no device memory to give and cannot
 * obtain any.  (This entry point has no counterpart in the reference, whose host functions allocate
 * their outputs and workspaces with torch on every call.)  Two kinds of host are meant: an inference
 * server that hands the whole device to its KV-cache pool at start-up, so that a later cudaMalloc
 * fails or fragments the pool; and a plugin host that passes the plugin its input and output buffers
 * but no allocator, where a cudaMalloc from inside the plugin would also stall the device, because
 * cudaMalloc synchronises it.
 *
 * The `workspace`, `workspace_bytes`, `counters` and `counters_len` fields of `args` are ignored: the
 * scratch is a fixed array of FA_DECODE_STATIC_SCRATCH_BYTES inside the library's device image.  The
 * call allocates nothing (no cudaMalloc / cudaFree, no library routine that allocates).
 *   - Limits: at most 16384 (sequence, KV head, 16-row tile) units per call, i.e. B * H_kv *
 *     ceil((H_q / H_kv) * N_q / 16) <= 16384, and the partial results of split sequences
 *     (fa_decode_workspace_bytes) must fit in the remaining FA_DECODE_STATIC_SCRATCH_BYTES - 65792 bytes;
 *     beyond either limit the call returns FA_ERR_WORKSPACE and launches nothing.  Every argument is
 *     checked before the call touches the array.
 *   - The first call on each device looks up the array's device address; make that first call outside
 *     any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *     streams, different threads) race on it and give wrong results.  Serialise them, or use
 *     fa_paged_decode_fwd with one scratch buffer per concurrent call.
 *   - The device status word of these calls lives in the array too and is kept until it is read:
 *     fa_paged_decode_static_status copies it to `status_host`, optionally clears it, and waits for
 *     `stream` (the one call of this header that synchronises). */
#define FA_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
FA_API int fa_paged_decode_fwd_static(const fa_decode_args* args);
FA_API int fa_paged_decode_static_status(int32_t* status_host, int clear, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Merge of normalised partial outputs over disjoint key ranges (the algebra of the reference merge
 * kernels, e.g. kernels/v8_gqa_ss/gqa_ss_attention.cu:209-231, with (m, l) folded into LSE).
 * Used after the all-gather of per-GPU partials when one sequence's keys are spread over GPUs.
 *   o_parts  : device float32, part s at o_parts + s * o_part_stride, each [rows, D]
 *   lse_parts: device float32, part s at lse_parts + s * lse_part_stride, each [rows]
 *              (strides in floats; <= 0 means densely packed [n_parts, rows, D] / [n_parts, rows])
 *   out      : device [rows, D] in out_dtype          lse_out   : optional float32 [rows]
 * ---------------------------------------------------------------------------------------------- */
FA_API int fa_merge_partials(const float* o_parts, const float* lse_parts, int n_parts, int64_t rows, int D,
                             int64_t o_part_stride, int64_t lse_part_stride, void* out, int out_dtype,
                             float* lse_out, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Dense attention forward (optionally causal) on tcgen05 tensor cores.
 * Replaces `forward(q, k, v, scale, causal)` of kernels/v1_naive/binding.cpp:7-14 ... v6 (the call at
 * fa_kernels/__init__.py:41-42).  q [B,H,N_q,D], k/v [B,H,N_k,D] contiguous, f16 or bf16, D in {64,128},
 * 16-byte aligned.  causal masks key j when j > i (top-left aligned, kernels/v5_wmma/wmma_attention.cu:159).
 * out [B,H,N_q,D] in out_dtype (FA_F32 = reference behaviour); lse optional float32 [B,H,N_q].
 * status: optional device int; a non-zero value after the kernel names a pipeline wait that timed out
 * (the kernel then ends early instead of hanging; the output is invalid).
 * ---------------------------------------------------------------------------------------------- */
typedef struct fa_dense_args {
  const void* q;
  const void* k;
  const void* v;
  int dtype;
  int B, H, N_q, N_k, D;
  float softmax_scale;
  int causal;
  void* out;
  int out_dtype;
  float* lse;
  int* status;
  void* stream;
} fa_dense_args;
FA_API int fa_dense_fwd(const fa_dense_args* args);

/* ------------------------------------------------------------------------------------------------
 * MLA latent-KV decode: MQA of H_q heads over one shared latent per token; scores over DQK dims, values
 * = the first DV dims of the same latent.  Replaces `forward` of kernels/v11_mla/binding.cpp and
 * kernels/v12_mla_tc/binding.cpp:11-27 (the calls at fa_kernels/paged.py:338-340, 373-376).
 *   q       : device [B, H_q, N_q, DQK], FA_BF16 with a bf16 latent, FA_F16 otherwise
 *   l_pool  : device [num_blocks, page_size, 1, DX]: bf16 (DX = DQK), uint8 E4M3 (DX = DQK) or packed
 *             NVFP4 nibbles (DX = DQK/2, with l_micro [.., 1, DQK/16] E4M3 micro-scales — the reference
 *             layout of build_paged_kv_mla, paged.py:287-309)
 *   l_scale : per-tensor scale (`scale_l`); l_token_scale: optional float32 [num_blocks, page_size, 1]
 *             per-token scales of an E4M3 latent (multiply l_scale)
 *   (DQK, DV) in {(576,512), (160,128), (96,64)} as in kernels/v11_mla/mla_attention.cu:383-397.
 * Plan, workspace and counters as for fa_paged_decode_fwd, with H_kv = 1 and 32-row tiles: call
 * fa_decode_plan(..., H_kv = 1, rows = 16 * ceil(H_q * N_q / 32), chunk_hint <= fa_mla_pair_max_range(page_size)
 * to allow the tcgen05 kernel), workspace bytes = fa_mla_workspace_bytes(n_slots, H_q, N_q, DV), counters =
 * fa_mla_counters_len(B, H_q, N_q) (word 0 is the device status word).
 * ---------------------------------------------------------------------------------------------- */
typedef struct fa_mla_args {
  const void* q;
  int q_dtype;
  const void* l_pool;
  int latent_dtype;
  const void* l_micro;
  float l_scale;
  const float* l_token_scale;
  const int32_t* block_table;
  int n_logical;
  int num_blocks;
  int page_size;
  int B, H_q, N_q, DQK, DV;
  float softmax_scale;
  int causal;
  int q_offset;
  const int32_t* q_offsets;
  const fa_decode_item* items;
  int n_items;
  int n_slots;
  int max_range_keys;
  void* out;
  int out_dtype;
  float* lse;
  void* workspace;
  size_t workspace_bytes;
  int32_t* counters;
  size_t counters_len;
  void* stream;
  int engine_hint;   /* 0 = choose (tcgen05 on a CTA pair where it applies); 2 = force the mma.sync kernel.
                        The tcgen05 kernels need a (576, 512) latent in bf16 (bf16 q) or E4M3 (fp16 q, pool
                        16-byte aligned; per-token or per-tensor scales), page_size a power of two >= 64 and
                        key ranges <= fa_mla_pair_max_range; everything else (NVFP4 latents read in place, the
                        (160, 128) and (96, 64) geometries, other page sizes) runs on the mma.sync kernel */
} fa_mla_args;
FA_API size_t fa_mla_counters_len(int B, int H_q, int N_q);
FA_API size_t fa_mla_workspace_bytes(int n_slots, int H_q, int N_q, int DV);
FA_API int fa_mla_pair_max_range(int page_size);   /* longest key range of the CTA-pair kernel */
FA_API int fa_mla_decode_fwd(const fa_mla_args* args);
/* Expand the tokens of the planned key ranges of a quantised latent pool into a bf16 pool of the same
 * shape [num_blocks, page_size, 1, dqk] (rows of other tokens are not touched), the operand of the
 * tensor-core MLA kernels:
 *   FA_E4M3 : out[row, :] = bf16(e4m3(l_pool[row, :]) * token_scale[row])   (token_scale null: tensor_scale)
 *   FA_NVFP4: out[row, 16 j + i] = bf16(e2m1(code) * e4m3(l_micro[row, j]) * tensor_scale), two codes per byte
 * `items` are the ranges of fa_decode_plan (device memory).  The dequantisation is the one the reference
 * oracle applies to the same bytes (fa_kernels/reference.py:84-111: dequantize_nvfp4 / FP8 x scale), rounded
 * once to bf16. */
FA_API int fa_mla_expand_latent(const void* l_pool, int latent_dtype, const uint8_t* l_micro, const float* token_scale,
                                float tensor_scale, const int32_t* block_table, int n_logical, int num_blocks, int page_size,
                                const fa_decode_item* items, int n_items, int dqk, void* out_bf16, void* stream);

/* ------------------------------------------------------------------------------------------------
 * KV-cache formats and the paged layout (bit-exact with the reference's torch functions).
 * ---------------------------------------------------------------------------------------------- */

/* FP8 E4M3 quantise — `quantize_fp8_e4m3`, fa_kernels/paged.py:94-109.
 *   per_row == 0 : one scale for the tensor, scale = float32(max(amax, 1e-12) / 448) -> scales[0]
 *   per_row  > 0 : one scale per row of per_row elements (per token per head) -> scales[n / per_row]
 *   x: device f32/f16/bf16 [n]; out: device uint8 [n]; scratch4: device, 4 bytes (per-tensor mode). */
FA_API int fa_quantize_fp8_e4m3(const void* x, int x_dtype, int64_t n, int per_row, uint8_t* out, float* scales,
                                void* scratch4, void* stream);
/* `dequantize_fp8_e4m3`, fa_kernels/paged.py:112-118: out[i] = e4m3(bytes[i]) * scale (or row_scales). */
FA_API int fa_dequantize_fp8_e4m3(const uint8_t* bytes, int64_t n, float scale, const float* row_scales, int per_row,
                                  float* out, void* stream);
/* NVFP4 quantise — `quantize_nvfp4`, fa_kernels/paged.py:136-170.  n elements, the last dimension a
 * multiple of 16; packed: uint8 [n/2] (low nibble = even element), micro: uint8 [n/16] E4M3,
 * scale_out: device float32[1] = max(amax, 1e-12) / (6 * 448). */
FA_API int fa_quantize_nvfp4(const void* x, int x_dtype, int64_t n, uint8_t* packed, uint8_t* micro, float* scale_out,
                             void* scratch4, void* stream);
/* `dequantize_nvfp4`, fa_kernels/paged.py:173-189. */
FA_API int fa_dequantize_nvfp4(const uint8_t* packed, const uint8_t* micro, int64_t n, float scale, float* out, void* stream);
/* Dense [B, H, N, row_bytes] -> pool [num_blocks, page_size, H, row_bytes] with
 * pool[block_table[b][j / page], j % page] = dense[b, :, j]; the tail of the last page is zeroed.
 * The scatter of `build_paged_kv`, fa_kernels/paged.py:75-88 (the permutation is the caller's). */
FA_API int fa_paged_scatter(const void* dense, void* pool, const int32_t* block_table, int B, int H, int N, int row_bytes,
                            int page_size, int n_logical, int num_blocks, void* stream);
/* The inverse: the gather every kernel performs (kernels/v7_paged/paged_attention.cu:118-131). */
FA_API int fa_paged_gather(const void* pool, void* dense, const int32_t* block_table, int B, int H, int N, int row_bytes,
                           int page_size, int n_logical, int num_blocks, void* stream);

/* Quantise-dequantise to signed E2M1 levels in fp32 with one scale = amax / 6 per tensor (0), per channel =
 * last-dimension index (1) or per token = row (2), the scale optionally rounded through E4M3 —
 * `fake_quant_nvfp4` for the granularities "tensor" / "channel" / "token" of the reference's
 * fa_kernels/nvfp4_recipes.py:42-73 ("block16" is fa_quantize_nvfp4 + fa_dequantize_nvfp4).
 * x, out: device float32 [rows, d]; scratch: device, 4 bytes per scale. */
FA_API int fa_fake_quant_e2m1(const float* x, int64_t rows, int d, int granularity, int e4m3_scale, float* out,
                              void* scratch, size_t scratch_bytes, void* stream);

/* KV-cache write path: append T new tokens of every sequence to a paged pool, converting / quantising on the
 * way (the reference only has whole-tensor offline quantisers, fa_kernels/paged.py:94-170; the formulas are
 * the same, applied per row).  x: device [B, H, T, d] f32/f16/bf16; positions: device int32[B], logical
 * position of the first new token; pool_dtype FA_F16 / FA_BF16 (convert), FA_E4M3 (one fp32 scale per token
 * per head = amax/448 into scale_pool [num_blocks, page, H]), FA_NVFP4 (E2M1 codes + E4M3 micro-scales into
 * micro_pool [.., H, d/16], relative to the caller's fixed tensor_scale).  status: optional device int, bit 0
 * = bad block-table entry, bit 1 = position outside the table (the row is skipped). */
FA_API int fa_kv_append(const void* x, int x_dtype, const int32_t* positions, const int32_t* block_table, int B, int H,
                        int T, int d, int page_size, int n_logical, int num_blocks, int pool_dtype, float tensor_scale,
                        void* pool, float* scale_pool, uint8_t* micro_pool, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
