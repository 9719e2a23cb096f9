/*
 * pypto_b200 — C ABI of the B200 (sm_100a) implementation of the quantized DeepSeek-V3.2
 * sparse-attention decode path: lightning-indexer score -> exact top-k -> sparse MLA attention.
 *
 * Every entry point replaces one operator of the reference's
 * examples/models/deepseek_v32_exp package (the reference binds its operators through
 * `pypto.jit`, python/pypto/runtime.py:218-253, which launches on the current stream with device
 * pointers taken from `pypto.from_torch`, python/pypto/converter.py:36-112). The contract is the
 * same here: all pointers are DEVICE pointers owned by the caller, outputs are written in place,
 * the call is asynchronous on `stream`, nothing is retained after the call returns.
 *
 * Conventions
 *   - return value: 0 on success, a negative PTO_ERR_* code otherwise; no exception crosses the
 *     ABI. `pto_last_error()` gives a thread-local detail string for the last failing call.
 *   - `workspace` is caller-allocated device scratch of at least `*_workspace_bytes(...)` bytes,
 *     256-byte aligned. Its first PTO_STATUS_WORDS int32 words are a device status area that the
 *     kernels set on a rejected page-table entry or an expired bounded wait; read it with
 *     `pto_workspace_status` (which synchronises the stream).
 *   - the library allocates no device memory; the indexer, attention and fused entry points keep no
 *     state between calls and are re-entrant (calls on different streams need different
 *     workspaces). The prolog entry point is the exception: per device it creates, at its first
 *     call, a second stream and three events, and its calls on one device are serialised by a
 *     per-device mutex while they enqueue. A prolog call must not be enqueued on a device while
 *     another stream of that device is capturing a prolog call: both would use the same side
 *     stream.
 *   - t = b * s1 query tokens; the tokens of sequence `bi` are rows bi*s1 .. bi*s1+s1-1.
 */
#ifndef PYPTO_B200_H_
#define PYPTO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* pto_stream_t; /* cudaStream_t */

#define PTO_ABI_VERSION 1

#define PTO_OK 0
#define PTO_ERR_INVALID (-1)     /* bad argument (null pointer, unsupported shape, misalignment) */
#define PTO_ERR_WORKSPACE (-2)   /* workspace null or too small */
#define PTO_ERR_CUDA (-3)        /* a CUDA runtime call or launch failed */
#define PTO_ERR_UNSUPPORTED (-4) /* device is not sm_100 / feature not built */
#define PTO_ERR_DRIVER (-5)      /* tensor-map encoding through the driver failed */

/* dtype of idx_query_scale / idx_key_scale / idx_weight */
#define PTO_DT_F16 0
#define PTO_DT_F32 1

/* flags of the indexer entry points */
#define PTO_LI_SCORE_SIMT 0x1 /* score stage on CUDA cores (dp4a) instead of tcgen05; validation aid */
#define PTO_LI_UNSORTED 0x2   /* leave the selected indices unordered (default: value-descending) */
#define PTO_LI_FP16_CHAIN 0x4 /* the older formulation of the score, LightningIndexerTopkImpl
                               * (framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:150-196):
                               * fp16(dot * 2^-11), x q_scale, x k_scale, relu, x weight all in fp16, head sum in
                               * fp32; scales and weights must be fp16 */
#define PTO_LI_EPILOGUE_HIST 0x8 /* decode / fused entries with at most two query tokens per sequence: the score
                               * kernel also leaves a 4096-bin histogram of every row (top 12 bits of the
                               * order-preserving image of the score) and the selection starts from it instead
                               * of scanning the row for min/max and its own histogram. Same results. Measured
                               * 1.3 us slower per step on the benchmark configuration (the scans it saves read
                               * L2-resident rows; the histogram costs a memset, shared-memory atomics in the score
                               * epilogue and a flush), so it is off unless asked for. */

/* device status area at the start of every workspace */
#define PTO_STATUS_WORDS 8
#define PTO_ST_BAD_PAGE 0x1    /* a block-table entry or top-k index outside its range was skipped */
#define PTO_ST_WAIT_EXPIRED 0x2 /* a bounded mbarrier wait gave up; results are incomplete */

int pto_abi_version(void);
const char* pto_strerror(int code);
const char* pto_last_error(void);
/* Kernels of this library enqueued so far by this process (every kernel of every entry point): a
 * diagnostic that a call reached the CUDA path. A launch recorded during stream capture counts once, at
 * capture time. No counterpart in the reference. */
long long pto_launch_count(void);

/* Copies the status words of `workspace` to `host_out[PTO_STATUS_WORDS]` and synchronises `stream`. */
int pto_workspace_status(const void* workspace, int32_t* host_out, pto_stream_t stream);
/* Clears the status area (asynchronous on `stream`). */
int pto_workspace_reset(void* workspace, pto_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Lightning indexer. Replaces `lightning_indexer_decode`
 * (examples/models/deepseek_v32_exp/lightning_indexer_quant_impl.py:315-346; score stage :138-194,
 * top-k stage :196-312; golden deepseekv32_lightning_indexer_quant.py:184-269).
 *
 *   idx_query        int8  [t, n_heads=64, head_dim=128]
 *   idx_query_scale  f16|f32 [t, 64]
 *   idx_key_cache    int8  [block_num, block_size=128, 1, 128]
 *   idx_key_scale    f16|f32 [block_num, 128, 1]
 *   idx_weight       f16|f32 [t, 64]
 *   act_seq_key      int32 [b]
 *   block_table      int32 [b, max_blocks]   (-1 in unused slots)
 *   topk_res         int32 [t, 1, selected_count]   out; value-descending, -1 padded
 *
 * score[pos] = k_scale[pos] * sum_h fp32(q_scale_h*weight_h) * fp32(fp16(relu(q_h.k[pos]) / 2048)),
 * top-k over pos < S_b - (s1 - 1 - i).
 * ------------------------------------------------------------------------------------------ */
size_t pto_li_workspace_bytes(int t, int max_blocks, int block_size);

int pto_li_decode(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                  const void* idx_key_scale, const void* idx_weight, int scale_dtype,
                  const int32_t* act_seq_key, const int32_t* block_table, int32_t* topk_res,
                  int b, int s1, int n_heads, int head_dim, int block_size, int block_num,
                  int max_blocks, int selected_count, int flags,
                  void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* Score stage alone (the reference ST's `mm_out` hook,
 * framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_lightning_indexer.py:282-360).
 * scores: f32 [t, max_blocks*block_size]; positions >= S_b are left untouched.
 * first_mm (optional, may be NULL; SIMT path only): f16 [t*64, max_blocks*block_size]. */
int pto_li_scores(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                  const void* idx_key_scale, const void* idx_weight, int scale_dtype,
                  const int32_t* act_seq_key, const int32_t* block_table, float* scores, void* first_mm,
                  int b, int s1, int n_heads, int head_dim, int block_size, int block_num,
                  int max_blocks, int flags, void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* Non-quantised lightning indexer. Replaces `LightningIndexerTopk` / `LightningIndexerTopkImpl` with isQuant = false
 * (framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:113-147, :23-58; golden
 * `indexer_topk_compute(is_quant=False)`,
 * framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_lightning_indexer.py:189-279).
 *
 *   idx_query      bf16 [t, 64, 128]       idx_key_cache  bf16 [block_num, 128, 1, 128]
 *   idx_weight     bf16 [t, 64]            no scale tensors
 *
 * score[pos] = sum_h fp32(weight_h) * relu(fp32(q_h . k[pos])), top-k as above. `flags`: PTO_LI_UNSORTED only.
 * `pto_li_scores_bf16` is the score stage alone (the reference's `tmpOut` hook, lightning_indexer.cpp:142-145):
 * scores f32 [t, max_blocks*block_size], positions >= S_b left untouched. */
int pto_li_decode_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                       const int32_t* act_seq_key, const int32_t* block_table, int32_t* topk_res,
                       int b, int s1, int n_heads, int head_dim, int block_size, int block_num,
                       int max_blocks, int selected_count, int flags,
                       void* workspace, size_t workspace_bytes, pto_stream_t stream);
int pto_li_scores_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                       const int32_t* act_seq_key, const int32_t* block_table, float* scores,
                       int b, int s1, int n_heads, int head_dim, int block_size, int block_num,
                       int max_blocks, int flags, void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* Lightning indexer for callers that cannot allocate device memory. No counterpart in the
 * reference: it exists for hosts of this library that run where cudaMalloc is off limits - inside
 * a serving engine whose memory pool owns all of HBM, or in a process that must not touch the
 * allocator while another component is capturing a CUDA graph. Same arguments and results as
 * `pto_li_decode`, minus the workspace: the fp32 score rows and the status words live in a
 * file-scope `static __device__` array of PTO_LI_STATIC_SCRATCH_BYTES that every GPU loading the
 * library holds until the process exits.
 *   - limit: t * max_blocks * block_size * 4 bytes of score rows may not exceed 8 MiB (the array is
 *     8 MiB + 256 bytes of status words), otherwise PTO_ERR_WORKSPACE is returned and nothing is
 *     launched (t = 16 tokens at 131072 keys, or 64 tokens at 32768 keys, just fit);
 *   - the first call on a device resolves the array's device address (cudaGetSymbolAddress, with
 *     that device current) and caches it; make that first call outside of any stream capture;
 *   - all calls share the one array and it keeps the previous call's contents; the status words
 *     are cleared at the start of each call, every score that is read is written first. Two calls
 *     that overlap on the GPU (different streams) race on it: serialise them;
 *   - `status_out` (host, PTO_STATUS_WORDS ints, may be NULL) receives the status words after the
 *     call; passing it synchronises the stream, so it is refused (PTO_ERR_INVALID) while `stream`
 *     is being captured. With NULL, read the words later with `pto_li_static_status`, before the
 *     next call clears them. After PTO_ST_WAIT_EXPIRED the indices are undefined. */
#define PTO_LI_STATIC_SCRATCH_BYTES ((8u << 20) + 256u)
int pto_li_decode_static(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                         const void* idx_key_scale, const void* idx_weight, int scale_dtype,
                         const int32_t* act_seq_key, const int32_t* block_table, int32_t* topk_res,
                         int b, int s1, int n_heads, int head_dim, int block_size, int block_num,
                         int max_blocks, int selected_count, int flags, int32_t* status_out,
                         pto_stream_t stream);

/* Status words left by the last `pto_li_decode_static` call on the current device (synchronises
 * `stream`; no counterpart in the reference). */
int pto_li_static_status(int32_t* host_out, pto_stream_t stream);

/* Top-k stage alone over f32 score rows with row stride `row_stride` elements
 * (TopKSort/Merge/Extract semantics, lightning_indexer_quant_impl.py:196-312: exact, -1 padded). */
int pto_li_topk(const float* scores, int64_t row_stride, const int32_t* act_seq_key, int32_t* topk_res,
                int b, int s1, int selected_count, int flags, void* workspace, size_t workspace_bytes,
                pto_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Sparse MLA attention over the selected rows. Replaces `sparse_flash_attention_quant_d/_p`
 * (examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:420-476, :479-538; body
 * :45-207; golden deepseekv32_sparse_flash_attention_quant.py:169-254).
 *
 *   query_nope     bf16 [t*nq, 512]       query_rope   bf16 [t*nq, 64]
 *   key_nope_2d    int8 [n_rows, 512]     key_rope_2d  bf16 [n_rows, 64]
 *   k_nope_scales  f32  [n_rows, 4]       topk_indices int32 [t, topk]
 *   block_table    int32 [b, max_blocks]  kv_act_seqs  int32 [b]
 *   attention_out  bf16 [b, s1, nq, 512]  out (rows of tokens that see no key are zeroed)
 *
 * Head slices: the query and output arrays hold `nq_total` heads per token; the call processes
 * heads [head_begin, head_begin + nq) of every token and touches no other output row. Pass
 * nq_total = nq and head_begin = 0 for whole tokens.
 * ------------------------------------------------------------------------------------------ */
size_t pto_sfa_workspace_bytes(int t, int nq);

int pto_sfa_quant(const void* query_nope, const void* query_rope, const int8_t* key_nope_2d,
                  const void* key_rope_2d, const float* k_nope_scales, const int32_t* topk_indices,
                  const int32_t* block_table, const int32_t* kv_act_seqs, void* attention_out,
                  int b, int s1, int nq, int n_kv, float softmax_scale, int topk, int block_size,
                  int64_t n_rows, int max_blocks, int nq_total, int head_begin,
                  void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* Non-quantised latent cache: the same operator called with a bf16 `key_nope_2d` [n_rows, 512]
 * (sparse_flash_attention_quant_impl.py:149-153 and :199-202 take the rows as they are when the dtype
 * is not int8; golden deepseekv32_sparse_flash_attention_quant.py:216-221 with is_kn_quant = 0). No
 * scales. Only nq == 128 (all heads of a token); other widths return PTO_ERR_UNSUPPORTED. */
int pto_sfa_bf16(const void* query_nope, const void* query_rope, const void* key_nope_2d,
                 const void* key_rope_2d, const int32_t* topk_indices, const int32_t* block_table,
                 const int32_t* kv_act_seqs, void* attention_out, int b, int s1, int nq, int n_kv,
                 float softmax_scale, int topk, int block_size, int64_t n_rows, int max_blocks,
                 int nq_total, int head_begin, void* workspace, size_t workspace_bytes,
                 pto_stream_t stream);

/* Packed-row variant. Replaces `sparse_attention_antiquant_d/_p`
 * (examples/models/deepseek_v32_exp/sparse_attention_antiquant_impl.py:246-358; golden
 * deepseekv32_sparse_attention_antiquant.py:49-136). nope_cache: int8 [n_rows, 656] =
 * 512 int8 latent | 64 bf16 rope | 4 f32 scales. */
int pto_sfa_packed(const void* query_nope, const void* query_rope, const int8_t* nope_cache,
                   const int32_t* topk_indices, const int32_t* block_table, const int32_t* kv_act_seqs,
                   void* attention_out, int b, int s1, int nq, int n_kv, float softmax_scale, int topk,
                   int block_size, int64_t n_rows, int max_blocks, int nq_total, int head_begin,
                   void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * MLA + lightning-indexer prolog: produces every input of the entry points above from the
 * token's hidden state and writes the token's rows into the paged caches. Replaces
 * `mla_indexer_prolog_quant_d/_p` (examples/models/deepseek_v32_exp/
 * mla_indexer_prolog_quant_impl.py:37-139, :142-256; bodies mla_prolog_quant_impl.py:502-707 and
 * lightning_indexer_prolog_quant_impl.py:325-504; goldens deepseekv32_mla_indexer_prolog_quant.py
 * :409-541 and :544-614), in the configuration the example runs: bf16 down-projections, int8
 * up-projection of the normalised query with per-column scales, int8 latent cache.
 *
 *   token_x   bf16 [t, hidden]                 cos, sin   bf16 [t, 64]      cache_index int64 [t]
 *   w_dq      bf16 [hidden, q_lora]            w_uqqr     int8 [q_lora, 128*192], w_qb_scale f32 [128*192]
 *   w_uk      bf16 [128, 128, 512]             w_dkvkr    bf16 [hidden, 576]
 *   gamma_cq  bf16 [q_lora]                    gamma_ckv  bf16 [512]
 *   w_idx_qb  int8 [q_lora, 64*128], w_idx_qb_scale f32 [64*128]
 *   w_idx_k   bf16 [hidden, 128]               w_idx_proj bf16 [hidden, 64]
 *   ln_gamma, ln_beta bf16 [128]               hadamard_q, hadamard_k bf16 [128, 128]
 * updated in place (row cache_index[i] of each, rows outside [0, cache_rows) are skipped and
 * reported as PTO_ST_BAD_PAGE):
 *   kv_cache int8 [cache_rows, 512]   kr_cache bf16 [cache_rows, 64]   kv_scale_cache f32 [cache_rows, 4]
 *   idx_k_cache int8 [cache_rows, 128]   idx_k_scale_cache f16 [cache_rows]
 * outputs:
 *   query_nope_out bf16 [t, 128, 512]   query_rope_out bf16 [t, 128, 64]
 *   q_int8_out int8 [t, 64, 128]        q_scale_out f16 [t, 64]        weights_out f16 [t, 64]
 *
 * The seven projections and everything between them are this library's kernels (no GEMM library is loaded):
 * the bf16 projections of the hidden state are split over K and leave fp32 partials in the workspace that the
 * kernels reading them add in a fixed order, so the call is deterministic. No allocation: the call can be
 * recorded into a CUDA graph.
 * ------------------------------------------------------------------------------------------ */
size_t pto_prolog_workspace_bytes(int t, int hidden, int q_lora);

/* The packed cache format as the native one: converts the three split arrays (int8 [n_rows, 512], bf16
 * [n_rows, 64], f32 [n_rows, 4]) into the 656-byte rows `pto_sfa_packed` reads (packing of
 * deepseekv32_sparse_attention_antiquant.py:258-268); afterwards the prolog keeps the packed cache current
 * through its `packed_kv_cache` argument. */
int pto_kv_pack_rows(const int8_t* key_nope_2d, const void* key_rope_2d, const float* k_nope_scales,
                     int64_t n_rows, int8_t* nope_cache, pto_stream_t stream);

/* Optional one-time weight preparation (the counterpart of the reference's cast of these weights to its
 * NZ format, deepseekv32_mla_indexer_prolog_quant.py:696-698, :721-725): the four projections of the token
 * share their left operand, so their weights are laid side by side, packed bf16
 * [hidden, q_lora + 576 + 128 + 64] = w_dq | w_dkvkr | w_idx_k | w_idx_proj, and become one product. */
int pto_prolog_pack_weights(const void* w_dq, const void* w_dkvkr, const void* w_idx_k,
                            const void* w_idx_proj, int hidden, int q_lora, void* packed,
                            pto_stream_t stream);

int pto_mla_indexer_prolog_quant(
    const void* token_x, const void* w_dq, const int8_t* w_uqqr, const float* w_qb_scale,
    const void* w_uk, const void* w_dkvkr, const void* gamma_cq, const void* gamma_ckv,
    const void* cos, const void* sin, const int64_t* cache_index, int8_t* kv_cache, void* kr_cache,
    float* kv_scale_cache, const int8_t* w_idx_qb, const float* w_idx_qb_scale, const void* w_idx_k,
    const void* w_idx_proj, const void* ln_gamma, const void* ln_beta, const void* hadamard_q,
    const void* hadamard_k, int8_t* idx_k_cache, void* idx_k_scale_cache, void* query_nope_out,
    void* query_rope_out, int8_t* q_int8_out, void* q_scale_out, void* weights_out,
    const void* w_x_packed /* from pto_prolog_pack_weights, or NULL: four separate products */,
    int8_t* packed_kv_cache /* int8 [cache_rows, 656] or NULL: the token's row is also written there */,
    int t, int hidden, int q_lora, int64_t cache_rows, float eps_cq, float eps_ckv, float ln_eps,
    void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* The two prologs in front of the non-quantised chain, in one call: `MlaPrologComputeV32` without
 * quantisation (framework/src/operator/models/deepseek_v3.2_exp/dynamic_mla_v32.cpp:187-345) and
 * `LightningIndexerPrologCompute` (.../lightning_indexer_prolog.cpp:129-227) on its normalised query, as
 * `DecodeIndexerAttention` runs them (.../decode_indexer_attention.cpp:85-106). Arithmetic of the system tests'
 * goldens (framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_mla_prolog_golden_v32.py:176-303,
 * gen_lightning_indexer_prolog.py:253-293): every product is rounded to bf16 once, all ropes de-interleave,
 * the indexer key is LayerNorm(fp32 product) -> bf16 -> rope, the weights are bf16(x . w_idx_proj).
 *
 *   as pto_mla_indexer_prolog_quant, except:
 *   w_uqqr bf16 [q_lora, 128*192]    w_idx_qb bf16 [q_lora, 64*128]    no scales, no Hadamard matrices
 *   kv_cache bf16 [cache_rows, 512]  kr_cache bf16 [cache_rows, 64]    idx_k_cache bf16 [cache_rows, 128]
 *   idx_query_out bf16 [t, 64, 128]  weights_out bf16 [t, 64]
 *   q_norm_out bf16 [t, q_lora] or NULL: the normalised query (the reference's `rmsRes`)
 *
 * The outputs are what pto_li_decode_bf16 / pto_sfa_bf16 / pto_decode_fused_bf16 take. Same workspace rules as
 * the quantised prolog; size from pto_prolog_nonquant_workspace_bytes. */
size_t pto_prolog_nonquant_workspace_bytes(int t, int hidden, int q_lora);

int pto_mla_indexer_prolog(
    const void* token_x, const void* w_dq, const void* w_uqqr, const void* w_uk, const void* w_dkvkr,
    const void* gamma_cq, const void* gamma_ckv, const void* cos, const void* sin, const int64_t* cache_index,
    void* kv_cache, void* kr_cache, const void* w_idx_qb, const void* w_idx_k, const void* w_idx_proj,
    const void* ln_gamma, const void* ln_beta, void* idx_k_cache, void* query_nope_out, void* query_rope_out,
    void* idx_query_out, void* weights_out, void* q_norm_out,
    const void* w_x_packed /* from pto_prolog_pack_weights, or NULL */,
    int t, int hidden, int q_lora, int64_t cache_rows, float eps_cq, float eps_ckv, float ln_eps,
    void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Fused decode chain: indexer -> top-k -> sparse attention on one stream, the order of
 * `DeepSeekIndexerAttentionQuant`
 * (framework/src/operator/models/deepseek_v3.2_exp/deepseek_indexer_attention_quant.cpp:170-250).
 * Both caches share `block_table` / `act_seq`. topk_res (int32 [t,1,selected_count]) is written
 * too (unordered unless PTO_LI_UNSORTED is cleared in `flags`).
 * ------------------------------------------------------------------------------------------ */
size_t pto_decode_workspace_bytes(int t, int max_blocks, int block_size, int nq);

int pto_decode_fused(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                     const void* idx_key_scale, const void* idx_weight, int scale_dtype,
                     const void* query_nope, const void* query_rope, const int8_t* key_nope_2d,
                     const void* key_rope_2d, const float* k_nope_scales,
                     const int32_t* act_seq, const int32_t* block_table,
                     int32_t* topk_res, void* attention_out,
                     int b, int s1, int block_num, int max_blocks, int selected_count, int nq,
                     float softmax_scale, int flags,
                     void* workspace, size_t workspace_bytes, pto_stream_t stream);

/* The non-quantised chain: bf16 indexer -> top-k -> sparse attention over the bf16 latent cache, the part of
 * `DecodeIndexerAttention` behind its two prologs
 * (framework/src/operator/models/deepseek_v3.2_exp/decode_indexer_attention.cpp:108-129:
 * LightningIndexerTopk -> GatherAfterPrologCompute -> SparseFlashAttentionCompute). key_nope_2d is
 * bf16 [block_num*128, 512]; nq must be 128. Workspace: pto_decode_workspace_bytes. */
int pto_decode_fused_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                          const void* query_nope, const void* query_rope, const void* key_nope_2d,
                          const void* key_rope_2d, const int32_t* act_seq, const int32_t* block_table,
                          int32_t* topk_res, void* attention_out,
                          int b, int s1, int block_num, int max_blocks, int selected_count, int nq,
                          float softmax_scale, int flags,
                          void* workspace, size_t workspace_bytes, pto_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PYPTO_B200_H_ */
