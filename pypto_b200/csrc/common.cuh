// Shared device helpers: PTX wrappers for mbarrier, TMA (no multicast), tcgen05/TMEM, plus the
// parameter blocks passed from the C ABI to the kernels. sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pypto_b200.h"

namespace pto {

// ---------------------------------------------------------------------------------------------
// status area (first PTO_STATUS_WORDS int32 of every workspace)
// word 0: OR of PTO_ST_* flags; word 1: first offending value; word 2: site id of an expired wait
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void set_status(int32_t* status, int flag, int detail, int site = 0) {
  if (status == nullptr) return;
  int old = atomicOr(status, flag);
  if ((old & flag) == 0) {
    status[1] = detail;
    status[2] = site;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// non-blocking probe of a phase
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream still runs; `pdl_wait` blocks until that predecessor has completed and
// its writes are visible (a no-op in a kernel launched the ordinary way). `pdl_trigger` lets the successor
// start early. Rule kept throughout: a kernel triggers only after its own wait, and the first kernel of a
// chain is launched the ordinary way, so a successor that is running implies that everything before the
// chain has completed.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Bounded wait: gives up after ~`kWaitBudgetCycles` SM clocks and returns false. Every spin in the
// library goes through this, so a protocol error turns into a status word, not a hang.
constexpr long long kWaitBudgetCycles = 2000000000LL;  // about one second at 2 GHz

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

// Same bound, but polling with the non-blocking probe: a blocked try_wait was measured to resume
// about a microsecond after the phase completes, which is too slow for per-tile hand-offs.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      if (mbar_test_wait(bar, parity)) return true;
    }
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

// Warp-wide form (all 32 lanes call it, converged): every lane polls and the outcome is made uniform.
// Polling from one lane while the others wait at a shuffle was measured slower (the divergent
// section costs more than the 31 extra probes).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait_spin(bar, parity));
}

// ---------------------------------------------------------------------------------------------
// TMA: tiled 2-D load global -> shared, completion on an mbarrier. No multicast anywhere.
// x is the innermost (contiguous) coordinate and must make x * elem_size a multiple of 16 bytes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// The same load for data that is read once (a stream much larger than L2): the lines are the first to be evicted,
// so that what the kernel writes for its successor stays in L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const void* tmap, int x, int y, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
// untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrives (count 1) on the mbarrier once all previously issued tcgen05.mma of this thread completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, int8 x int8 -> int32
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// bf16/f16 x bf16/f16 -> f32
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes, groups of
// 8 rows 1024 bytes apart (tile base 1024-byte aligned). Advance along K inside the 128-byte row by
// adding (bytes >> 4) to the low word.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// Instruction descriptor fields (dense, no negate, no saturate)
constexpr uint32_t kCFmtF32 = 1, kCFmtS32 = 2;
constexpr uint32_t kABFmtBF16 = 1, kABFmtS8 = 1;
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                  uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// TMEM -> registers: this warp's 32 lanes, 32 consecutive 32-bit columns each
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred)
      :
      : "memory");
  return pred != 0;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// kernel launchers (defined in the .cu files, called from capi.cu)
// ---------------------------------------------------------------------------------------------
// Every launcher counts the kernels it enqueues (read back through pto_launch_count): a caller can check
// that its call reached this library's kernels, and how many of them.
void count_launch(int n = 1);

struct LiParams {
  const int8_t* q;          // [t*64, 128]
  const void* q_scale;      // [t, 64]
  const int8_t* k_cache;    // [block_num*128, 128]
  const void* k_scale;      // [block_num*128]
  const void* weight;       // [t, 64]
  int scale_dtype;          // PTO_DT_*
  const int32_t* act_seq;   // [b]
  const int32_t* block_table;  // [b, max_blocks]
  float* scores;            // [t, row_stride]
  void* first_mm;           // optional f16 [t*64, row_stride] (SIMT path)
  int64_t row_stride;
  int b, s1, block_num, max_blocks;
  int fp16_chain;  // PTO_LI_FP16_CHAIN: the older formulation of the score
  int bf16;        // non-quantised formulation: q, k_cache and weight are bf16, the scales are not read
  int s1_total;    // query tokens per sequence in memory (>= s1)
  int tok_offset;  // first token of each sequence handled by this launch
  int groups;      // token groups of s1 tokens taken by one launch (grid y; tensor-core kernel), >= 1
  // optional, tensor-core kernel with s1 <= 2 per launch: per query token a histogram [t, kLiHistBins] (zeroed by the
  // caller) of the scores at positions below the token's causal end, binned by the top 12 bits of the
  // order-preserving image of the float; the top-k kernel starts from it instead of scanning the row for one
  unsigned int* hist;
  int32_t* status;
};
constexpr int kLiHistBins = 4096;
constexpr int kLiHistShift = 20;  // bin = order(score) >> 20: sign, exponent, three mantissa bits
constexpr int kLiHistMaxS1 = 2;   // tokens per launch the score kernel keeps a shared-memory histogram for
__device__ __forceinline__ unsigned int li_float_order(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct TopkParams {
  const float* scores;
  int64_t row_stride;
  const int32_t* act_seq;
  int32_t* out;  // [t, k]
  int b, s1, k, flags;
  const unsigned int* hist;  // optional [t, kLiHistBins] from the score kernel (see LiParams::hist)
  int32_t* status;
};

struct SfaParams {
  const __nv_bfloat16* q_nope;  // [t*nq_total, 512]
  const __nv_bfloat16* q_rope;  // [t*nq_total, 64]
  const int8_t* kn;             // [n_rows, 512]   (packed rows when packed != 0; bf16 [n_rows, 512] when kn_bf16 != 0)
  const __nv_bfloat16* kr;      // [n_rows, 64]
  const float* kn_scales;       // [n_rows, 4]     (unused when kn_bf16 != 0)
  const int32_t* topk;          // [t, topk]
  const int32_t* block_table;   // [b, max_blocks]
  const int32_t* act_seq;       // [b]
  __nv_bfloat16* out;           // [t, nq_total, 512]
  float* part_o;                // [t, n_split, nq, 512]
  float* part_ml;               // [t, n_split, nq, 2]
  int b, s1, nq, nq_total, head_begin, topk_k, block_size, max_blocks, n_split, packed, kn_bf16;
  int pdl;  // launched behind the top-k kernel with programmatic serialization: setup overlaps the selection
  int64_t n_rows;
  float scale_log2;  // softmax_scale * log2(e)
  int32_t* status;
};

cudaError_t launch_li_score_tc(const LiParams& p, const void* tmap_k, const void* tmap_q, int num_sms,
                               cudaStream_t stream);
cudaError_t launch_li_score_simt(const LiParams& p, cudaStream_t stream);
cudaError_t launch_li_topk(const TopkParams& p, int num_sms, cudaStream_t stream);
cudaError_t launch_sfa(const SfaParams& p, cudaStream_t stream);
cudaError_t launch_sfa_pair(const SfaParams& p, cudaStream_t stream);     // nq == 128, any cache format: 2-SM MMAs, heads split over the pair
int sfa_pair_split(int t, int num_sms);

// Launch with the programmatic-serialization attribute when `pdl`: the grid may be scheduled while the kernel
// before it in the stream drains, and must execute pdl_wait() before it touches global memory that kernel wrote.
template <typename... KArgs, typename... Args>
cudaError_t launch_maybe_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Prolog stages between the projections (prolog.cu). Fixed widths: 128 heads x (128 + 64), latent 512,
// rope 64, indexer 64 x 128. `ld`: row stride (elements) of the fp32 projection results, which arrive as `n_split`
// K-split partials `split_stride` elements apart and are added in split order by the kernels that read them.
cudaError_t launch_prolog_qnorm_quant(const float* qa, int ld, int n_split, long long split_stride, const void* gamma_cq,
                                      int t, int q_lora, float eps, int8_t* q_norm, float* q_norm_scale,
                                      cudaStream_t stream, bool pdl = false);
cudaError_t launch_prolog_qb_dequant_rope(const int32_t* qb_i32, const float* q_norm_scale, const float* w_scale,
                                          const void* cos, const void* sin, int t, void* q_b, void* q_rope,
                                          cudaStream_t stream, bool pdl = false);
cudaError_t launch_prolog_kv(const float* kv, const float* ki, const float* wp, int ld, int n_split,
                             long long split_stride, const void* gamma_ckv, const void* cos, const void* sin, const void* ln_gamma, const void* ln_beta, const void* hadamard_k,
                             const int64_t* cache_index, int64_t cache_rows, int t, float eps_ckv, float ln_eps,
                             int8_t* kv_cache, void* kr_cache, float* kv_scale_cache, int8_t* idx_k_cache,
                             void* idx_k_scale_cache, void* weights, int8_t* packed_cache, int32_t* status,
                             cudaStream_t stream);
// both int8 up-projections of the prolog in one tcgen05 launch (prolog_gemm.cu); t <= 64 token rows
bool prolog_i8_gemm_supported(int t, int k);
cudaError_t launch_prolog_i8_gemm(const void* tmap_w0, const void* tmap_w1, const void* tmap_x, int32_t* out0, int n0,
                                  int32_t* out1, int n1, int k, int t, int num_sms, int32_t* status, cudaStream_t stream,
                                  bool pdl = false);
// the weight-streaming products of the prolog (prolog_sgemm.cu)
int prolog_sgemm_rows(int t);
int prolog_sgemm_splits(int t, int n, int k, int num_sms);
cudaError_t launch_prolog_sgemm(int kind, const void* tmap_w, const void* tmap_x, void* out, int t, int n, int k,
                                int batch, int w_batch_rows, int x_batch_bytes, long long out_batch, long long ld_out,
                                int splits, long long split_stride, int num_sms, int32_t* status, cudaStream_t stream,
                                bool pdl = false);
cudaError_t launch_kv_pack_rows(const int8_t* kv, const void* kr, const float* sc, int64_t rows, int8_t* packed,
                                int num_sms, cudaStream_t stream);
cudaError_t launch_prolog_idxq(const int32_t* qi_i32, const float* q_norm_scale, const float* w_scale, const void* cos,
                               const void* sin, const void* hadamard_q, int t, int8_t* q_int8, void* q_scale,
                               cudaStream_t stream);
// stages of the two non-quantised prologs (bf16 caches, bf16 indexer query and weights)
cudaError_t launch_prolog_qnorm_bf16(const float* qa, int ld, int n_split, long long split_stride, const void* gamma_cq,
                                     int t, int q_lora, float eps, void* q_norm, cudaStream_t stream, bool pdl = false);
cudaError_t launch_prolog_kv_bf16(const float* kv, const float* ki, const float* wp, int ld, int n_split,
                                  long long split_stride, const void* gamma_ckv, const void* cos, const void* sin,
                                  const void* ln_gamma, const void* ln_beta, const int64_t* cache_index,
                                  int64_t cache_rows, int t, float eps_ckv, float ln_eps, void* kv_cache, void* kr_cache,
                                  void* idx_k_cache, void* weights, int32_t* status, cudaStream_t stream);
cudaError_t launch_prolog_rope_bf16(const void* q_b, const void* cos, const void* sin, int t, void* q_rope,
                                    void* idx_query, cudaStream_t stream, bool pdl = false);

}  // namespace pto
