// C ABI (include/pypto_b200.h): argument validation, workspace carving, TMA tensor maps, launches.
// No device memory is allocated here and nothing is kept between calls except cached device
// attributes.
#include <cuda.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pto {
int li_max_s1();
int li_max_sequences();
int topk_max_k();
}  // namespace pto

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define PTO_REQUIRE(cond, ...) \
  do {                         \
    if (!(cond)) return fail(PTO_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define PTO_CUDA(expr)                                                                       \
  do {                                                                                       \
    cudaError_t e__ = (expr);                                                                \
    if (e__ != cudaSuccess) return fail(PTO_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

constexpr size_t kStatusBytes = 256;
static_assert(PTO_STATUS_WORDS * sizeof(int32_t) <= kStatusBytes, "status area");

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceInfo {
  int device = -1;
  int cc_major = 0;
  int num_sms = 0;
};

int get_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = 0;
  PTO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(PTO_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev].device != dev) {
    DeviceInfo d;
    PTO_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    PTO_CUDA(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev));
    d.device = dev;
    cache[dev] = d;
  }
  *out = cache[dev];
  if (out->cc_major != 10) return fail(PTO_ERR_UNSUPPORTED, "compute capability %d.x: this library is sm_100a only", out->cc_major);
  return PTO_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* fn) {
  static std::mutex mu;
  static EncodeTiledFn cached = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cached == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || sym == nullptr) {
      return fail(PTO_ERR_DRIVER, "cuTensorMapEncodeTiled not available from the driver");
    }
    cached = reinterpret_cast<EncodeTiledFn>(sym);
  }
  *fn = cached;
  return PTO_OK;
}

// 2-D map over a byte matrix [rows, 128] with a [box_rows, 128] box and 128-byte swizzle.
int make_rows128_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn enc;
  int rc = get_encode_fn(&enc);
  if (rc != PTO_OK) return rc;
  cuuint64_t dims[2] = {128, rows};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PTO_ERR_DRIVER, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
  return PTO_OK;
}

size_t li_scores_bytes(int t, int max_blocks, int block_size) {
  return align_up(static_cast<size_t>(t) * max_blocks * block_size * sizeof(float), 256);
}

int sfa_split(int t, int nq) {
  const int n_hb = (nq + 63) / 64;
  const long long ctas = static_cast<long long>(t) * n_hb;
  if (ctas >= 148) return 1;
  long long s = 148 / (ctas > 0 ? ctas : 1);
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  return static_cast<int>(s);
}

size_t sfa_part_bytes(int t, int nq) {
  const int ns = sfa_split(t, nq);
  if (ns == 1) return 0;
  const size_t rows = static_cast<size_t>(t) * ns * nq;
  return align_up(rows * 2 * sizeof(float), 256) + align_up(rows * 512 * sizeof(float), 256);
}

int check_li_common(const void* q, const void* qs, const void* kc, const void* ks, const void* w, int scale_dtype,
                    const void* act, const void* bt, int b, int s1, int n_heads, int head_dim, int block_size,
                    int block_num, int max_blocks) {
  PTO_REQUIRE(q && qs && kc && ks && w && act && bt, "null tensor pointer");
  PTO_REQUIRE(scale_dtype == PTO_DT_F16 || scale_dtype == PTO_DT_F32, "scale_dtype %d is neither f16 nor f32", scale_dtype);
  PTO_REQUIRE(n_heads == 64 && head_dim == 128, "indexer shape %dx%d: only 64 heads x 128 dims", n_heads, head_dim);
  PTO_REQUIRE(block_size == 128, "block_size %d: only 128", block_size);
  PTO_REQUIRE(b >= 1 && b <= pto::li_max_sequences(), "batch %d outside [1, %d]", b, pto::li_max_sequences());
  PTO_REQUIRE(s1 >= 1, "s1 %d < 1", s1);
  PTO_REQUIRE(block_num >= 1 && max_blocks >= 1, "block_num %d / max_blocks %d", block_num, max_blocks);
  PTO_REQUIRE(static_cast<long long>(max_blocks) * block_size <= (1ll << 24), "context of %lld keys is too long",
              static_cast<long long>(max_blocks) * block_size);
  PTO_REQUIRE(aligned16(q) && aligned16(kc) && aligned16(ks), "idx_query / idx_key_cache / idx_key_scale must be 16-byte aligned");
  return PTO_OK;
}

// Score stage for tokens-per-sequence s1 (any s1 >= 1: groups of up to 4 tokens per launch).
int run_li_scores(const int8_t* q, const void* qs, const int8_t* kc, const void* ks, const void* w, int scale_dtype,
                  const int32_t* act, const int32_t* bt, float* scores, void* first_mm, int b, int s1, int block_num,
                  int max_blocks, int flags, int32_t* status, cudaStream_t stream) {
  pto::LiParams p{};
  p.q = q;
  p.q_scale = qs;
  p.k_cache = kc;
  p.k_scale = ks;
  p.weight = w;
  p.scale_dtype = scale_dtype;
  p.act_seq = act;
  p.block_table = bt;
  p.scores = scores;
  p.first_mm = first_mm;
  p.row_stride = static_cast<int64_t>(max_blocks) * 128;
  p.b = b;
  p.block_num = block_num;
  p.max_blocks = max_blocks;
  p.status = status;
  const bool simt = (flags & PTO_LI_SCORE_SIMT) != 0;
  PTO_REQUIRE(simt || first_mm == nullptr, "first_mm is only produced with PTO_LI_SCORE_SIMT");
  DeviceInfo di;
  CUtensorMap tmap_k, tmap_q;
  const int group = s1 < pto::li_max_s1() ? s1 : pto::li_max_s1();
  if (!simt) {
    int rc = get_device_info(&di);
    if (rc != PTO_OK) return rc;
    rc = make_rows128_map(&tmap_k, kc, static_cast<uint64_t>(block_num) * 128, 128);
    if (rc != PTO_OK) return rc;
  }
  // more than four query tokens per sequence (prefill chunks): one launch per group of tokens
  p.s1_total = s1;
  for (int off = 0; off < s1; off += group) {
    p.tok_offset = off;
    p.s1 = (s1 - off) < group ? (s1 - off) : group;
    if (simt) {
      PTO_CUDA(pto::launch_li_score_simt(p, stream));
    } else {
      int rc = make_rows128_map(&tmap_q, q, static_cast<uint64_t>(b) * s1 * 64, static_cast<uint32_t>(64 * p.s1));
      if (rc != PTO_OK) return rc;
      PTO_CUDA(pto::launch_li_score_tc(p, &tmap_k, &tmap_q, di.num_sms, stream));
    }
  }
  return PTO_OK;
}

int run_li_topk(const float* scores, int64_t row_stride, const int32_t* act, int32_t* out, int b, int s1, int k,
                int flags, int32_t* status, cudaStream_t stream) {
  PTO_REQUIRE(k >= 1 && k <= pto::topk_max_k(), "selected_count %d outside [1, %d]", k, pto::topk_max_k());
  PTO_REQUIRE(row_stride % 4 == 0 && aligned16(scores), "score rows must be 16-byte aligned");
  pto::TopkParams p{};
  p.scores = scores;
  p.row_stride = row_stride;
  p.act_seq = act;
  p.out = out;
  p.b = b;
  p.s1 = s1;
  p.k = k;
  p.flags = flags;
  p.status = status;
  DeviceInfo di;
  const int rc = get_device_info(&di);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(pto::launch_li_topk(p, di.num_sms, stream));
  return PTO_OK;
}

// `layout`: how the latent cache is stored
enum { kSfaSplitInt8 = 0, kSfaPackedInt8 = 1, kSfaSplitBf16 = 2 };

int run_sfa(const void* qn, const void* qr, const void* kn, const void* kr, const float* sc, int layout,
            const int32_t* topk_idx, const int32_t* bt, const int32_t* act, void* out, int b, int s1, int nq, int n_kv,
            float softmax_scale, int topk, int block_size, int64_t n_rows, int max_blocks, int nq_total, int head_begin,
            uint8_t* part_base, size_t part_bytes, int32_t* status, cudaStream_t stream) {
  PTO_REQUIRE(qn && qr && kn && topk_idx && bt && act && out, "null tensor pointer");
  const bool packed = layout == kSfaPackedInt8, bf16 = layout == kSfaSplitBf16;
  PTO_REQUIRE(packed || (kr && (sc || bf16)), "null tensor pointer");
  PTO_REQUIRE(n_kv == 1, "n_kv %d: only 1 (MLA latent cache)", n_kv);
  PTO_REQUIRE(b >= 1 && s1 >= 1, "b %d / s1 %d", b, s1);
  PTO_REQUIRE(nq >= 1 && nq % 16 == 0, "nq %d must be a positive multiple of 16", nq);
  PTO_REQUIRE(nq_total >= nq && head_begin >= 0 && head_begin + nq <= nq_total, "head slice [%d, %d) of %d", head_begin,
              head_begin + nq, nq_total);
  PTO_REQUIRE(topk >= 1 && block_size >= 1 && max_blocks >= 1 && n_rows >= 1, "topk/block_size/max_blocks/n_rows");
  PTO_REQUIRE(softmax_scale > 0.f, "softmax_scale %f", softmax_scale);
  PTO_REQUIRE(aligned16(qn) && aligned16(qr) && aligned16(kn) && aligned16(out) &&
                  (packed || (aligned16(kr) && (bf16 || aligned16(sc)))),
              "attention tensors must be 16-byte aligned");
  if (bf16 && nq != 128) {
    return fail(PTO_ERR_UNSUPPORTED, "bf16 latent cache: nq %d, only all 128 heads of a token are supported", nq);
  }
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != PTO_OK) return rc;
  const int t = b * s1;
  const int ns = sfa_split(t, nq);
  if (ns > 1 && part_bytes < sfa_part_bytes(t, nq)) return fail(PTO_ERR_WORKSPACE, "attention workspace too small");
  pto::SfaParams p{};
  p.q_nope = reinterpret_cast<const __nv_bfloat16*>(qn);
  p.q_rope = reinterpret_cast<const __nv_bfloat16*>(qr);
  p.kn = reinterpret_cast<const int8_t*>(kn);
  p.kr = reinterpret_cast<const __nv_bfloat16*>(kr);
  p.kn_scales = sc;
  p.topk = topk_idx;
  p.block_table = bt;
  p.act_seq = act;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  if (ns > 1) {
    const size_t rows = static_cast<size_t>(t) * ns * nq;
    p.part_ml = reinterpret_cast<float*>(part_base);
    p.part_o = reinterpret_cast<float*>(part_base + align_up(rows * 2 * sizeof(float), 256));
  }
  p.b = b;
  p.s1 = s1;
  p.nq = nq;
  p.nq_total = nq_total;
  p.head_begin = head_begin;
  p.topk_k = topk;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.n_split = ns;
  p.packed = packed ? 1 : 0;
  p.kn_bf16 = bf16 ? 1 : 0;
  p.n_rows = n_rows;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  PTO_CUDA(pto::launch_sfa(p, stream));
  return PTO_OK;
}

// Scratch of `pto_li_decode_static`: status words + fp32 score rows. In host code this name is only
// a stand-in for the device object; its device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_li_static_scratch[PTO_LI_STATIC_SCRATCH_BYTES];

// Device address of the static scratch on the current device, resolved once per device.
int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cache[64] = {nullptr};
  int dev = 0;
  PTO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(PTO_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_li_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      return fail(PTO_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    }
    cache[dev] = ptr;
  }
  *out = cache[dev];
  return PTO_OK;
}

int check_workspace(void* ws, size_t have, size_t need) {
  if (ws == nullptr) return fail(PTO_ERR_WORKSPACE, "workspace is null");
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return fail(PTO_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (have < need) return fail(PTO_ERR_WORKSPACE, "workspace of %zu bytes, %zu needed", have, need);
  return PTO_OK;
}

}  // namespace

extern "C" {

int pto_abi_version(void) { return PTO_ABI_VERSION; }

const char* pto_strerror(int code) {
  switch (code) {
    case PTO_OK: return "ok";
    case PTO_ERR_INVALID: return "invalid argument";
    case PTO_ERR_WORKSPACE: return "workspace null, misaligned or too small";
    case PTO_ERR_CUDA: return "CUDA runtime error";
    case PTO_ERR_UNSUPPORTED: return "unsupported device or feature";
    case PTO_ERR_DRIVER: return "driver tensor-map encoding failed";
    default: return "unknown error";
  }
}

const char* pto_last_error(void) { return g_err; }

int pto_workspace_status(const void* workspace, int32_t* host_out, pto_stream_t stream) {
  if (workspace == nullptr || host_out == nullptr) return fail(PTO_ERR_INVALID, "null pointer");
  PTO_CUDA(cudaMemcpyAsync(host_out, workspace, PTO_STATUS_WORDS * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  PTO_CUDA(cudaStreamSynchronize(stream));
  return PTO_OK;
}

int pto_workspace_reset(void* workspace, pto_stream_t stream) {
  if (workspace == nullptr) return fail(PTO_ERR_WORKSPACE, "workspace is null");
  PTO_CUDA(cudaMemsetAsync(workspace, 0, kStatusBytes, stream));
  return PTO_OK;
}

size_t pto_li_workspace_bytes(int t, int max_blocks, int block_size) {
  if (t < 1 || max_blocks < 1 || block_size < 1) return 0;
  return kStatusBytes + li_scores_bytes(t, max_blocks, block_size);
}

int pto_li_scores(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                  const void* idx_key_scale, const void* idx_weight, int scale_dtype, const int32_t* act_seq_key,
                  const int32_t* block_table, float* scores, void* first_mm, int b, int s1, int n_heads, int head_dim,
                  int block_size, int block_num, int max_blocks, int flags, void* workspace, size_t workspace_bytes,
                  pto_stream_t stream) {
  int rc = check_li_common(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype,
                           act_seq_key, block_table, b, s1, n_heads, head_dim, block_size, block_num, max_blocks);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(scores != nullptr && aligned16(scores), "scores must be a 16-byte aligned device pointer");
  rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq_key,
                       block_table, scores, first_mm, b, s1, block_num, max_blocks, flags,
                       reinterpret_cast<int32_t*>(workspace), stream);
}

int pto_li_topk(const float* scores, int64_t row_stride, const int32_t* act_seq_key, int32_t* topk_res, int b, int s1,
                int selected_count, int flags, void* workspace, size_t workspace_bytes, pto_stream_t stream) {
  PTO_REQUIRE(scores && act_seq_key && topk_res, "null tensor pointer");
  PTO_REQUIRE(b >= 1 && s1 >= 1 && row_stride >= 1, "b %d / s1 %d / row_stride %lld", b, s1, static_cast<long long>(row_stride));
  int rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_li_topk(scores, row_stride, act_seq_key, topk_res, b, s1, selected_count, flags,
                     reinterpret_cast<int32_t*>(workspace), stream);
}

int pto_li_decode(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                  const void* idx_key_scale, const void* idx_weight, int scale_dtype, const int32_t* act_seq_key,
                  const int32_t* block_table, int32_t* topk_res, int b, int s1, int n_heads, int head_dim,
                  int block_size, int block_num, int max_blocks, int selected_count, int flags, void* workspace,
                  size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_li_common(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype,
                           act_seq_key, block_table, b, s1, n_heads, head_dim, block_size, block_num, max_blocks);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(topk_res != nullptr, "topk_res is null");
  rc = check_workspace(workspace, workspace_bytes, pto_li_workspace_bytes(b * s1, max_blocks, block_size));
  if (rc != PTO_OK) return rc;
  int32_t* status = reinterpret_cast<int32_t*>(workspace);
  float* scores = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kStatusBytes);
  rc = run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq_key,
                     block_table, scores, nullptr, b, s1, block_num, max_blocks, flags, status, stream);
  if (rc != PTO_OK) return rc;
  return run_li_topk(scores, static_cast<int64_t>(max_blocks) * block_size, act_seq_key, topk_res, b, s1,
                     selected_count, flags, status, stream);
}

int pto_li_decode_static(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                         const void* idx_key_scale, const void* idx_weight, int scale_dtype,
                         const int32_t* act_seq_key, const int32_t* block_table, int32_t* topk_res, int b, int s1,
                         int n_heads, int head_dim, int block_size, int block_num, int max_blocks,
                         int selected_count, int flags, int32_t* status_out, pto_stream_t stream) {
  int rc = check_li_common(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype,
                           act_seq_key, block_table, b, s1, n_heads, head_dim, block_size, block_num, max_blocks);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(topk_res != nullptr, "topk_res is null");
  const size_t need = pto_li_workspace_bytes(b * s1, max_blocks, block_size);
  if (need == 0 || need > PTO_LI_STATIC_SCRATCH_BYTES) {
    return fail(PTO_ERR_WORKSPACE,
                "%d tokens x %d keys need %zu bytes of scratch, the static array holds %u: use pto_li_decode with "
                "a caller-allocated workspace",
                b * s1, max_blocks * block_size, need, static_cast<unsigned>(PTO_LI_STATIC_SCRATCH_BYTES));
  }
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);  // first call on this device: resolves and caches the address
  if (rc != PTO_OK) return rc;
  PTO_CUDA(cudaMemsetAsync(scratch, 0, kStatusBytes, stream));  // the status words must start at zero
  int32_t* status = reinterpret_cast<int32_t*>(scratch);
  float* scores = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + kStatusBytes);
  rc = run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq_key,
                     block_table, scores, nullptr, b, s1, block_num, max_blocks, flags, status, stream);
  if (rc != PTO_OK) return rc;
  rc = run_li_topk(scores, static_cast<int64_t>(max_blocks) * block_size, act_seq_key, topk_res, b, s1,
                   selected_count, flags, status, stream);
  if (rc != PTO_OK) return rc;
  if (status_out != nullptr) {
    PTO_CUDA(cudaMemcpyAsync(status_out, scratch, PTO_STATUS_WORDS * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    PTO_CUDA(cudaStreamSynchronize(stream));
  }
  return PTO_OK;
}

size_t pto_sfa_workspace_bytes(int t, int nq) {
  if (t < 1 || nq < 1) return 0;
  return kStatusBytes + sfa_part_bytes(t, nq);
}

int pto_sfa_quant(const void* query_nope, const void* query_rope, const int8_t* key_nope_2d, const void* key_rope_2d,
                  const float* k_nope_scales, const int32_t* topk_indices, const int32_t* block_table,
                  const int32_t* kv_act_seqs, void* attention_out, int b, int s1, int nq, int n_kv, float softmax_scale,
                  int topk, int block_size, int64_t n_rows, int max_blocks, int nq_total, int head_begin,
                  void* workspace, size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, 0, topk_indices, block_table,
                 kv_act_seqs, attention_out, b, s1, nq, n_kv, softmax_scale, topk, block_size, n_rows, max_blocks,
                 nq_total, head_begin, reinterpret_cast<uint8_t*>(workspace) + kStatusBytes,
                 workspace_bytes - kStatusBytes, reinterpret_cast<int32_t*>(workspace), stream);
}

int pto_sfa_bf16(const void* query_nope, const void* query_rope, const void* key_nope_2d, const void* key_rope_2d,
                 const int32_t* topk_indices, const int32_t* block_table, const int32_t* kv_act_seqs,
                 void* attention_out, int b, int s1, int nq, int n_kv, float softmax_scale, int topk, int block_size,
                 int64_t n_rows, int max_blocks, int nq_total, int head_begin, void* workspace,
                 size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, nullptr, kSfaSplitBf16, topk_indices, block_table,
                 kv_act_seqs, attention_out, b, s1, nq, n_kv, softmax_scale, topk, block_size, n_rows, max_blocks,
                 nq_total, head_begin, reinterpret_cast<uint8_t*>(workspace) + kStatusBytes,
                 workspace_bytes - kStatusBytes, reinterpret_cast<int32_t*>(workspace), stream);
}

int pto_sfa_packed(const void* query_nope, const void* query_rope, const int8_t* nope_cache,
                   const int32_t* topk_indices, const int32_t* block_table, const int32_t* kv_act_seqs,
                   void* attention_out, int b, int s1, int nq, int n_kv, float softmax_scale, int topk, int block_size,
                   int64_t n_rows, int max_blocks, int nq_total, int head_begin, void* workspace,
                   size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, nope_cache, nullptr, nullptr, 1, topk_indices, block_table, kv_act_seqs,
                 attention_out, b, s1, nq, n_kv, softmax_scale, topk, block_size, n_rows, max_blocks, nq_total,
                 head_begin, reinterpret_cast<uint8_t*>(workspace) + kStatusBytes, workspace_bytes - kStatusBytes,
                 reinterpret_cast<int32_t*>(workspace), stream);
}

size_t pto_decode_workspace_bytes(int t, int max_blocks, int block_size, int nq) {
  if (t < 1 || max_blocks < 1 || block_size < 1 || nq < 1) return 0;
  return kStatusBytes + li_scores_bytes(t, max_blocks, block_size) + sfa_part_bytes(t, nq);
}

int pto_decode_fused(const int8_t* idx_query, const void* idx_query_scale, const int8_t* idx_key_cache,
                     const void* idx_key_scale, const void* idx_weight, int scale_dtype, const void* query_nope,
                     const void* query_rope, const int8_t* key_nope_2d, const void* key_rope_2d,
                     const float* k_nope_scales, const int32_t* act_seq, const int32_t* block_table,
                     int32_t* topk_res, void* attention_out, int b, int s1, int block_num, int max_blocks,
                     int selected_count, int nq, float softmax_scale, int flags, void* workspace,
                     size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_li_common(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq,
                           block_table, b, s1, 64, 128, 128, block_num, max_blocks);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(topk_res != nullptr, "topk_res is null");
  rc = check_workspace(workspace, workspace_bytes, pto_decode_workspace_bytes(b * s1, max_blocks, 128, nq));
  if (rc != PTO_OK) return rc;
  uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(base);
  float* scores = reinterpret_cast<float*>(base + kStatusBytes);
  uint8_t* part = base + kStatusBytes + li_scores_bytes(b * s1, max_blocks, 128);
  rc = run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq,
                     block_table, scores, nullptr, b, s1, block_num, max_blocks, flags, status, stream);
  if (rc != PTO_OK) return rc;
  rc = run_li_topk(scores, static_cast<int64_t>(max_blocks) * 128, act_seq, topk_res, b, s1, selected_count, flags,
                   status, stream);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, 0, topk_res, block_table, act_seq,
                 attention_out, b, s1, nq, 1, softmax_scale, selected_count, 128, static_cast<int64_t>(block_num) * 128,
                 max_blocks, nq, 0, part, sfa_part_bytes(b * s1, nq), status, stream);
}

}  // extern "C"
