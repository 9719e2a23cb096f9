// C ABI (include/pypto_b200.h): argument validation, workspace carving, TMA tensor maps, launches.
// No device memory is allocated here and nothing is kept between calls except cached device
// attributes.
#include <cuda.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdlib>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pto {
static std::atomic<long long> g_launch_count{0};
void count_launch(int n) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }
int li_max_s1();
int li_max_s1_bf16();
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

// 2-D map over a byte matrix [outer, inner] (row pitch `pitch` bytes) with an [box_outer, box_inner] box and
// 128-byte swizzle; box_inner must be 128.
int make_bytes_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch, uint32_t box_outer) {
  EncodeTiledFn enc;
  int rc = get_encode_fn(&enc);
  if (rc != PTO_OK) return rc;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {128, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PTO_ERR_DRIVER, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
  return PTO_OK;
}

// histogram rows the score kernel leaves for the top-k kernel (LiParams::hist), at the end of a workspace
size_t li_hist_bytes(int t) { return align_up(static_cast<size_t>(t) * pto::kLiHistBins * sizeof(unsigned int), 256); }

size_t li_scores_bytes(int t, int max_blocks, int block_size) {
  return align_up(static_cast<size_t>(t) * max_blocks * block_size * sizeof(float), 256);
}

int sfa_split(int t, int nq) {
  if (nq == 128) return pto::sfa_pair_split(t, 148);  // one cluster of two CTAs per (token, split)
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

// Internal flag (never part of the ABI's `flags`): the non-quantised formulation, bf16 q / k_cache / weight.
constexpr int kLiFlagBf16 = 0x1000;

int check_li_bf16(const void* q, const void* kc, const void* w, const void* act, const void* bt, int b, int s1,
                  int n_heads, int head_dim, int block_size, int block_num, int max_blocks, int flags) {
  PTO_REQUIRE((flags & (PTO_LI_SCORE_SIMT | PTO_LI_FP16_CHAIN)) == 0,
              "flags 0x%x: the non-quantised indexer has one formulation and runs on the tensor cores only", flags);
  // the shape checks of the quantised entry, with the key cache standing in for the absent scale tensors
  return check_li_common(q, kc, kc, kc, w, PTO_DT_F16, act, bt, b, s1, n_heads, head_dim, block_size, block_num,
                         max_blocks);
}

// Score stage for tokens-per-sequence s1 (any s1 >= 1: groups of up to 4 tokens per launch).
int run_li_scores(const int8_t* q, const void* qs, const int8_t* kc, const void* ks, const void* w, int scale_dtype,
                  const int32_t* act, const int32_t* bt, float* scores, void* first_mm, int b, int s1, int block_num,
                  int max_blocks, int flags, int32_t* status, cudaStream_t stream, unsigned int* hist = nullptr) {
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
  if (hist != nullptr) {  // li_hist_usable() said yes: every launch below takes all s1 tokens of a sequence
    p.hist = hist;
    PTO_CUDA(cudaMemsetAsync(hist, 0, li_hist_bytes(b * s1), stream));
  }
  p.fp16_chain = (flags & PTO_LI_FP16_CHAIN) != 0 ? 1 : 0;
  p.bf16 = (flags & kLiFlagBf16) != 0 ? 1 : 0;
  PTO_REQUIRE(!p.fp16_chain || scale_dtype == PTO_DT_F16, "PTO_LI_FP16_CHAIN needs fp16 scales and weights");
  PTO_REQUIRE(!p.fp16_chain || first_mm == nullptr, "first_mm is not produced with PTO_LI_FP16_CHAIN");
  DeviceInfo di;
  CUtensorMap tmap_k, tmap_q;
  const int max_group = p.bf16 ? pto::li_max_s1_bf16() : pto::li_max_s1();
  const int group = s1 < max_group ? s1 : max_group;
  if (!simt) {
    int rc = get_device_info(&di);
    if (rc != PTO_OK) return rc;
    // bf16 rows are 256 bytes: the map's box is one 128-byte half of 128 rows
    rc = p.bf16 ? make_bytes_map(&tmap_k, kc, 256, static_cast<uint64_t>(block_num) * 128, 256, 128)
                : make_rows128_map(&tmap_k, kc, static_cast<uint64_t>(block_num) * 128, 128);
    if (rc != PTO_OK) return rc;
  }
  // more than four query tokens per sequence (prefill chunks): groups of four tokens; the tensor-core kernel
  // takes up to sixteen full groups per launch (grid y), a last partial group gets a launch of its own
  p.s1_total = s1;
  int off = 0;
  while (off < s1) {
    p.tok_offset = off;
    p.s1 = (s1 - off) < group ? (s1 - off) : group;
    p.groups = 1;
    if (simt) {
      PTO_CUDA(pto::launch_li_score_simt(p, stream));
    } else {
      const int full = (s1 - off) / group;
      if (p.s1 == group && full > 1) p.groups = full < 16 ? full : 16;
      int rc = p.bf16 ? make_bytes_map(&tmap_q, q, 256, static_cast<uint64_t>(b) * s1 * 64, 256, static_cast<uint32_t>(64 * p.s1))
                      : make_rows128_map(&tmap_q, q, static_cast<uint64_t>(b) * s1 * 64, static_cast<uint32_t>(64 * p.s1));
      if (rc != PTO_OK) return rc;
      PTO_CUDA(pto::launch_li_score_tc(p, &tmap_k, &tmap_q, di.num_sms, stream));
    }
    off += p.s1 * p.groups;
  }
  return PTO_OK;
}

// Whether the score stage of this call leaves a histogram for the top-k stage: tensor-core kernel, one launch
// that takes every query token of a sequence.
bool li_hist_usable(int s1, int flags) {
  return (flags & PTO_LI_EPILOGUE_HIST) != 0 && (flags & PTO_LI_SCORE_SIMT) == 0 && s1 <= pto::kLiHistMaxS1;
}

int run_li_topk(const float* scores, int64_t row_stride, const int32_t* act, int32_t* out, int b, int s1, int k,
                int flags, int32_t* status, cudaStream_t stream, const unsigned int* hist = nullptr) {
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
  p.hist = hist;
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
            uint8_t* part_base, size_t part_bytes, int32_t* status, cudaStream_t stream, int behind_topk = 0) {
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
  p.pdl = behind_topk;
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

// ---- per-device side stream of the prolog ------------------------------------------------------------
// The per-token kernel and the indexer-query kernel run beside the chain of products they do not depend on: a
// second stream and fork/join events per device, created at the first prolog call on that device.
struct PrologSide {
  cudaStream_t side[64] = {nullptr};
  cudaEvent_t ev[64][3] = {{nullptr}};
  std::mutex mu;          // guards the per-device set-up
  std::mutex dev_mu[64];  // a device's calls enqueue one after the other (they share its side stream and events)
};

PrologSide& prolog_side() {
  static PrologSide s;
  return s;
}

int prolog_side_stream(int* device) {
  PrologSide& b = prolog_side();
  std::lock_guard<std::mutex> lock(b.mu);
  int dev = 0;
  PTO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(PTO_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (b.side[dev] == nullptr) {
    PTO_CUDA(cudaStreamCreateWithFlags(&b.side[dev], cudaStreamNonBlocking));
    for (int i = 0; i < 3; ++i) PTO_CUDA(cudaEventCreateWithFlags(&b.ev[dev][i], cudaEventDisableTiming));
  }
  *device = dev;
  return PTO_OK;
}

// One weight-streaming product (prolog_sgemm.cu): out = x[t, k] . W[k, n] per problem of the batch.
// kind 0: bf16 -> fp32 partials, 1: bf16 -> bf16, 2: int8 -> int32. Row pitches in bytes.
int run_sgemm(int kind, const void* x, size_t x_pitch, const void* w, size_t w_pitch, int64_t w_rows, void* out, int t,
              int n, int k, int batch, int w_batch_rows, int x_batch_bytes, long long out_batch, long long ld_out,
              int splits, long long split_stride, int num_sms, int32_t* status, cudaStream_t stream, bool pdl = false) {
  alignas(64) CUtensorMap map_w, map_x;
  int rc = make_bytes_map(&map_w, w, w_pitch, static_cast<uint64_t>(w_rows), w_pitch, kind == 2 ? 128 : 64);
  if (rc != PTO_OK) return rc;
  rc = make_bytes_map(&map_x, x, x_pitch, static_cast<uint64_t>(t), x_pitch, static_cast<uint32_t>(pto::prolog_sgemm_rows(t)));
  if (rc != PTO_OK) return rc;
  PTO_CUDA(pto::launch_prolog_sgemm(kind, &map_w, &map_x, out, t, n, k, batch, w_batch_rows, x_batch_bytes, out_batch,
                                    ld_out, splits, split_stride, num_sms, status, stream, pdl));
  return PTO_OK;
}

// SM count the K-split of the hidden-state projections is planned for (the workspace size must not depend on the
// device the call later runs on; this library targets the 148-SM B200 only)
constexpr int kPlanSms = 148;

struct PrologWs {
  size_t status, xproj, q_norm, q_norm_scale, qb_i32, q_b, qi_i32, total;
  int splits;  // K-split partials of the hidden-state projections
};
constexpr int kXProjExtra = 576 + 128 + 64;  // columns after the q_lora ones: latent+rope key | indexer key | weights

// Rows of the int8 activation buffer: the resident-activation kernel's tensor map covers whole 16-row groups.
inline int prolog_int8_rows(int t) { return t < 64 ? 64 : t; }

PrologWs prolog_ws(int t, int hidden, int q_lora) {
  PrologWs w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align_up(bytes, 256);
    return at;
  };
  const size_t tt = static_cast<size_t>(t);
  const size_t tp = static_cast<size_t>(prolog_int8_rows(t));
  w.status = take(kStatusBytes);
  w.splits = pto::prolog_sgemm_splits(t, q_lora + kXProjExtra, hidden, kPlanSms);
  w.xproj = take(w.splits * tt * (q_lora + kXProjExtra) * 4);  // fp32 [splits, t, q_lora | 576 | 128 | 64]
  w.q_norm = take(tp * q_lora);
  w.q_norm_scale = take(tt * 4);
  w.qb_i32 = take(tp * 128 * 192 * 4);
  w.q_b = take(tt * 128 * 192 * 2);
  w.qi_i32 = take(tp * 64 * 128 * 4);
  w.total = off;
  return w;
}

struct PrologNqWs {
  size_t status, xproj, q_norm, q_b, total;
  int splits;
};

PrologNqWs prolog_nq_ws(int t, int hidden, int q_lora) {
  PrologNqWs w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align_up(bytes, 256);
    return at;
  };
  const size_t tt = static_cast<size_t>(t);
  w.status = take(kStatusBytes);
  w.splits = pto::prolog_sgemm_splits(t, q_lora + kXProjExtra, hidden, kPlanSms);
  w.xproj = take(w.splits * tt * (q_lora + kXProjExtra) * 4);
  w.q_norm = take(tt * q_lora * 2);      // bf16 [t, q_lora]
  w.q_b = take(tt * 128 * 192 * 2);      // bf16 [t, 128, 192]
  w.total = off;
  return w;
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

long long pto_launch_count(void) { return pto::g_launch_count.load(std::memory_order_relaxed); }

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
  return kStatusBytes + li_scores_bytes(t, max_blocks, block_size) + li_hist_bytes(t);
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
  unsigned int* hist = nullptr;  // behind the score rows
  if (li_hist_usable(s1, flags)) {
    hist = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(workspace) + kStatusBytes +
                                           li_scores_bytes(b * s1, max_blocks, block_size));
  }
  rc = run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq_key,
                     block_table, scores, nullptr, b, s1, block_num, max_blocks, flags, status, stream, hist);
  if (rc != PTO_OK) return rc;
  return run_li_topk(scores, static_cast<int64_t>(max_blocks) * block_size, act_seq_key, topk_res, b, s1,
                     selected_count, flags, status, stream, hist);
}

int pto_li_scores_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                       const int32_t* act_seq_key, const int32_t* block_table, float* scores, int b, int s1, int n_heads,
                       int head_dim, int block_size, int block_num, int max_blocks, int flags, void* workspace,
                       size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_li_bf16(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table, b, s1, n_heads, head_dim,
                         block_size, block_num, max_blocks, flags);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(scores != nullptr && aligned16(scores), "scores must be a 16-byte aligned device pointer");
  rc = check_workspace(workspace, workspace_bytes, kStatusBytes);
  if (rc != PTO_OK) return rc;
  return run_li_scores(reinterpret_cast<const int8_t*>(idx_query), nullptr, reinterpret_cast<const int8_t*>(idx_key_cache),
                       nullptr, idx_weight, PTO_DT_F16, act_seq_key, block_table, scores, nullptr, b, s1, block_num,
                       max_blocks, kLiFlagBf16, reinterpret_cast<int32_t*>(workspace), stream);
}

int pto_li_decode_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                       const int32_t* act_seq_key, const int32_t* block_table, int32_t* topk_res, int b, int s1,
                       int n_heads, int head_dim, int block_size, int block_num, int max_blocks, int selected_count,
                       int flags, void* workspace, size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_li_bf16(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table, b, s1, n_heads, head_dim,
                         block_size, block_num, max_blocks, flags);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(topk_res != nullptr, "topk_res is null");
  rc = check_workspace(workspace, workspace_bytes, pto_li_workspace_bytes(b * s1, max_blocks, block_size));
  if (rc != PTO_OK) return rc;
  int32_t* status = reinterpret_cast<int32_t*>(workspace);
  float* scores = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kStatusBytes);
  unsigned int* hist = nullptr;  // behind the score rows
  if (li_hist_usable(s1, flags)) {
    hist = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(workspace) + kStatusBytes +
                                           li_scores_bytes(b * s1, max_blocks, block_size));
  }
  rc = run_li_scores(reinterpret_cast<const int8_t*>(idx_query), nullptr, reinterpret_cast<const int8_t*>(idx_key_cache),
                     nullptr, idx_weight, PTO_DT_F16, act_seq_key, block_table, scores, nullptr, b, s1, block_num,
                     max_blocks, kLiFlagBf16, status, stream, hist);
  if (rc != PTO_OK) return rc;
  return run_li_topk(scores, static_cast<int64_t>(max_blocks) * block_size, act_seq_key, topk_res, b, s1,
                     selected_count, flags, status, stream, hist);
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
  if (status_out != nullptr) {  // reading the words back synchronises the stream, which a capture forbids
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    PTO_CUDA(cudaStreamIsCapturing(stream, &cap));
    PTO_REQUIRE(cap == cudaStreamCaptureStatusNone,
                "status_out must be NULL while the stream is being captured (read the words with pto_li_static_status)");
  }
  // status words and score rows; this entry keeps no histogram (the selection scans the row for its own)
  const size_t need = (b < 1 || s1 < 1) ? 0 : kStatusBytes + li_scores_bytes(b * s1, max_blocks, block_size);
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

int pto_li_static_status(int32_t* host_out, pto_stream_t stream) {
  PTO_REQUIRE(host_out != nullptr, "null pointer");
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(cudaMemcpyAsync(host_out, scratch, PTO_STATUS_WORDS * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  PTO_CUDA(cudaStreamSynchronize(stream));
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

size_t pto_prolog_workspace_bytes(int t, int hidden, int q_lora) {
  if (t < 1 || hidden < 1 || q_lora < 1) return 0;
  return prolog_ws(t, hidden, q_lora).total;
}

int pto_kv_pack_rows(const int8_t* key_nope_2d, const void* key_rope_2d, const float* k_nope_scales, int64_t n_rows,
                     int8_t* nope_cache, pto_stream_t stream) {
  PTO_REQUIRE(key_nope_2d && key_rope_2d && k_nope_scales && nope_cache, "null tensor pointer");
  PTO_REQUIRE(n_rows >= 1, "n_rows");
  PTO_REQUIRE(aligned16(key_nope_2d) && aligned16(key_rope_2d) && aligned16(k_nope_scales) && aligned16(nope_cache),
              "cache tensors must be 16-byte aligned");
  DeviceInfo di;
  const int rc = get_device_info(&di);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(pto::launch_kv_pack_rows(key_nope_2d, key_rope_2d, k_nope_scales, n_rows, nope_cache, di.num_sms, stream));
  return PTO_OK;
}

int pto_prolog_pack_weights(const void* w_dq, const void* w_dkvkr, const void* w_idx_k, const void* w_idx_proj, int hidden,
                            int q_lora, void* packed, pto_stream_t stream) {
  PTO_REQUIRE(w_dq && w_dkvkr && w_idx_k && w_idx_proj && packed, "null tensor pointer");
  PTO_REQUIRE(hidden >= 1 && q_lora >= 1, "hidden / q_lora");
  const size_t ld = static_cast<size_t>(q_lora + kXProjExtra) * 2;  // bytes per packed row (bf16)
  uint8_t* dst = reinterpret_cast<uint8_t*>(packed);
  const void* src[4] = {w_dq, w_dkvkr, w_idx_k, w_idx_proj};
  const size_t width[4] = {static_cast<size_t>(q_lora) * 2, 576 * 2, 128 * 2, 64 * 2};
  size_t off = 0;
  for (int i = 0; i < 4; ++i) {
    PTO_CUDA(cudaMemcpy2DAsync(dst + off, ld, src[i], width[i], width[i], hidden, cudaMemcpyDeviceToDevice, stream));
    off += width[i];
  }
  return PTO_OK;
}

int pto_mla_indexer_prolog_quant(const void* token_x, const void* w_dq, const int8_t* w_uqqr, const float* w_qb_scale,
                                 const void* w_uk, const void* w_dkvkr, const void* gamma_cq, const void* gamma_ckv,
                                 const void* cos, const void* sin, const int64_t* cache_index, int8_t* kv_cache,
                                 void* kr_cache, float* kv_scale_cache, const int8_t* w_idx_qb,
                                 const float* w_idx_qb_scale, const void* w_idx_k, const void* w_idx_proj,
                                 const void* ln_gamma, const void* ln_beta, const void* hadamard_q,
                                 const void* hadamard_k, int8_t* idx_k_cache, void* idx_k_scale_cache,
                                 void* query_nope_out, void* query_rope_out, int8_t* q_int8_out, void* q_scale_out,
                                 void* weights_out, const void* w_x_packed, int8_t* packed_kv_cache, int t, int hidden,
                                 int q_lora,
                                 int64_t cache_rows, float eps_cq, float eps_ckv, float ln_eps, void* workspace,
                                 size_t workspace_bytes, pto_stream_t stream) {
  PTO_REQUIRE(token_x && w_dq && w_uqqr && w_qb_scale && w_uk && w_dkvkr && gamma_cq && gamma_ckv && cos && sin &&
                  cache_index && kv_cache && kr_cache && kv_scale_cache && w_idx_qb && w_idx_qb_scale && w_idx_k &&
                  w_idx_proj && ln_gamma && ln_beta && hadamard_q && hadamard_k && idx_k_cache && idx_k_scale_cache &&
                  query_nope_out && query_rope_out && q_int8_out && q_scale_out && weights_out,
              "null tensor pointer");
  PTO_REQUIRE(t >= 1 && t <= 65535, "t %d: 1..65535 tokens per call", t);
  PTO_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden %d must be a positive multiple of 8", hidden);
  PTO_REQUIRE(q_lora >= 16 && q_lora % 16 == 0 && q_lora <= 12288, "q_lora %d must be a multiple of 16, at most 12288",
              q_lora);
  PTO_REQUIRE(cache_rows >= 1, "cache_rows");
  PTO_REQUIRE(packed_kv_cache == nullptr || aligned16(packed_kv_cache), "packed_kv_cache must be 16-byte aligned");
  PTO_REQUIRE(eps_cq >= 0.f && eps_ckv >= 0.f && ln_eps >= 0.f, "negative epsilon");
  PTO_REQUIRE(aligned16(token_x) && aligned16(w_dq) && aligned16(w_uqqr) && aligned16(w_uk) && aligned16(w_dkvkr) &&
                  aligned16(w_idx_qb) && aligned16(w_idx_k) && aligned16(w_idx_proj) && aligned16(kv_cache) && aligned16(gamma_cq) &&
                  aligned16(query_nope_out),
              "prolog tensors must be 16-byte aligned");
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != PTO_OK) return rc;
  const PrologWs w = prolog_ws(t, hidden, q_lora);
  rc = check_workspace(workspace, workspace_bytes, w.total);
  if (rc != PTO_OK) return rc;
  uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(base + w.status);
  const int ld = q_lora + kXProjExtra;
  float* qa = reinterpret_cast<float*>(base + w.xproj);
  float* kv = qa + q_lora;
  float* ki = kv + 576;
  float* wp = ki + 128;
  int8_t* q_norm = reinterpret_cast<int8_t*>(base + w.q_norm);
  float* q_norm_scale = reinterpret_cast<float*>(base + w.q_norm_scale);
  int32_t* qb_i32 = reinterpret_cast<int32_t*>(base + w.qb_i32);
  void* q_b = base + w.q_b;
  int32_t* qi_i32 = reinterpret_cast<int32_t*>(base + w.qi_i32);

  int dev = 0;
  rc = prolog_side_stream(&dev);
  if (rc != PTO_OK) return rc;
  std::lock_guard<std::mutex> lock(prolog_side().dev_mu[dev]);
  cudaStream_t side = prolog_side().side[dev];
  cudaEvent_t* ev = prolog_side().ev[dev];

  // projections of the token: fp32 partials [splits][t, q_lora | 576 | 128 | 64] (K split over CTAs), added and
  // rounded where the golden rounds by the kernels that read them. One product when the caller has packed the four
  // weights side by side, else four.
  const int splits = w.splits;
  const long long split_stride = static_cast<long long>(t) * ld;
  const size_t x_pitch = static_cast<size_t>(hidden) * 2;
  if (w_x_packed != nullptr) {
    PTO_REQUIRE(aligned16(w_x_packed), "w_x_packed must be 16-byte aligned");
    rc = run_sgemm(0, token_x, x_pitch, w_x_packed, static_cast<size_t>(ld) * 2, hidden, qa, t, ld, hidden, 1, 0, 0, 0, ld,
                   splits, split_stride, di.num_sms, status, stream);
    if (rc != PTO_OK) return rc;
  } else {
    const void* ws[4] = {w_dq, w_dkvkr, w_idx_k, w_idx_proj};
    float* outs[4] = {qa, kv, ki, wp};
    const int ns[4] = {q_lora, 576, 128, 64};
    for (int i = 0; i < 4; ++i) {
      rc = run_sgemm(0, token_x, x_pitch, ws[i], static_cast<size_t>(ns[i]) * 2, hidden, outs[i], t, ns[i], hidden, 1, 0, 0,
                     0, ld, splits, split_stride, di.num_sms, status, stream);
      if (rc != PTO_OK) return rc;
    }
  }
  // fork: the per-token kernel (caches, indexer key, weights) needs only the projections
  PTO_CUDA(cudaEventRecord(ev[0], stream));
  PTO_CUDA(cudaStreamWaitEvent(side, ev[0], 0));
  PTO_CUDA(pto::launch_prolog_kv(kv, ki, wp, ld, splits, split_stride, gamma_ckv, cos, sin, ln_gamma, ln_beta, hadamard_k,
                                 cache_index, cache_rows, t, eps_ckv, ln_eps, kv_cache, kr_cache, kv_scale_cache,
                                 idx_k_cache, idx_k_scale_cache, weights_out, packed_kv_cache, status, side));
  // from here on every kernel of the caller's stream follows a kernel of this call: each may be scheduled while
  // the one before it drains (it waits before it reads)
  PTO_CUDA(pto::launch_prolog_qnorm_quant(qa, ld, splits, split_stride, gamma_cq, t, q_lora, eps_cq, q_norm, q_norm_scale,
                                          stream, /*pdl=*/true));
  // int8 up-projections of the normalised query: one launch for both with the activations resident in shared
  // memory when the token rows fit (decode), else one streaming product per weight over blocks of 256 tokens
  const int tp = prolog_int8_rows(t);
  if (pto::prolog_i8_gemm_supported(t, q_lora)) {
    alignas(64) CUtensorMap map_w0, map_w1, map_x;
    rc = make_bytes_map(&map_w0, w_uqqr, 128 * 192, q_lora, 128 * 192, 128);
    if (rc != PTO_OK) return rc;
    rc = make_bytes_map(&map_w1, w_idx_qb, 64 * 128, q_lora, 64 * 128, 128);
    if (rc != PTO_OK) return rc;
    rc = make_bytes_map(&map_x, q_norm, q_lora, tp, q_lora, static_cast<uint32_t>((t + 15) / 16 * 16));
    if (rc != PTO_OK) return rc;
    PTO_CUDA(pto::launch_prolog_i8_gemm(&map_w0, &map_w1, &map_x, qb_i32, 128 * 192, qi_i32, 64 * 128, q_lora, t,
                                        di.num_sms, status, stream, /*pdl=*/true));
  } else {
    rc = run_sgemm(2, q_norm, q_lora, w_uqqr, 128 * 192, q_lora, qb_i32, t, 128 * 192, q_lora, 1, 0, 0, 0, 128 * 192, 1, 0,
                   di.num_sms, status, stream, /*pdl=*/true);
    if (rc != PTO_OK) return rc;
    rc = run_sgemm(2, q_norm, q_lora, w_idx_qb, 64 * 128, q_lora, qi_i32, t, 64 * 128, q_lora, 1, 0, 0, 0, 64 * 128, 1, 0,
                   di.num_sms, status, stream, /*pdl=*/true);
    if (rc != PTO_OK) return rc;
  }
  // the indexer-query kernel joins the side stream; the attention query finishes on the caller's
  PTO_CUDA(cudaEventRecord(ev[1], stream));
  PTO_CUDA(cudaStreamWaitEvent(side, ev[1], 0));
  PTO_CUDA(pto::launch_prolog_idxq(qi_i32, q_norm_scale, w_idx_qb_scale, cos, sin, hadamard_q, t, q_int8_out, q_scale_out,
                                   side));
  PTO_CUDA(cudaEventRecord(ev[2], side));
  PTO_CUDA(pto::launch_prolog_qb_dequant_rope(qb_i32, q_norm_scale, w_qb_scale, cos, sin, t, q_b, query_rope_out, stream,
                                              /*pdl=*/true));
  // absorbed nope part: per head [t, 128] (row pitch 128*192, head pitch 192 elements) @ w_uk[head] [128, 512] -> bf16
  rc = run_sgemm(1, q_b, 128 * 192 * 2, w_uk, 512 * 2, 128 * 128, query_nope_out, t, 512, 128, 128, 128, 192 * 2, 512,
                 128 * 512, 1, 0, di.num_sms, status, stream, /*pdl=*/true);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(cudaStreamWaitEvent(stream, ev[2], 0));  // join: everything is ordered before what the caller enqueues next
  return PTO_OK;
}

size_t pto_prolog_nonquant_workspace_bytes(int t, int hidden, int q_lora) {
  if (t < 1 || hidden < 1 || q_lora < 1) return 0;
  return prolog_nq_ws(t, hidden, q_lora).total;
}

int pto_mla_indexer_prolog(const void* token_x, const void* w_dq, const void* w_uqqr, const void* w_uk,
                           const void* w_dkvkr, const void* gamma_cq, const void* gamma_ckv, const void* cos,
                           const void* sin, const int64_t* cache_index, void* kv_cache, void* kr_cache,
                           const void* w_idx_qb, const void* w_idx_k, const void* w_idx_proj, const void* ln_gamma,
                           const void* ln_beta, void* idx_k_cache, void* query_nope_out, void* query_rope_out,
                           void* idx_query_out, void* weights_out, void* q_norm_out, const void* w_x_packed, int t,
                           int hidden, int q_lora, int64_t cache_rows, float eps_cq, float eps_ckv, float ln_eps,
                           void* workspace, size_t workspace_bytes, pto_stream_t stream) {
  PTO_REQUIRE(token_x && w_dq && w_uqqr && w_uk && w_dkvkr && gamma_cq && gamma_ckv && cos && sin && cache_index &&
                  kv_cache && kr_cache && w_idx_qb && w_idx_k && w_idx_proj && ln_gamma && ln_beta && idx_k_cache &&
                  query_nope_out && query_rope_out && idx_query_out && weights_out,
              "null tensor pointer");
  PTO_REQUIRE(t >= 1 && t <= 65535, "t %d: 1..65535 tokens per call", t);
  PTO_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden %d must be a positive multiple of 8", hidden);
  PTO_REQUIRE(q_lora >= 16 && q_lora % 16 == 0 && q_lora <= 12288, "q_lora %d must be a multiple of 16, at most 12288",
              q_lora);
  PTO_REQUIRE(cache_rows >= 1, "cache_rows");
  PTO_REQUIRE(eps_cq >= 0.f && eps_ckv >= 0.f && ln_eps >= 0.f, "negative epsilon");
  PTO_REQUIRE(aligned16(token_x) && aligned16(w_dq) && aligned16(w_uqqr) && aligned16(w_uk) && aligned16(w_dkvkr) &&
                  aligned16(w_idx_qb) && aligned16(w_idx_k) && aligned16(w_idx_proj) && aligned16(kv_cache) &&
                  aligned16(gamma_cq) && aligned16(query_nope_out) && aligned16(idx_query_out) &&
                  (q_norm_out == nullptr || aligned16(q_norm_out)),
              "prolog tensors must be 16-byte aligned");
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != PTO_OK) return rc;
  const PrologNqWs w = prolog_nq_ws(t, hidden, q_lora);
  rc = check_workspace(workspace, workspace_bytes, w.total);
  if (rc != PTO_OK) return rc;
  uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(base + w.status);
  const int ld = q_lora + kXProjExtra;
  float* qa = reinterpret_cast<float*>(base + w.xproj);
  float* kv = qa + q_lora;
  float* ki = kv + 576;
  float* wp = ki + 128;
  void* q_norm = q_norm_out != nullptr ? q_norm_out : static_cast<void*>(base + w.q_norm);
  void* q_b = base + w.q_b;

  int dev = 0;
  rc = prolog_side_stream(&dev);
  if (rc != PTO_OK) return rc;
  std::lock_guard<std::mutex> lock(prolog_side().dev_mu[dev]);
  cudaStream_t side = prolog_side().side[dev];
  cudaEvent_t* ev = prolog_side().ev[dev];

  // projections of the token, as in the quantised prolog: fp32 K-split partials [splits][t, q_lora | 576 | 128 | 64]
  const int splits = w.splits;
  const long long split_stride = static_cast<long long>(t) * ld;
  const size_t x_pitch = static_cast<size_t>(hidden) * 2;
  if (w_x_packed != nullptr) {
    PTO_REQUIRE(aligned16(w_x_packed), "w_x_packed must be 16-byte aligned");
    rc = run_sgemm(0, token_x, x_pitch, w_x_packed, static_cast<size_t>(ld) * 2, hidden, qa, t, ld, hidden, 1, 0, 0, 0, ld,
                   splits, split_stride, di.num_sms, status, stream);
    if (rc != PTO_OK) return rc;
  } else {
    const void* ws[4] = {w_dq, w_dkvkr, w_idx_k, w_idx_proj};
    float* outs[4] = {qa, kv, ki, wp};
    const int ns[4] = {q_lora, 576, 128, 64};
    for (int i = 0; i < 4; ++i) {
      rc = run_sgemm(0, token_x, x_pitch, ws[i], static_cast<size_t>(ns[i]) * 2, hidden, outs[i], t, ns[i], hidden, 1, 0, 0,
                     0, ld, splits, split_stride, di.num_sms, status, stream);
      if (rc != PTO_OK) return rc;
    }
  }
  // fork: caches, indexer key and weights need only the projections
  PTO_CUDA(cudaEventRecord(ev[0], stream));
  PTO_CUDA(cudaStreamWaitEvent(side, ev[0], 0));
  PTO_CUDA(pto::launch_prolog_kv_bf16(kv, ki, wp, ld, splits, split_stride, gamma_ckv, cos, sin, ln_gamma, ln_beta,
                                      cache_index, cache_rows, t, eps_ckv, ln_eps, kv_cache, kr_cache, idx_k_cache,
                                      weights_out, status, side));
  // caller's stream: normalised query -> attention up-projection (bf16 in, bf16 out) -> ropes -> absorbed nope part.
  // The indexer's up-projection (64 column tiles) runs on the side stream beside the attention one (192 tiles on
  // 148 CTAs: its second wave leaves two thirds of the SMs free), behind the per-token kernel.
  PTO_CUDA(pto::launch_prolog_qnorm_bf16(qa, ld, splits, split_stride, gamma_cq, t, q_lora, eps_cq, q_norm, stream,
                                         /*pdl=*/true));
  PTO_CUDA(cudaEventRecord(ev[1], stream));
  const size_t qn_pitch = static_cast<size_t>(q_lora) * 2;
  rc = run_sgemm(1, q_norm, qn_pitch, w_uqqr, 128 * 192 * 2, q_lora, q_b, t, 128 * 192, q_lora, 1, 0, 0, 0, 128 * 192, 1, 0,
                 di.num_sms, status, stream);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(cudaStreamWaitEvent(side, ev[1], 0));
  rc = run_sgemm(1, q_norm, qn_pitch, w_idx_qb, 64 * 128 * 2, q_lora, idx_query_out, t, 64 * 128, q_lora, 1, 0, 0, 0,
                 64 * 128, 1, 0, di.num_sms, status, side);
  if (rc != PTO_OK) return rc;
  PTO_CUDA(cudaEventRecord(ev[2], side));
  PTO_CUDA(cudaStreamWaitEvent(stream, ev[2], 0));  // the rope kernel reads both products
  PTO_CUDA(pto::launch_prolog_rope_bf16(q_b, cos, sin, t, query_rope_out, idx_query_out, stream));
  rc = run_sgemm(1, q_b, 128 * 192 * 2, w_uk, 512 * 2, 128 * 128, query_nope_out, t, 512, 128, 128, 128, 192 * 2, 512,
                 128 * 512, 1, 0, di.num_sms, status, stream, /*pdl=*/true);
  if (rc != PTO_OK) return rc;
  return PTO_OK;  // (the side stream was joined in front of the rope kernel)
}

size_t pto_decode_workspace_bytes(int t, int max_blocks, int block_size, int nq) {
  if (t < 1 || max_blocks < 1 || block_size < 1 || nq < 1) return 0;
  return kStatusBytes + li_scores_bytes(t, max_blocks, block_size) + sfa_part_bytes(t, nq) + li_hist_bytes(t);
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
  unsigned int* hist =  // behind the attention partials
      li_hist_usable(s1, flags) ? reinterpret_cast<unsigned int*>(part + sfa_part_bytes(b * s1, nq)) : nullptr;
  rc = run_li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, scale_dtype, act_seq,
                     block_table, scores, nullptr, b, s1, block_num, max_blocks, flags, status, stream, hist);
  if (rc != PTO_OK) return rc;
  rc = run_li_topk(scores, static_cast<int64_t>(max_blocks) * 128, act_seq, topk_res, b, s1, selected_count, flags,
                   status, stream, hist);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, 0, topk_res, block_table, act_seq,
                 attention_out, b, s1, nq, 1, softmax_scale, selected_count, 128, static_cast<int64_t>(block_num) * 128,
                 max_blocks, nq, 0, part, sfa_part_bytes(b * s1, nq), status, stream, /*behind_topk=*/1);
}

int pto_decode_fused_bf16(const void* idx_query, const void* idx_key_cache, const void* idx_weight,
                          const void* query_nope, const void* query_rope, const void* key_nope_2d,
                          const void* key_rope_2d, const int32_t* act_seq, const int32_t* block_table,
                          int32_t* topk_res, void* attention_out, int b, int s1, int block_num, int max_blocks,
                          int selected_count, int nq, float softmax_scale, int flags, void* workspace,
                          size_t workspace_bytes, pto_stream_t stream) {
  int rc = check_li_bf16(idx_query, idx_key_cache, idx_weight, act_seq, block_table, b, s1, 64, 128, 128, block_num,
                         max_blocks, flags);
  if (rc != PTO_OK) return rc;
  PTO_REQUIRE(topk_res != nullptr, "topk_res is null");
  rc = check_workspace(workspace, workspace_bytes, pto_decode_workspace_bytes(b * s1, max_blocks, 128, nq));
  if (rc != PTO_OK) return rc;
  uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(base);
  float* scores = reinterpret_cast<float*>(base + kStatusBytes);
  uint8_t* part = base + kStatusBytes + li_scores_bytes(b * s1, max_blocks, 128);
  unsigned int* hist =  // behind the attention partials
      li_hist_usable(s1, flags) ? reinterpret_cast<unsigned int*>(part + sfa_part_bytes(b * s1, nq)) : nullptr;
  rc = run_li_scores(reinterpret_cast<const int8_t*>(idx_query), nullptr, reinterpret_cast<const int8_t*>(idx_key_cache),
                     nullptr, idx_weight, PTO_DT_F16, act_seq, block_table, scores, nullptr, b, s1, block_num, max_blocks,
                     kLiFlagBf16, status, stream, hist);
  if (rc != PTO_OK) return rc;
  rc = run_li_topk(scores, static_cast<int64_t>(max_blocks) * 128, act_seq, topk_res, b, s1, selected_count, flags,
                   status, stream, hist);
  if (rc != PTO_OK) return rc;
  return run_sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, nullptr, kSfaSplitBf16, topk_res, block_table,
                 act_seq, attention_out, b, s1, nq, 1, softmax_scale, selected_count, 128,
                 static_cast<int64_t>(block_num) * 128, max_blocks, nq, 0, part, sfa_part_bytes(b * s1, nq), status, stream,
                 /*behind_topk=*/1);
}

}  // extern "C"
