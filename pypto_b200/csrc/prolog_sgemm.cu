// Weight-streaming products of the prolog on tcgen05, one kernel for its three shapes:
//
//   * the projections of the hidden state, out[t, N] (fp32) = x[t, K] (bf16) . W[K, N] (bf16), K = 7168 split over
//     CTAs (every split writes its own fp32 partial; the kernels that read the result add the partials in a fixed
//     order, so the sum does not depend on which CTA finished first);
//   * the absorbed query, per head h: out[t, h, 512] (bf16) = q_b[t, h, 0:128] (bf16) . w_uk[h] [128, 512] (bf16);
//   * the int8 up-projections for more token rows than the resident-activation kernel takes,
//     out[t, N] (int32) = x[t, K] (int8) . W[K, N] (int8).
//
// (reference: examples/models/deepseek_v32_exp/mla_prolog_quant_impl.py:502-707,
// lightning_indexer_prolog_quant_impl.py:325-504.)
//
// The weights are the large operand, so the product is taken transposed, D[n, tok] = W^T[n, k] . x^T[k, tok]:
// 128 weight columns are the M dimension of the MMA, up to 256 token rows its N dimension. W is row-major [K, N],
// i.e. an MN-major A operand, which TMA delivers in the canonical 128-byte-swizzled layout (box of k-rows x 128
// bytes of n). A ring stage holds one 16 KB weight tile (128 k x 128 n int8, or 64 k x 128 n bf16 as two 64-column
// boxes) and the matching [token rows x 128 bytes] slice of x; rows and columns outside the tensors read as zeros.
// Work items (token block, problem of the batch, 128-column tile, K split) are dealt round-robin to persistent CTAs.
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue (TMEM lane quarter = warp & 3); two
// accumulators in tensor memory. Every wait is bounded and reports PTO_ST_WAIT_EXPIRED.
#include <cuda.h>

#include "sfa_common.cuh"

namespace pto {

namespace {

constexpr int kSTileN = 128;          // weight columns per tile (MMA M)
constexpr int kSWBytes = 16384;       // weight tile bytes per stage
constexpr int kSMaxStages = 8;
constexpr int kSRingBytes = 192 * 1024;
constexpr int kSThreads = 192;
constexpr int kSMaxRows = 256;        // token rows per block (MMA N)

enum { kOutF32 = 0, kOutBf16 = 1, kOutI32 = 2 };

struct SCtl {
  uint64_t full[kSMaxStages];
  uint64_t empty[kSMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
};

constexpr int kSSmemMax = kSRingBytes + sizeof(SCtl) + 1024;

struct SGemmParams {
  int n_tiles;            // 128-column tiles per problem
  int chunks;             // K chunks in all (64 bf16 / 128 int8 per chunk)
  int per_split;          // chunks per split
  int splits;
  int batch;              // problems (heads), >= 1
  int tok_blocks;
  int t;                  // token rows in all
  int t_pad;              // rows per token block = MMA N (multiple of 16, <= 256)
  int n;                  // valid output columns per problem
  int w_batch_rows;       // rows of W between problems
  int x_batch_bytes;      // bytes along a row of x between problems
  long long out_batch;    // output elements between problems
  long long ld_out;       // output elements between token rows
  long long split_stride; // output elements between the partials of two splits
  void* out;
  int n_stages;
  uint32_t stage_bytes;   // kSWBytes + t_pad * 128
  uint32_t tmem_cols;
  int32_t* status;
};

struct SItem {
  int tb, b, tile, split;
};
__device__ __forceinline__ SItem s_item(const SGemmParams& p, int item) {
  SItem it;
  it.split = item % p.splits;
  int r = item / p.splits;
  it.tile = r % p.n_tiles;
  r /= p.n_tiles;
  it.b = r % p.batch;
  it.tb = r / p.batch;
  return it;
}

template <bool kI8, int kOut>
__global__ void __launch_bounds__(kSThreads, 1)
prolog_sgemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const SGemmParams p) {
  extern __shared__ uint8_t sgemm_smem_raw[];
  const uint32_t raw = smem_u32(sgemm_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = sgemm_smem_raw + (base - raw);
  SCtl* ctl = reinterpret_cast<SCtl*>(smem + p.n_stages * p.stage_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.tok_blocks * p.batch * p.n_tiles * p.splits;
  constexpr int kChunkK = kI8 ? 128 : 64;  // k rows per weight tile
  const uint32_t x_bytes = static_cast<uint32_t>(p.t_pad) * 128u;

  if (tid == 0) {
    for (int i = 0; i < kSMaxStages; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[i]), 4);
    }
    ctl->abort = 0;
    fence_mbar_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  // the set-up above overlaps the tail of the kernel before it; its results are read (and buffers it may still
  // read are overwritten) from here on
  pdl_wait();
  if (tid == 0) pdl_trigger();

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      // weights are read once per call: first to leave L2, so that activations and partial sums stay there
      const uint64_t w_policy = l2_policy_evict_first();
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const SItem w = s_item(p, item);
        const int k0 = w.split * p.per_split;
        const int kn = min(p.per_split, p.chunks - k0);
        const int n0 = w.tile * kSTileN;
        for (int c = 0; c < kn; ++c, ++it) {
          const uint32_t s = it % p.n_stages;
          if (it >= static_cast<uint32_t>(p.n_stages)) {
            ok = mbar_wait(smem_u32(&ctl->empty[s]), ((it / p.n_stages) - 1) & 1);
            if (!ok) break;
          }
          const uint32_t bar = smem_u32(&ctl->full[s]);
          const uint32_t dst = base + s * p.stage_bytes;
          const int krow = w.b * p.w_batch_rows + (k0 + c) * kChunkK;
          mbar_arrive_expect_tx(bar, kSWBytes + x_bytes);
          if (kI8) {
            tma_load_2d_hint(dst, &tmap_w, n0, krow, bar, w_policy);
          } else {
            tma_load_2d_hint(dst, &tmap_w, n0 * 2, krow, bar, w_policy);
            tma_load_2d_hint(dst + kSWBytes / 2, &tmap_w, n0 * 2 + 128, krow, bar, w_policy);
          }
          tma_load_2d(dst + kSWBytes, &tmap_x, w.b * p.x_batch_bytes + (k0 + c) * 128, w.tb * p.t_pad, bar);
        }
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 73);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = kI8 ? umma_idesc(kCFmtS32, kABFmtS8, kABFmtS8, 1, 0, kSTileN, static_cast<uint32_t>(p.t_pad))
                                 : umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 1, 0, kSTileN, static_cast<uint32_t>(p.t_pad));
      bool ok = true;
      uint32_t it = 0, ti = 0;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ti) {
        const SItem w = s_item(p, item);
        const int kn = min(p.per_split, p.chunks - w.split * p.per_split);
        const uint32_t acc = ti & 1;
        if (ti >= 2) {
          ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), ((ti >> 1) - 1) & 1);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * static_cast<uint32_t>(p.t_pad);
        for (int c = 0; c < kn; ++c, ++it) {
          const uint32_t s = it % p.n_stages;
          ok = mbar_wait(smem_u32(&ctl->full[s]), (it / p.n_stages) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a = base + s * p.stage_bytes;
          const uint64_t b_desc = umma_desc_kmajor_sw128(a + kSWBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (kI8) {  // K = 32 per instruction: 32 k-rows of A (4 KB), 32 bytes along x's rows
              mma_i8_ss(d, desc_mnmajor_sw128(a + j * 4096, 16, 1024), b_desc + 2 * j, idesc, (c | j) != 0 ? 1u : 0u);
            } else {    // K = 16: 16 k-rows of each 64-column half (2 KB), the halves 8 KB apart
              mma_f16_ss(d, desc_mnmajor_sw128(a + j * 2048, kSWBytes / 2, 1024), b_desc + 2 * j, idesc,
                         (c | j) != 0 ? 1u : 0u);
            }
          }
          tc_commit(smem_u32(&ctl->empty[s]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&ctl->acc_full[acc]));
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 74);
      }
    }
  } else {
    // ---------------- epilogue: accumulator rows (one weight column per lane) -> output ----------------
    const int q = warp & 3;  // TMEM lanes 32q .. 32q+31
    bool ok = true;
    uint32_t ti = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++ti) {
      const SItem w = s_item(p, item);
      const uint32_t acc = ti & 1;
      ok = mbar_wait_warp(smem_u32(&ctl->acc_full[acc]), (ti >> 1) & 1);
      if (!ok || ctl->abort) break;
      tc_fence_after();
      const int n = w.tile * kSTileN + q * 32 + lane;
      const bool col_ok = n < p.n;
      const long long col = static_cast<long long>(w.b) * p.out_batch + n + static_cast<long long>(w.split) * p.split_stride;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * static_cast<uint32_t>(p.t_pad);
      const int tok0 = w.tb * p.t_pad;
      for (int c0 = 0; c0 < p.t_pad && tok0 + c0 < p.t; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(taddr + c0, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int tok = tok0 + c0 + e;
          if (tok < p.t && col_ok) {  // 32 lanes: consecutive columns of one token row
            const long long at = static_cast<long long>(tok) * p.ld_out + col;
            if (kOut == kOutF32) reinterpret_cast<float*>(p.out)[at] = __uint_as_float(v[e]);
            if (kOut == kOutBf16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(__uint_as_float(v[e]));
            if (kOut == kOutI32) reinterpret_cast<int32_t*>(p.out)[at] = static_cast<int32_t>(v[e]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 75);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort) {
    // give copies still in flight time to land before the CTA's shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

template <bool kI8, int kOut>
cudaError_t launch_one(const void* tmap_w, const void* tmap_x, const SGemmParams& p, int grid, cudaStream_t stream,
                       bool pdl) {
  auto kernel = prolog_sgemm_kernel<kI8, kOut>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSSmemMax);
  if (e != cudaSuccess) return e;
  const size_t smem = static_cast<size_t>(p.n_stages) * p.stage_bytes + sizeof(SCtl) + 1024;
  count_launch();
  return launch_maybe_pdl(kernel, dim3(grid), dim3(kSThreads), smem, stream, pdl,
                          *reinterpret_cast<const CUtensorMap*>(tmap_w), *reinterpret_cast<const CUtensorMap*>(tmap_x), p);
}

}  // namespace

int prolog_sgemm_rows(int t) {
  const int r = (t + 15) / 16 * 16;
  return r < kSMaxRows ? r : kSMaxRows;
}

// K splits of the hidden-state projections for t token rows and n output columns: as many as fill the SMs once,
// at most 8 and at most one per K chunk. A pure function of the shapes, so that the workspace size, the product and
// the kernels that add the partials agree.
int prolog_sgemm_splits(int t, int n, int k, int num_sms) {
  const int rows = prolog_sgemm_rows(t);
  const int items = ((t + rows - 1) / rows) * ((n + kSTileN - 1) / kSTileN);
  const int chunks = (k + 63) / 64;
  int s = num_sms / (items < 1 ? 1 : items);
  s = s < 1 ? 1 : (s > 8 ? 8 : s);
  s = s > chunks ? chunks : s;
  for (;;) {  // a count every split of which has work: s = ceil(chunks / ceil(chunks / s))
    const int per = (chunks + s - 1) / s;
    const int again = (chunks + per - 1) / per;
    if (again == s) return s;
    s = again;
  }
}

// kind: 0 = bf16 x bf16 -> fp32 (with `splits` partials `split_stride` elements apart), 1 = bf16 x bf16 -> bf16,
// 2 = int8 x int8 -> int32. The tensor maps are byte matrices: W with a [k rows x 128 B] box (64 rows for bf16, 128
// for int8), x with a [prolog_sgemm_rows(t) x 128 B] box.
cudaError_t launch_prolog_sgemm(int kind, const void* tmap_w, const void* tmap_x, void* out, int t, int n, int k,
                                int batch, int w_batch_rows, int x_batch_bytes, long long out_batch, long long ld_out,
                                int splits, long long split_stride, int num_sms, int32_t* status, cudaStream_t stream,
                                bool pdl) {
  SGemmParams p{};
  const bool i8 = kind == kOutI32;
  p.n_tiles = (n + kSTileN - 1) / kSTileN;
  p.chunks = i8 ? (k + 127) / 128 : (k + 63) / 64;
  p.splits = splits < 1 ? 1 : splits;
  p.per_split = (p.chunks + p.splits - 1) / p.splits;
  if ((p.chunks + p.per_split - 1) / p.per_split != p.splits) return cudaErrorInvalidValue;  // a split without work
  p.batch = batch < 1 ? 1 : batch;
  p.t = t;
  p.t_pad = prolog_sgemm_rows(t);
  p.tok_blocks = (t + p.t_pad - 1) / p.t_pad;
  p.n = n;
  p.w_batch_rows = w_batch_rows;
  p.x_batch_bytes = x_batch_bytes;
  p.out_batch = out_batch;
  p.ld_out = ld_out;
  p.split_stride = split_stride;
  p.out = out;
  p.stage_bytes = kSWBytes + static_cast<uint32_t>(p.t_pad) * 128u;
  p.n_stages = kSRingBytes / static_cast<int>(p.stage_bytes);
  if (p.n_stages > kSMaxStages) p.n_stages = kSMaxStages;
  p.status = status;
  const long long items = static_cast<long long>(p.tok_blocks) * p.batch * p.n_tiles * p.splits;
  int grid = static_cast<int>(items < num_sms ? items : num_sms);
  uint32_t accs = 2;
  if (items > num_sms && p.per_split <= 4 && items <= (1 << 20)) {
    // many small items (the per-head products: two chunks each): one CTA per item with a ring just large enough,
    // so that several CTAs share an SM and their load, product and store latencies overlap instead of queueing
    // behind one CTA's epilogue warps
    grid = static_cast<int>(items);
    p.n_stages = p.per_split < 2 ? 2 : p.per_split;
    accs = 1;
  }
  uint32_t cols = 32;
  while (cols < accs * static_cast<uint32_t>(p.t_pad)) cols <<= 1;
  p.tmem_cols = cols;
  if (kind == kOutF32) return launch_one<false, kOutF32>(tmap_w, tmap_x, p, grid, stream, pdl);
  if (kind == kOutBf16) return launch_one<false, kOutBf16>(tmap_w, tmap_x, p, grid, stream, pdl);
  return launch_one<true, kOutI32>(tmap_w, tmap_x, p, grid, stream, pdl);
}

}  // namespace pto
