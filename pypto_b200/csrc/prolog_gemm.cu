// Skinny int8 products of the prolog on tcgen05: out[t, N] (int32) = x[t, K] (int8) . W[K, N] (int8) for up to
// 64 token rows, both up-projections of the normalised query (w_uqqr and w_idx_qb) in one launch.
//
// The weights are the large operand (50 MB against 98 KB of activations), so the kernel is a weight stream:
// the product is taken transposed, D[n, t] = W^T[n, k] . x^T[k, t], with 128 weight columns as the M dimension
// of the MMA and the tokens as its N dimension. W is row-major [K, N], i.e. for the A operand the M index is the
// contiguous one: an MN-major operand, which TMA delivers in exactly the canonical 128-byte-swizzled layout
// (box of 128 k-rows x 128 bytes of n: row k at k*128, 16-byte chunks XORed with k mod 8). x stays resident in
// shared memory for the whole kernel (K-major, one [t_pad x 128 B] slab per 128 k), each CTA walks its weight
// tiles once: 12 stages of 16 KB per tile at K = 1536.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue (TMEM lane quarter = warp & 3); two
// accumulators in tensor memory so that the epilogue of a tile overlaps the MMAs of the next. Every wait is
// bounded and reports PTO_ST_WAIT_EXPIRED.
#include <cuda.h>

#include "sfa_common.cuh"

namespace pto {

namespace {

constexpr int kGTileN = 128;              // weight columns per tile (MMA M)
constexpr int kGTileK = 128;              // k rows per stage
constexpr int kGStageBytes = kGTileN * kGTileK;  // 16 KB
constexpr int kGMaxStages = 10;           // ring stages: as many as fit beside the activations, see kGDataBudget
constexpr int kGXBytesMax = 96 * 1024;    // resident activations: (K / 128) * t_pad * 128 bytes
// Ring + activations: at most kGDataMax. With more than 32 token rows they stay within kGDataBudget, so that a
// block of the prolog's per-token kernel (33 KB of shared memory, launched on a second stream just before this
// kernel) fits on the same SM: with all of shared memory taken here, those blocks (one per token) kept their SMs to
// themselves and this kernel's CTAs there started 5 us late (64 tokens: 63.3 -> 60.5 us per prolog call; with 8 or
// 32 tokens sharing costs about 1 us more than it returns, so fewer tokens keep the larger ring).
constexpr int kGDataBudget = 176 * 1024;
constexpr int kGDataMax = 192 * 1024;
constexpr int kGThreads = 192;

struct GemmCtl {
  uint64_t full[kGMaxStages];
  uint64_t empty[kGMaxStages];
  uint64_t x_full;
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
};

constexpr int kGSmemBytes = kGDataMax + sizeof(GemmCtl) + 1024;
static_assert(kGXBytesMax + 2 * kGStageBytes <= kGDataBudget, "no room for a ring beside the activations");

struct GemmParams {
  int32_t* out[2];   // [t, ld] row-major
  int ld[2];         // N of each product
  int tiles[2];      // N / 128
  int k;             // contraction length, multiple of 128
  int t;             // token rows that are stored
  int t_pad;         // MMA N: t rounded up to 16, <= 64
  int n_stages;      // ring stages of this launch
  int data_bytes;    // ring + activations area of this launch (the control block follows it)
  int32_t* status;
};

__global__ void __launch_bounds__(kGThreads, 1)
prolog_i8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1,
                      const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  extern __shared__ uint8_t gemm_smem_raw[];
  const uint32_t raw = smem_u32(gemm_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = gemm_smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t n_stages = static_cast<uint32_t>(p.n_stages);
  const uint32_t x_base = base + n_stages * kGStageBytes;
  GemmCtl* ctl = reinterpret_cast<GemmCtl*>(smem + p.data_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunks = p.k / kGTileK;
  const int n_tiles = p.tiles[0] + p.tiles[1];
  const uint32_t x_slab = static_cast<uint32_t>(p.t_pad) * 128u;

  if (tid == 0) {
    for (int i = 0; i < kGMaxStages; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 1);
    }
    mbar_init(smem_u32(&ctl->x_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[i]), 4);
    }
    ctl->abort = 0;
    fence_mbar_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_w0);
    tma_prefetch_desc(&tmap_w1);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  // the set-up above overlaps the tail of the kernel before it; its results are read from here on
  pdl_wait();
  if (tid == 0) pdl_trigger();

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      bool ok = true;
      mbar_arrive_expect_tx(smem_u32(&ctl->x_full), static_cast<uint32_t>(chunks) * x_slab);
      for (int c = 0; c < chunks; ++c) tma_load_2d(x_base + c * x_slab, &tmap_x, c * kGTileK, 0, smem_u32(&ctl->x_full));
      uint32_t it = 0;
      const uint64_t w_policy = l2_policy_evict_first();  // weights are read once per call
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const bool second = tile >= p.tiles[0];
        const CUtensorMap* tm = second ? &tmap_w1 : &tmap_w0;
        const int n0 = (second ? tile - p.tiles[0] : tile) * kGTileN;
        for (int c = 0; c < chunks; ++c, ++it) {
          const uint32_t s = it % n_stages;
          if (it >= n_stages) {
            ok = mbar_wait(smem_u32(&ctl->empty[s]), ((it / n_stages) - 1) & 1);
            if (!ok) break;
          }
          mbar_arrive_expect_tx(smem_u32(&ctl->full[s]), kGStageBytes);
          tma_load_2d_hint(a_base + s * kGStageBytes, tm, n0, c * kGTileK, smem_u32(&ctl->full[s]), w_policy);
        }
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 70);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kCFmtS32, kABFmtS8, kABFmtS8, 1, 0, kGTileN, static_cast<uint32_t>(p.t_pad));
      bool ok = mbar_wait(smem_u32(&ctl->x_full), 0);
      uint32_t it = 0, ti = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++ti) {
        const uint32_t acc = ti & 1;
        if (ti >= 2) {
          ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), ((ti >> 1) - 1) & 1);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * 64u;
        for (int c = 0; c < chunks; ++c, ++it) {
          const uint32_t s = it % n_stages;
          ok = mbar_wait(smem_u32(&ctl->full[s]), (it / n_stages) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint64_t b_desc = umma_desc_kmajor_sw128(x_base + c * x_slab);
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // K = 32 per instruction: 32 k-rows of A (4 KB), 32 bytes along B's rows
            const uint64_t a_desc = desc_mnmajor_sw128(a_base + s * kGStageBytes + j * 4096, 16, 1024);
            mma_i8_ss(d, a_desc, b_desc + 2 * j, idesc, (c | j) != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&ctl->empty[s]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&ctl->acc_full[acc]));
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 71);
      }
    }
  } else {
    // ---------------- epilogue: accumulator -> int32 rows ----------------
    const int q = warp & 3;  // TMEM lanes 32q .. 32q+31
    bool ok = true;
    uint32_t ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const uint32_t acc = ti & 1;
      ok = mbar_wait_warp(smem_u32(&ctl->acc_full[acc]), (ti >> 1) & 1);
      if (!ok || ctl->abort) break;
      tc_fence_after();
      const bool second = tile >= p.tiles[0];
      const int which = second ? 1 : 0;
      const int n = (second ? tile - p.tiles[0] : tile) * kGTileN + q * 32 + lane;
      int32_t* dst = p.out[which] + n;
      const int64_t ld = p.ld[which];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 64u;
      for (int c0 = 0; c0 < p.t_pad; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(taddr + c0, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (c0 + e < p.t) dst[(c0 + e) * ld] = static_cast<int32_t>(v[e]);  // 32 lanes: 128 contiguous bytes
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 72);
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
    tmem_dealloc(tmem_base, 128);
  }
}

}  // namespace

bool prolog_i8_gemm_supported(int t, int k) {
  if (t < 1 || t > 64 || k < kGTileK || k % kGTileK != 0) return false;
  const int t_pad = (t + 15) / 16 * 16;
  return static_cast<long long>(k / kGTileK) * t_pad * 128 <= kGXBytesMax;
}

cudaError_t launch_prolog_i8_gemm(const void* tmap_w0, const void* tmap_w1, const void* tmap_x, int32_t* out0, int n0,
                                  int32_t* out1, int n1, int k, int t, int num_sms, int32_t* status, cudaStream_t stream,
                                  bool pdl) {
  cudaError_t e = cudaFuncSetAttribute(prolog_i8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGSmemBytes);
  if (e != cudaSuccess) return e;
  GemmParams p{};
  p.out[0] = out0;
  p.out[1] = out1;
  p.ld[0] = n0;
  p.ld[1] = n1;
  p.tiles[0] = n0 / kGTileN;
  p.tiles[1] = n1 / kGTileN;
  p.k = k;
  p.t = t;
  p.t_pad = (t + 15) / 16 * 16;
  const int x_bytes = (k / kGTileK) * p.t_pad * 128;
  p.data_bytes = p.t_pad > 32 ? kGDataBudget : kGDataMax;
  p.n_stages = (p.data_bytes - x_bytes) / kGStageBytes;
  if (p.n_stages > kGMaxStages) p.n_stages = kGMaxStages;
  const int smem_bytes = p.data_bytes + static_cast<int>(sizeof(GemmCtl)) + 1024;
  p.status = status;
  const int n_tiles = p.tiles[0] + p.tiles[1];
  const int grid = n_tiles < num_sms ? n_tiles : num_sms;
  count_launch();
  return launch_maybe_pdl(prolog_i8_gemm_kernel, dim3(grid), dim3(kGThreads), smem_bytes, stream, pdl,
                          *reinterpret_cast<const CUtensorMap*>(tmap_w0), *reinterpret_cast<const CUtensorMap*>(tmap_w1),
                          *reinterpret_cast<const CUtensorMap*>(tmap_x), p);
}

}  // namespace pto
