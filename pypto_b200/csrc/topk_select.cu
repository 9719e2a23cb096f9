// Exact per-row top-k over the fp32 score rows of the lightning indexer.
//
// Semantics (reference: examples/models/deepseek_v32_exp/lightning_indexer_quant_impl.py:196-312,
// golden deepseekv32_lightning_indexer_quant.py:244-262): row (b, i) selects over positions
// [0, eff), eff = S_b - (s1 - 1 - i); output is value-descending; when eff < k the first eff entries
// are valid and the rest is -1; eff <= 0 gives all -1. Ties are broken toward the smaller position,
// which makes the result deterministic (torch.topk leaves tie order unspecified).
//
// One CTA per row. Every element is mapped to a unique 64-bit key (order-preserving image of the
// float in the high word, ~position in the low word), so "the k largest keys" is well defined.
//   1. min/max of the row                    2. 2048-bin histogram over a monotone linear bucket map
//   3. bucket above the threshold bucket -> selected; threshold bucket -> candidate buffer (shared)
//   4. candidates sorted (bitonic) and the best `need` appended; if the threshold bucket does not
//      fit the buffer (massive ties), an MSB-first radix select over the 64-bit keys runs on the row
//   5. the k selected keys are sorted (bitonic) and the positions written.
#include "common.cuh"

namespace pto {

namespace {

constexpr int kTopkThreads = 1024;
constexpr int kBins = 2048;
constexpr int kMaxK = 2048;
constexpr int kCandCap = 4096;

struct TopkSmem {
  unsigned long long sel[kMaxK];
  unsigned long long cand[kCandCap];
  unsigned int hist[kBins];
  unsigned int warp_tot[32];
  float red_min[32];
  float red_max[32];
  unsigned int n_sel;
  unsigned int n_cand;
  int thr_bin;
  unsigned int thr_above;
  unsigned int thr_count;
};

__device__ __forceinline__ unsigned int float_order(float f) {
  unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long make_key(float f, int pos) {
  return (static_cast<unsigned long long>(float_order(f)) << 32) | static_cast<unsigned int>(~static_cast<unsigned int>(pos));
}
__device__ __forceinline__ int key_pos(unsigned long long key) {
  return static_cast<int>(~static_cast<unsigned int>(key & 0xffffffffull));
}

// descending bitonic sort of n (power of two) keys in shared memory; all threads of the CTA call it.
// Pair t of a stage is handled by thread t (and t + blockDim, ...), so for strides below 64 warp w only
// touches the 64-key blocks w, w + 32, ...: those stages need a warp barrier only, unless the previous
// stage had a larger stride and other warps wrote into the block.
__device__ void bitonic_sort_desc(unsigned long long* buf, int n) {
  __syncthreads();
  int prev_stride = 64;
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= 64 || prev_stride >= 64) __syncthreads(); else __syncwarp();
      prev_stride = stride;
      for (int t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));  // index with the `stride` bit clear
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const unsigned long long a = buf[lo], b = buf[hi];
        if ((a < b) == desc) {
          buf[lo] = b;
          buf[hi] = a;
        }
      }
    }
  }
  __syncthreads();
}

// Finds, scanning the histogram from the top bin down, the bin where the running count reaches
// `need`. Results in sm->thr_bin (bin), thr_above (count in bins above it), thr_count (its count).
__device__ void find_threshold_bin(TopkSmem* sm, unsigned int need) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  // thread t owns bins (kBins-1-2t) and (kBins-2-2t): a descending walk is a prefix scan over t
  const unsigned int c0 = sm->hist[kBins - 1 - 2 * tid];
  const unsigned int c1 = sm->hist[kBins - 2 - 2 * tid];
  const unsigned int s = c0 + c1;
  unsigned int incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) sm->warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    unsigned int w = sm->warp_tot[lane];
    unsigned int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    sm->warp_tot[lane] = wi - w;  // exclusive
  }
  __syncthreads();
  const unsigned int excl = sm->warp_tot[warp] + incl - s;
  if (excl < need && need <= excl + c0) {
    sm->thr_bin = kBins - 1 - 2 * tid;
    sm->thr_above = excl;
    sm->thr_count = c0;
  } else if (excl + c0 < need && need <= excl + s) {
    sm->thr_bin = kBins - 2 - 2 * tid;
    sm->thr_above = excl + c0;
    sm->thr_count = c1;
  }
  __syncthreads();
}

// Applies f(value, position) to every element of row[0, eff). Loads go through the read-only path
// and are issued four 16-byte loads at a time before the bodies run, so the latency of one batch is
// paid once (the bodies contain shared-memory atomics the compiler will not move loads across).
template <typename F>
__device__ __forceinline__ void for_each_element(const float* row, int eff, F&& f) {
  const int tid = threadIdx.x;
  const int n4 = eff & ~3;
  constexpr int kStep = kTopkThreads * 4;
  for (int j0 = tid * 4; j0 < n4; j0 += 4 * kStep) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kStep;
      if (j < n4) v[u] = __ldg(reinterpret_cast<const float4*>(row + j));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kStep;
      if (j < n4) {
        f(v[u].x, j);
        f(v[u].y, j + 1);
        f(v[u].z, j + 2);
        f(v[u].w, j + 3);
      }
    }
  }
  for (int j = n4 + tid; j < eff; j += kTopkThreads) f(__ldg(row + j), j);
}

__global__ void __launch_bounds__(kTopkThreads, 1)
li_topk_kernel(TopkParams p) {
  extern __shared__ __align__(16) uint8_t topk_smem_raw[];
  TopkSmem* sm = reinterpret_cast<TopkSmem*>(topk_smem_raw);
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int row_id = blockIdx.x;
  const int bi = row_id / p.s1;
  const int i = row_id % p.s1;
  const int k = p.k;
  int32_t* out = p.out + static_cast<int64_t>(row_id) * k;
  const float* row = p.scores + static_cast<int64_t>(row_id) * p.row_stride;
  int eff = p.act_seq[bi] - (p.s1 - 1 - i);
  if (eff > p.row_stride) eff = static_cast<int>(p.row_stride);

  if (eff <= 0) {
    for (int j = tid; j < k; j += kTopkThreads) out[j] = -1;
    return;
  }
  int kpow2 = 1;
  while (kpow2 < k) kpow2 <<= 1;

  if (eff <= k) {
    for (int j = tid; j < kpow2; j += kTopkThreads) sm->sel[j] = (j < eff) ? make_key(row[j], j) : 0ull;
    if ((p.flags & PTO_LI_UNSORTED) == 0) bitonic_sort_desc(sm->sel, kpow2); else __syncthreads();
    for (int j = tid; j < k; j += kTopkThreads) out[j] = (j < eff) ? key_pos(sm->sel[j]) : -1;
    return;
  }

  // ---- 1. row min / max -------------------------------------------------------------------
  float vmin = INFINITY, vmax = -INFINITY;
  for_each_element(row, eff, [&](float v, int) {
    vmin = fminf(vmin, v);
    vmax = fmaxf(vmax, v);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
  }
  if (lane == 0) {
    sm->red_min[warp] = vmin;
    sm->red_max[warp] = vmax;
  }
  for (int j = tid; j < kBins; j += kTopkThreads) sm->hist[j] = 0;
  if (tid == 0) {
    sm->n_sel = 0;
    sm->n_cand = 0;
  }
  __syncthreads();
  vmin = sm->red_min[lane];
  vmax = sm->red_max[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
  }
  // monotone bucket map: floor((v - vmin) * inv), clamped. Non-finite range -> everything in bin 0
  // and the radix fallback resolves it.
  float inv = 0.f;
  {
    const float range = vmax - vmin;
    if (range > 0.f && range < INFINITY) inv = static_cast<float>(kBins - 1) / range;
    if (!(inv < INFINITY)) inv = 0.f;
  }
  auto bucket = [&](float v) -> int {
    const float x = (v - vmin) * inv;
    int bkt = static_cast<int>(x);
    bkt = max(0, min(kBins - 1, bkt));
    return bkt;
  };

  // ---- 2. histogram -----------------------------------------------------------------------
  for_each_element(row, eff, [&](float v, int) { atomicAdd(&sm->hist[bucket(v)], 1u); });
  __syncthreads();
  find_threshold_bin(sm, static_cast<unsigned int>(k));
  const int thr_bin = sm->thr_bin;
  const unsigned int above = sm->thr_above;
  const unsigned int thr_count = sm->thr_count;
  const unsigned int need = static_cast<unsigned int>(k) - above;  // to take from the threshold bucket

  if (thr_count <= static_cast<unsigned int>(kCandCap)) {
    // ---- 3. collect -------------------------------------------------------------------------
    for_each_element(row, eff, [&](float v, int pos) {
      const int bkt = bucket(v);
      if (bkt > thr_bin) {
        sm->sel[atomicAdd(&sm->n_sel, 1u)] = make_key(v, pos);
      } else if (bkt == thr_bin) {
        sm->cand[atomicAdd(&sm->n_cand, 1u)] = make_key(v, pos);
      }
    });
    __syncthreads();
    // ---- 4. best `need` of the candidates ---------------------------------------------------
    if (need == thr_count) {
      for (unsigned int j = tid; j < need; j += kTopkThreads) sm->sel[above + j] = sm->cand[j];
    } else {
      int cpow2 = 1;
      while (cpow2 < static_cast<int>(thr_count)) cpow2 <<= 1;
      for (int j = thr_count + tid; j < cpow2; j += kTopkThreads) sm->cand[j] = 0ull;
      bitonic_sort_desc(sm->cand, cpow2);
      for (unsigned int j = tid; j < need; j += kTopkThreads) sm->sel[above + j] = sm->cand[j];
    }
    __syncthreads();
  } else {
    // ---- 4'. massive ties: MSB-first radix select on the 64-bit keys of the threshold bucket ----
    // digits: 11/11/10 bits of the value word, then 11/11/10 bits of the inverted position.
    // invariant: keys in the bucket with (key >> shift) > prefix are selected; `remaining` more are
    // needed among those with (key >> shift) == prefix.
    unsigned long long prefix = 0ull;
    int shift = 64;
    unsigned int remaining = need;
    const int widths[6] = {11, 11, 10, 11, 11, 10};
    bool exact = false;
    for (int pass = 0; pass < 6 && !exact; ++pass) {
      const int w = widths[pass];
      const int new_shift = shift - w;
      for (int j = tid; j < kBins; j += kTopkThreads) sm->hist[j] = 0;
      __syncthreads();
      for_each_element(row, eff, [&](float v, int pos) {
        if (bucket(v) != thr_bin) return;
        const unsigned long long key = make_key(v, pos);
        if (shift < 64 && (key >> shift) != prefix) return;
        atomicAdd(&sm->hist[static_cast<unsigned int>(key >> new_shift) & ((1u << w) - 1u)], 1u);
      });
      __syncthreads();
      find_threshold_bin(sm, remaining);
      remaining -= sm->thr_above;
      exact = (sm->thr_count == remaining);
      prefix = (prefix << w) | static_cast<unsigned long long>(sm->thr_bin);
      shift = new_shift;
      __syncthreads();
    }
    // every key with (key >> shift) >= prefix inside the bucket, plus all higher buckets
    for_each_element(row, eff, [&](float v, int pos) {
      const int bkt = bucket(v);
      if (bkt < thr_bin) return;
      const unsigned long long key = make_key(v, pos);
      if (bkt > thr_bin || (key >> shift) >= prefix) {
        const unsigned int slot = atomicAdd(&sm->n_sel, 1u);
        if (slot < static_cast<unsigned int>(kMaxK)) sm->sel[slot] = key;
      }
    });
    __syncthreads();
  }

  // ---- 5. order and write -------------------------------------------------------------------
  if ((p.flags & PTO_LI_UNSORTED) == 0) {
    for (int j = k + tid; j < kpow2; j += kTopkThreads) sm->sel[j] = 0ull;
    bitonic_sort_desc(sm->sel, kpow2);
  }
  for (int j = tid; j < k; j += kTopkThreads) out[j] = key_pos(sm->sel[j]);
}

}  // namespace

cudaError_t launch_li_topk(const TopkParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(li_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(TopkSmem)));
  if (e != cudaSuccess) return e;
  li_topk_kernel<<<p.b * p.s1, kTopkThreads, sizeof(TopkSmem), stream>>>(p);
  return cudaGetLastError();
}

int topk_max_k() { return kMaxK; }

}  // namespace pto
