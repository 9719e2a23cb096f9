// Exact per-row top-k over the fp32 score rows of the lightning indexer.
//
// Semantics (reference: examples/models/deepseek_v32_exp/lightning_indexer_quant_impl.py:196-312,
// golden deepseekv32_lightning_indexer_quant.py:244-262): row (b, i) selects over positions
// [0, eff), eff = S_b - (s1 - 1 - i); output is value-descending; when eff < k the first eff entries
// are valid and the rest is -1; eff <= 0 gives all -1. Ties are broken toward the smaller position,
// which makes the result deterministic (torch.topk leaves tie order unspecified).
//
// One cluster of 1, 2, 4 or 8 CTAs per row (as many as keep the grid within one wave of SMs). The
// scanning passes (1-3) are split over the CTAs of the cluster by position range; what they must agree
// on travels through distributed shared memory: the range's min/max, the histogram (added into rank
// every other rank's with remote atomics), the per-rank counts. In the unordered mode every rank writes
// the positions it selected straight to the output at its offset and pushes only its candidates of
// the threshold bucket into rank 0's list; in the ordered mode the selected keys are pushed too.
// Every element is mapped to a unique 64-bit key (order-preserving image of the
// float in the high word, ~position in the low word), so "the k largest keys" is well defined.
//   1. min/max of the row                    2. 2048-bin histogram over a monotone linear bucket map
//   3. bucket above the threshold bucket -> selected; threshold bucket -> candidate buffer (shared)
//   4. candidates sorted (bitonic) and the best `need` appended; if the threshold bucket does not
//      fit the buffer (massive ties), an MSB-first radix select over the 64-bit keys runs on the row
//   5. the k selected keys are sorted (bitonic) and the positions written.
// When the score kernel has left a histogram of the row (4096 bins over the top 12 bits of the order-preserving
// image of the float, counted over the positions below the row's causal end), passes 1 and 2 are skipped: the
// threshold bin comes from that histogram and pass 3 is the only scan of the row. The histogram is used only if
// its total equals the row's length and its threshold bin fits the candidate buffer; otherwise passes 1-2 run.
#include <cstdlib>

#include "common.cuh"

namespace pto {

namespace {

// -DPTO_TOPK_TIMELINE: clock64 stamps of thread 0 of CTA 0 at the phase boundaries (development aid, read back
// through pto_debug_topk_timeline; not part of the ABI)
#ifdef PTO_TOPK_TIMELINE
__device__ long long g_topk_tl[16];
#define TKT(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_topk_tl[i] = clock64(); } while (0)
#else
#define TKT(i) do { } while (0)
#endif

constexpr int kTopkThreads = 1024;
constexpr int kBins = 2048;
constexpr int kHistSlots = kLiHistBins > kBins ? kLiHistBins : kBins;
constexpr int kMaxK = 2048;
constexpr int kCandCap = 4096;
constexpr int kRowCap = 32768;  // positions of a rank's share that stay in shared memory between the scans

struct TopkSmem {
  unsigned long long sel[kMaxK];
  unsigned long long cand[kCandCap];
  unsigned int hist[kHistSlots];
  unsigned int warp_tot[32];
  unsigned int hist_total;
  float red_min[32];
  float red_max[32];
  unsigned int n_sel;
  unsigned int n_cand;
  unsigned int n_sel2, n_cand2;  // second radix step over the candidates of a coarse bin
  // values every rank of the cluster publishes into every other rank's copy (remote stores, made visible
  // by the next cluster barrier), so that nobody waits for a chain of remote loads
  float all_min[8], all_max[8];
  unsigned int all_sel[8], all_cand[8];
  int thr_bin;
  unsigned int thr_above;
  unsigned int thr_count;
  // this rank's share of the row, kept from the first scan for the other two (when it fits)
  __align__(16) float row[kRowCap];
};

__device__ __forceinline__ unsigned int cluster_rank() {
  unsigned int r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned int cluster_size() {
  unsigned int r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// all threads of all CTAs of the cluster; orders shared-memory accesses across the cluster
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(const void* local, unsigned int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_peer_u64(uint32_t a, unsigned long long v) {
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(a), "l"(v) : "memory");
}
__device__ __forceinline__ void st_peer_u32(uint32_t a, unsigned int v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void red_peer_add_u32(uint32_t a, unsigned int v) {
  asm volatile("red.relaxed.cluster.shared::cluster.add.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

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

// Descending bitonic sort of n (power of two) keys in shared memory; all threads of the CTA call it.
// Shared-memory version: pair t of a stage is handled by thread t (and t + blockDim, ...), so for strides
// below 64 warp w only touches the 64-key blocks w, w + 32, ...: those stages need a warp barrier only,
// unless the previous stage had a larger stride and other warps wrote into the block.
__device__ void bitonic_sort_desc_smem(unsigned long long* buf, int n) {
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

// Register version for n <= 2 * blockDim: thread t keeps keys 2t and 2t+1. Stride 1 is a compare inside
// the thread, strides 2..32 exchange with lane (t ^ stride/2) by shuffle (a warp holds 64 consecutive
// keys), and only strides >= 64 (15 of the 66 stages at n = 2048) go through shared memory and a block
// barrier. Lanes beyond n/2 carry zeros and are never paired with a real key (i ^ stride < n).
__device__ void bitonic_sort_desc(unsigned long long* buf, int n) {
  if (n > 2 * static_cast<int>(blockDim.x) || n < 2) {
    bitonic_sort_desc_smem(buf, n);
    return;
  }
  __syncthreads();
  const int t = threadIdx.x;
  const int i0 = 2 * t;
  const bool live = i0 < n;
  unsigned long long e0 = live ? buf[i0] : 0ull, e1 = live ? buf[i0 + 1] : 0ull;
  for (int size = 2; size <= n; size <<= 1) {
    int stride = size >> 1;
    if (stride >= 64) {
      if (live) {
        buf[i0] = e0;
        buf[i0 + 1] = e1;
      }
      for (; stride >= 64; stride >>= 1) {
        __syncthreads();
        if (t < (n >> 1)) {
          const int lo = 2 * t - (t & (stride - 1));
          const int hi = lo + stride;
          const bool desc = (lo & size) == 0;
          const unsigned long long a = buf[lo], b = buf[hi];
          if ((a < b) == desc) {
            buf[lo] = b;
            buf[hi] = a;
          }
        }
      }
      __syncthreads();
      if (live) {
        e0 = buf[i0];
        e1 = buf[i0 + 1];
      }
    }
    const bool desc = (i0 & size) == 0;  // the same for both keys of the thread (size >= 2)
    for (; stride >= 2; stride >>= 1) {
      const unsigned long long o0 = __shfl_xor_sync(0xffffffffu, e0, stride >> 1);
      const unsigned long long o1 = __shfl_xor_sync(0xffffffffu, e1, stride >> 1);
      const bool keep_max = ((i0 & stride) == 0) == desc;
      e0 = keep_max ? (e0 > o0 ? e0 : o0) : (e0 < o0 ? e0 : o0);
      e1 = keep_max ? (e1 > o1 ? e1 : o1) : (e1 < o1 ? e1 : o1);
    }
    {
      const unsigned long long hi = e0 > e1 ? e0 : e1, lo = e0 > e1 ? e1 : e0;
      e0 = desc ? hi : lo;
      e1 = desc ? lo : hi;
    }
  }
  if (live) {
    buf[i0] = e0;
    buf[i0 + 1] = e1;
  }
  __syncthreads();
}

// Finds, scanning the histogram of kPer * 1024 bins from the top bin down, the bin where the running count reaches
// `need`. Results in sm->thr_bin (bin), thr_above (count in bins above it), thr_count (its count), hist_total.
template <int kPer>
__device__ void find_threshold_bin(TopkSmem* sm, unsigned int need) {
  constexpr int kN = kPer * kTopkThreads;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  // thread t owns bins kN-1-kPer*t down to kN-kPer-kPer*t: a descending walk is a prefix scan over t
  unsigned int c[kPer];
  unsigned int s = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    c[e] = sm->hist[kN - 1 - kPer * tid - e];
    s += c[e];
  }
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
    if (lane == 31) sm->hist_total = wi;
  }
  __syncthreads();
  unsigned int run = sm->warp_tot[warp] + incl - s;  // count in the bins above this thread's first
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    if (run < need && need <= run + c[e]) {
      sm->thr_bin = kN - 1 - kPer * tid - e;
      sm->thr_above = run;
      sm->thr_count = c[e];
    }
    run += c[e];
  }
  __syncthreads();
}

// Applies f(value, position) to every element of row[0, eff). Loads go through the read-only path
// and are issued four 16-byte loads at a time before the bodies run, so the latency of one batch is
// paid once (the bodies contain shared-memory atomics the compiler will not move loads across).
template <bool kGlobal, typename F>
__device__ __forceinline__ void for_each_element(const float* row, int begin, int end, F&& f) {
  const int tid = threadIdx.x;
  const int n4 = begin + ((end - begin) & ~3);  // begin is a multiple of 4
  constexpr int kStep = kTopkThreads * 4;
  for (int j0 = begin + tid * 4; j0 < n4; j0 += 4 * kStep) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kStep;
      if (j < n4) v[u] = kGlobal ? __ldg(reinterpret_cast<const float4*>(row + j)) : *reinterpret_cast<const float4*>(row + j);
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
  for (int j = n4 + tid; j < end; j += kTopkThreads) f(kGlobal ? __ldg(row + j) : row[j], j);
}

__global__ void __launch_bounds__(kTopkThreads, 1)
li_topk_kernel(TopkParams p) {
  extern __shared__ __align__(16) uint8_t topk_smem_raw[];
  TopkSmem* sm = reinterpret_cast<TopkSmem*>(topk_smem_raw);
  // launched with programmatic serialization: the score kernel before it may still be running
  TKT(0);
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const unsigned int csize = cluster_size();
  const unsigned int rank = cluster_rank();
  const int row_id = blockIdx.x / csize;
  const int bi = row_id / p.s1;
  const int i = row_id % p.s1;
  const int k = p.k;
  int32_t* out = p.out + static_cast<int64_t>(row_id) * k;
  const float* row = p.scores + static_cast<int64_t>(row_id) * p.row_stride;
  // the row's length is an input of the call, not a result of the score kernel: its trip to memory runs while
  // this grid still waits for that kernel
  int eff = p.act_seq[bi] - (p.s1 - 1 - i);
  if (eff > p.row_stride) eff = static_cast<int>(p.row_stride);
  const bool unsorted = (p.flags & PTO_LI_UNSORTED) != 0;
  pdl_wait();
  pdl_trigger();
  TKT(1);

  // short rows: rank 0 alone, no cluster barrier on this path (every CTA of the cluster takes it)
  if (eff <= k) {
    if (rank != 0) return;
    if (eff <= 0) {
      for (int j = tid; j < k; j += kTopkThreads) out[j] = -1;
      return;
    }
    int kpow2 = 1;
    while (kpow2 < k) kpow2 <<= 1;
    for (int j = tid; j < kpow2; j += kTopkThreads) sm->sel[j] = (j < eff) ? make_key(row[j], j) : 0ull;
    if (!unsorted) bitonic_sort_desc(sm->sel, kpow2); else __syncthreads();
    for (int j = tid; j < k; j += kTopkThreads) out[j] = (j < eff) ? key_pos(sm->sel[j]) : -1;
    return;
  }
  int kpow2 = 1;
  while (kpow2 < k) kpow2 <<= 1;

  // this rank's share of the positions (a multiple of 4 so that 16-byte loads stay aligned)
  const int chunk = (((eff + static_cast<int>(csize) - 1) / static_cast<int>(csize)) + 3) & ~3;
  const int begin = min(eff, static_cast<int>(rank) * chunk);
  const int end = min(eff, begin + chunk);

  // ---- 0. the score kernel's histogram of the row, when there is one ------------------------------
  bool coarse = false;
  float vmin = 0.f, inv = 0.f;
  if (p.hist != nullptr) {
    const uint4* h4 = reinterpret_cast<const uint4*>(p.hist + static_cast<int64_t>(row_id) * kLiHistBins);
    static_assert(kLiHistBins == 4 * kTopkThreads, "one 16-byte load per thread");
    reinterpret_cast<uint4*>(sm->hist)[tid] = __ldg(h4 + tid);
    if (tid == 0) {
      sm->n_sel = 0;
      sm->n_cand = 0;
    }
    __syncthreads();
    find_threshold_bin<kLiHistBins / kTopkThreads>(sm, static_cast<unsigned int>(k));
    // usable if it counted exactly this row's positions and its threshold bin fits the candidate buffer; the
    // same answer in every rank of the cluster (all read the same histogram)
    coarse = sm->hist_total == static_cast<unsigned int>(eff) && sm->thr_count <= static_cast<unsigned int>(kCandCap);
    __syncthreads();  // every thread has read the outcome before the histogram area is reused
  }
  auto bucket = [&](float v) -> int {
    if (coarse) return static_cast<int>(float_order(v) >> kLiHistShift);
    const float x = (v - vmin) * inv;
    int bkt = static_cast<int>(x);
    bkt = max(0, min(kBins - 1, bkt));
    return bkt;
  };
  // the share stays in shared memory between the scans when it fits (not when the first scan is skipped)
  const bool resident = !coarse && (end - begin) <= kRowCap;
  TKT(2);
  if (!coarse) {
    // ---- 1. row min / max -------------------------------------------------------------------
    vmin = INFINITY;
    float vmax = -INFINITY;
    {
      // the one scan that reads the row from global memory (L2): this rank's share also goes into shared memory,
      // where the other two scans read it (three trips to L2 were three of the latencies this kernel consists of)
      const int n4 = begin + ((end - begin) & ~3);
      constexpr int kStep = kTopkThreads * 4;
      for (int j0 = begin + tid * 4; j0 < n4; j0 += 4 * kStep) {
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
            vmin = fminf(fminf(vmin, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
            vmax = fmaxf(fmaxf(vmax, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
            if (resident) *reinterpret_cast<float4*>(sm->row + (j - begin)) = v[u];
          }
        }
      }
      for (int j = n4 + tid; j < end; j += kTopkThreads) {
        const float v = __ldg(row + j);
        vmin = fminf(vmin, v);
        vmax = fmaxf(vmax, v);
        if (resident) sm->row[j - begin] = v;
      }
    }
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
    if (csize > 1) {
      if (tid < csize) {  // thread r tells rank r
        st_peer_u32(peer_addr(&sm->all_min[rank], tid), __float_as_uint(vmin));
        st_peer_u32(peer_addr(&sm->all_max[rank], tid), __float_as_uint(vmax));
      }
      cluster_barrier();
      for (unsigned int r = 0; r < csize; ++r) {  // every rank arrives at the same pair
        vmin = fminf(vmin, sm->all_min[r]);
        vmax = fmaxf(vmax, sm->all_max[r]);
      }
    }
    // monotone bucket map: floor((v - vmin) * inv), clamped. Non-finite range -> everything in bin 0
    // and the radix fallback resolves it.
    {
      const float range = vmax - vmin;
      if (range > 0.f && range < INFINITY) inv = static_cast<float>(kBins - 1) / range;
      if (!(inv < INFINITY)) inv = 0.f;
    }

    TKT(3);
    // ---- 2. histogram -----------------------------------------------------------------------
    {
      auto count = [&](float v, int) { atomicAdd(&sm->hist[bucket(v)], 1u); };
      if (resident) for_each_element<false>(sm->row - begin, begin, end, count);
      else for_each_element<true>(row, begin, end, count);
    }
    __syncthreads();
    if (csize == 2) {
      // two ranks: each stores its counts into the free upper half of the other's histogram area (plain remote
      // stores, all bins), one cluster barrier, and adds what it received to its own
      static_assert(kHistSlots >= 2 * kBins, "no room for the peer's counts");
#pragma unroll
      for (int u = 0; u < kBins / kTopkThreads; ++u) {
        const int bin = tid + u * kTopkThreads;
        st_peer_u32(peer_addr(&sm->hist[kBins + bin], rank ^ 1u), sm->hist[bin]);
      }
      cluster_barrier();
#pragma unroll
      for (int u = 0; u < kBins / kTopkThreads; ++u) {
        const int bin = tid + u * kTopkThreads;
        sm->hist[bin] += sm->hist[kBins + bin];
      }
      __syncthreads();
    } else if (csize > 1) {
      // every rank adds its counts into every other rank's histogram; a rank must not receive additions
      // before its own pass is over (they would be indistinguishable from its own counts only after it)
      unsigned int mine[kBins / kTopkThreads];
#pragma unroll
      for (int u = 0; u < kBins / kTopkThreads; ++u) mine[u] = sm->hist[tid + u * kTopkThreads];
      cluster_barrier();  // all local histograms complete and read into registers
#pragma unroll
      for (int u = 0; u < kBins / kTopkThreads; ++u) {
        if (mine[u] != 0) {
          for (unsigned int r = 0; r < csize; ++r) {
            if (r != rank) red_peer_add_u32(peer_addr(&sm->hist[tid + u * kTopkThreads], r), mine[u]);
          }
        }
      }
      cluster_barrier();  // every rank holds the row's histogram
    }
    TKT(4);
    find_threshold_bin<kBins / kTopkThreads>(sm, static_cast<unsigned int>(k));  // the same answer in every rank
  }
  TKT(5);
  const int thr_bin = sm->thr_bin;
  const unsigned int above = sm->thr_above;
  const unsigned int thr_count = sm->thr_count;
  const unsigned int need = static_cast<unsigned int>(k) - above;  // to take from the threshold bucket

  if (thr_count <= static_cast<unsigned int>(kCandCap)) {
    // ---- 3. collect (this rank's positions) ---------------------------------------------------
    {
      auto collect = [&](float v, int pos) {
        const int bkt = bucket(v);
        if (bkt > thr_bin) {
          sm->sel[atomicAdd(&sm->n_sel, 1u)] = make_key(v, pos);
        } else if (bkt == thr_bin) {
          sm->cand[atomicAdd(&sm->n_cand, 1u)] = make_key(v, pos);
        }
      };
      if (resident) for_each_element<false>(sm->row - begin, begin, end, collect);
      else for_each_element<true>(row, begin, end, collect);
    }
    __syncthreads();
    TKT(6);
    unsigned int direct_base = above;  // first output slot of the keys chosen among the candidates (direct mode)
    if (csize == 2 && unsorted) {
      // Two ranks, unordered output: ONE cluster barrier. Rank 1 writes its selected positions from the END of
      // the output row and pushes its candidates to the END of rank 0's candidate buffer (neither needs rank 0's
      // counts), with its count; after the barrier rank 0 moves them behind its own and fills the slots between
      // its selected positions and rank 1's with the chosen candidates.
      const unsigned int my_sel = sm->n_sel, my_cand = sm->n_cand;
      if (rank == 1) {
        for (unsigned int j = tid; j < my_sel; j += kTopkThreads) out[k - 1 - static_cast<int>(j)] = key_pos(sm->sel[j]);
        for (unsigned int j = tid; j < my_cand; j += kTopkThreads) st_peer_u64(peer_addr(&sm->cand[kCandCap - 1 - j], 0), sm->cand[j]);
        if (tid == 0) st_peer_u32(peer_addr(&sm->all_cand[1], 0), my_cand);
      } else {
        for (unsigned int j = tid; j < my_sel; j += kTopkThreads) out[j] = key_pos(sm->sel[j]);
      }
      cluster_barrier();  // rank 0 holds every candidate and rank 1's count
      if (rank != 0) return;
      const unsigned int c1 = sm->all_cand[1];
      // (thr_count = my_cand + c1 <= kCandCap, so the two segments cannot overlap)
      // (the two regions can overlap when there are many candidates: all reads, a barrier, then the writes)
      unsigned long long moved[kCandCap / kTopkThreads];
#pragma unroll
      for (int u = 0; u < kCandCap / kTopkThreads; ++u) {
        const unsigned int j = tid + u * kTopkThreads;
        moved[u] = j < c1 ? sm->cand[kCandCap - 1 - j] : 0ull;
      }
      __syncthreads();
#pragma unroll
      for (int u = 0; u < kCandCap / kTopkThreads; ++u) {
        const unsigned int j = tid + u * kTopkThreads;
        if (j < c1) sm->cand[my_cand + j] = moved[u];
      }
      direct_base = my_sel;
      __syncthreads();
    } else if (csize > 1) {
      if (tid < csize) {
        st_peer_u32(peer_addr(&sm->all_sel[rank], tid), sm->n_sel);
        st_peer_u32(peer_addr(&sm->all_cand[rank], tid), sm->n_cand);
      }
      cluster_barrier();  // every rank's lists are complete and all counts are known everywhere
      // offsets of this rank's lists in the row's lists
      unsigned int sel_off = 0, cand_off = 0;
      for (unsigned int r = 0; r < rank; ++r) {
        sel_off += sm->all_sel[r];
        cand_off += sm->all_cand[r];
      }
      // the candidates (and, for ordered output, the selected keys) of ranks 1.. are pushed into rank 0's
      // lists at their offsets: remote stores from all ranks at once, completed by the barrier below
      if (rank != 0) {
        const unsigned int my_cand = sm->n_cand;
        for (unsigned int j = tid; j < my_cand; j += kTopkThreads) st_peer_u64(peer_addr(&sm->cand[cand_off + j], 0), sm->cand[j]);
      }
      const unsigned int my_sel = sm->n_sel;
      if (unsorted) {
        // the selected positions go straight to the output
        for (unsigned int j = tid; j < my_sel; j += kTopkThreads) out[sel_off + j] = key_pos(sm->sel[j]);
      } else if (rank != 0) {
        for (unsigned int j = tid; j < my_sel; j += kTopkThreads) st_peer_u64(peer_addr(&sm->sel[sel_off + j], 0), sm->sel[j]);
      }
      cluster_barrier();  // rank 0's lists are complete; the other ranks are done
      if (rank != 0) return;
      __syncthreads();
    }
    TKT(7);
    // ---- 4. best `need` of the candidates (rank 0) --------------------------------------------
    // a chosen key goes to its place among the selected ones: straight to the output when every rank wrote its own
    // part there (unordered, cluster), else behind the `above` keys already in `sel`
    const bool direct = unsorted && csize > 1;
    auto emit = [&](unsigned int j, unsigned long long key) {
      if (direct) out[direct_base + j] = key_pos(key); else sm->sel[above + j] = key;
    };
    bool refined = false;
    if (coarse && need != thr_count && thr_count > 256u) {
      // The candidates of a coarse bin share the top 12 bits of their value word and are many (the bin is wide):
      // one more radix step inside shared memory instead of sorting them all. Digit: the next 11 bits of the value.
      constexpr int kFineShift = 32 + kLiHistShift - 11;
      for (int j = tid; j < kBins; j += kTopkThreads) sm->hist[j] = 0;
      if (tid == 0) {
        sm->n_sel2 = 0;
        sm->n_cand2 = 0;
      }
      __syncthreads();
      for (unsigned int j = tid; j < thr_count; j += kTopkThreads) {
        atomicAdd(&sm->hist[static_cast<unsigned int>(sm->cand[j] >> kFineShift) & (kBins - 1)], 1u);
      }
      __syncthreads();
      find_threshold_bin<kBins / kTopkThreads>(sm, need);
      const unsigned int fine_bin = static_cast<unsigned int>(sm->thr_bin), fine_above = sm->thr_above, fine_count = sm->thr_count;
      __syncthreads();  // the histogram area becomes the list of the keys in the fine threshold bin
      unsigned long long* tmp = reinterpret_cast<unsigned long long*>(sm->hist);
      constexpr unsigned int kTmpCap = kHistSlots * sizeof(unsigned int) / sizeof(unsigned long long);
      if (fine_count <= kTmpCap) {
        for (unsigned int j = tid; j < thr_count; j += kTopkThreads) {
          const unsigned long long key = sm->cand[j];
          const unsigned int f = static_cast<unsigned int>(key >> kFineShift) & (kBins - 1);
          if (f > fine_bin) emit(atomicAdd(&sm->n_sel2, 1u), key);
          else if (f == fine_bin) tmp[atomicAdd(&sm->n_cand2, 1u)] = key;
        }
        __syncthreads();
        const unsigned int need2 = need - fine_above;
        if (need2 != fine_count) {
          int cpow2 = 2;
          while (cpow2 < static_cast<int>(fine_count)) cpow2 <<= 1;
          for (int j = fine_count + tid; j < cpow2; j += kTopkThreads) tmp[j] = 0ull;
          bitonic_sort_desc(tmp, cpow2);
        }
        for (unsigned int j = tid; j < need2; j += kTopkThreads) emit(fine_above + j, tmp[j]);
        refined = true;
      }
    }
    if (!refined) {
      if (need != thr_count && thr_count <= 512u) {
        // few candidates (the usual case: a fine bucket holds a few dozen): every candidate counts the candidates
        // above it (keys are unique, so the counts are the ranks) and the first `need` ranks go out. All threads
        // read the same candidate at a time (a broadcast); no barrier inside, where a bitonic sort of 1024 threads
        // spends its time.
        __syncthreads();
        if (static_cast<unsigned int>(tid) < thr_count) {
          const unsigned long long mine = sm->cand[tid];
          unsigned int rank_of = 0;
          for (unsigned int j = 0; j < thr_count; ++j) rank_of += sm->cand[j] > mine ? 1u : 0u;
          if (rank_of < need) emit(rank_of, mine);
        }
      } else {
        if (need != thr_count) {
          int cpow2 = 1;
          while (cpow2 < static_cast<int>(thr_count)) cpow2 <<= 1;
          for (int j = thr_count + tid; j < cpow2; j += kTopkThreads) sm->cand[j] = 0ull;
          bitonic_sort_desc(sm->cand, cpow2);
        }
        for (unsigned int j = tid; j < need; j += kTopkThreads) emit(j, sm->cand[j]);
      }
    }
    TKT(8);
    if (direct) return;
    __syncthreads();
  } else {
    // ---- 4'. massive ties: MSB-first radix select on the 64-bit keys of the threshold bucket ----
    // (rank 0 alone, over the whole row; the decision above is the same in every rank)
    if (rank != 0) return;
    if (tid == 0) sm->n_sel = 0;
    __syncthreads();
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
      for_each_element<true>(row, 0, eff, [&](float v, int pos) {
        if (bucket(v) != thr_bin) return;
        const unsigned long long key = make_key(v, pos);
        if (shift < 64 && (key >> shift) != prefix) return;
        atomicAdd(&sm->hist[static_cast<unsigned int>(key >> new_shift) & ((1u << w) - 1u)], 1u);
      });
      __syncthreads();
      find_threshold_bin<kBins / kTopkThreads>(sm, remaining);
      remaining -= sm->thr_above;
      exact = (sm->thr_count == remaining);
      prefix = (prefix << w) | static_cast<unsigned long long>(sm->thr_bin);
      shift = new_shift;
      __syncthreads();
    }
    // every key with (key >> shift) >= prefix inside the bucket, plus all higher buckets
    for_each_element<true>(row, 0, eff, [&](float v, int pos) {
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
  if (!unsorted) {
    for (int j = k + tid; j < kpow2; j += kTopkThreads) sm->sel[j] = 0ull;
    bitonic_sort_desc(sm->sel, kpow2);
  }
  for (int j = tid; j < k; j += kTopkThreads) out[j] = key_pos(sm->sel[j]);
}

}  // namespace

cudaError_t launch_li_topk(const TopkParams& p, int num_sms, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(li_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(TopkSmem)));
  if (e != cudaSuccess) return e;
  // as many CTAs per row as keep the grid within one wave (portable cluster sizes: up to 8)
  const int rows = p.b * p.s1;
  int csize = 1;
  while (csize < 8 && rows * csize * 2 <= num_sms) csize *= 2;
  // ordered output ends in a 2048-key sort on rank 0 that dwarfs the scans of short rows: measured, a
  // cluster only pays there for rows beyond ~40 K positions
  if ((p.flags & PTO_LI_UNSORTED) == 0 && p.row_stride <= 40960) csize = 1;
  static const int forced = [] {  // PTO_TOPK_CLUSTER=1|2|4|8 in the environment: CTAs per row (A/B timing aid)
    const char* v = getenv("PTO_TOPK_CLUSTER");
    const int want = v != nullptr ? atoi(v) : 0;
    return (want == 1 || want == 2 || want == 4 || want == 8) ? want : 0;
  }();
  if (forced != 0) csize = forced;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * csize), 1, 1);
  cfg.blockDim = dim3(kTopkThreads, 1, 1);
  cfg.dynamicSmemBytes = sizeof(TopkSmem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(csize);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // may be scheduled while the kernel before it drains; it waits (first instruction) before it reads anything
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  count_launch();
  return cudaLaunchKernelEx(&cfg, li_topk_kernel, p);
}

int topk_max_k() { return kMaxK; }

#ifdef PTO_TOPK_TIMELINE
extern "C" int pto_debug_topk_timeline(long long* host, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_topk_tl, sizeof(long long) * n));
}
#endif

}  // namespace pto
