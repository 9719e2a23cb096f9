// Sparse MLA attention for all 128 heads of a token on a PAIR of SMs that share every matrix product
// (tcgen05.mma.cta_group::2): the two CTAs of a cluster split the token's HEADS, 64 each.
//
// Arithmetic as in sfa_decode.cu (reference:
// examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:45-207; golden
// deepseekv32_sparse_flash_attention_quant.py:169-254).
//
// Why a pair: the fp32 output of 128 heads x 512 values is 256 KB, all of one SM's tensor memory. With the
// heads split, CTA c keeps O for its 64 heads (256 columns) and two score buffers (2 x 64 columns), and the
// whole 576-wide contraction is local to the pair's MMA: no score ever crosses between the CTAs, and nothing
// else does either except four "ready" notices per tile. A 2-SM MMA reads half of its B operand from
// each CTA's shared memory:
//   q.K^T  (M = 128 heads, N = 128 keys of a tile, K = 576): A = this CTA's 64 query rows, B = the tile's keys,
//          of which CTA c gathers and dequantises keys [64c, 64c+64) in full width (9 chunks of 64 dims).
//   P.V    (M = 128 heads, N = 256 of the 512 values per MMA, K = 128 keys): A = this CTA's P, B = V, of which
//          CTA c supplies the value columns [256c, 256c+256) of ALL 128 keys. Shared memory between the SMs
//          moves about 7 bytes per clock (measured: a 32 KB bulk copy to the peer takes 4-5 k cycles), far too
//          slow to ship the other CTA's keys over, so a second group of producers gathers that half of all
//          128 rows again (an L2 hit: the other CTA has just fetched the row) and dequantises it.
// Tensor memory of a 2-SM MMA with 64 rows per CTA: lanes 0-63 hold the first half of the N columns, lanes
// 64-127 the second half (row = lane % 64). So of a score tile lane l holds (head l % 64, keys 64 (l / 64) ..+63),
// and of O lane l holds (head l % 64, values 256 (l / 64) ..+255).
//   warp 0          CTA 0: issues the q.K^T MMAs of a tile as soon as its keys are ready and a score buffer is free
//   warp 2          CTA 0: issues the P.V MMAs of a tile as soon as P is written and the values are ready
//                   (two issuing threads on two schedulers: neither queue waits behind the other's barrier)
//   warp 1          CTA 1: forwards the "ready" events of its own CTA to CTA 0 (tcgen05.commit arrivals on CTA 0's barriers)
//   warps 4..11     softmax: four threads per head (two TMEM lanes x two column halves), P goes to shared memory
//   warps 12..19    K producers: 16-byte gathers of the CTA's 64 rows, int8 -> bf16 in registers, swizzled stores
//   warps 20..27    V producers: this CTA's half of the value columns of all 128 rows
// Cache formats: int8 latent + bf16 rope + fp32 scales in three arrays, the same as packed 656-byte rows, or bf16
// latent + rope arrays (the non-quantised cache): there the producers dequantise nothing, they copy the rows' bytes
// from L2 to the same swizzled places with cp.async once a buffer half is free. The MMAs, the softmax and the
// output are the same code, so the bf16 cache of dequantised values gives the int8 cache's output bit for bit.
// Roles are uniform within each group of four warps so that registers can be moved between them (setmaxnreg):
// 72 per thread at launch (seven warps share one scheduler's file of 512 x 32), then 24 / 104 / 72 / 64:
// nothing spills (a spilled register costs a trip to L2: beside 227 KB of shared memory there is no L1 to speak of).
// All waits are bounded.
#include "common.cuh"
#include "sfa_common.cuh"

namespace pto {

namespace {

// Developer aid: -DPTO_PAIR_TIMELINE records clock64() at 16 points of the first 24 tiles of cluster 0.
#ifdef PTO_PAIR_TIMELINE
__device__ long long g_pair_tl[2 * 24 * 16];
#define TLP(slot, j) do { if (blockIdx.x < 2 && (j) >= 0 && (j) < 24) g_pair_tl[((blockIdx.x & 1) * 24 + (j)) * 16 + (slot)] = clock64(); } while (0)
#else
#define TLP(slot, j) do { } while (0)
#endif

constexpr int kPT = 128;                 // selected rows per tile (64 per CTA)
constexpr int kPRows = 64;               // rows a CTA gathers in full width per tile; also heads per CTA
constexpr int kChunk = kPRows * 128;     // 64 rows x 64 bf16 (128-byte rows, 128-byte swizzle): 8 KB
constexpr int kQChunks = 9;              // 8 latent chunks + 1 rope chunk
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + kQChunks * kChunk;        // 73,728
constexpr int kSmemV = kSmemK + kQChunks * kChunk;        // 147,456: two regions (keys 0-63, keys 64-127) of 4 chunks
constexpr int kSmemP = kSmemV + 8 * kChunk;               // 212,992: two chunks (keys 0-63, keys 64-127)
constexpr int kSmemCtl = kSmemP + 2 * kChunk;             // 229,376
constexpr int kVHalfBytes = 4 * kChunk;                   // 32 KB: 64 keys x 256 values
constexpr int kPairSoftmaxWarp0 = 4, kPairSoftmaxWarps = 8;
constexpr int kPairKWarp0 = 12, kPairKWarps = 8;
constexpr int kPairVWarp0 = 20, kPairVWarps = 8;
constexpr int kPairThreads = 32 * 28;
constexpr uint32_t kPairTmemCols = 512;
constexpr uint32_t kPairColO = 0, kPairColS = 256;        // S buffer b at kPairColS + 64 b
constexpr float kPairRescale = 8.0f;

struct PairCtl {
  // The K chunks and the V regions are each handed over in two halves, so that a refill runs behind the MMAs that
  // read the other half: K half 0 = chunks 0-3, half 1 = chunks 4-8 (with the rope chunk); V half h = keys 64h..+63.
  uint64_t kfull[2];   // K producers filled half h of this CTA's K chunks of tile j     (8 warps)
  uint64_t kfree[2];   // the q.K^T MMAs that read half h are complete                   (tcgen05.commit, both CTAs)
  uint64_t vfull[2];   // V producers filled this CTA's V region of key half h           (8 warps)
  uint64_t vfree[2];   // the P.V MMAs that read key half h are complete                 (tcgen05.commit, both CTAs)
  uint64_t sfull[2];   // q.K^T of a tile complete (score buffer b)                      (tcgen05.commit, both CTAs)
  uint64_t pvdone;     // P.V of a tile complete                                        (tcgen05.commit, both CTAs)
  uint64_t pfull;      // this CTA's P of tile j written                                (8 warps)
  uint64_t sread[2];   // this CTA's softmax warps have the scores in registers         (8 warps)
  // in CTA 0 only: the same events of CTA 1, forwarded (one arrival each)
  uint64_t kpeer[2], vpeer[2], ppeer, speer[2];
  uint32_t tmem_base;
  int abort;
  int go[3][2];        // outcome of a role's latest waits (softmax, K producers, V producers)
  float mt[2][4][64];  // [tile parity][key half * 2 + column half][head]: partial maxima; partial sums at the end
};
static_assert(kSmemCtl + sizeof(PairCtl) <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
constexpr size_t kPairSmemBytes = 232448;

__device__ __forceinline__ uint32_t pair_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void pair_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Notice from CTA 1 to CTA 0: a tcgen05.commit of no outstanding operation arrives at once on the mbarrier at this
// offset in CTA 0 (mask 1). It travels on the tensor pipe's own path: measured one way 390 cycles, as fast as an
// asynchronous remote store, but unlike that store it does not queue behind the SM's gathers in the load/store
// unit (under load the store took 2000-3300 cycles to arrive; a remote mbarrier arrive holds the lane ~1400).
__device__ __forceinline__ void pair_signal(uint32_t bar_local) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar_local), "h"(static_cast<uint16_t>(1))
               : "memory");
}

__device__ __forceinline__ void mma2_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (count 1) on the mbarrier at this offset in BOTH CTAs once all MMAs issued so far have completed
__device__ __forceinline__ void tc2_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3))
               : "memory");
}

// Warp-wide bounded wait that sleeps between probes. A probe is a shared-memory access and a handful of
// instructions; two dozen warps probing back to back take issue slots and shared-memory cycles from the warps
// that have work.
template <int kSleepNs>
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity) {
  bool ok = true;
  if (!mbar_test_wait(bar, parity)) {
    const long long t0 = clock64();
    while (true) {
      __nanosleep(kSleepNs);
      if (mbar_test_wait(bar, parity)) break;
      if (clock64() - t0 > kWaitBudgetCycles) {
        ok = false;
        break;
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

// Wait of a whole role (kThreads threads = full warps, named barrier kBarId): only the role's first warp probes the
// mbarrier, the others block at the named barrier without issuing anything. The first warp publishes the outcome
// in one of two slots (alternating: a thread is never more than one wait behind), every thread of the role reads
// the same slot after the barrier, so the whole role takes the same branch; the barrier itself depends on no data
// and every thread of the role reaches it on every path.
template <int kSleepNs, int kBarId, int kThreads, int kRole>
__device__ __forceinline__ bool pair_group_wait(PairCtl* ctl, uint32_t& nwait, uint32_t bar, uint32_t parity, bool first_warp) {
  volatile int* go = &ctl->go[kRole][nwait & 1u];
  ++nwait;
  if (first_warp) {
    const bool ok = pair_wait<kSleepNs>(bar, parity);
    if ((threadIdx.x & 31) == 0) *go = ok ? 1 : 0;
  }
  asm volatile("bar.sync %0, %1;" ::"n"(kBarId), "n"(kThreads) : "memory");
  return *go != 0;
}

// 8 int8 (two words) -> 8 bf16 of (value * scale), as `dequant16` but with the subtraction and the multiplication on pairs
// (fp32x2 instructions): the byte placed in the mantissa of 2^23 gives 2^23 + 128 + x exactly, subtracting 8388736
// leaves x, one fp32 multiply and one rounding to bf16: bf16(fp32(x) * scale) as the golden computes it.
__device__ __forceinline__ uint4 pair_dequant8(const uint32_t w0, const uint32_t w1, const float scale) {
  const float2 off = make_float2(-8388736.0f, -8388736.0f), sc = make_float2(scale, scale);
  uint4 o;
  {
    const uint32_t w = w0 ^ 0x80808080u;
    float2 a = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)));
    float2 b = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)));
    a = __fmul2_rn(__fadd2_rn(a, off), sc);
    b = __fmul2_rn(__fadd2_rn(b, off), sc);
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(b.x, b.y);
  }
  {
    const uint32_t w = w1 ^ 0x80808080u;
    float2 a = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)));
    float2 b = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)));
    a = __fmul2_rn(__fadd2_rn(a, off), sc);
    b = __fmul2_rn(__fadd2_rn(b, off), sc);
    o.z = pack_bf16x2(a.x, a.y);
    o.w = pack_bf16x2(b.x, b.y);
  }
  return o;
}

// Paged row of a selected position, in 32 bits (the host side refuses caches of 2^31 rows or more): -1 for a
// padding index or a rejected one (reported once through the status words).
__device__ __forceinline__ int pair_row(const SfaParams& p, int idx, int entry) {
  if (entry == kTableSkip) return -1;
  const long long r = static_cast<long long>(entry) * p.block_size + idx % p.block_size;
  if (entry < 0 || r >= p.n_rows) {
    set_status(p.status, PTO_ST_BAD_PAGE, entry, 21);
    return -1;
  }
  return static_cast<int>(r);
}

struct PairCtx {
  PairCtl* ctl;
  const int32_t* idx_row;  // this token's selected positions
  int64_t q_row0;          // first query/output row of the token
  uint32_t base, tmem_base, crank;
  int ntiles, begin, end, ti, sp, bi;
};

// The one meeting of all threads of the pair before the tile loop: barriers initialised, tensor memory allocated,
// both Q halves in shared memory. Every role calls it exactly once; the producers call it after they have
// requested their first rows, so that the index -> block table -> row chain of the first tile (three dependent
// trips to memory) runs beside the set-up instead of after it.
__device__ __forceinline__ uint32_t pair_setup_sync(PairCtl* ctl) {
  tc_fence_before();
  __syncthreads();
  pair_cluster_sync();
  tc_fence_after();
  // the kernel behind this one (the merge of the split partials) may be scheduled from here on; it waits for
  // this grid to complete before it reads anything
  if (threadIdx.x == 0) pdl_trigger();
  if (threadIdx.x == 0) TLP(1, 20);  // roles start
  return ctl->tmem_base;
}

// ================================ MMA issuers (CTA 0) ===========================================
// Two threads on two different schedulers: warp 0 issues the score products, warp 2 the value products.
//   q.K^T first half  (chunks 0-3: 16 MMAs)  needs K half 0 of the tile and the score buffer it overwrites read
//   q.K^T second half (chunks 4-8: 20 MMAs)  needs K half 1; completes the tile's scores
//   P.V first half    (keys 0-63:   8 MMAs)  needs P of the tile and V key half 0
//   P.V second half   (keys 64-127: 8 MMAs)  needs V key half 1; completes the tile's P.V
// After each action a commit hands the half it read back to its producers, so that the refill for the next tile
// runs behind the MMAs that read the other half. One thread issuing everything (an event loop over the four
// actions) was what a tile waited for: 36 + 16 MMAs kept it busy for 8.7 k cycles per tile; side by side the two
// threads take 3.2-4.0 k and 1.5-2.7 k (80.1 -> 77.7 us on 64 tokens x 2048 rows). The products of the two threads
// are independent (different accumulators), every dependency between them goes through the mbarriers, and a
// commit covers the MMAs of the thread that executes it.
// (No cluster-scope fence before the MMAs: measured, `fence.acq_rel.cluster` holds a thread for 2000-3700 cycles
// per use. The order is kept by the chain itself: CTA 1's writers fence for the async proxy and arrive on their
// own barrier, its forwarding thread observes that barrier before it sends the notice, and the MMA issued here
// after the notice reads CTA 1's shared memory from CTA 1's side.)
__device__ __forceinline__ bool pair_poll(uint32_t bar, uint32_t parity) {  // one thread, bounded
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    __nanosleep(20);
    if (mbar_test_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

__device__ __forceinline__ void pair_role_issue_qk(const SfaParams& p, PairCtx c) {
  PairCtl* ctl = c.ctl;
  const int ntiles = c.ntiles;
  c.tmem_base = pair_setup_sync(ctl);
  if ((threadIdx.x & 31) == 0) {
    const uint32_t idesc_qk = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 0, 128, kPT);
    const uint32_t q_base = c.base + kSmemQ, k_base = c.base + kSmemK;
    auto issue_qk_chunks = [&](int j, int ch0, int ch1) {
      const uint32_t d = c.tmem_base + kPairColS + 64 * (j & 1);
#pragma unroll 1
      for (int ch = ch0; ch < ch1; ++ch) {
        const uint64_t a_desc = umma_desc_kmajor_sw128(q_base + ch * kChunk);
        const uint64_t b_desc = umma_desc_kmajor_sw128(k_base + ch * kChunk);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma2_f16_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc_qk, (ch | k) != 0 ? 1u : 0u);
      }
    };
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const uint32_t ph = j & 1;
      ok = pair_poll(smem_u32(&ctl->kfull[0]), ph) && pair_poll(smem_u32(&ctl->kpeer[0]), ph);
      if (ok && j >= 2) {  // the score buffer it overwrites has been read in both CTAs
        const uint32_t sp = ((j - 2) >> 1) & 1;
        ok = pair_poll(smem_u32(&ctl->sread[j & 1]), sp) && pair_poll(smem_u32(&ctl->speer[j & 1]), sp);
      }
      if (!ok) break;
      tc_fence_after();
      TLP(6, j);
      issue_qk_chunks(j, 0, 4);
      tc2_commit(smem_u32(&ctl->kfree[0]));
      ok = pair_poll(smem_u32(&ctl->kfull[1]), ph) && pair_poll(smem_u32(&ctl->kpeer[1]), ph);
      if (!ok) break;
      tc_fence_after();
      issue_qk_chunks(j, 4, kQChunks);
      tc2_commit(smem_u32(&ctl->kfree[1]));
      tc2_commit(smem_u32(&ctl->sfull[j & 1]));
      TLP(7, j);
    }
    if (!ok) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 50);
    }
  }
  __syncwarp();
}

__device__ __forceinline__ void pair_role_issue_pv(const SfaParams& p, PairCtx c) {
  PairCtl* ctl = c.ctl;
  const int ntiles = c.ntiles;
  c.tmem_base = pair_setup_sync(ctl);
  if ((threadIdx.x & 31) == 0) {
    const uint32_t idesc_pv = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 1, 128, 256);
    const uint32_t v_base = c.base + kSmemV, p_base = c.base + kSmemP;
    auto issue_pv_half = [&](int j, int kh) {  // keys 64 kh .. +63 into both pairs of value columns
      const uint64_t a_desc = umma_desc_kmajor_sw128(p_base + kh * kChunk);
#pragma unroll 1
      for (int dp = 0; dp < 2; ++dp) {
        const uint64_t b_desc = desc_mnmajor_sw128(v_base + kh * kVHalfBytes + dp * 2 * kChunk, kChunk, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          mma2_f16_ss(c.tmem_base + kPairColO + 128 * dp, a_desc + 2 * k, b_desc + k * ((16 * 128) >> 4), idesc_pv,
                      (j > 0 || kh > 0 || k > 0) ? 1u : 0u);
        }
      }
    };
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const uint32_t ph = j & 1;
      ok = pair_poll(smem_u32(&ctl->pfull), ph) && pair_poll(smem_u32(&ctl->ppeer), ph) &&
           pair_poll(smem_u32(&ctl->vfull[0]), ph) && pair_poll(smem_u32(&ctl->vpeer[0]), ph);
      if (!ok) break;
      tc_fence_after();
      TLP(8, j);
      issue_pv_half(j, 0);
      tc2_commit(smem_u32(&ctl->vfree[0]));
      ok = pair_poll(smem_u32(&ctl->vfull[1]), ph) && pair_poll(smem_u32(&ctl->vpeer[1]), ph);
      if (!ok) break;
      tc_fence_after();
      issue_pv_half(j, 1);
      tc2_commit(smem_u32(&ctl->vfree[1]));
      tc2_commit(smem_u32(&ctl->pvdone));
      TLP(9, j);
    }
    if (!ok) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 55);
    }
  }
  __syncwarp();
}

// ================================ forwarding (CTA 1) ============================================
// One thread: whenever one of this CTA's per-tile events completes, tell CTA 0.
__device__ __forceinline__ void pair_role_relay(const SfaParams& p, PairCtx c) {
  PairCtl* ctl = c.ctl;
  const int ntiles = c.ntiles;
  pair_setup_sync(ctl);
  if ((threadIdx.x & 31) == 0) {
    int k_i[2] = {0, 0}, v_i[2] = {0, 0}, p_i = 0, s_i = 0;  // s_i: scores of tile s_i read (only tiles that have a successor two on)
    const int s_n = ntiles > 2 ? ntiles - 2 : 0;
    long long t_last = clock64();
    bool ok = true;
    while (k_i[0] < ntiles || k_i[1] < ntiles || v_i[0] < ntiles || v_i[1] < ntiles || p_i < ntiles || s_i < s_n) {
      bool progressed = false;
      if (p_i < ntiles && mbar_test_wait(smem_u32(&ctl->pfull), p_i & 1)) {
        pair_signal(smem_u32(&ctl->ppeer));
        ++p_i;
        progressed = true;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (k_i[h] < ntiles && mbar_test_wait(smem_u32(&ctl->kfull[h]), k_i[h] & 1)) {
          pair_signal(smem_u32(&ctl->kpeer[h]));
          ++k_i[h];
          progressed = true;
        }
        if (v_i[h] < ntiles && mbar_test_wait(smem_u32(&ctl->vfull[h]), v_i[h] & 1)) {
          pair_signal(smem_u32(&ctl->vpeer[h]));
          ++v_i[h];
          progressed = true;
        }
      }
      if (s_i < s_n && mbar_test_wait(smem_u32(&ctl->sread[s_i & 1]), (s_i >> 1) & 1)) {
        pair_signal(smem_u32(&ctl->speer[s_i & 1]));
        ++s_i;
        progressed = true;
      }
      if (progressed) {
        t_last = clock64();
      } else {
        __nanosleep(20);
        if (clock64() - t_last > kWaitBudgetCycles) {
          ok = false;
          break;
        }
      }
    }
    if (!ok) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 54);
    }
  }
  __syncwarp();
}

// ================================ softmax =======================================================
// Thread (TMEM lane L, column half ch): head L % 64, keys 64 (L / 64) + 32 ch .. +31 of the 128-key tile.
__device__ __forceinline__ void pair_role_softmax(const SfaParams& p, PairCtx c) {
  PairCtl* ctl = c.ctl;
  const uint32_t tmem_base = pair_setup_sync(ctl);
  const int ntiles = c.ntiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = warp & 3;                            // TMEM lane quarter this warp may access
  const int ch = (warp - kPairSoftmaxWarp0) >> 2;      // column half
  const int kh = sub >> 1;                             // key half of the tile
  const int hg = sub & 1;                              // head group: heads 32 hg .. +31
  const int head = 32 * hg + lane;
  const int slot = kh * 2 + ch;                        // which of the head's four threads
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(sub * 32) << 16);
  const uint32_t p_row = c.base + kSmemP + kh * kChunk + head * 128;
  const int psw = head & 7;
  const bool tl = threadIdx.x == 32 * kPairSoftmaxWarp0;
  float m_seen = -INFINITY;  // the head's reference max (identical in its four threads)
  float l_run = 0.f;         // this thread's share of the row sum
  bool ok = true;
  const bool first_warp = warp == kPairSoftmaxWarp0;
  uint32_t nwait = 0;
  auto meet = [&]() {  // the four warps of a head group: orders their mt writes before the reads (named barriers 4, 5)
    if (hg == 0) asm volatile("bar.sync 4, 128;" ::: "memory");
    else asm volatile("bar.sync 5, 128;" ::: "memory");
  };
  for (int j = 0; j < ntiles; ++j) {
    const int b = j & 1;
    ok = pair_group_wait<20, 1, 256, 0>(ctl, nwait, smem_u32(&ctl->sfull[b]), (j >> 1) & 1, first_warp);
    if (!ok) break;
    if (tl) TLP(10, j);
    tc_fence_after();
    float s[32];
    {
      uint32_t v[32];
      tmem_ld_32x32b_x32(lane_addr + kPairColS + 64 * b + 32 * ch, v);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(v[i]);
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->sread[b]));  // the score buffer may be overwritten
    // ---- mask rows past the token's selected count (last tile only) --------------------------------
    const int key0 = c.begin + j * kPT + 64 * kh + 32 * ch;
    if (key0 + 32 > c.end) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (key0 + i >= c.end) s[i] = -INFINITY;
      }
    }
    float mt2[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; ++i) mt2[i & 1] = fmaxf(mt2[i & 1], s[i]);
    const float mt_part = fmaxf(mt2[0], mt2[1]) * p.scale_log2;  // scale > 0
    ctl->mt[b][slot][head] = mt_part;
    // ---- exponentials against a speculative reference (corrected by one factor once the head's max is known) --
    float m_spec = (m_seen == -INFINITY || mt_part > m_seen + kPairRescale) ? mt_part : m_seen;
    if (m_spec == -INFINITY) m_spec = 0.f;
    const float neg_spec = -m_spec;
    float ls2[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s[i] = ex2f(fmaf(s[i], p.scale_log2, neg_spec));
      ls2[i & 1] += s[i];
    }
    const float lsum = ls2[0] + ls2[1];
    if (tl) TLP(11, j);
    meet();
    if (tl) TLP(12, j);
    const float mt = fmaxf(fmaxf(ctl->mt[b][0][head], ctl->mt[b][1][head]), fmaxf(ctl->mt[b][2][head], ctl->mt[b][3][head]));
    const float m_new = fmaxf(m_seen, mt);
    const bool need = (m_new > m_seen + kPairRescale) || (m_seen == -INFINITY && m_new > -INFINITY);
    float alpha = 1.f;
    if (need) {
      alpha = (m_seen == -INFINITY) ? 0.f : ex2f(m_seen - m_new);
      m_seen = m_new;
    }
    const float m_ref = (m_seen == -INFINITY) ? 0.f : m_seen;
    const float factor = ex2f(m_spec - m_ref);
    l_run = l_run * alpha + lsum * factor;
    // ---- the previous tile's P.V is complete: P may be overwritten, O is at rest ----------------------
    if (j > 0) {
      ok = pair_group_wait<20, 1, 256, 0>(ctl, nwait, smem_u32(&ctl->pvdone), (j - 1) & 1, first_warp);
      if (!ok) break;
      tc_fence_after();
    }
    if (tl) TLP(13, j);
    if (j > 0 && __any_sync(0xffffffffu, need)) {  // rare: rescale this thread's 128 output columns
#pragma unroll 1
      for (int cc = 0; cc < 8; ++cc) {
        uint32_t o[16];
        tmem_ld_32x32b_x16(lane_addr + kPairColO + ch * 128 + cc * 16, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32b_x16(lane_addr + kPairColO + ch * 128 + cc * 16, o);
      }
      tc_wait_st();
    }
    // ---- P row piece into shared memory (A operand of P.V): 32 keys = four 16-byte units 4 ch .. 4 ch + 3 ----
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint4 w;
      w.x = pack_bf16x2(s[8 * u] * factor, s[8 * u + 1] * factor);
      w.y = pack_bf16x2(s[8 * u + 2] * factor, s[8 * u + 3] * factor);
      w.z = pack_bf16x2(s[8 * u + 4] * factor, s[8 * u + 5] * factor);
      w.w = pack_bf16x2(s[8 * u + 6] * factor, s[8 * u + 7] * factor);
      sts_v4u(p_row + (((4 * ch + u) ^ psw) << 4), w);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->pfull));
    if (tl) TLP(14, j);
  }
  // ---- output ---------------------------------------------------------------------------------------
  if (ok) ok = pair_group_wait<20, 1, 256, 0>(ctl, nwait, smem_u32(&ctl->pvdone), (ntiles - 1) & 1, first_warp);
  if (tl) TLP(5, 20);  // last P.V complete
  float l_tot = 0.f;
  if (ok) {
    ctl->mt[ntiles & 1][slot][head] = l_run;
    meet();
    const int b = ntiles & 1;
    l_tot = (ctl->mt[b][0][head] + ctl->mt[b][1][head]) + (ctl->mt[b][2][head] + ctl->mt[b][3][head]);
  }
  // The rows go out through shared memory: a thread holds 128 values of ONE row, so direct stores put every lane of
  // a warp on its own 128-byte line (4096 lines per CTA, about 4 k cycles); staged, a warp writes 512 contiguous
  // bytes. Staging area: the K chunks (all q.K^T of this cluster are complete once the last P.V is), rows of
  // 1 KB + 16 B (the pad keeps the lanes of a warp, which write different rows, on different banks); a row holds
  // the 256-byte pieces of the head's four threads. bf16 rows take one pass, fp32 partial rows two.
  {
    const uint32_t stage = c.base + kSmemK;
    constexpr uint32_t kStageRow = 1024 + 16;
    static_assert(64 * kStageRow <= kQChunks * kChunk, "output staging exceeds the K chunks");
    const int stid = threadIdx.x - 32 * kPairSoftmaxWarp0;       // 0..255
    const uint32_t my_piece = stage + head * kStageRow + slot * 256;
    const bool direct = p.n_split == 1;
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    const int npass = direct ? 1 : 2;
    if (ok) tc_fence_after();
#pragma unroll 1
    for (int ps = 0; ps < npass; ++ps) {
      if (ok) {
#pragma unroll 1
        for (int cc = 0; cc < (direct ? 4 : 2); ++cc) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kPairColO + ch * 128 + (direct ? cc : 2 * ps + cc) * 32, o);
          tc_wait_ld();
          if (direct) {  // 32 values -> 64 bytes
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              sts_v4u(my_piece + cc * 64 + i * 2, w);
            }
          } else {       // 32 values -> 128 bytes
#pragma unroll
            for (int i = 0; i < 32; i += 4) sts_v4u(my_piece + cc * 128 + i * 4, make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]));
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");  // (every softmax thread reaches it, also after an expired wait)
      if (ok) {
        // 64 rows x 64 units of 16 bytes; consecutive threads take consecutive units of a row
        uint8_t* gbase;
        int64_t grow_bytes;  // bytes between rows in global memory
        if (direct) {
          gbase = reinterpret_cast<uint8_t*>(p.out + (c.q_row0 + 64 * static_cast<int>(c.crank)) * 512);
          grow_bytes = 1024;
        } else {
          const int64_t prow0 = (static_cast<int64_t>(c.ti) * p.n_split + c.sp) * p.nq + 64 * static_cast<int>(c.crank);
          gbase = reinterpret_cast<uint8_t*>(p.part_o + prow0 * 512);
          grow_bytes = 2048;
        }
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int e = it * 256 + stid;
          const int r = e >> 6, unit = e & 63;        // unit: 16 bytes of the staged row; piece = unit / 16
          const uint4 w = lds_v4u(stage + r * kStageRow + unit * 16);
          // bf16: the row's bytes in order. fp32: piece q of pass ps holds floats 128 q + 64 ps .. + 63 of the row
          const int64_t off = direct ? unit * 16 : ((unit >> 4) * 512 + ps * 256 + (unit & 15) * 16);
          *reinterpret_cast<uint4*>(gbase + r * grow_bytes + off) = w;
        }
      }
      if (ps + 1 < npass) asm volatile("bar.sync 1, 256;" ::: "memory");  // staging area reused by the next pass
    }
    if (ok && !direct && slot == 0) {
      const int64_t prow = (static_cast<int64_t>(c.ti) * p.n_split + c.sp) * p.nq + 64 * static_cast<int>(c.crank) + head;
      p.part_ml[prow * 2] = m_seen;
      p.part_ml[prow * 2 + 1] = l_tot;
    }
  }
  if (!ok && lane == 0) {
    ctl->abort = 1;
    set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 51);
  }
}

// ================================ K producers ===================================================
// 256 threads; warp w owns rows 8w .. 8w+7 of this CTA's 64. A gather instruction reads half a row's latent bytes
// (256 = two whole 128-byte lines) of TWO rows: lane l takes unit l % 16 of row 2m + l / 16, once for the first
// half of the row (chunks 0-3) and once for the second (chunks 4-7), so a thread holds unit l % 16 and unit
// 16 + l % 16 of four rows. (Four threads per row, each reading its own 16 bytes of eight different lines, cost
// eight lines per instruction; with the V producers' gathers on top, the load/store unit's queue then delayed
// the tensor core's operand reads: q.K^T took 5-6 k cycles instead of 2.5 k.)
// Unit u (16 int8 -> 16 bf16 = two 16-byte stores) goes to chunk u / 4, store units 2 (u % 4) and 2 (u % 4) + 1 of
// the row's 128 bytes; the lanes of an odd chunk store the second half first, so that the eight lanes of a
// quarter-warp (two chunks, same row) hit eight different bank groups. The first-half units are stored when the
// q.K^T of the previous tile has read chunks 0-3, the second-half units and the rope when it has read the rest.
// Lane r % 8 also walks the look-ahead chain of row 8w + r % 8: the selected index four tiles ahead, its
// block-table entry three tiles ahead, an L2 prefetch of the row two tiles ahead, the row itself (by all lanes)
// one tile ahead.
// kFmt: 0 = int8 latent, bf16 rope and fp32 scales in three arrays, 1 = packed 656-byte rows, 2 = bf16 latent and
// rope arrays (the non-quantised cache). With a bf16 cache nothing passes through registers: when a half of the
// buffer is free every lane issues its 16-byte `cp.async` copies from L2 (the rows were prefetched there two tiles
// ago) straight to the swizzled places the dequantised units would go, waits for them, fences and arrives.
template <int kFmt>
__device__ __forceinline__ void pair_role_kproducer(const SfaParams& p, const PairCtx c) {
  constexpr bool kPacked = kFmt == 1, kBf = kFmt == 2;
  PairCtl* ctl = c.ctl;
  const int ntiles = c.ntiles, bi = c.bi;
  const int lane = threadIdx.x & 31;
  const int ptid = threadIdx.x - kPairKWarp0 * 32;
  const int w = ptid >> 5;
  const int u = lane & 15, s2 = lane >> 4;
  const int my_row = 64 * static_cast<int>(c.crank) + 8 * w + (lane & 7);  // key of the tile this lane looks ahead for
  const int32_t* idx_ptr = c.idx_row + c.begin + my_row;
  const int n_mine = c.end - (c.begin + my_row);  // entry j * 128 of idx_ptr is valid iff j * 128 < n_mine
  constexpr int stride_n = kPacked ? 656 : (kBf ? 1024 : 512), stride_r = kPacked ? 656 : 128, stride_s = kPacked ? 656 : 16;
  // (the base pointers are read from the parameter block where they are used: they would otherwise occupy six
  // registers across the whole tile loop)
#define PAIR_KN reinterpret_cast<const uint8_t*>(p.kn)
#define PAIR_ROPE (kPacked ? PAIR_KN + 512 : reinterpret_cast<const uint8_t*>(p.kr))
#define PAIR_SCL (kPacked ? PAIR_KN + 640 : reinterpret_cast<const uint8_t*>(p.kn_scales))
  struct RowRegs {
    uint4 d[2][4];  // [row half][m]: unit 16 half + u of row 8w + 2m + s2
    uint4 r[2];     // rope unit lane % 8 of rows 8w + 4i + lane / 8
    float sc;       // scale lane % 4 of row 8w + lane / 4
  };
  auto load_idx = [&](int j) -> int { return (j < ntiles && j * kPT < n_mine) ? ldg_pinned_i32(idx_ptr + j * kPT) : -1; };
  // `phys`: this lane's look-ahead row of the tile (-1: padding or rejected -> zeros with scale 0)
  auto issue_loads = [&](RowRegs& r, int phys) {
    if (kBf) return;  // (copied from L2 when the buffer is free)
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int pm = __shfl_sync(0xffffffffu, phys, 2 * m + s2);
      r.d[0][m] = make_uint4(0, 0, 0, 0);
      r.d[1][m] = make_uint4(0, 0, 0, 0);
      if (pm >= 0) {
        const uint8_t* a = PAIR_KN + static_cast<int64_t>(pm) * stride_n + u * 16;
        r.d[0][m] = ldg_pinned_v4(a);
        r.d[1][m] = ldg_pinned_v4(a + 256);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int pr = __shfl_sync(0xffffffffu, phys, 4 * i + (lane >> 3));
      r.r[i] = make_uint4(0, 0, 0, 0);
      if (pr >= 0) r.r[i] = ldg_pinned_v4(PAIR_ROPE + static_cast<int64_t>(pr) * stride_r + (lane & 7) * 16);
    }
    const int ps = __shfl_sync(0xffffffffu, phys, lane >> 2);
    r.sc = 0.f;
    if (ps >= 0) asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(r.sc) : "l"(PAIR_SCL + static_cast<int64_t>(ps) * stride_s + (lane & 3) * 4));
  };
  auto prefetch_row = [&](int phys) {  // lanes r, r+8, r+16, r+24 share a row: one of its four latent lines each, two of them the rest
    if (phys < 0) return;
    if (kBf) {  // eight latent lines and the rope line of the row
      const uint8_t* a = PAIR_KN + static_cast<int64_t>(phys) * 1024;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a + (lane >> 3) * 128));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a + 512 + (lane >> 3) * 128));
      if (lane < 8) asm volatile("prefetch.global.L2 [%0];" ::"l"(PAIR_ROPE + static_cast<int64_t>(phys) * 128));
    } else if (kPacked) {
      const uint8_t* a = PAIR_KN + static_cast<int64_t>(phys) * 656;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a + (lane >> 3) * 128));
      if (lane < 16) asm volatile("prefetch.global.L2 [%0];" ::"l"(a + 512 + (lane >> 3) * 128));
    } else {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(PAIR_KN + static_cast<int64_t>(phys) * 512 + (lane >> 3) * 128));
      if (lane < 8) asm volatile("prefetch.global.L2 [%0];" ::"l"(PAIR_ROPE + static_cast<int64_t>(phys) * 128));
      else if (lane < 16) asm volatile("prefetch.global.L2 [%0];" ::"l"(PAIR_SCL + static_cast<int64_t>(phys) * 16));
    }
  };
  const uint32_t k_rows = c.base + kSmemK + (u >> 2) * kChunk + 8 * w * 128;  // row 8w of this lane's chunk of half 0
  const bool odd = ((u >> 2) & 1) != 0;
  bool ok = true;
  uint32_t nwait = 0;
  RowRegs ra;
  pdl_wait();          // the selected indices come from the kernel before this one, which may still be running
  if (ptid == 0) TLP(3, 21);
  int row_cur;         // this lane's row of tile j (bf16 cache: the copies are issued when the buffer is free)
  int row_n;           // this lane's row of tile j+1
  int idx_a, entry_a;  // tile j+2
  int idx_b;           // tile j+3
  {
    const int idx0 = load_idx(0), idx1 = load_idx(1);
    idx_a = load_idx(2);
    idx_b = load_idx(3);
    if (ptid == 0 && idx0 + idx1 + idx_a + idx_b != -12345) TLP(4, 21);
    const int e0 = tc_table_entry(p, bi, idx0);
    const int e1 = tc_table_entry(p, bi, idx1);
    entry_a = tc_table_entry(p, bi, idx_a);
    if (ptid == 0 && e0 + e1 + entry_a != -12345) TLP(5, 21);
    row_cur = pair_row(p, idx0, e0);
    issue_loads(ra, row_cur);
    if (kBf) prefetch_row(row_cur);
    row_n = pair_row(p, idx1, e1);
    prefetch_row(row_n);
    if (ptid == 0) TLP(6, 21);
  }
  if (!kBf && ptid == 0 && ra.d[0][0].x != 0x7fffffffu) TLP(7, 21);  // first rows arrived
  pair_setup_sync(ctl);
  for (int j = 0; j < ntiles && ok; ++j) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (j > 0) {  // the q.K^T MMAs of the previous tile that read this half of the chunks are complete
        ok = pair_group_wait<32, 2, 256, 1>(ctl, nwait, smem_u32(&ctl->kfree[half]), (j - 1) & 1, ptid < 32);
        if (!ok) break;
      }
      if (ptid == 0 && half == 0) TLP(0, j);
#pragma unroll
      for (int m = 0; m < 4; ++m) {  // row 8w + 2m + s2 (its swizzle term is 2m + s2); scale 2 half + u / 8 of that row
        const int x = 2 * m + s2;
        const uint32_t row_addr = k_rows + half * 4 * kChunk + x * 128;
        const uint32_t a = ((2 * (u & 3)) ^ x) << 4, b = ((2 * (u & 3) + 1) ^ x) << 4;
        if (kBf) {  // the unit's 16 values are 32 bytes of the bf16 row: two copies
          const int pm = __shfl_sync(0xffffffffu, row_cur, x);
          const uint8_t* src = PAIR_KN + (pm >= 0 ? static_cast<int64_t>(pm) * 1024 + half * 512 + u * 32 : 0);
          cp_async_16(row_addr + a, src, pm >= 0 ? 16u : 0u);
          cp_async_16(row_addr + b, src + (pm >= 0 ? 16 : 0), pm >= 0 ? 16u : 0u);
        } else {
          const float scale = __shfl_sync(0xffffffffu, ra.sc, 4 * x + 2 * half + (u >> 3));
          const uint4 v = ra.d[half][m];
          // first half of the unit (bytes 0-7) belongs at `a`, second half at `b`; odd chunks store the second first
          sts_v4u(row_addr + (odd ? b : a), pair_dequant8(odd ? v.z : v.x, odd ? v.w : v.y, scale));
          sts_v4u(row_addr + (odd ? a : b), pair_dequant8(odd ? v.x : v.z, odd ? v.y : v.w, scale));
        }
      }
      if (half == 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // rope of row 8w + 4i + lane / 8
          const int r8 = 4 * i + (lane >> 3);
          const uint32_t dst = c.base + kSmemK + 8 * kChunk + (8 * w + r8) * 128 + (((lane & 7) ^ r8) << 4);
          if (kBf) {
            const int pr = __shfl_sync(0xffffffffu, row_cur, r8);
            cp_async_16(dst, PAIR_ROPE + (pr >= 0 ? static_cast<int64_t>(pr) * 128 + (lane & 7) * 16 : 0), pr >= 0 ? 16u : 0u);
          } else {
            sts_v4u(dst, ra.r[i]);
          }
        }
      }
      if (kBf) asm volatile("cp.async.wait_all;" ::: "memory");
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->kfull[half]));
      if (ptid == 0 && half == 1) TLP(1, j);
    }
    if (!ok) break;
    if (j + 1 < ntiles) issue_loads(ra, row_n);  // rows of tile j+1 (in L2: prefetched a tile ago)
    row_cur = row_n;
    row_n = pair_row(p, idx_a, entry_a);         // tile j+2: into L2
    prefetch_row(row_n);
    idx_a = idx_b;
    entry_a = tc_table_entry(p, bi, idx_a);      // block-table entries of tile j+3
    idx_b = load_idx(j + 4);
  }
  if (!ok && lane == 0) {
    ctl->abort = 1;
    set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 52);
  }
}

// ================================ V producers ===================================================
// 256 threads; warp w owns rows 8w .. 8w+7 of EACH key half of the tile (keys 64 h + 8w ..). A gather instruction
// reads this CTA's half of the value columns (256 of the 512 latent bytes) of TWO rows: lane l takes unit l % 16
// of row 2m + l / 16, again whole 128-byte lines (the other CTA's K producers have fetched or are fetching the
// same lines: L2 hits). Unit u goes to V chunk u / 4 of the row's key half, store units 2 (u % 4) and 2 (u % 4) + 1,
// second half first in odd chunks as in the K producers. Key half 0 is stored when the P.V of the previous tile
// has read keys 0-63, key half 1 when it has read the rest. Lane r % 16 walks the look-ahead chain of row
// 64 (r / 8) + 8w + r % 8 (no L2 prefetch: the row's owner issues it).
template <int kFmt>
__device__ __forceinline__ void pair_role_vproducer(const SfaParams& p, const PairCtx c) {
  constexpr bool kPacked = kFmt == 1, kBf = kFmt == 2;
  PairCtl* ctl = c.ctl;
  const int ntiles = c.ntiles;
  const int lane = threadIdx.x & 31;
  const int vtid = threadIdx.x - kPairVWarp0 * 32;
  const int w = vtid >> 5;
  const int u = lane & 15, s2 = lane >> 4;
  const int my_row = 64 * ((lane >> 3) & 1) + 8 * w + (lane & 7);  // key of the tile this lane looks ahead for
  const int32_t* idx_ptr = c.idx_row + c.begin + my_row;
  const int n_mine = c.end - (c.begin + my_row);
  const int col0 = 256 * static_cast<int>(c.crank);  // first latent byte of this CTA's value columns
  constexpr int stride_n = kPacked ? 656 : (kBf ? 1024 : 512), stride_s = kPacked ? 656 : 16;
  struct RowRegs {
    uint4 d[2][4];  // [key half][m]: unit u of row 64 half + 8w + 2m + s2
    float sc;       // scale lane % 2 (of this CTA's two) of the row lane / 2 (chain order: half * 8 + r)
  };
  auto load_idx = [&](int j) -> int { return (j < ntiles && j * kPT < n_mine) ? ldg_pinned_i32(idx_ptr + j * kPT) : -1; };
  auto issue_loads = [&](RowRegs& r, int phys) {
    if (kBf) return;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int pm = __shfl_sync(0xffffffffu, phys, 8 * half + 2 * m + s2);
        r.d[half][m] = make_uint4(0, 0, 0, 0);
        if (pm >= 0) r.d[half][m] = ldg_pinned_v4(PAIR_KN + static_cast<int64_t>(pm) * stride_n + col0 + u * 16);
      }
    }
    const int ps = __shfl_sync(0xffffffffu, phys, lane >> 1);
    r.sc = 0.f;
    if (ps >= 0) asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(r.sc) : "l"(PAIR_SCL + static_cast<int64_t>(ps) * stride_s + (col0 >> 5) + (lane & 1) * 4));
  };
  // row 8w of chunk u / 4 in the V region of key half 0
  const uint32_t v_rows = c.base + kSmemV + (u >> 2) * kChunk + 8 * w * 128;
  const bool odd = ((u >> 2) & 1) != 0;
  bool ok = true;
  uint32_t nwait = 0;
  RowRegs ra;
  pdl_wait();
  int row_cur, row_n, idx_a, entry_a;  // this lane's row of tiles j and j+1; index and block-table entry of tile j+2
  {
    const int idx0 = load_idx(0), idx1 = load_idx(1);
    idx_a = load_idx(2);
    const int e0 = tc_table_entry(p, c.bi, idx0);
    const int e1 = tc_table_entry(p, c.bi, idx1);
    entry_a = tc_table_entry(p, c.bi, idx_a);
    row_cur = pair_row(p, idx0, e0);
    issue_loads(ra, row_cur);
    row_n = pair_row(p, idx1, e1);
  }
  pair_setup_sync(ctl);
  for (int j = 0; j < ntiles && ok; ++j) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (j > 0) {  // the P.V MMAs of the previous tile that read this key half are complete
        ok = pair_group_wait<32, 3, 256, 2>(ctl, nwait, smem_u32(&ctl->vfree[half]), (j - 1) & 1, vtid < 32);
        if (!ok) break;
      }
      if (vtid == 0 && half == 0) TLP(4, j);
#pragma unroll
      for (int m = 0; m < 4; ++m) {  // row 64 half + 8w + 2m + s2: swizzle term 2m + s2, scale held by lane 2 (8 half + 2m + s2) + u / 8
        const int x = 2 * m + s2;
        const uint32_t row_addr = v_rows + half * kVHalfBytes + x * 128;
        const uint32_t a = ((2 * (u & 3)) ^ x) << 4, b = ((2 * (u & 3) + 1) ^ x) << 4;
        if (kBf) {
          const int pm = __shfl_sync(0xffffffffu, row_cur, 8 * half + x);
          const uint8_t* src = PAIR_KN + (pm >= 0 ? static_cast<int64_t>(pm) * 1024 + 2 * col0 + u * 32 : 0);
          cp_async_16(row_addr + a, src, pm >= 0 ? 16u : 0u);
          cp_async_16(row_addr + b, src + (pm >= 0 ? 16 : 0), pm >= 0 ? 16u : 0u);
        } else {
          const float scale = __shfl_sync(0xffffffffu, ra.sc, 2 * (8 * half + x) + (u >> 3));
          const uint4 v = ra.d[half][m];
          sts_v4u(row_addr + (odd ? b : a), pair_dequant8(odd ? v.z : v.x, odd ? v.w : v.y, scale));
          sts_v4u(row_addr + (odd ? a : b), pair_dequant8(odd ? v.x : v.z, odd ? v.y : v.w, scale));
        }
      }
      if (kBf) asm volatile("cp.async.wait_all;" ::: "memory");
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->vfull[half]));
      if (vtid == 0 && half == 1) TLP(5, j);
    }
    if (!ok) break;
    if (j + 1 < ntiles) issue_loads(ra, row_n);
    row_cur = row_n;
    row_n = pair_row(p, idx_a, entry_a);
    idx_a = load_idx(j + 3);
    entry_a = tc_table_entry(p, c.bi, idx_a);  // (the index was requested this iteration: one trip to L2 here, after the
                                               // tile's stores, a whole tile before the next wait)
  }
  if (!ok && lane == 0) {
    ctl->abort = 1;
    set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 53);
  }
}

__global__ void __launch_bounds__(kPairThreads, 1)
sfa_pair_kernel(const __grid_constant__ SfaParams p) {
  extern __shared__ __align__(1024) uint8_t sfa_pair_smem[];
  const uint32_t base = smem_u32(sfa_pair_smem);
  if ((base & 1023u) != 0) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(base), 55);
    return;
  }
  if (threadIdx.x == 0) TLP(0, 20);  // kernel entry
  PairCtx c;
  c.base = base;
  c.ctl = reinterpret_cast<PairCtl*>(sfa_pair_smem + kSmemCtl);
  PairCtl* ctl = c.ctl;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  c.crank = pair_ctarank();
  const uint32_t crank = c.crank;
  const int bid = blockIdx.x >> 1;  // cluster index
  c.sp = bid % p.n_split;
  c.ti = bid / p.n_split;
  c.bi = c.ti / p.s1;
  const int si = c.ti % p.s1;

  int n = p.act_seq[c.bi] - p.s1 + 1 + si;
  n = max(0, min(n, p.topk_k));
  const int tiles_total = (n + kPT - 1) / kPT;
  const int tiles_per_split = (tiles_total + p.n_split - 1) / p.n_split;
  c.begin = min(n, c.sp * tiles_per_split * kPT);
  c.end = min(n, (c.sp + 1) * tiles_per_split * kPT);
  c.ntiles = (c.end - c.begin + kPT - 1) / kPT;
  c.idx_row = p.topk + static_cast<int64_t>(c.ti) * p.topk_k;
  c.q_row0 = static_cast<int64_t>(c.ti) * p.nq_total + p.head_begin;

  if (c.ntiles == 0) {  // same decision in both CTAs of the pair
    if (p.n_split == 1) {
      for (int e = tid; e < 64 * 64; e += kPairThreads) {
        const int r = e >> 6, cc = e & 63;
        *reinterpret_cast<uint4*>(p.out + (c.q_row0 + 64 * crank + r) * 512 + cc * 8) = make_uint4(0, 0, 0, 0);
      }
    } else {
      for (int r = tid; r < 64; r += kPairThreads) {
        float* ml = p.part_ml + ((static_cast<int64_t>(c.ti) * p.n_split + c.sp) * p.nq + 64 * crank + r) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }

  // ---- setup ------------------------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(smem_u32(&ctl->pvdone), 1);
    mbar_init(smem_u32(&ctl->pfull), kPairSoftmaxWarps);
    mbar_init(smem_u32(&ctl->ppeer), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->kfull[b]), kPairKWarps);
      mbar_init(smem_u32(&ctl->vfull[b]), kPairVWarps);
      mbar_init(smem_u32(&ctl->kfree[b]), 1);
      mbar_init(smem_u32(&ctl->vfree[b]), 1);
      mbar_init(smem_u32(&ctl->sfull[b]), 1);
      mbar_init(smem_u32(&ctl->sread[b]), kPairSoftmaxWarps);
      mbar_init(smem_u32(&ctl->kpeer[b]), 1);
      mbar_init(smem_u32(&ctl->vpeer[b]), 1);
      mbar_init(smem_u32(&ctl->speer[b]), 1);
    }
    ctl->abort = 0;
    fence_mbar_init();
    TLP(0, 21);
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kPairTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    if (tid == 0) TLP(1, 21);
  }
  // this CTA's 64 query rows into shared memory, nine swizzled chunks of 64 dims (A operand of q.K^T): 64 x 72
  // 16-byte units, twelve per thread of the twelve warps that are not producers, all loads in flight before the
  // first store. The producers go straight to their first rows.
  if (warp < kPairKWarp0) {
    constexpr int kLoaders = 32 * kPairKWarp0;
    const int64_t row0 = c.q_row0 + 64 * crank;
    uint4 w[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) {
      const int e = tid + i * kLoaders;
      const int r = e / 72, u = e % 72;
      w[i] = (u < 64) ? __ldg(reinterpret_cast<const uint4*>(p.q_nope + (row0 + r) * 512) + u)
                      : __ldg(reinterpret_cast<const uint4*>(p.q_rope + (row0 + r) * 64) + (u - 64));
    }
#pragma unroll
    for (int i = 0; i < 12; ++i) {
      const int e = tid + i * kLoaders;
      const int r = e / 72, u = e % 72;
      sts_v4u(base + kSmemQ + (u >> 3) * kChunk + r * 128 + (((u & 7) ^ (r & 7)) << 4), w[i]);
    }
    fence_proxy_async();
    if (tid == 0) TLP(2, 21);
  }
  static_assert(12 * 32 * kPairKWarp0 == 64 * 72, "Q units per loader thread");

#define PAIR_SETREG(x) asm volatile(x)
  if (warp < kPairSoftmaxWarp0) {
    PAIR_SETREG("setmaxnreg.dec.sync.aligned.u32 24;");
    if (warp == 0 && crank == 0) pair_role_issue_qk(p, c);
    else if (warp == 2 && crank == 0) pair_role_issue_pv(p, c);
    else if (warp == 1 && crank == 1) pair_role_relay(p, c);
    else pair_setup_sync(ctl);
  } else if (warp < kPairKWarp0) {
    PAIR_SETREG("setmaxnreg.inc.sync.aligned.u32 104;");
    pair_role_softmax(p, c);
  } else if (warp < kPairVWarp0) {
    PAIR_SETREG("setmaxnreg.inc.sync.aligned.u32 72;");  // (no change of the count; without it ptxas spills in this role)
    if (p.kn_bf16) pair_role_kproducer<2>(p, c);
    else if (p.packed) pair_role_kproducer<1>(p, c);
    else pair_role_kproducer<0>(p, c);
  } else {
    PAIR_SETREG("setmaxnreg.dec.sync.aligned.u32 64;");
    if (p.kn_bf16) pair_role_vproducer<2>(p, c);
    else if (p.packed) pair_role_vproducer<1>(p, c);
    else pair_role_vproducer<0>(p, c);
  }

  // ---- teardown: neither CTA may leave while the peer's MMAs can still read its shared memory --------
  // (nothing is kept in registers across the roles: what the teardown needs is read again)
  if (threadIdx.x == 32 * kPairSoftmaxWarp0) TLP(2, 20);  // first softmax warp done with its output
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TLP(3, 20);
  pair_cluster_sync();
  if ((threadIdx.x >> 5) == 0) {
    tc_fence_after();
    const uint32_t tmem = reinterpret_cast<const PairCtl*>(sfa_pair_smem + kSmemCtl)->tmem_base;
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPairTmemCols) : "memory");
  }
  if (threadIdx.x == 0) TLP(4, 20);  // exit
}

}  // namespace

#ifdef PTO_PAIR_TIMELINE
extern "C" int pto_debug_pair_timeline(long long* host, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_pair_tl, sizeof(long long) * n));
}
#endif

// split of a token's selected rows over clusters so that the grid fills the SM pairs once
int sfa_pair_split(int t, int num_sms) {
  const int pairs = num_sms / 2;
  if (t >= pairs) return 1;
  int s = pairs / (t > 0 ? t : 1);
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

cudaError_t launch_sfa_pair(const SfaParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(sfa_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kPairSmemBytes));
  if (e != cudaSuccess) return e;
  const int t = p.b * p.s1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(t) * p.n_split * 2, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 2 : 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, sfa_pair_kernel, p);
}

}  // namespace pto
