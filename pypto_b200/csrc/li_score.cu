// Lightning-indexer score stage.
//
//   d[h, pos]  = int32( q[h, :] . k[pos, :] )                    64 heads x 128 dims, int8
//   h16        = fp16( relu(d) * 2^-11 )
//   score[pos] = k_scale[pos] * sum_h fp32(ws_h) * fp32(h16),    ws_h = q_scale_h * weight_h
//
// (reference: examples/models/deepseek_v32_exp/lightning_indexer_quant_impl.py:138-194; golden
// deepseekv32_lightning_indexer_quant.py:205-241).
//
// Tensor-core kernel: persistent CTAs, each owning a contiguous range of the flattened
// (sequence, page) list. Per page: one TMA load of the 16 KB key page (128 keys x 128 B,
// 128-byte swizzle) -> four tcgen05.mma kind::i8 (M = 128 keys, N = 64*s1 heads, K = 32) into a
// TMEM accumulator -> epilogue warps read their key's row (one TMEM lane = one key), apply
// ReLU/2^-11/fp16 rounding and the weighted head sum, and write the fp32 score.
// Warp roles: warp 0 TMA producer, warps 1..2 MMA issuers (alternate pages; warp 1 owns TMEM),
// warps 3..18 epilogue (four groups of four warps that take pages round-robin; a single warp is
// latency-bound on the conversion chain, so thread-level parallelism has to come from many warps).
// A ring of 8 slots pairs one shared-memory stage with one TMEM accumulator. All waits are bounded.
//
// Non-quantised formulation (bf16 queries, keys and weights; reference LightningIndexerTopkImpl with isQuant =
// false, framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:113-147, golden
// indexer_topk_compute(is_quant=False), framework/tests/st/operator/src/test_deepseek_v3.2_exp/
// gen_lightning_indexer.py:189-279):   score[pos] = sum_h fp32(w_h) * relu( fp32( q[h, :] . k[pos, :] ) ).
// Same kernel and ring, mode kLiBf16: a key page is 32 KB (two 128-byte-swizzled halves of the 128 dims), the
// product is tcgen05.mma kind::f16 (bf16 x bf16 -> fp32, eight MMAs of K = 16 per page), four ring slots, at
// most two query tokens of a sequence per launch, and the epilogue is max/fma on the fp32 accumulators.
#include <cuda.h>

#include "common.cuh"

namespace pto {

namespace {

constexpr int kLiSlots = 8;            // ring of (smem stage, TMEM accumulator) pairs
constexpr int kPageKeys = 128;
constexpr int kPageBytes = kPageKeys * 128;
constexpr int kStageBytes = kPageBytes + 1024;  // key page + the page's 128 key scales (<= 512 B), 1024-aligned
constexpr int kHeads = 64;
constexpr int kQBytesPerToken = kHeads * 128;
constexpr int kLiMmaWarps = 2;         // warps 1..2: issuer for pages n with n % 2 == warp - 1
constexpr int kLiEpilogueGroups = 4;   // groups of four warps; a slot is always served by the same group (below)
constexpr int kLiEpilogueWarp0 = 1 + kLiMmaWarps;
constexpr int kLiThreads = 32 * (kLiEpilogueWarp0 + 4 * kLiEpilogueGroups);
constexpr int kMaxS1 = 4;
constexpr int kMaxSeqPerLaunch = 2048;
constexpr int kTmemCols = 512;
// score formulations the tensor-core kernel is instantiated for
enum { kLiQuant = 0, kLiChain = 1, kLiBf16 = 2 };
constexpr int kBf16PageBytes = kPageKeys * 256;  // one stage of the bf16 ring: the page's two 16 KB halves
constexpr int kBf16Slots = 4;                    // 4 x 32 KB fit where the int8 ring keeps 8 x 17 KB
constexpr int kBf16MaxS1 = 2;                    // 2 tokens x 64 heads x 256 B of queries fit the int8 Q area
static_assert(kBf16Slots * kBf16PageBytes <= kLiSlots * kStageBytes, "bf16 ring exceeds the stage area");
static_assert(kBf16MaxS1 * kHeads * 256 <= kMaxS1 * kQBytesPerToken, "bf16 queries exceed the Q area");

struct LiCtl {
  uint64_t full[kLiSlots];     // TMA bytes of the slot's page landed
  uint64_t accfull[kLiSlots];  // the slot's MMAs completed (tcgen05.commit)
  uint64_t empty[kLiSlots];    // the slot's epilogue warps finished reading TMEM and the scales
  uint64_t qfull;
  uint32_t tmem_base;
  int abort;
  int prefix[kMaxSeqPerLaunch + 1];
  __align__(16) float ws[kMaxS1 * kHeads];
};

constexpr size_t kLiHistSmemBytes = static_cast<size_t>(kLiHistMaxS1) * kLiHistBins * sizeof(unsigned int) + 16;  // 32 KB (+ alignment of its start)
constexpr size_t kLiSmemBytes = 1024 /*alignment slack*/ + kLiSlots * kStageBytes + kMaxS1 * kQBytesPerToken + sizeof(LiCtl);
static_assert(kLiSmemBytes + kLiHistSmemBytes <= 227 * 1024, "score kernel shared memory");

__device__ __forceinline__ float load_scale(const void* base, int dtype, int64_t i) {
  if (dtype == PTO_DT_F16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
  return reinterpret_cast<const float*>(base)[i];
}

// ws = q_scale * weight, the product taken in the tensors' own dtype (fp16 product is rounded to
// fp16 before widening, as the golden does).
__device__ __forceinline__ float load_ws(const void* qs, const void* w, int dtype, int64_t i) {
  if (dtype == PTO_DT_F16) {
    return __half2float(__hmul(reinterpret_cast<const __half*>(qs)[i], reinterpret_cast<const __half*>(w)[i]));
  }
  return __fmul_rn(reinterpret_cast<const float*>(qs)[i], reinterpret_cast<const float*>(w)[i]);
}

// relu(d) * 2^-11 rounded to fp16, for two dots at once; exact for |d| < 2^21:
// adding d to the bit pattern of 6144.0f (ulp 2^-11) and subtracting 6144 gives d * 2^-11.
__device__ __forceinline__ float2 relu_scale_round(int d0, int d1) {
  // the two subtractions as one packed fp32 instruction (each half is an ordinary IEEE subtraction)
  const float2 f = __fadd2_rn(make_float2(__int_as_float(0x45C00000 + d0), __int_as_float(0x45C00000 + d1)),
                              make_float2(-6144.0f, -6144.0f));
  uint32_t packed;  // round to fp16 and clamp negatives to zero in one conversion (f.x in the low half)
  asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(f.y), "f"(f.x));
  return __half22float2(*reinterpret_cast<const __half2*>(&packed));
}

// The older formulation for 32 heads of one key: table entries come in pairs, (q_scale_2p, q_scale_2p+1) and
// (weight_2p, weight_2p+1) as half2 bit patterns; d * 2^-11 is exact by the same magic number as above.
__device__ __forceinline__ float chain_sum_32(const uint32_t (&v)[32], const float* table, __half2 ks2) {
  const uint32_t* tb = reinterpret_cast<const uint32_t*>(table);
  float acc = 0.f;
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    const float f0 = __int_as_float(0x45C00000 + static_cast<int>(v[c])) - 6144.0f;
    const float f1 = __int_as_float(0x45C00000 + static_cast<int>(v[c + 1])) - 6144.0f;
    const uint32_t qs_bits = tb[c], w_bits = tb[c + 1];
    const __half2 qs2 = *reinterpret_cast<const __half2*>(&qs_bits);
    const __half2 w2 = *reinterpret_cast<const __half2*>(&w_bits);
    __half2 a = __hmul2(__hmul2(__floats2half2_rn(f0, f1), qs2), ks2);
    a = __hmax2(a, __float2half2_rn(0.0f));
    const float2 m = __half22float2(__hmul2(a, w2));
    acc = __fadd_rn(__fadd_rn(acc, m.x), m.y);
  }
  return acc;
}

__device__ __forceinline__ float weighted_sum_32(const uint32_t (&v)[32], const float* ws) {
  // four running sums as two packed pairs: one packed FMA per two heads (the same four chains of ordinary FMAs)
  float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    const float4 w = *reinterpret_cast<const float4*>(ws + c);
    const float2 x = relu_scale_round(static_cast<int>(v[c]), static_cast<int>(v[c + 1]));
    const float2 y = relu_scale_round(static_cast<int>(v[c + 2]), static_cast<int>(v[c + 3]));
    a01 = __ffma2_rn(make_float2(w.x, w.y), x, a01);
    a23 = __ffma2_rn(make_float2(w.z, w.w), y, a23);
  }
  return (a01.x + a01.y) + (a23.x + a23.y);
}

// Non-quantised formulation, 32 heads of one key: the accumulators are fp32 dots.
__device__ __forceinline__ float weighted_relu_sum_32(const uint32_t (&v)[32], const float* ws) {
  float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    const float4 w = *reinterpret_cast<const float4*>(ws + c);
    a01 = __ffma2_rn(make_float2(w.x, w.y),
                     make_float2(fmaxf(__uint_as_float(v[c]), 0.f), fmaxf(__uint_as_float(v[c + 1]), 0.f)), a01);
    a23 = __ffma2_rn(make_float2(w.z, w.w),
                     make_float2(fmaxf(__uint_as_float(v[c + 2]), 0.f), fmaxf(__uint_as_float(v[c + 3]), 0.f)), a23);
  }
  return (a01.x + a01.y) + (a23.x + a23.y);
}

template <int kMode>
__global__ void __launch_bounds__(kLiThreads, 1)
li_score_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q, LiParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t stage_base = base;
  const uint32_t q_base = base + kLiSlots * kStageBytes;
  LiCtl* ctl = reinterpret_cast<LiCtl*>(smem + kLiSlots * kStageBytes + kMaxS1 * kQBytesPerToken);
  // per-CTA histogram of the current sequence's scores (present only when the launch asked for it)
  unsigned int* hist_sm = reinterpret_cast<unsigned int*>(smem + kLiSlots * kStageBytes + kMaxS1 * kQBytesPerToken +
                                                          ((sizeof(LiCtl) + 15) & ~size_t(15)));
  const bool with_hist = p.hist != nullptr;

  constexpr bool kChain = kMode == kLiChain;
  constexpr bool kBf16 = kMode == kLiBf16;
  constexpr uint32_t kStage = kBf16 ? kBf16PageBytes : kStageBytes;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // this kernel is launched the ordinary way (everything before it has completed); the top-k kernel behind it
  // may be scheduled as soon as SMs drain and waits there for this grid to complete
  if (tid == 0) pdl_trigger();
  const int s1 = p.s1;
  const int n_cols = kHeads * s1;                                // accumulator columns per page
  const uint32_t n_slots = min(kBf16 ? kBf16Slots : kLiSlots, kTmemCols / n_cols);   // int8: 8, 4, 2, 2 for s1 = 1..4

  if (tid == 0) {
    for (int i = 0; i < kLiSlots; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->accfull[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 4);
    }
    mbar_init(smem_u32(&ctl->qfull), 1);
    ctl->abort = 0;
    fence_mbar_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_q);
  }
  if (with_hist) {
    for (int j = tid; j < s1 * kLiHistBins; j += kLiThreads) hist_sm[j] = 0u;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (warp == kLiEpilogueWarp0) {
    // exclusive prefix of pages per sequence
    int carry = 0;
    for (int b0 = 0; b0 < p.b; b0 += 32) {
      int v = 0;
      if (b0 + lane < p.b) {
        int s = p.act_seq[b0 + lane];
        s = max(s, 0);
        v = min((s + kPageKeys - 1) / kPageKeys, p.max_blocks);
      }
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (b0 + lane < p.b) ctl->prefix[b0 + lane] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) ctl->prefix[p.b] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  const int total = ctl->prefix[p.b];
  const int it0 = static_cast<int>(static_cast<long long>(total) * blockIdx.x / gridDim.x);
  const int it1 = static_cast<int>(static_cast<long long>(total) * (blockIdx.x + 1) / gridDim.x);

  const uint32_t idesc = kBf16 ? umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 0, 128, n_cols)
                               : umma_idesc(kCFmtS32, kABFmtS8, kABFmtS8, 0, 0, 128, n_cols);
  const uint32_t scale_bytes = kBf16 ? 0u : kPageKeys * (p.scale_dtype == PTO_DT_F16 ? 2u : 4u);
  const uint32_t q_half_bytes = static_cast<uint32_t>(n_cols) * 128u;  // bf16: one 64-dim half of the query tile

  int cur = it0;
  int bi = 0;
  if (cur < it1) {
    int lo = 0, hi = p.b;  // largest bi with prefix[bi] <= cur
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (ctl->prefix[mid] <= cur) lo = mid; else hi = mid;
    }
    bi = lo;
  }
  uint32_t n_item = 0;
  uint32_t seg = 0;
  int64_t prev_tok0 = 0;
  // adds this CTA's counts of the tokens tok_first .. tok_first + s1 - 1 into the global histogram and clears them
  auto flush_hist = [&](int64_t tok_first) {
    // (not the producer warp: it does not take part in the barrier that orders the flush before new counts)
    for (int j = tid - 32; j >= 0 && j < s1 * kLiHistBins; j += kLiThreads - 32) {
      const unsigned int c = hist_sm[j];
      if (c != 0u) {
        atomicAdd(p.hist + tok_first * kLiHistBins + j, c);
        hist_sm[j] = 0u;
      }
    }
  };

  while (cur < it1) {
    while (ctl->prefix[bi + 1] <= cur) ++bi;
    const int seg_end = min(it1, ctl->prefix[bi + 1]);
    const int page0 = cur - ctl->prefix[bi];
    const int npages = seg_end - cur;
    const int seq_len = p.act_seq[bi];
    // (grid y: further groups of s1 tokens of the same sequences, prefill chunks)
    const int64_t tok0 = static_cast<int64_t>(bi) * p.s1_total + p.tok_offset + static_cast<int>(blockIdx.y) * p.s1;

    // The producer warp takes no part in the two barriers of a segment: the ring's own barriers order its loads, so
    // the next segment's first pages are on their way while this one drains and the scale products are fetched.
    // previous segment fully drained: Q tile and ws may be overwritten
    if (warp != 0) asm volatile("bar.sync 1, %0;" ::"n"(kLiThreads - 32) : "memory");
    if (with_hist && seg > 0) flush_hist(prev_tok0);  // (the barrier below orders it before the next segment's counts)
    prev_tok0 = tok0;
    const bool aborted = ctl->abort != 0;
    if (!aborted) {
      if (warp == 1 && lane == 0) {
        if (kBf16) {
          mbar_arrive_expect_tx(smem_u32(&ctl->qfull), 2 * q_half_bytes);
          tma_load_2d(q_base, &tmap_q, 0, static_cast<int>(tok0) * kHeads, smem_u32(&ctl->qfull));
          tma_load_2d(q_base + q_half_bytes, &tmap_q, 128, static_cast<int>(tok0) * kHeads, smem_u32(&ctl->qfull));
        } else {
          mbar_arrive_expect_tx(smem_u32(&ctl->qfull), s1 * kQBytesPerToken);
          tma_load_2d(q_base, &tmap_q, 0, static_cast<int>(tok0) * kHeads, smem_u32(&ctl->qfull));
        }
      }
      const int e = tid - 32 * kLiEpilogueWarp0;
      if (e >= 0 && e < s1 * kHeads) {
        if (kBf16) {
          ctl->ws[e] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.weight)[tok0 * kHeads + e]);
        } else if (kChain) {
          // pairs of heads: even slot = the two query scales, odd slot = the two weights (fp16 bit patterns)
          const __half* src = reinterpret_cast<const __half*>((e & 1) ? p.weight : p.q_scale) + tok0 * kHeads + (e & ~1);
          const __half2 two = __halves2half2(src[0], src[1]);
          reinterpret_cast<uint32_t*>(ctl->ws)[e] = *reinterpret_cast<const uint32_t*>(&two);
        } else {
          ctl->ws[e] = load_ws(p.q_scale, p.weight, p.scale_dtype, tok0 * kHeads + e);
        }
      }
    }
    // the scale products are visible to the MMA and epilogue warps
    if (warp != 0) asm volatile("bar.sync 1, %0;" ::"n"(kLiThreads - 32) : "memory");

    if (!aborted) {
      if (warp == 0) {
        // ---------------- TMA producer ----------------
        const int32_t* bt = p.block_table + static_cast<int64_t>(bi) * p.max_blocks + page0;
        // key pages are read once: first to leave L2, so that the score rows written for the selection stay there
        const uint64_t stream_policy = l2_policy_evict_first();
        bool ok = true;
        for (int j0 = 0; j0 < npages && ok; j0 += 32) {
          const int mine = (j0 + lane < npages) ? bt[j0 + lane] : 0;
          const int cnt = min(32, npages - j0);
          for (int jj = 0; jj < cnt; ++jj) {
            int phys = __shfl_sync(0xffffffffu, mine, jj);
            if (lane == 0) {
              const uint32_t n = n_item + j0 + jj;
              const uint32_t slot = n % n_slots;
              const uint32_t ph = (n / n_slots) & 1u;
              if (!mbar_wait(smem_u32(&ctl->empty[slot]), ph ^ 1u)) {
                ok = false;
                ctl->abort = 1;
                set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(n), 1);
              } else {
                int scale_page = phys;
                if (phys < 0 || phys >= p.block_num) {
                  set_status(p.status, PTO_ST_BAD_PAGE, phys, 1);
                  phys = p.block_num;  // out of range of the tensor map: the page reads as zeros
                  scale_page = 0;      // any valid scales: the dots are zero
                }
                const uint32_t bar = smem_u32(&ctl->full[slot]);
                const uint32_t dst = stage_base + slot * kStage;
                if (kBf16) {
                  mbar_arrive_expect_tx(bar, kBf16PageBytes);
                  tma_load_2d_hint(dst, &tmap_k, 0, phys * kPageKeys, bar, stream_policy);
                  tma_load_2d_hint(dst + kPageBytes, &tmap_k, 128, phys * kPageKeys, bar, stream_policy);
                } else {
                  mbar_arrive_expect_tx(bar, kPageBytes + scale_bytes);
                  tma_load_2d_hint(dst, &tmap_k, 0, phys * kPageKeys, bar, stream_policy);
                  bulk_load_1d(dst + kPageBytes,
                               reinterpret_cast<const uint8_t*>(p.k_scale) + static_cast<int64_t>(scale_page) * scale_bytes,
                               scale_bytes, bar);
                }
              }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
          }
        }
      } else if (warp < kLiEpilogueWarp0) {
        // ---------------- MMA issuers: warp w takes pages n with n % 2 == w - 1 ----------------
        if (lane == 0) {
          bool ok = mbar_wait(smem_u32(&ctl->qfull), seg & 1u);
          if (!ok) set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(seg), 2);
          const uint64_t b_desc = umma_desc_kmajor_sw128(q_base);
          const uint64_t a_desc0 = umma_desc_kmajor_sw128(stage_base);
          for (int j = 0; j < npages && ok; ++j) {
            const uint32_t n = n_item + j;
            if (static_cast<int>(n % kLiMmaWarps) != warp - 1) continue;
            const uint32_t slot = n % n_slots;
            const uint32_t ph = (n / n_slots) & 1u;
            if (!mbar_wait(smem_u32(&ctl->full[slot]), ph)) {
              ok = false;
              set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(n), 3);
              break;
            }
            tc_fence_after();
            const uint64_t a_desc = a_desc0 + ((slot * kStage) >> 4);
            const uint32_t d = tmem_base + slot * n_cols;
            if (kBf16) {
              // K = 16 bf16 (32 bytes) per instruction: four steps inside each 64-dim half
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint64_t a = a_desc + ((k >> 2) * (kPageBytes >> 4)) + 2 * (k & 3);
                const uint64_t bq = b_desc + ((k >> 2) * (q_half_bytes >> 4)) + 2 * (k & 3);
                mma_f16_ss(d, a, bq, idesc, k > 0 ? 1u : 0u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) mma_i8_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
            }
            tc_commit(smem_u32(&ctl->accfull[slot]));
          }
          if (!ok) ctl->abort = 1;
        }
        __syncwarp();
      } else {
        // ---------------- epilogue ----------------
        const int grp = (warp - kLiEpilogueWarp0) >> 2;
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        const int row = quarter * 32 + lane;
        // A slot belongs to one group, so that the group sees every use of the slot and consecutive waits on its
        // barriers alternate in parity. (Taking pages n % 4 == grp is the same thing for 8 and 4 slots, but with
        // the two slots of s1 = 3, 4 a group met only every second use of a slot: two waits in a row on the same
        // parity, of which the second returned at once, before the page's products were there.) The ring has 8, 4
        // or 2 slots, so group g owns the pages n with n % min(slots, 4) == g and walks them directly: stepping
        // through every page and skipping three of four cost a tenth of the kernel's instructions.
        const int gstride = static_cast<int>(n_slots < 4u ? n_slots : 4u);
        const uint32_t slot_shift = 31u - static_cast<uint32_t>(__clz(static_cast<int>(n_slots)));
        for (int j = (grp - static_cast<int>(n_item % static_cast<uint32_t>(gstride)) + gstride) % gstride;
             grp < gstride && j < npages; j += gstride) {
          const uint32_t n = n_item + j;
          const uint32_t slot = n & (n_slots - 1u);
          const uint32_t ph = (n >> slot_shift) & 1u;
          if (!mbar_wait(smem_u32(&ctl->accfull[slot]), ph)) {
            ctl->abort = 1;
            set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(n), 4);
            break;
          }
          tc_fence_after();
          // the page's scales came in with the page; its `full` phase has completed (the MMA issuer
          // waited on it); observing it here orders this thread after the bulk copy
          if (!kBf16) mbar_wait(smem_u32(&ctl->full[slot]), ph);
          const uint8_t* sc_smem = smem + slot * kStage + kPageBytes;
          float ks = 1.f;
          if (!kBf16) {
            ks = (p.scale_dtype == PTO_DT_F16) ? __half2float(reinterpret_cast<const __half*>(sc_smem)[row])
                                               : reinterpret_cast<const float*>(sc_smem)[row];
          }
          const int pos = (page0 + j) * kPageKeys + row;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + slot * n_cols;
          float res[kMaxS1];
#pragma unroll
          for (int i = 0; i < kMaxS1; ++i) {
            if (i < s1) {
              uint32_t v0[32], v1[32];
              tmem_ld_32x32b_x32(taddr + i * kHeads, v0);
              tmem_ld_32x32b_x32(taddr + i * kHeads + 32, v1);
              tc_wait_ld();
              if (i == s1 - 1) {
                // TMEM and the scale row are read: hand the slot back before the arithmetic
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->empty[slot]));
              }
              if (kBf16) {
                res[i] = weighted_relu_sum_32(v0, ctl->ws + i * kHeads) + weighted_relu_sum_32(v1, ctl->ws + i * kHeads + 32);
              } else if (kChain) {
                const __half2 ks2 = __half2half2(reinterpret_cast<const __half*>(sc_smem)[row]);
                res[i] = __fadd_rn(chain_sum_32(v0, ctl->ws + i * kHeads, ks2), chain_sum_32(v1, ctl->ws + i * kHeads + 32, ks2));
              } else {
                res[i] = (weighted_sum_32(v0, ctl->ws + i * kHeads) + weighted_sum_32(v1, ctl->ws + i * kHeads + 32)) * ks;
              }
            }
          }
          if (pos < seq_len) {
#pragma unroll
            for (int i = 0; i < kMaxS1; ++i) {
              if (i < s1) p.scores[(tok0 + i) * p.row_stride + pos] = res[i];
            }
          }
          if (with_hist) {
            // counts for the top-k kernel: positions below the token's causal end
#pragma unroll
            for (int i = 0; i < kLiHistMaxS1; ++i) {
              if (i < s1) {
                const int eff = seq_len - (p.s1_total - 1 - (p.tok_offset + static_cast<int>(blockIdx.y) * p.s1 + i));
                if (pos < eff) atomicAdd(&hist_sm[i * kLiHistBins + (li_float_order(res[i]) >> kLiHistShift)], 1u);
              }
            }
          }
        }
      }
    }
    n_item += npages;
    cur = seg_end;
    ++seg;
  }

  // teardown
  tc_fence_before();
  __syncthreads();
  if (with_hist && seg > 0) flush_hist(prev_tok0);
  if (ctl->abort) {
    // give copies still in flight time to land before the CTA's shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// CUDA-core variant (dp4a), one thread per key position. Used to cross-check the tensor-core
// kernel bit for bit and to produce the `first_mm` debug tile.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
li_score_simt_kernel(LiParams p) {
  __shared__ __align__(16) int8_t qs[kMaxS1 * kQBytesPerToken];
  __shared__ float ws[kMaxS1 * kHeads];
  __shared__ __half qsc[kMaxS1 * kHeads], wgt[kMaxS1 * kHeads];  // older formulation: scales and weights apart
  const int bi = blockIdx.y;
  const int page = blockIdx.x;
  const int seq_len = p.act_seq[bi];
  if (page * kPageKeys >= seq_len) return;
  const int s1 = p.s1;
  const int tid = threadIdx.x;
  {
    const int64_t tok0 = static_cast<int64_t>(bi) * p.s1_total + p.tok_offset;
    const int4* src = reinterpret_cast<const int4*>(p.q + tok0 * kQBytesPerToken);
    int4* dst = reinterpret_cast<int4*>(qs);
    for (int i = tid; i < s1 * kQBytesPerToken / 16; i += blockDim.x) dst[i] = src[i];
    for (int e = tid; e < s1 * kHeads; e += blockDim.x) {
      if (p.fp16_chain) {
        qsc[e] = reinterpret_cast<const __half*>(p.q_scale)[tok0 * kHeads + e];
        wgt[e] = reinterpret_cast<const __half*>(p.weight)[tok0 * kHeads + e];
      } else {
        ws[e] = load_ws(p.q_scale, p.weight, p.scale_dtype, tok0 * kHeads + e);
      }
    }
  }
  __syncthreads();
  const int phys = p.block_table[static_cast<int64_t>(bi) * p.max_blocks + page];
  const int pos = page * kPageKeys + tid;
  if (phys < 0 || phys >= p.block_num) {
    // a rejected page scores 0 for every token, as in the tensor-core kernel (where the page reads as zeros):
    // the top-k stage never ranks what an earlier call left in the buffer
    if (tid == 0) set_status(p.status, PTO_ST_BAD_PAGE, phys, 5);
    if (pos < seq_len) {
      for (int i = 0; i < s1; ++i) {
        p.scores[(static_cast<int64_t>(bi) * p.s1_total + p.tok_offset + i) * p.row_stride + pos] = 0.f;
      }
    }
    return;
  }
  if (pos >= seq_len) return;
  int4 kreg[8];
  const int4* krow = reinterpret_cast<const int4*>(p.k_cache + (static_cast<int64_t>(phys) * kPageKeys + tid) * 128);
#pragma unroll
  for (int c = 0; c < 8; ++c) kreg[c] = krow[c];
  const float ks = load_scale(p.k_scale, p.scale_dtype, static_cast<int64_t>(phys) * kPageKeys + tid);
  for (int i = 0; i < s1; ++i) {
    float acc = 0.f;
    for (int h = 0; h < kHeads; ++h) {
      const int4* qrow = reinterpret_cast<const int4*>(qs + (i * kHeads + h) * 128);
      int d = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int4 qv = qrow[c];
        d = __dp4a(kreg[c].x, qv.x, d);
        d = __dp4a(kreg[c].y, qv.y, d);
        d = __dp4a(kreg[c].z, qv.z, d);
        d = __dp4a(kreg[c].w, qv.w, d);
      }
      if (p.fp16_chain) {
        const __half ksh = reinterpret_cast<const __half*>(p.k_scale)[static_cast<int64_t>(phys) * kPageKeys + tid];
        __half a = __hmul(__hmul(__float2half_rn(static_cast<float>(d) * (1.0f / 2048.0f)), qsc[i * kHeads + h]), ksh);
        a = __hmax(a, __float2half_rn(0.0f));
        acc = __fadd_rn(acc, __half2float(__hmul(a, wgt[i * kHeads + h])));
        continue;
      }
      const float f = fmaxf(static_cast<float>(d), 0.f) * (1.0f / 2048.0f);
      const __half hh = __float2half_rn(f);
      if (p.first_mm != nullptr) {
        reinterpret_cast<__half*>(p.first_mm)[((static_cast<int64_t>(bi) * p.s1_total + p.tok_offset + i) * kHeads + h) * p.row_stride + pos] = hh;
      }
      acc = fmaf(ws[i * kHeads + h], __half2float(hh), acc);
    }
    p.scores[(static_cast<int64_t>(bi) * p.s1_total + p.tok_offset + i) * p.row_stride + pos] = p.fp16_chain ? acc : acc * ks;
  }
}

}  // namespace

cudaError_t launch_li_score_tc(const LiParams& p, const void* tmap_k, const void* tmap_q, int num_sms,
                               cudaStream_t stream) {
  auto kernel = p.bf16 ? li_score_tc_kernel<kLiBf16>
                       : (p.fp16_chain ? li_score_tc_kernel<kLiChain> : li_score_tc_kernel<kLiQuant>);
  if (p.hist != nullptr && p.s1 > kLiHistMaxS1) return cudaErrorInvalidValue;
  const size_t smem_bytes = kLiSmemBytes + (p.hist != nullptr ? kLiHistSmemBytes : 0);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kLiSmemBytes + kLiHistSmemBytes));
  if (e != cudaSuccess) return e;
  // a launch that takes several token groups gives each group its share of the SMs: every CTA then walks more
  // pages and the fixed cost of a launch (about 8 us) is paid once for all of them
  const int groups = p.groups < 1 ? 1 : p.groups;
  long long max_items = static_cast<long long>(p.b) * p.max_blocks;
  const int per_group = num_sms / groups < 1 ? 1 : num_sms / groups;
  int gx = static_cast<int>(max_items < per_group ? max_items : per_group);
  if (gx < 1) gx = 1;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(groups), 1);
  count_launch();
  kernel<<<grid, kLiThreads, smem_bytes, stream>>>(*reinterpret_cast<const CUtensorMap*>(tmap_k),
                                                                 *reinterpret_cast<const CUtensorMap*>(tmap_q), p);
  return cudaGetLastError();
}

cudaError_t launch_li_score_simt(const LiParams& p, cudaStream_t stream) {
  dim3 grid(p.max_blocks, p.b);
  count_launch();
  li_score_simt_kernel<<<grid, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

int li_max_s1() { return kMaxS1; }
int li_max_s1_bf16() { return kBf16MaxS1; }
int li_max_sequences() { return kMaxSeqPerLaunch; }

}  // namespace pto
