// Sparse MLA attention for 128 heads: a cluster of two CTAs per (token, split) that splits the
// 576-wide q.K^T contraction between the CTAs.
//
// Arithmetic as in sfa_decode.cu (reference:
// examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:45-207; golden
// deepseekv32_sparse_flash_attention_quant.py:169-254).
//
// CTA c of the pair owns latent dims [256c, 256c+256) and rope dims [32c, 32c+32): it holds that
// half of Q (in tensor memory, as the A operand of q.K^T), gathers and
// dequantises only that half of every selected row, computes the partial scores S_c = Q_c . K_c^T
// for all 128 heads (tcgen05, M = 128, N = 64 rows per tile), and owns the 256-wide half of the
// output (P . V_c, V_c = the latent half it already has in shared memory). The two partial score
// tiles are exchanged through distributed shared memory by four exchange warps, off the softmax
// chain: as soon as the q.K^T of a tile completes, each exchange warp copies its 32 rows of the
// partial scores from TMEM into its 8 KB send slice and bulk-copies the slice into the peer CTA's
// receive slice (completing on the peer's mbarrier). A softmax thread adds its own partials (send
// slice) and the peer's (receive slice): fp32 addition commutes, so both CTAs get bit-identical
// scores, maxima and P. Nothing is computed twice except the softmax itself.
//   warp 0          issues every MMA (event loop over "K tile filled" and "P written")
//   warps 1..3, 20  exchange: one TMEM lane quarter each (quarter = warp & 3)
//   warps 4..11     softmax, two threads per head row (32 of the tile's 64 columns each); P goes to TMEM
//   warps 12..19    producers: 16-byte gathers, int8 -> bf16 in registers, swizzled stores (3 K buffers)
// Roles are uniform within each group of four warps so that registers can be moved between them
// (setmaxnreg): the kernel starts with 80 per thread (six warps share one scheduler's file), warps
// 0..3 drop to 64 and the softmax warps rise to 88. Nothing may spill: beside ~210 KB of shared
// memory the L1 is too small to hold the stack, and a spilled register costs a trip to L2.
// Tensor memory: O 256 columns | Q latent 128 | Q rope 16 | partial scores 64 | P 32 (bf16 pairs).
// Every MMA takes its A operand (Q or P) from tensor memory and its B operand (the K tile) from
// shared memory.
// All waits are bounded; local waits that order peer writes use cluster-scope acquire.
#include "common.cuh"
#include "sfa_common.cuh"

namespace pto {

namespace {

// Developer aid: -DPTO_SFA_TIMELINE records clock64() at up to 40 points of tiles 8..23 of CTA 0.
#ifdef PTO_SFA_TIMELINE
__device__ long long g_sfa_timeline[16 * 40];
#define TL(slot, j) do { if (blockIdx.x == 0 && (j) >= 8 && (j) < 24) g_sfa_timeline[((j) - 8) * 40 + (slot)] = clock64(); } while (0)
#define TLM(k) do { if (blockIdx.x == 0) g_sfa_timeline[(k) * 40 + 39] = clock64(); } while (0)
#else
#define TLM(k) do { } while (0)
#define TL(slot, j) do { } while (0)
#endif

constexpr int kCT = 64;                          // selected rows per tile
constexpr int kKNopeChunk = kCT * 128;           // 64 rows x 64 dims bf16, 128-byte rows
constexpr int kKRope = kCT * 64;
constexpr int kKBuf = 4 * kKNopeChunk + kKRope;  // 36,864
constexpr int kNK = 3;                           // K buffers
constexpr int kXSlice = 32 * 256;                // 32 head rows x 64 fp32 partial scores
constexpr int kXBuf = 4 * kXSlice;               // send area; two receive areas of the same size follow it
constexpr int kClXWarps = 4;
constexpr int kClSoftmaxWarp0 = 4;
constexpr int kClSoftmaxWarps = 8;   // two warps per TMEM lane quarter: columns 0-31 and 32-63 of the tile
constexpr int kClProducerWarp0 = kClSoftmaxWarp0 + kClSoftmaxWarps;
constexpr int kClProducerWarps = 8;
constexpr int kClLastXWarp = kClProducerWarp0 + kClProducerWarps;  // 20: lane quarter 0
constexpr int kClThreads = 32 * (kClLastXWarp + 1);                // 672
constexpr uint32_t kClTmemCols = 512;
constexpr uint32_t kClColO = 0;
constexpr uint32_t kClColQ = 256;   // 128 columns: this CTA's 256 latent dims of Q as bf16 pairs
constexpr uint32_t kClColQR = 384;  // 16 columns: its 32 rope dims
constexpr uint32_t kClColS = 400;   // 64 columns: partial scores of the tile in flight
constexpr uint32_t kClColP = 464;   // 32 columns: P of the tile in flight as bf16 pairs
constexpr float kClRescale = 8.0f;

struct ClCtl {
  uint64_t k_full[kNK];  // producers filled K buffer                          (count: producer warps)
  uint64_t k_free[kNK];  // the P.V that read K buffer is complete             (tcgen05.commit)
  uint64_t s_full;       // partial scores complete                             (tcgen05.commit)
  uint64_t s_free;       // exchange warps have copied the scores out           (count 4 warps)
  uint64_t pv_done;      // P.V of a tile complete: P may be overwritten, O is at rest (tcgen05.commit)
  uint64_t p_full;       // P written                                           (count 8 warps)
  uint64_t xs_full[4];      // own partials of lane quarter q staged in the send slice   (1 arrival)
  uint64_t xs_free[4];      // both softmax warps of the quarter have read the send slice (2 arrivals)
  uint64_t xr_full[4][2];   // the peer's partials landed in receive slice [q][tile parity] (1 arming arrival + tx bytes)
  uint64_t xr_free[4][2];   // the PEER's two softmax warps have read what I copied into its slice [q][parity] (2 remote arrivals)
  uint64_t pair_bar[4];  // the two softmax warps of a lane quarter meet here (count 2), bounded like every wait
  uint32_t tmem_base;
  int abort;
  __align__(16) unsigned char k_valid[kNK][kCT];
  float pair_mt[2][2][128];  // [tile parity][column half][row]: tile max of each half; the halves' sums at the end
};

constexpr size_t kClSmemBytes = kNK * kKBuf + 3 * kXBuf + sizeof(ClCtl);
static_assert(kClSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA may use");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_peer(uint32_t local_smem_addr, uint32_t peer_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(peer_rank));
  return r;
}
// bulk copy of this CTA's shared memory into the peer's, completing (tx bytes) on the peer's mbarrier
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, uint32_t src_local, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src_local), "r"(bytes), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// no ordering of this thread's earlier writes is needed (the peer only waits for reads to have happened)
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Waits on barriers that a peer CTA completes (bulk-copy bytes, remote arrivals): polled with the
// plain CTA-scope test like any other barrier - a cluster-scope acquire in the polling loop slows the
// whole SM's memory pipeline - and followed by one cluster-scope acquire fence once the phase is over.
__device__ __forceinline__ bool mbar_wait_peer(uint32_t bar, uint32_t parity) {  // one thread
  const bool ok = mbar_wait_spin(bar, parity);
  asm volatile("fence.acquire.sync_restrict::shared::cluster.cluster;" ::: "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait_peer_warp(uint32_t bar, uint32_t parity) {  // a converged warp
  return __all_sync(0xffffffffu, mbar_wait_peer(bar, parity));
}

// Values every role needs, set up once per CTA.
struct ClCtx {
  uint8_t* k_ptr;
  uint8_t* x_ptr;
  ClCtl* ctl;
  const int32_t* idx_row;  // this token's selected positions
  int64_t q_row0;          // first query/output row of the token
  uint32_t k_base, x_base, tmem_base, crank, peer;
  int ntiles, begin, end, ti, sp, bi;
};

// One 128-byte line of a selected row per thread of the row's four (q = 0..3): two lines of this CTA's
// latent half, the rope half, the scales. With a bf16 latent cache the half is four lines, one per thread,
// and thread 0 also takes the rope half (there are no scales).
template <bool kBf16>
__device__ __forceinline__ void cl_prefetch_row(const SfaParams& p, long long phys, uint32_t crank, int q) {
  if (phys < 0) return;
  const uint8_t* kn_bytes = reinterpret_cast<const uint8_t*>(p.kn);
  if (kBf16) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kn_bytes + phys * 1024 + crank * 512 + q * 128));
    if (q == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(p.kr) + phys * 128 + crank * 64));
    return;
  }
  const uint8_t* a;
  if (q < 2) {
    a = (p.packed ? kn_bytes + phys * 656 : kn_bytes + phys * 512) + crank * 256 + q * 128;
  } else if (q == 2) {
    a = (p.packed ? kn_bytes + phys * 656 + 512 : reinterpret_cast<const uint8_t*>(p.kr) + phys * 128) + crank * 64;
  } else {
    a = (p.packed ? kn_bytes + phys * 656 + 640 : reinterpret_cast<const uint8_t*>(p.kn_scales) + phys * 16) + crank * 8;
  }
  asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

// ================================ MMA issuer ====================================================
// One thread, an event loop: P.V of the oldest tile whose P is written, else q.K^T of the next tile
// whose K buffer is filled (and whose score columns the exchange warps have released).
__device__ __forceinline__ void cl_role_mma(const SfaParams& p, const ClCtx c) {
  ClCtl* ctl = c.ctl;
  const uint32_t tmem_base = c.tmem_base, k_base = c.k_base;
  const int ntiles = c.ntiles;
  const int lane = threadIdx.x & 31;
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 0, 128, kCT);
      const uint32_t idesc_pv = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 1, 128, 256);
      auto issue_qk = [&](int j) {
        const uint32_t d = tmem_base + kClColS;
        const uint32_t kb = k_base + (j % kNK) * kKBuf;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const uint64_t b_desc = umma_desc_kmajor_sw128(kb + c * kKNopeChunk);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_f16_ts(d, tmem_base + kClColQ + c * 32 + k * 8, b_desc + 2 * k, idesc_qk, (c | k) != 0 ? 1u : 0u);
          }
        }
        const uint64_t b_desc = desc_kmajor_sw64(kb + 4 * kKNopeChunk);
#pragma unroll
        for (int k = 0; k < 2; ++k) mma_f16_ts(d, tmem_base + kClColQR + k * 8, b_desc + 2 * k, idesc_qk, 1u);
        tc_commit(smem_u32(&ctl->s_full));
      };
      auto issue_pv = [&](int j) {
        const uint64_t b_desc = desc_mnmajor_sw128(k_base + (j % kNK) * kKBuf, kKNopeChunk, 1024);
#pragma unroll
        for (int k = 0; k < kCT / 16; ++k) {
          mma_f16_ts(tmem_base + kClColO, tmem_base + kClColP + k * 8, b_desc + k * ((16 * 128) >> 4), idesc_pv,
                     (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&ctl->k_free[j % kNK]));
        tc_commit(smem_u32(&ctl->pv_done));
      };
      bool ok = true;
      int qk_i = 0, pv_i = 0;
      long long t_last = clock64();
      while (pv_i < ntiles) {
        bool progressed = false;
        if (pv_i < qk_i && mbar_test_wait(smem_u32(&ctl->p_full), pv_i & 1)) {
          TL(2, pv_i);
          tc_fence_after();
          issue_pv(pv_i);
          TL(3, pv_i);
          ++pv_i;
          progressed = true;
        }
        if (qk_i < ntiles && mbar_test_wait(smem_u32(&ctl->k_full[qk_i % kNK]), (qk_i / kNK) & 1) &&
            (qk_i == 0 || mbar_test_wait(smem_u32(&ctl->s_free), (qk_i - 1) & 1))) {
          TL(0, qk_i);
          tc_fence_after();
          issue_qk(qk_i);
          TL(1, qk_i);
          ++qk_i;
          progressed = true;
        }
        if (progressed) {
          t_last = clock64();
        } else {
          if (clock64() - t_last > kWaitBudgetCycles) {
            ok = false;
            break;
          }
        }
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 40);
      }
    }
  __syncwarp();
}

// ================================ exchange ======================================================
// Warp of lane quarter q: partial scores of each tile, TMEM -> 8 KB send slice -> the peer CTA's
// receive slice. A slice row is 16 units of 16 bytes, unit u stored at u ^ (lane & 7).
__device__ __forceinline__ void cl_role_exchange(const SfaParams& p, const ClCtx c) {
  ClCtl* ctl = c.ctl;
  const uint32_t tmem_base = c.tmem_base, x_base = c.x_base, peer = c.peer;
  uint8_t* x_ptr = c.x_ptr;
  const int ntiles = c.ntiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quarter = warp & 3;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint8_t* send_row = x_ptr + quarter * kXSlice + lane * 256;
    const uint32_t send_slice = x_base + quarter * kXSlice;
    const int xsw = lane & 7;
    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
      // the scores are complete and this CTA's softmax warps have read the previous tile's send slice
      ok = mbar_wait_warp(smem_u32(&ctl->s_full), t & 1);
      if (ok && t >= 1) ok = mbar_wait_warp(smem_u32(&ctl->xs_free[quarter]), (t - 1) & 1);
      if (!ok) break;
      if (lane == 0) bulk_wait_read_all();  // the previous copy has finished reading the send slice
      __syncwarp();
      if (warp == 1) TL(7, t);
      tc_fence_after();
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + kClColS + 32 * g, v);
        tc_wait_ld();
        if (g == 1) {  // all 64 columns are in registers: the next q.K^T may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->s_free));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          *reinterpret_cast<uint4*>(send_row + (((8 * g + u) ^ xsw) << 4)) = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&ctl->xs_full[quarter]));    // own partials staged
        if (warp == 1) TL(8, t);
        // the peer has read what went into this receive slice two tiles ago
        if (t >= 2) ok = mbar_wait_peer(smem_u32(&ctl->xr_free[quarter][t & 1]), ((t - 2) >> 1) & 1);
        if (ok) {
          bulk_copy_to_peer(map_to_peer(x_base + (1 + (t & 1)) * kXBuf + quarter * kXSlice, peer), send_slice, kXSlice,
                            map_to_peer(smem_u32(&ctl->xr_full[quarter][t & 1]), peer));
          bulk_commit();
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 1) TL(9, t);
    }
    if (lane == 0) bulk_wait_read_all();
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 44);
    }
}

// ================================ softmax =======================================================
// Thread (row, half): head row = TMEM lane, columns [32*half, 32*half+32) of the 64-row tile.
__device__ __forceinline__ void cl_role_softmax(const SfaParams& p, const ClCtx c) {
  ClCtl* ctl = c.ctl;
  const uint32_t tmem_base = c.tmem_base, peer = c.peer, crank = c.crank;
  uint8_t* x_ptr = c.x_ptr;
  const int ntiles = c.ntiles, ti = c.ti, sp = c.sp;
  const int64_t q_row0 = c.q_row0;
  const int tid = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = (warp - kClSoftmaxWarp0) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    // exchange slices of the lane quarter: own partials (send area) and the peer's (receive area);
    // a row is 16 units of 16 bytes, unit u stored at u ^ (lane & 7); this half reads units 8*half..+7
    const uint8_t* send_row = x_ptr + quarter * kXSlice + lane * 256;
    const uint8_t* recv_row0 = x_ptr + kXBuf + quarter * kXSlice + lane * 256;  // + kXBuf for odd tiles
    const int xsw = lane & 7;
    float m_seen = -INFINITY;  // the row's reference max (identical in both halves)
    float l_run = 0.f;         // this half's share of the row sum
    bool ok = true;
    uint32_t pair_phase = 0;
    auto pair_sync = [&]() -> bool {  // orders the pair_mt writes of both warps before the reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->pair_bar[quarter]));
      const bool w = mbar_wait_warp(smem_u32(&ctl->pair_bar[quarter]), pair_phase & 1u);
      ++pair_phase;
      return w;
    };
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      const int kb = j % kNK;
      // ---- scores = own partials (staged by an exchange warp) + the peer CTA's ----------------------
      ok = mbar_wait_warp(smem_u32(&ctl->xs_full[quarter]), j & 1) &&
           mbar_wait_peer_warp(smem_u32(&ctl->xr_full[quarter][b]), (j >> 1) & 1);
      if (!ok) break;
      const uint8_t* recv_row = recv_row0 + b * kXBuf;
      if (tid == 32 * kClSoftmaxWarp0) TL(10, j);
      float s[32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float4 a = *reinterpret_cast<const float4*>(send_row + (((8 * half + u) ^ xsw) << 4));
        s[4 * u] = a.x;
        s[4 * u + 1] = a.y;
        s[4 * u + 2] = a.z;
        s[4 * u + 3] = a.w;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float4 o = *reinterpret_cast<const float4*>(recv_row + (((8 * half + u) ^ xsw) << 4));
        s[4 * u] += o.x;
        s[4 * u + 1] += o.y;
        s[4 * u + 2] += o.z;
        s[4 * u + 3] += o.w;
      }
      __syncwarp();
      if (lane == 31) mbar_arrive(smem_u32(&ctl->xs_free[quarter]));  // the send slice may be refilled
      if (tid == 32 * kClSoftmaxWarp0) TL(11, j);
      // ---- scale, mask, max of this half ------------------------------------------------------------
      // (k_valid was written before the producers' arrival on k_full, which the MMA thread observed before
      // issuing the q.K^T whose completion led, through the exchange warp, to the xs_full phase just
      // acquired: release/acquire chains are cumulative, no further wait is needed to read it)
      // all rows valid (always, except in a token's last tile or after a rejected index): max on
      // the raw sums, scale folded into the exponent's FMA
      const uint4 va = *reinterpret_cast<const uint4*>(&ctl->k_valid[kb][32 * half]);
      const uint4 vb = *reinterpret_cast<const uint4*>(&ctl->k_valid[kb][32 * half + 16]);
      if ((va.x & va.y & va.z & va.w & vb.x & vb.y & vb.z & vb.w) != 0x01010101u) {
        const uint32_t vw[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (((vw[c >> 2] >> ((c & 3) * 8)) & 0xffu) == 0) s[c] = -INFINITY;
        }
      }
      float mt4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; ++c) mt4[c & 3] = fmaxf(mt4[c & 3], s[c]);
      const float mt_half = fmaxf(fmaxf(mt4[0], mt4[1]), fmaxf(mt4[2], mt4[3])) * p.scale_log2;  // scale > 0
      ctl->pair_mt[b][half][row] = mt_half;
      // ---- exponentials against a speculative reference ---------------------------------------------
      // The other half's maximum is not known yet; rescales are rare, so exp2 is taken now against the
      // row's current reference (never more than 2^8 below this half's maximum) and corrected by one
      // factor once the reference is final.
      float m_spec = (m_seen == -INFINITY || mt_half > m_seen + kClRescale) ? mt_half : m_seen;
      if (m_spec == -INFINITY) m_spec = 0.f;
      const float neg_spec = -m_spec;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        s[c] = ex2f(fmaf(s[c], p.scale_log2, neg_spec));
        ls4[c & 3] += s[c];
      }
      const float lsum = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      if (tid == 32 * kClSoftmaxWarp0) TL(12, j);
      // ---- join: the other half's maximum -------------------------------------------------------------
      ok = pair_sync();
      if (!ok) break;
      if (tid == 32 * kClSoftmaxWarp0) TL(13, j);
      const float mt = fmaxf(mt_half, ctl->pair_mt[b][half ^ 1][row]);
      const float m_new = fmaxf(m_seen, mt);
      const bool need = (m_new > m_seen + kClRescale) || (m_seen == -INFINITY && m_new > -INFINITY);
      float alpha = 1.f;
      if (need) {
        alpha = (m_seen == -INFINITY) ? 0.f : ex2f(m_seen - m_new);
        m_seen = m_new;
      }
      const float m_ref = (m_seen == -INFINITY) ? 0.f : m_seen;
      const float factor = ex2f(m_spec - m_ref);
      l_run = l_run * alpha + lsum * factor;
      // ---- the previous tile's P.V is complete: P may be overwritten, O is at rest ---------------------
      if (j > 0) {
        ok = mbar_wait_warp(smem_u32(&ctl->pv_done), (j - 1) & 1);
        if (!ok) break;
        tc_fence_after();
      }
      if (tid == 32 * kClSoftmaxWarp0) TL(14, j);
      if (j > 0 && __any_sync(0xffffffffu, need)) {  // rare: rescale the output accumulated so far
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {  // this half's 128 of the 256 output columns
          uint32_t o[16];
          tmem_ld_32x32b_x16(lane_addr + kClColO + half * 128 + ch * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st_32x32b_x16(lane_addr + kClColO + half * 128 + ch * 16, o);
        }
      }
      // ---- P row into tensor memory (A operand of P.V): column c = keys 2c, 2c+1; this half owns 16 columns
      {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) pk[c] = pack_bf16x2(s[2 * c] * factor, s[2 * c + 1] * factor);
        tmem_st_32x32b_x16(lane_addr + kClColP + 16 * half, pk);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
      if (tid == 32 * kClSoftmaxWarp0) TL(15, j);
      if (lane == 31) {
        // off the chain: arm this receive slice for the tile after next, then tell the peer that what it
        // copied into the slice has been read (it needs to know only two tiles from now)
        if (half == 0) mbar_arrive_expect_tx(smem_u32(&ctl->xr_full[quarter][b]), kXSlice);
        mbar_arrive_remote_relaxed(map_to_peer(smem_u32(&ctl->xr_free[quarter][b]), peer));
      }
    }
    // ---- output: row sum = both halves' shares; each half stores 128 of the CTA's 256 columns ---------
    if (tid == 32 * kClSoftmaxWarp0) TLM(4);
    if (ok) {
      ok = mbar_wait_warp(smem_u32(&ctl->pv_done), (ntiles - 1) & 1);
    }
    if (tid == 32 * kClSoftmaxWarp0) TLM(10);
    float l_last = 0.f;
    if (ok) {
      ctl->pair_mt[ntiles & 1][half][row] = l_run;
      ok = pair_sync();
      l_last = l_run + ctl->pair_mt[ntiles & 1][half ^ 1][row];
    }
    if (tid == 32 * kClSoftmaxWarp0) TLM(11);
    // The rows go out through shared memory (the K buffers are idle now): a thread owns a row, so direct
    // stores would touch 32 rows per instruction; staged, every store instruction writes 512 contiguous
    // bytes of one row. Staging row = 32 units of 16 bytes, unit u stored at u ^ (row & 31).
    // All eight softmax warps reach the barriers below whether or not their waits succeeded.
    const uint32_t stage = c.k_base;
    const int ws = warp - kClSoftmaxWarp0;
    if (ok) tc_fence_after();
    if (p.n_split == 1) {
      if (ok) {
        const float inv = l_last > 0.f ? 1.f / l_last : 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kClColO + half * 128 + ch * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int cc = 0; cc < 32; cc += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[cc]) * inv, __uint_as_float(o[cc + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[cc + 2]) * inv, __uint_as_float(o[cc + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[cc + 4]) * inv, __uint_as_float(o[cc + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[cc + 6]) * inv, __uint_as_float(o[cc + 7]) * inv);
            const int unit = 16 * half + ch * 4 + (cc >> 3);
            sts_v4u(stage + row * 512 + ((unit ^ (row & 31)) << 4), w);
          }
        }
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (ok) {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int r = ws * 16 + rr;
          const uint4 w = lds_v4u(stage + r * 512 + ((lane ^ (r & 31)) << 4));
          *reinterpret_cast<uint4*>(p.out + (q_row0 + r) * 512 + crank * 256 + lane * 8) = w;
        }
      }
    } else {
      const int64_t prow0 = (static_cast<int64_t>(ti) * p.n_split + sp) * p.nq;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {  // fp32 partials: one column half (128 floats = 512 bytes per row) per pass
        if (ok && half == h) {
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_addr + kClColO + half * 128 + ch * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int cc = 0; cc < 32; cc += 4) {
              const int unit = ch * 8 + (cc >> 2);
              sts_v4u(stage + row * 512 + ((unit ^ (row & 31)) << 4), make_uint4(o[cc], o[cc + 1], o[cc + 2], o[cc + 3]));
            }
          }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (ok) {
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int r = ws * 16 + rr;
            const uint4 w = lds_v4u(stage + r * 512 + ((lane ^ (r & 31)) << 4));
            *reinterpret_cast<uint4*>(p.part_o + (prow0 + r) * 512 + crank * 256 + h * 128 + lane * 4) = w;
          }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
      }
      if (ok && crank == 0 && half == 0) {
        p.part_ml[(prow0 + row) * 2] = m_seen;
        p.part_ml[(prow0 + row) * 2 + 1] = l_last;
      }
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 41);
    }
}

// ================================ producers =====================================================
// 256 threads, four per row: thread (row, q) owns latent units q, q+4, q+8, q+12 of this CTA's
// 256-dim half (unit = 16 int8 -> 16 bf16 = two 16-byte stores), rope unit q of the 32-dim half, and
// the half's two scales. Everything a tile needs is requested ahead of its use and nothing is
// branched on before it has had a tile's time to arrive: the selected index four tiles ahead, its
// block-table entry three tiles ahead, an L2 prefetch of the row two tiles ahead, the row itself one
// tile ahead (into the registers the current tile has just been dequantised out of).
// kBf16: the latent cache already holds bf16 (the operator's non-quantised key_nope_2d); thread (row, q)
// then owns bf16 units 2q and 2q+1 of each of the half's four 64-dim chunks. Nothing has to pass through
// registers: once the K buffer is free the nine 16-byte pieces go from L2 (the row was prefetched two
// tiles ago) to their swizzled places with `cp.async`, zero-filled for a padding row.
template <bool kBf16>
__device__ __forceinline__ void cl_role_producer(const SfaParams& p, const ClCtx c) {
  ClCtl* ctl = c.ctl;
  uint8_t* k_ptr = c.k_ptr;
  const uint32_t crank = c.crank;
  const int ntiles = c.ntiles, begin = c.begin, end = c.end, bi = c.bi;
  const int32_t* idx_row = c.idx_row;
  const int lane = threadIdx.x & 31;
  const int ptid = threadIdx.x - kClProducerWarp0 * 32;
  const int row = ptid >> 2;
  const int q = ptid & 3;
  const uint8_t* kn_bytes = reinterpret_cast<const uint8_t*>(p.kn);
  const uint8_t* kr_bytes = reinterpret_cast<const uint8_t*>(p.kr);
  const uint8_t* sc_bytes = reinterpret_cast<const uint8_t*>(p.kn_scales);
  struct RowRegs {
    uint4 d[kBf16 ? 1 : 4];
    uint4 r;
    float2 sc;
    long long phys;  // kBf16 only: the row to copy
    bool valid;
  };
  auto load_idx = [&](int j) -> int {
    const int e = begin + j * kCT + row;
    return (j < ntiles && e < end) ? ldg_pinned_i32(idx_row + e) : -1;
  };
  auto issue_loads = [&](RowRegs& r, long long phys) {
    r.valid = phys >= 0;
    if (!r.valid) return;
    if (kBf16) {
      r.phys = phys;
      return;
    }
    const uint8_t* nope = p.packed ? kn_bytes + phys * 656 : kn_bytes + phys * 512;
    const uint8_t* rope = p.packed ? kn_bytes + phys * 656 + 512 : kr_bytes + phys * 128;
    const uint8_t* scl = p.packed ? kn_bytes + phys * 656 + 640 : sc_bytes + phys * 16;
#pragma unroll
    for (int m = 0; m < 4; ++m) r.d[m] = ldg_pinned_v4(nope + crank * 256 + (q + 4 * m) * 16);
    r.r = ldg_pinned_v4(rope + crank * 64 + q * 16);
    r.sc = ldg_pinned_v2f(scl + crank * 8);
  };
  auto prefetch_row = [&](long long phys) { cl_prefetch_row<kBf16>(p, phys, crank, q); };
  const int sw = row & 7;
  const int rsw = (row >> 1) & 3;
  bool ok = true;
  RowRegs ra;
  pdl_wait();          // the selected indices come from the kernel before this one, which may still be running
  long long row_n;     // row of tile j+1
  int idx_a, entry_a;  // tile j+2
  int idx_b;           // tile j+3
  {
    const int idx0 = load_idx(0), idx1 = load_idx(1);
    idx_a = load_idx(2);
    idx_b = load_idx(3);
    const int e0 = tc_table_entry(p, bi, idx0);
    const int e1 = tc_table_entry(p, bi, idx1);
    entry_a = tc_table_entry(p, bi, idx_a);
    issue_loads(ra, tc_row_from_entry(p, idx0, e0));
    row_n = tc_row_from_entry(p, idx1, e1);
    prefetch_row(row_n);
  }
  for (int j = 0; j < ntiles; ++j) {
    const int kb = j % kNK;
    if (ptid == 0) TL(35, j);
    if (j >= kNK) {  // the P.V that read this buffer kNK tiles ago is complete
      ok = mbar_wait_warp(smem_u32(&ctl->k_free[kb]), ((j - kNK) / kNK) & 1);
      if (!ok) break;
    }
    if (ptid == 0) TL(5, j);
    // dequantise and store one latent unit at a time: nothing but the raw row stays in registers
    // (a spilled register costs a trip to L2 here: the L1 left beside 219 KB of shared memory is tiny)
    uint8_t* kbuf = k_ptr + kb * kKBuf;
    const bool valid = ra.valid;
    if (kBf16) {
      const uint32_t kaddr = c.k_base + kb * kKBuf;
      const uint32_t nbytes = valid ? 16u : 0u;  // 0: the 16 bytes are written as zeros, nothing is read
      const uint8_t* nope = kn_bytes + (valid ? ra.phys : 0) * 1024 + crank * 512 + q * 32;
      const uint8_t* rope = kr_bytes + (valid ? ra.phys : 0) * 128 + crank * 64 + q * 16;
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        cp_async_16(kaddr + m * kKNopeChunk + row * 128 + (((2 * q) ^ sw) << 4), nope + m * 128, nbytes);
        cp_async_16(kaddr + m * kKNopeChunk + row * 128 + (((2 * q + 1) ^ sw) << 4), nope + m * 128 + 16, nbytes);
      }
      cp_async_16(kaddr + 4 * kKNopeChunk + row * 64 + ((q ^ rsw) << 4), rope, nbytes);
      asm volatile("cp.async.wait_all;" ::: "memory");
    } else {
#pragma unroll
      for (int m = 0; m < 4; ++m) {  // latent unit q + 4m of the half: chunk m, bf16 units 2q, 2q+1
        uint4 c0 = make_uint4(0, 0, 0, 0), c1 = make_uint4(0, 0, 0, 0);
        if (valid) dequant16(ra.d[m], (m < 2) ? ra.sc.x : ra.sc.y, c0, c1);
        *reinterpret_cast<uint4*>(kbuf + m * kKNopeChunk + row * 128 + (((2 * q) ^ sw) << 4)) = c0;
        *reinterpret_cast<uint4*>(kbuf + m * kKNopeChunk + row * 128 + (((2 * q + 1) ^ sw) << 4)) = c1;
      }
      *reinterpret_cast<uint4*>(kbuf + 4 * kKNopeChunk + row * 64 + ((q ^ rsw) << 4)) = valid ? ra.r : make_uint4(0, 0, 0, 0);
    }
    if (q == 0) ctl->k_valid[kb][row] = valid ? 1 : 0;
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->k_full[kb]));
    if (ptid == 0) TL(6, j);
    if (ptid == 0 && j == 0) TLM(2);
    if (ptid == 0 && j == ntiles - 1) TLM(3);
    if (j + 1 < ntiles) issue_loads(ra, row_n);    // rows of tile j+1 (in L2: prefetched a tile ago)
    row_n = tc_row_from_entry(p, idx_a, entry_a);  // tile j+2: into L2
    prefetch_row(row_n);
    idx_a = idx_b;
    entry_a = tc_table_entry(p, bi, idx_a);        // block-table entries of tile j+3
    idx_b = load_idx(j + 4);
    if (ptid == 0) TL(4, j);
  }
  if (!ok && lane == 0) {
    ctl->abort = 1;
    set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 42);
  }
}

// 21 warps: six share one scheduler partition and 6 x 32 x 80 registers fit its file; bounds of 768 threads
// make the compiler start from 80 registers without capping the regions that raise their share
template <bool kBf16>
__global__ void __launch_bounds__(768, 1)
sfa_cluster_kernel(const __grid_constant__ SfaParams p) {
  // the swizzled operand tiles need a 1024-byte aligned base: the kernel has no static shared memory,
  // so the dynamic window starts aligned; a misaligned base is reported instead of computing garbage
  extern __shared__ __align__(1024) uint8_t sfa_cl_smem_raw[];
  const uint32_t base = smem_u32(sfa_cl_smem_raw);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(base), 43);
    return;
  }
  ClCtx c;
  c.k_base = base;
  c.x_base = c.k_base + kNK * kKBuf;
  c.k_ptr = sfa_cl_smem_raw;
  c.x_ptr = c.k_ptr + kNK * kKBuf;
  c.ctl = reinterpret_cast<ClCtl*>(c.x_ptr + 3 * kXBuf);
  ClCtl* ctl = c.ctl;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (tid == 0) TLM(0);
  c.crank = cluster_ctarank();  // which half of the dims this CTA owns
  c.peer = c.crank ^ 1u;
  const uint32_t crank = c.crank;
  const int bid = blockIdx.x >> 1;  // cluster index
  c.sp = bid % p.n_split;
  c.ti = bid / p.n_split;
  c.bi = c.ti / p.s1;
  const int si = c.ti % p.s1;

  int n = p.act_seq[c.bi] - p.s1 + 1 + si;
  n = max(0, min(n, p.topk_k));
  const int tiles_total = (n + kCT - 1) / kCT;
  const int tiles_per_split = (tiles_total + p.n_split - 1) / p.n_split;
  c.begin = min(n, c.sp * tiles_per_split * kCT);
  c.end = min(n, (c.sp + 1) * tiles_per_split * kCT);
  c.ntiles = (c.end - c.begin + kCT - 1) / kCT;
  c.idx_row = p.topk + static_cast<int64_t>(c.ti) * p.topk_k;
  c.q_row0 = static_cast<int64_t>(c.ti) * p.nq_total + p.head_begin;
  const int64_t q_row0 = c.q_row0;

  if (c.ntiles == 0) {  // same decision in both CTAs of the pair
    if (p.n_split == 1) {
      for (int e = tid; e < 128 * 32; e += kClThreads) {
        const int row = e >> 5, cc = e & 31;
        *reinterpret_cast<uint4*>(p.out + (q_row0 + row) * 512 + crank * 256 + cc * 8) = make_uint4(0, 0, 0, 0);
      }
    } else if (crank == 0) {
      for (int row = tid; row < 128; row += kClThreads) {
        float* ml = p.part_ml + ((static_cast<int64_t>(c.ti) * p.n_split + c.sp) * p.nq + row) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }

  // ---- before the setup: the softmax threads touch the Q rows they will copy into tensor memory, so
  // that the copy finds them in L2 (prefetches do not block; anything that waits here would hold up
  // the whole CTA's first barrier)
  if (warp >= kClSoftmaxWarp0 && warp < kClProducerWarp0) {
    const int qhalf = (warp - kClSoftmaxWarp0) >> 2;
    const int qrow = (warp & 3) * 32 + lane;
    const uint8_t* a = reinterpret_cast<const uint8_t*>(p.q_nope + (q_row0 + qrow) * 512 + crank * 256 + qhalf * 128);
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a + 128));
    if (qhalf == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q_rope + (q_row0 + qrow) * 64 + crank * 32));
  }

  // ---- setup ------------------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < kNK; ++i) {
      mbar_init(smem_u32(&ctl->k_full[i]), kClProducerWarps);
      mbar_init(smem_u32(&ctl->k_free[i]), 1);
    }
    mbar_init(smem_u32(&ctl->s_full), 1);
    mbar_init(smem_u32(&ctl->s_free), kClXWarps);
    mbar_init(smem_u32(&ctl->pv_done), 1);
    mbar_init(smem_u32(&ctl->p_full), kClSoftmaxWarps);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&ctl->xs_full[i]), 1);
      mbar_init(smem_u32(&ctl->xs_free[i]), 2);
      for (int b = 0; b < 2; ++b) {
        mbar_init(smem_u32(&ctl->xr_full[i][b]), 1);
        mbar_init(smem_u32(&ctl->xr_free[i][b]), 2);
        mbar_arrive_expect_tx(smem_u32(&ctl->xr_full[i][b]), kXSlice);  // armed for tiles 0 and 1
      }
      mbar_init(smem_u32(&ctl->pair_bar[i]), 2);
    }
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kClTmemCols);
    tmem_relinquish();
  }
  if (tid == 0) TLM(7);
  tc_fence_before();
  __syncthreads();
  if (tid == 0) TLM(8);
  cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
  if (tid == 0) TLM(9);
  tc_fence_after();
  c.tmem_base = ctl->tmem_base;
  const uint32_t tmem_base = c.tmem_base;
  // Q half into tensor memory (A operand of q.K^T): lane = head row, column c = dims 2c, 2c+1
  static_assert(32 * (kClSoftmaxWarps + 1) == 288, "named barrier 1: softmax warps + the MMA warp");
  if (warp >= kClSoftmaxWarp0 && warp < kClProducerWarp0) {
    const int qhalf = (warp - kClSoftmaxWarp0) >> 2;
    const int qrow = (warp & 3) * 32 + lane;
    const uint32_t dst = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kClColQ + 64 * qhalf;
    const uint4* src = reinterpret_cast<const uint4*>(p.q_nope + (q_row0 + qrow) * 512 + crank * 256 + qhalf * 128);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint32_t v[32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 w = __ldg(src + g * 8 + u);
        v[4 * u] = w.x;
        v[4 * u + 1] = w.y;
        v[4 * u + 2] = w.z;
        v[4 * u + 3] = w.w;
      }
      tmem_st_32x32b_x32(dst + 32 * g, v);
    }
    if (qhalf == 0) {  // rope half: 32 dims = 16 columns
      const uint4* rsrc = reinterpret_cast<const uint4*>(p.q_rope + (q_row0 + qrow) * 64 + crank * 32);
      uint32_t v[16];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint4 w = __ldg(rsrc + u);
        v[4 * u] = w.x;
        v[4 * u + 1] = w.y;
        v[4 * u + 2] = w.z;
        v[4 * u + 3] = w.w;
      }
      tmem_st_32x32b_x16(tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kClColQR, v);
    }
    tc_wait_st();
    tc_fence_before();
    asm volatile("bar.sync 1, 288;" ::: "memory");  // with the MMA warp: Q is in place
  } else if (warp == 0) {
    // only the MMA warp waits for Q; producers and exchange warps go straight to work, so the first
    // tile's index -> block-table -> row chain overlaps the Q loads instead of following them
    asm volatile("bar.sync 1, 288;" ::: "memory");
    tc_fence_after();
  }
  if (tid == 0) TLM(1);

  if (warp < kClSoftmaxWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 0) {
      cl_role_mma(p, c);
    } else {
      cl_role_exchange(p, c);
    }
  } else if (warp < kClProducerWarp0) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 88;");
    cl_role_softmax(p, c);
  } else if (warp < kClLastXWarp) {
    cl_role_producer<kBf16>(p, c);
  } else {
    cl_role_exchange(p, c);
  }

  // ---- teardown: neither CTA may leave while the peer can still write into its shared memory --------
  if (tid == 32 * kClSoftmaxWarp0) TLM(5);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (tid == 0) TLM(6);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kClTmemCols);
  }
}

}  // namespace

#ifdef PTO_SFA_TIMELINE
extern "C" int pto_debug_sfa_reset() {
  static long long zeros[16 * 40] = {0};
  return static_cast<int>(cudaMemcpyToSymbol(g_sfa_timeline, zeros, sizeof(zeros)));
}
extern "C" int pto_debug_sfa_timeline(long long* host, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_sfa_timeline, sizeof(long long) * n));
}
#endif

cudaError_t launch_sfa_cluster(const SfaParams& p, cudaStream_t stream) {
  // two instances of one kernel: int8 latent rows dequantised by the producers, or bf16 rows copied as they are
  void (*kernel)(SfaParams) = p.kn_bf16 ? sfa_cluster_kernel<true> : sfa_cluster_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kClSmemBytes));
  if (e != cudaSuccess) return e;
  const int t = p.b * p.s1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(t) * p.n_split * 2, 1, 1);
  cfg.blockDim = dim3(kClThreads, 1, 1);
  cfg.dynamicSmemBytes = kClSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // behind the top-k kernel of the fused chain: tensor-memory allocation, barrier set-up and the copy of Q run
  // while the selection finishes; only the producers read its output, and they wait first
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 2 : 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace pto
