// Sparse MLA attention for 128 heads: a cluster of two CTAs per (token, split) that splits the
// 576-wide q.K^T contraction between the CTAs.
//
// Arithmetic as in sfa_decode.cu (reference:
// examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:45-207; golden
// deepseekv32_sparse_flash_attention_quant.py:169-254).
//
// CTA c of the pair owns latent dims [256c, 256c+256) and rope dims [32c, 32c+32): it holds that
// half of Q (72 KB), gathers and dequantises only that half of every selected row, computes the
// partial scores S_c = Q_c . K_c^T for all 128 heads (tcgen05, M = 128, N = 64 rows per tile), and
// owns the 256-wide half of the output (P . V_c, V_c = the latent half it already has in shared
// memory). The two partial score tiles are exchanged through distributed shared memory: every
// softmax thread (one per head row) writes its 64 fp32 partials into the peer's exchange buffer,
// signals the peer's mbarrier, waits for the peer's partials in its own buffer and adds them (fp32
// addition commutes, so both CTAs get bit-identical scores, maxima and P). Nothing is computed
// twice except the softmax itself.
//   warp 0        MMA issuer (owns TMEM: O 256 columns + two 64-column score buffers)
//   warps 1..8    softmax, two threads per head row (32 of the tile's 64 columns each)
//   warps 9..16   producers: 16-byte gathers, int8 -> bf16 in registers, swizzled stores (2 K buffers)
// All waits are bounded; local waits that order peer writes use cluster-scope acquire.
#include "common.cuh"
#include "sfa_common.cuh"

namespace pto {

namespace {


constexpr int kCT = 64;                          // selected rows per tile
constexpr int kQNopeChunk = 128 * 128;           // 128 heads x 64 dims bf16, 128-byte rows
constexpr int kQRope = 128 * 64;                 // 128 heads x 32 dims bf16, 64-byte rows
constexpr int kQBytes = 4 * kQNopeChunk + kQRope;  // 73,728
constexpr int kKNopeChunk = kCT * 128;
constexpr int kKRope = kCT * 64;
constexpr int kKBuf = 4 * kKNopeChunk + kKRope;  // 36,864
constexpr int kPBuf = 128 * 128;                 // 128 heads x 64 rows bf16
constexpr int kXBuf = 128 * 256;                 // 128 heads x 64 fp32 partial scores
constexpr int kClSoftmaxWarp0 = 1;
constexpr int kClSoftmaxWarps = 8;   // two warps per TMEM lane quarter: columns 0-31 and 32-63 of the tile
constexpr int kClProducerWarp0 = 1 + kClSoftmaxWarps;
constexpr int kClProducerWarps = 8;
constexpr int kClThreads = 32 * (kClProducerWarp0 + kClProducerWarps);  // 544
constexpr uint32_t kClTmemCols = 512;
constexpr uint32_t kClColO = 0;
constexpr uint32_t kClColS = 256;  // + 64 * buffer
constexpr float kClRescale = 8.0f;

struct ClCtl {
  uint64_t k_full[2];   // producers filled K buffer b                      (count: producer warps)
  uint64_t s_full[2];   // partial scores of buffer b complete               (tcgen05.commit)
  uint64_t s_free[2];   // softmax warps have read score buffer b             (count 8 warps)
  uint64_t pv_done[2];  // P.V of a tile with parity b complete              (tcgen05.commit)
  uint64_t p_full;      // P tile written                                    (count 8 warps)
  uint64_t x_full[8];   // peer's partials of softmax warp w landed in my receive buffer (1 arming arrive + 4096 tx bytes)
  uint64_t x_free[8];   // peer's warp w has consumed what my warp w sent             (1 remote arrival)
  uint32_t tmem_base;
  int abort;
  __align__(16) unsigned char k_valid[2][kCT];
  uint64_t pair_bar[4];  // the two softmax warps of a lane quarter meet here (count 2), bounded like every wait
  float pair_mt[2][2][128];  // [tile parity][column half][row]: tile max of each half; the halves' sums at the end
};

constexpr size_t kClSmemBytes = kQBytes + 2 * kKBuf + kPBuf + 2 * kXBuf + sizeof(ClCtl);
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
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
// bulk copy of this CTA's shared memory into the peer's, completing (tx bytes) on the peer's mbarrier
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, uint32_t src_local, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src_local), "r"(bytes), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// no ordering of this thread's earlier writes is needed (the peer only waits for reads to have happened)
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  if (mbar_test_wait_cluster(bar, parity)) return true;
  const long long t0s = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      if (mbar_test_wait_cluster(bar, parity)) return true;
    }
    if (clock64() - t0s > kWaitBudgetCycles) return false;
  }
}
__device__ __forceinline__ bool mbar_wait_cluster_blocking(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_cluster(bar, parity)) return true;
    }
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

__global__ void __launch_bounds__(kClThreads, 1)
sfa_cluster_kernel(SfaParams p) {
  // the swizzled operand tiles need a 1024-byte aligned base: the kernel has no static shared memory,
  // so the dynamic window starts aligned; a misaligned base is reported instead of computing garbage
  extern __shared__ __align__(1024) uint8_t sfa_cl_smem_raw[];
  const uint32_t base = smem_u32(sfa_cl_smem_raw);
  uint8_t* smem = sfa_cl_smem_raw;
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(p.status, PTO_ST_WAIT_EXPIRED, static_cast<int>(base), 43);
    return;
  }
  const uint32_t q_base = base;
  const uint32_t k_base = q_base + kQBytes;
  const uint32_t p_base = k_base + 2 * kKBuf;
  const uint32_t x_base = p_base + kPBuf;
  uint8_t* q_ptr = smem;
  uint8_t* k_ptr = q_ptr + kQBytes;
  uint8_t* p_ptr = k_ptr + 2 * kKBuf;
  uint8_t* x_ptr = p_ptr + kPBuf;
  ClCtl* ctl = reinterpret_cast<ClCtl*>(x_ptr + 2 * kXBuf);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t crank = cluster_ctarank();  // which half of the dims this CTA owns
  const uint32_t peer = crank ^ 1u;
  int bid = blockIdx.x >> 1;  // cluster index
  const int sp = bid % p.n_split;
  const int ti = bid / p.n_split;
  const int bi = ti / p.s1;
  const int si = ti % p.s1;

  int n = p.act_seq[bi] - p.s1 + 1 + si;
  n = max(0, min(n, p.topk_k));
  const int tiles_total = (n + kCT - 1) / kCT;
  const int tiles_per_split = (tiles_total + p.n_split - 1) / p.n_split;
  const int begin = min(n, sp * tiles_per_split * kCT);
  const int end = min(n, (sp + 1) * tiles_per_split * kCT);
  const int ntiles = (end - begin + kCT - 1) / kCT;
  const int32_t* idx_row = p.topk + static_cast<int64_t>(ti) * p.topk_k;
  const int64_t q_row0 = static_cast<int64_t>(ti) * p.nq_total + p.head_begin;

  if (ntiles == 0) {  // same decision in both CTAs of the pair
    if (p.n_split == 1) {
      for (int e = tid; e < 128 * 32; e += kClThreads) {
        const int row = e >> 5, c = e & 31;
        *reinterpret_cast<uint4*>(p.out + (q_row0 + row) * 512 + crank * 256 + c * 8) = make_uint4(0, 0, 0, 0);
      }
    } else if (crank == 0) {
      for (int row = tid; row < 128; row += kClThreads) {
        float* ml = p.part_ml + ((static_cast<int64_t>(ti) * p.n_split + sp) * p.nq + row) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }

  // ---- setup ------------------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->k_full[i]), kClProducerWarps);
      mbar_init(smem_u32(&ctl->s_full[i]), 1);
      mbar_init(smem_u32(&ctl->s_free[i]), kClSoftmaxWarps);
      mbar_init(smem_u32(&ctl->pv_done[i]), 1);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(smem_u32(&ctl->x_full[i]), 1);
      mbar_init(smem_u32(&ctl->x_free[i]), 1);
      mbar_arrive_expect_tx(smem_u32(&ctl->x_full[i]), 32 * 128);  // armed for the first tile
    }
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&ctl->pair_bar[i]), 2);
    mbar_init(smem_u32(&ctl->p_full), kClSoftmaxWarps);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kClTmemCols);
    tmem_relinquish();
  }
  // Q half: four 64-dim latent chunks (128-byte rows, unit u at u ^ (h & 7)) and the 32-dim rope
  // half (64-byte rows, unit u at u ^ ((h >> 1) & 3))
  for (int e = tid; e < 128 * 36; e += kClThreads) {
    const int h = e / 36, uu = e % 36;
    if (uu < 32) {
      const int c = uu >> 3, u = uu & 7;
      const uint4 v = *reinterpret_cast<const uint4*>(p.q_nope + (q_row0 + h) * 512 + crank * 256 + c * 64 + u * 8);
      *reinterpret_cast<uint4*>(q_ptr + c * kQNopeChunk + h * 128 + ((u ^ (h & 7)) << 4)) = v;
    } else {
      const int u = uu - 32;
      const uint4 v = *reinterpret_cast<const uint4*>(p.q_rope + (q_row0 + h) * 64 + crank * 32 + u * 8);
      *reinterpret_cast<uint4*>(q_ptr + 4 * kQNopeChunk + h * 64 + ((u ^ ((h >> 1) & 3)) << 4)) = v;
    }
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ================================ MMA issuer ================================================
    const uint32_t idesc_qk = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 0, 128, kCT);
    const uint32_t idesc_pv = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 1, 128, 256);
    if (lane == 0) {
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int b = j & 1;
        const uint32_t d = tmem_base + kClColS + kCT * b;
        const uint32_t kb = k_base + b * kKBuf;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const uint64_t a_desc = umma_desc_kmajor_sw128(q_base + c * kQNopeChunk);
          const uint64_t b_desc = umma_desc_kmajor_sw128(kb + c * kKNopeChunk);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc_qk, (c | k) != 0 ? 1u : 0u);
        }
        const uint64_t a_desc = desc_kmajor_sw64(q_base + 4 * kQNopeChunk);
        const uint64_t b_desc = desc_kmajor_sw64(kb + 4 * kKNopeChunk);
#pragma unroll
        for (int k = 0; k < 2; ++k) mma_f16_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc_qk, 1u);
        tc_commit(smem_u32(&ctl->s_full[b]));
      };
      auto issue_pv = [&](int j) {
        const int b = j & 1;
        const uint64_t a_desc = umma_desc_kmajor_sw128(p_base);
        const uint64_t b_desc = desc_mnmajor_sw128(k_base + b * kKBuf, kKNopeChunk, 1024);
#pragma unroll
        for (int k = 0; k < kCT / 16; ++k) {
          mma_f16_ss(tmem_base + kClColO, a_desc + 2 * k, b_desc + k * ((16 * 128) >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&ctl->pv_done[b]));
      };
      // q.K^T of tile j+1 is issued before P.V of tile j; a score buffer is reused two tiles later,
      // after the softmax set that read it has arrived on s_free
      auto qk_ready = [&](int j) -> bool {
        if (!mbar_wait_spin(smem_u32(&ctl->k_full[j & 1]), (j >> 1) & 1)) return false;
        if (j >= 2 && !mbar_wait_spin(smem_u32(&ctl->s_free[j & 1]), ((j - 2) >> 1) & 1)) return false;
        tc_fence_after();
        return true;
      };
      ok = qk_ready(0);
      if (ok) issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          ok = qk_ready(j + 1);
          if (!ok) break;
          issue_qk(j + 1);
        }
        ok = mbar_wait_spin(smem_u32(&ctl->p_full), j & 1);
        if (!ok) break;
        tc_fence_after();
        issue_pv(j);
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 40);
      }
    }
    __syncwarp();
  } else if (warp < kClProducerWarp0) {
    // ================================ softmax ===================================================
    // Thread (row, half): head row = TMEM lane, columns [32*half, 32*half+32) of the 64-row tile.
    const int half = (warp - kClSoftmaxWarp0) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int wslot = half * 4 + quarter;  // this warp's exchange slice and barriers
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    // exchange: send area = first half of X, receive area = second half; a warp owns a 4 KB slice
    // (32 rows x 128 B) in both. A row is 8 units of 16 bytes, unit u stored at u ^ (lane & 7).
    uint8_t* send_row = x_ptr + wslot * 4096 + lane * 128;
    const uint8_t* recv_row = x_ptr + kXBuf + wslot * 4096 + lane * 128;
    const uint32_t send_slice = x_base + wslot * 4096;
    const uint32_t recv_slice_peer = map_to_peer(x_base + kXBuf + wslot * 4096, peer);
    const uint32_t xfull_local = smem_u32(&ctl->x_full[wslot]);
    const uint32_t xfull_peer = map_to_peer(xfull_local, peer);
    const uint32_t xfree_local = smem_u32(&ctl->x_free[wslot]);
    const uint32_t xfree_peer = map_to_peer(xfree_local, peer);
    const int xsw = lane & 7;
    float m_seen = -INFINITY;  // the row's reference max (identical in both halves)
    float l_run = 0.f;         // this half's share of the row sum
    bool ok = true;
    uint32_t pair_phase = 0;
    auto pair_sync = [&]() -> bool {  // orders the pair_mt writes of both warps before the reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->pair_bar[quarter]));
      const bool w = mbar_wait_spin(smem_u32(&ctl->pair_bar[quarter]), pair_phase & 1u);
      ++pair_phase;
      return __all_sync(0xffffffffu, w);
    };
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      ok = mbar_wait_spin(smem_u32(&ctl->s_full[b]), (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float s[32];
      {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + kClColS + kCT * b + 32 * half, v);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(v[c]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->s_free[b]));
      // ---- exchange the partial scores with the peer CTA (per warp: 32 rows x 32 columns, 4 KB) ------
      {
        if (lane == 0) bulk_wait_read_all();  // the previous tile's copy has finished reading the send slice
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          *reinterpret_cast<float4*>(send_row + ((u ^ xsw) << 4)) = make_float4(s[4 * u], s[4 * u + 1], s[4 * u + 2], s[4 * u + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          // the peer's warp must have consumed the previous tile before its receive slice is overwritten
          if (j >= 1 && !mbar_wait_cluster(xfree_local, (j - 1) & 1)) ok = false;
          if (ok) {
            bulk_copy_to_peer(recv_slice_peer, send_slice, 4096, xfull_peer);
            bulk_commit();
          }
        }
        ok = ok && mbar_wait_cluster(xfull_local, j & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 o = *reinterpret_cast<const float4*>(recv_row + ((u ^ xsw) << 4));
          s[4 * u] += o.x;
          s[4 * u + 1] += o.y;
          s[4 * u + 2] += o.z;
          s[4 * u + 3] += o.w;
        }
        __syncwarp();
        if (lane == 31) {
          mbar_arrive_expect_tx(xfull_local, 4096);  // arm the receive barrier for the next tile, then
          mbar_arrive_remote_relaxed(xfree_peer);     // tell the peer this warp's slice has been consumed
        }
      }
      // ---- scale, mask, max of this half ------------------------------------------------------------
      mbar_wait_spin(smem_u32(&ctl->k_full[b]), (j >> 1) & 1);  // already complete: orders the k_valid reads
      // all rows valid (always, except in a token's last tile or after a rejected index): max on
      // the raw sums, scale folded into the exponent's FMA
      const uint4 va = *reinterpret_cast<const uint4*>(&ctl->k_valid[b][32 * half]);
      const uint4 vb = *reinterpret_cast<const uint4*>(&ctl->k_valid[b][32 * half + 16]);
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
      // The previous tile's P.V may still be running and the other half's maximum is not known yet;
      // rescales are rare, so exp2 is taken now against the row's current reference (never more than
      // 2^8 below this half's maximum) and corrected by one factor once the reference is final.
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
      // ---- join: the other half's maximum, then the previous tile's P.V (P buffer free, O at rest) -----
      ok = pair_sync();
      if (!ok) break;
      const float mt = fmaxf(mt_half, ctl->pair_mt[b][half ^ 1][row]);
      if (j > 0) {
        ok = mbar_wait_spin(smem_u32(&ctl->pv_done[(j - 1) & 1]), ((j - 1) >> 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
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
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {  // this half's 128 of the 256 output columns
          uint32_t o[16];
          tmem_ld_32x32b_x16(lane_addr + kClColO + half * 128 + ch * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st_32x32b_x16(lane_addr + kClColO + half * 128 + ch * 16, o);
        }
        tc_wait_st();
      }
      // ---- P row (bf16, 128-byte row, unit u at u ^ (row & 7)); this half owns units 4*half .. +3 ------
      uint8_t* prow = p_ptr + row * 128;
      const int psw = row & 7;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 w;
        w.x = pack_bf16x2(s[8 * u] * factor, s[8 * u + 1] * factor);
        w.y = pack_bf16x2(s[8 * u + 2] * factor, s[8 * u + 3] * factor);
        w.z = pack_bf16x2(s[8 * u + 4] * factor, s[8 * u + 5] * factor);
        w.w = pack_bf16x2(s[8 * u + 6] * factor, s[8 * u + 7] * factor);
        *reinterpret_cast<uint4*>(prow + (((4 * half + u) ^ psw) << 4)) = w;
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
    }
    if (lane == 0) bulk_wait_read_all();
    // ---- output: row sum = both halves' shares; each half stores 128 of the CTA's 256 columns ---------
    if (ok) {
      ok = mbar_wait_spin(smem_u32(&ctl->pv_done[(ntiles - 1) & 1]), ((ntiles - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    float l_last = 0.f;
    if (ok) {
      ctl->pair_mt[ntiles & 1][half][row] = l_run;
      ok = pair_sync();
      l_last = l_run + ctl->pair_mt[ntiles & 1][half ^ 1][row];
    }
    if (ok) {
      tc_fence_after();
      if (p.n_split == 1) {
        const float inv = l_last > 0.f ? 1.f / l_last : 0.f;
        __nv_bfloat16* dst = p.out + (q_row0 + row) * 512 + crank * 256 + half * 128;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kClColO + half * 128 + ch * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + ch * 32 + c) = w;
          }
        }
      } else {
        const int64_t prow_i = (static_cast<int64_t>(ti) * p.n_split + sp) * p.nq + row;
        float* dst = p.part_o + prow_i * 512 + crank * 256 + half * 128;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kClColO + half * 128 + ch * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            *reinterpret_cast<uint4*>(dst + ch * 32 + c) = make_uint4(o[c], o[c + 1], o[c + 2], o[c + 3]);
          }
        }
        if (crank == 0 && half == 0) {
          p.part_ml[prow_i * 2] = m_seen;
          p.part_ml[prow_i * 2 + 1] = l_last;
        }
      }
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 41);
    }
  } else {
    // ================================ producers =================================================
    // 256 threads, four per row: thread (row, q) owns latent units q, q+4, q+8, q+12 of this CTA's
    // 256-dim half (unit = 16 int8 -> 16 bf16 = two 16-byte stores), rope unit q of the 32-dim
    // half, and the half's two scales. The next tile's loads are issued as soon as the current
    // registers are dequantised; only the stores sit behind the buffer wait.
    const int ptid = tid - kClProducerWarp0 * 32;
    const int row = ptid >> 2;
    const int q = ptid & 3;
    auto load_idx = [&](int j) -> int {
      const int e = begin + j * kCT + row;
      return (j < ntiles && e < end) ? idx_row[e] : -1;
    };
    const uint8_t* kn_bytes = reinterpret_cast<const uint8_t*>(p.kn);
    const uint8_t* kr_bytes = reinterpret_cast<const uint8_t*>(p.kr);
    const uint8_t* sc_bytes = reinterpret_cast<const uint8_t*>(p.kn_scales);
    struct RowRegs {
      uint4 d[4];
      uint4 r;
      float2 sc;
      bool valid;
    };
    auto issue_loads = [&](RowRegs& r, long long phys) {
      r.valid = phys >= 0;
      if (!r.valid) return;
      const uint8_t* nope = p.packed ? kn_bytes + phys * 656 : kn_bytes + phys * 512;
      const uint8_t* rope = p.packed ? kn_bytes + phys * 656 + 512 : kr_bytes + phys * 128;
      const uint8_t* scl = p.packed ? kn_bytes + phys * 656 + 640 : sc_bytes + phys * 16;
#pragma unroll
      for (int m = 0; m < 4; ++m) r.d[m] = __ldg(reinterpret_cast<const uint4*>(nope + crank * 256 + (q + 4 * m) * 16));
      r.r = __ldg(reinterpret_cast<const uint4*>(rope + crank * 64 + q * 16));
      r.sc = __ldg(reinterpret_cast<const float2*>(scl + crank * 8));
    };
    const int sw = row & 7;
    const int rsw = (row >> 1) & 3;
    bool ok = true;
    RowRegs ra;
    long long phys_next = tc_physical_row(p, bi, load_idx(1));
    int idx_n2 = load_idx(2);
    issue_loads(ra, tc_physical_row(p, bi, load_idx(0)));
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      uint4 cv[8];
      const bool valid = ra.valid;
      if (valid) {
#pragma unroll
        for (int m = 0; m < 4; ++m) dequant16(ra.d[m], (m < 2) ? ra.sc.x : ra.sc.y, cv[2 * m], cv[2 * m + 1]);
      } else {
#pragma unroll
        for (int m = 0; m < 8; ++m) cv[m] = make_uint4(0, 0, 0, 0);
      }
      const uint4 rr = valid ? ra.r : make_uint4(0, 0, 0, 0);
      if (j + 1 < ntiles) issue_loads(ra, phys_next);
      phys_next = tc_physical_row(p, bi, idx_n2);
      idx_n2 = load_idx(j + 3);
      if (j >= 2) {
        ok = mbar_wait_spin(smem_u32(&ctl->pv_done[b]), ((j - 2) >> 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      uint8_t* kbuf = k_ptr + b * kKBuf;
#pragma unroll
      for (int m = 0; m < 4; ++m) {  // latent unit q + 4m of the half: chunk m, bf16 units 2q, 2q+1
        *reinterpret_cast<uint4*>(kbuf + m * kKNopeChunk + row * 128 + (((2 * q) ^ sw) << 4)) = cv[2 * m];
        *reinterpret_cast<uint4*>(kbuf + m * kKNopeChunk + row * 128 + (((2 * q + 1) ^ sw) << 4)) = cv[2 * m + 1];
      }
      *reinterpret_cast<uint4*>(kbuf + 4 * kKNopeChunk + row * 64 + ((q ^ rsw) << 4)) = rr;
      if (q == 0) ctl->k_valid[b][row] = valid ? 1 : 0;
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->k_full[b]));
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 42);
    }
  }

  // ---- teardown: neither CTA may leave while the peer can still write into its shared memory --------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kClTmemCols);
  }
}

}  // namespace

cudaError_t launch_sfa_cluster(const SfaParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(sfa_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kClSmemBytes));
  if (e != cudaSuccess) return e;
  const int t = p.b * p.s1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(t) * p.n_split * 2, 1, 1);
  cfg.blockDim = dim3(kClThreads, 1, 1);
  cfg.dynamicSmemBytes = kClSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, sfa_cluster_kernel, p);
}

}  // namespace pto
