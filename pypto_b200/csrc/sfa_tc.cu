// Sparse MLA attention for 128 heads on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Same arithmetic as sfa_decode.cu (reference:
// examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:45-207; golden
// deepseekv32_sparse_flash_attention_quant.py:169-254): per query token the first n selected rows
// are gathered from the paged cache, kn = bf16(int8 * scale), s = q.[kn|rope]^T * scale,
// online softmax with P rounded once to bf16, O = P.kn accumulated in fp32.
//
// One CTA per (token, half of the 512 value dims, split of the selected rows). TMEM cannot hold a
// 128 x 512 fp32 output next to the scores, so the output is split in two 256-wide halves; each CTA
// computes the full 128 x 32 score tile (M = 128 heads) and its half of P.V.
//   warp 0       : issues tcgen05.mma (q.K^T: 36 x (128x32x16), P.V: 2 x (128x256x16)), owns TMEM
//   warps 1..4   : softmax, one thread per head row (TMEM lane): S from TMEM, P to shared (bf16),
//                  lazy rescale of the O accumulator in TMEM, final normalisation and store
//   warps 5..12  : producers in two groups (one per K buffer): 16-byte loads of the selected rows,
//                  int8 -> bf16 dequantisation in registers, swizzled stores into the K tile
// Shared memory: Q 128 x 576 bf16 as nine 64-wide K-major chunks (128-byte swizzle); two K tiles of
// 32 rows in the same chunked layout, which serves both as the K-major B operand of q.K^T and as
// the MN-major B operand (V) of P.V; P 128 x 32 bf16 (64-byte swizzle). All waits are bounded.
#include "common.cuh"
#include "sfa_common.cuh"

namespace pto {

namespace {

constexpr int kT = 32;
constexpr int kChunks = 9;
constexpr int kQChunkBytes = 128 * 128;
constexpr int kKChunkBytes = kT * 128;
constexpr int kKBufBytes = kChunks * kKChunkBytes;
constexpr int kPBytes = 128 * 64;
constexpr int kProducerWarp0 = 5;
constexpr int kProducerWarps = 8;
constexpr int kTcThreads = 32 * (kProducerWarp0 + kProducerWarps);  // 416
constexpr uint32_t kTmemColsTc = 512;
constexpr uint32_t kColO = 0;
constexpr uint32_t kColS = 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P stays below 2^8 between rescales

struct TcCtl {
  uint64_t k_full[2];
  uint64_t s_full[2];
  uint64_t pv_done[2];
  uint64_t p_full;
  uint32_t tmem_base;
  int abort;
  __align__(16) unsigned char k_valid[2][kT];
};

constexpr size_t kTcSmemBytes = 1024 + kChunks * kQChunkBytes + 2 * kKBufBytes + kPBytes + sizeof(TcCtl);

__global__ void __launch_bounds__(kTcThreads, 1)
sfa_tc_kernel(SfaParams p) {
  extern __shared__ uint8_t sfa_tc_smem_raw[];
  const uint32_t raw = smem_u32(sfa_tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = sfa_tc_smem_raw + (base - raw);
  const uint32_t q_base = base;
  const uint32_t k_base = base + kChunks * kQChunkBytes;
  const uint32_t p_base = k_base + 2 * kKBufBytes;
  uint8_t* q_ptr = smem;
  uint8_t* k_ptr = smem + kChunks * kQChunkBytes;
  uint8_t* p_ptr = k_ptr + 2 * kKBufBytes;
  TcCtl* ctl = reinterpret_cast<TcCtl*>(p_ptr + kPBytes);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  int bid = blockIdx.x;
  const int sp = bid % p.n_split;
  bid /= p.n_split;
  const int dvh = bid & 1;
  const int ti = bid >> 1;
  const int bi = ti / p.s1;
  const int si = ti % p.s1;

  int n = p.act_seq[bi] - p.s1 + 1 + si;
  n = max(0, min(n, p.topk_k));
  const int tiles_total = (n + kT - 1) / kT;
  const int tiles_per_split = (tiles_total + p.n_split - 1) / p.n_split;
  const int begin = min(n, sp * tiles_per_split * kT);
  const int end = min(n, (sp + 1) * tiles_per_split * kT);
  const int ntiles = (end - begin + kT - 1) / kT;
  const int32_t* idx_row = p.topk + static_cast<int64_t>(ti) * p.topk_k;
  const int64_t q_row0 = static_cast<int64_t>(ti) * p.nq_total + p.head_begin;

  if (ntiles == 0) {
    if (p.n_split == 1) {
      for (int e = tid; e < 128 * 32; e += kTcThreads) {  // 128 rows x 32 uint4 (256 bf16)
        const int row = e >> 5, c = e & 31;
        *reinterpret_cast<uint4*>(p.out + (q_row0 + row) * 512 + dvh * 256 + c * 8) = make_uint4(0, 0, 0, 0);
      }
    } else if (dvh == 0) {
      for (int row = tid; row < 128; row += kTcThreads) {
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
      mbar_init(smem_u32(&ctl->k_full[i]), kProducerWarps / 2);  // one producer group per buffer
      mbar_init(smem_u32(&ctl->s_full[i]), 1);
      mbar_init(smem_u32(&ctl->pv_done[i]), 1);
    }
    mbar_init(smem_u32(&ctl->p_full), 4);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemColsTc);
    tmem_relinquish();
  }
  // Q: 128 heads x 576, chunk c = dims [64c, 64c+64), row h at h*128 B, 16-byte unit u at (u ^ (h & 7))
  for (int e = tid; e < 128 * 72; e += kTcThreads) {
    const int h = e / 72, uu = e % 72;
    const int c = uu >> 3, u = uu & 7;
    const uint4 v = (c < 8) ? *reinterpret_cast<const uint4*>(p.q_nope + (q_row0 + h) * 512 + c * 64 + u * 8)
                            : *reinterpret_cast<const uint4*>(p.q_rope + (q_row0 + h) * 64 + u * 8);
    *reinterpret_cast<uint4*>(q_ptr + c * kQChunkBytes + h * 128 + ((u ^ (h & 7)) << 4)) = v;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ================================ MMA issuer ================================================
    const uint32_t idesc_qk = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 0, 128, kT);
    const uint32_t idesc_pv = umma_idesc(kCFmtF32, kABFmtBF16, kABFmtBF16, 0, 1, 128, 256);
    bool ok = true;
    auto issue_qk = [&](int j) {
      const int b = j & 1;
      const uint32_t d = tmem_base + kColS + kT * b;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        const uint64_t a_desc = umma_desc_kmajor_sw128(q_base + c * kQChunkBytes);
        const uint64_t b_desc = umma_desc_kmajor_sw128(k_base + b * kKBufBytes + c * kKChunkBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if ((p.debug & 64) && k > 0) break;
          mma_f16_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc_qk, (c | k) != 0 ? 1u : 0u);
        }
      }
      tc_commit(smem_u32(&ctl->s_full[b]));
    };
    auto issue_pv = [&](int j) {
      const int b = j & 1;
      const uint64_t a_desc = desc_kmajor_sw64(p_base);
      const uint64_t b_desc = desc_mnmajor_sw128(k_base + b * kKBufBytes + dvh * 4 * kKChunkBytes, kKChunkBytes, 1024);
#pragma unroll
      for (int k = 0; k < kT / 16; ++k) {
        mma_f16_ss(tmem_base + kColO, a_desc + 2 * k, b_desc + k * ((16 * 128) >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
      }
      tc_commit(smem_u32(&ctl->pv_done[b]));
    };
    if (lane == 0) {
      if (!mbar_wait(smem_u32(&ctl->k_full[0]), 0)) {
        ok = false;
      } else {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          if (!mbar_wait(smem_u32(&ctl->k_full[(j + 1) & 1]), ((j + 1) >> 1) & 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_qk(j + 1);
        }
        if (!mbar_wait(smem_u32(&ctl->p_full), j & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        issue_pv(j);
      }
      if (!ok) {
        ctl->abort = 1;
        set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 30);
      }
    }
    __syncwarp();
  } else if (warp < kProducerWarp0) {
    // ================================ softmax ===================================================
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      ok = mbar_wait(smem_u32(&ctl->s_full[b]), (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32b_x32(lane_addr + kColS + kT * b, v);
      tc_wait_ld();
      mbar_wait(smem_u32(&ctl->k_full[b]), (j >> 1) & 1);  // already complete: orders the k_valid reads
      const uint4 va = *reinterpret_cast<const uint4*>(&ctl->k_valid[b][0]);
      const uint4 vb = *reinterpret_cast<const uint4*>(&ctl->k_valid[b][16]);
      const uint32_t vw[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      float s[32];
      float mt = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const bool valid = ((vw[c >> 2] >> ((c & 3) * 8)) & 0xffu) != 0;
        s[c] = valid ? __uint_as_float(v[c]) * p.scale_log2 : -INFINITY;
        mt = fmaxf(mt, s[c]);
      }
      const float m_new = fmaxf(m_used, mt);
      const bool need = (m_new > m_used + kRescaleThreshold) || (m_used == -INFINITY && m_new > -INFINITY);
      if (j > 0) {
        ok = mbar_wait(smem_u32(&ctl->pv_done[(j - 1) & 1]), ((j - 1) >> 1) & 1);  // P buffer free, O at rest
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      float alpha = 1.f;
      if (need) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
        l *= alpha;
        m_used = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kColO + ch * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st_32x32b_x32(lane_addr + kColO + ch * 32, o);
        }
        tc_wait_st();
      }
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float lsum = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = (p.debug & 16) ? s[c] : ex2f(s[c] - mref), p1 = (p.debug & 16) ? s[c + 1] : ex2f(s[c + 1] - mref);
        lsum += p0 + p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l += lsum;
      uint8_t* prow = p_ptr + row * 64;
      const int sw = (row >> 1) & 3;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        *reinterpret_cast<uint4*>(prow + ((u ^ sw) << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
    }
    if (ok) {
      ok = mbar_wait(smem_u32(&ctl->pv_done[(ntiles - 1) & 1]), ((ntiles - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      if (p.n_split == 1) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + (q_row0 + row) * 512 + dvh * 256;
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kColO + ch * 32, o);
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
        const int64_t prow = (static_cast<int64_t>(ti) * p.n_split + sp) * p.nq + row;
        float* dst = p.part_o + prow * 512 + dvh * 256;
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + kColO + ch * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            *reinterpret_cast<uint4*>(dst + ch * 32 + c) = make_uint4(o[c], o[c + 1], o[c + 2], o[c + 3]);
          }
        }
        if (dvh == 0) {
          p.part_ml[prow * 2] = m_used;
          p.part_ml[prow * 2 + 1] = l;
        }
      }
    } else if (lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 31);
    }
  } else {
    // ================================ producers =================================================
    // Two groups of four warps; group g fills the tiles j with j % 2 == g (always K buffer g). Each
    // thread owns a quarter of one row: ten 16-byte units (8 of int8 latent, 2 of bf16 rope) and the
    // row's four scales. The loads of the group's next tile are issued into a second register set
    // before the current tile is converted, so up to four tiles are in flight per CTA.
    const int ptid = tid - kProducerWarp0 * 32;
    const int grp = ptid >> 7;
    const int gt = ptid & 127;
    const int row = gt >> 2;  // row of the tile
    const int q = gt & 3;     // 16-byte lane: units q, q+4, ..., q+36 of the 41-unit row
    const int n_mine = (ntiles - grp + 1) / 2;  // tiles grp, grp+2, ...
    auto load_idx = [&](int i) -> int {  // i-th tile of this group
      const int e = begin + (grp + 2 * i) * kT + row;
      return (i < n_mine && e < end) ? idx_row[e] : -1;
    };
    const uint8_t* kn_bytes = reinterpret_cast<const uint8_t*>(p.kn);
    const uint8_t* kr_bytes = reinterpret_cast<const uint8_t*>(p.kr);
    const uint8_t* sc_bytes = reinterpret_cast<const uint8_t*>(p.kn_scales);
    struct RowRegs {
      uint4 d[10];
      float4 sc;
      bool valid;
    };
    auto issue_loads = [&](RowRegs& r, long long phys) {
      r.valid = phys >= 0;
      if (!r.valid) return;
      if (p.debug & 8) {  // experiment: no global loads
#pragma unroll
        for (int m = 0; m < 10; ++m) r.d[m] = make_uint4(0x01010101u * q, 2, 3, 4);
        r.sc = make_float4(1.f, 1.f, 1.f, 1.f);
        return;
      }
      if (p.packed) {
        const uint8_t* src = kn_bytes + phys * 656;
#pragma unroll
        for (int m = 0; m < 10; ++m) r.d[m] = __ldg(reinterpret_cast<const uint4*>(src + (q + 4 * m) * 16));
        r.sc = __ldg(reinterpret_cast<const float4*>(src + 640));
      } else {
#pragma unroll
        for (int m = 0; m < 8; ++m) r.d[m] = __ldg(reinterpret_cast<const uint4*>(kn_bytes + phys * 512 + (q + 4 * m) * 16));
        r.d[8] = __ldg(reinterpret_cast<const uint4*>(kr_bytes + phys * 128 + q * 16));
        r.d[9] = __ldg(reinterpret_cast<const uint4*>(kr_bytes + phys * 128 + (q + 4) * 16));
        r.sc = __ldg(reinterpret_cast<const float4*>(sc_bytes + phys * 16));
      }
    };
    uint8_t* kbuf = k_ptr + grp * kKBufBytes + row * 128;
    const int sw = row & 7;
    auto convert_store = [&](const RowRegs& r) {
      if (r.valid) {
        const float scl[4] = {r.sc.x, r.sc.y, r.sc.z, r.sc.w};
#pragma unroll
        for (int m = 0; m < 8; ++m) {  // int8 unit q + 4m: chunk m, bf16 units 2q and 2q+1, scale m / 2
          uint4 o0, o1;
          if (p.debug & 32) { o0 = r.d[m]; o1 = r.d[m]; } else
          dequant16(r.d[m], scl[m >> 1], o0, o1);
          *reinterpret_cast<uint4*>(kbuf + m * kKChunkBytes + (((2 * q) ^ sw) << 4)) = o0;
          *reinterpret_cast<uint4*>(kbuf + m * kKChunkBytes + (((2 * q + 1) ^ sw) << 4)) = o1;
        }
        *reinterpret_cast<uint4*>(kbuf + 8 * kKChunkBytes + ((q ^ sw) << 4)) = r.d[8];
        *reinterpret_cast<uint4*>(kbuf + 8 * kKChunkBytes + (((q + 4) ^ sw) << 4)) = r.d[9];
      } else {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          *reinterpret_cast<uint4*>(kbuf + m * kKChunkBytes + (((2 * q) ^ sw) << 4)) = z;
          *reinterpret_cast<uint4*>(kbuf + m * kKChunkBytes + (((2 * q + 1) ^ sw) << 4)) = z;
        }
        *reinterpret_cast<uint4*>(kbuf + 8 * kKChunkBytes + ((q ^ sw) << 4)) = z;
        *reinterpret_cast<uint4*>(kbuf + 8 * kKChunkBytes + (((q + 4) ^ sw) << 4)) = z;
      }
      if (q == 0) ctl->k_valid[grp][row] = r.valid ? 1 : 0;
    };
    bool ok = true;
    // i-th tile of the group: wait for the buffer (P.V of the group's previous tile), convert, publish
    auto finish_tile = [&](int i, const RowRegs& r) -> bool {
      if (i >= 1) {
        bool w = mbar_wait(smem_u32(&ctl->pv_done[grp]), (i - 1) & 1);
        w = __all_sync(0xffffffffu, w);
        if (!w) return false;
      }
      convert_store(r);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->k_full[grp]));
      return true;
    };
    if (n_mine > 0) {
      RowRegs ra, rb;
      long long phys_next = tc_physical_row(p, bi, load_idx(1));
      int idx_n2 = load_idx(2);
      issue_loads(ra, tc_physical_row(p, bi, load_idx(0)));
      for (int i = 0; i < n_mine && ok; i += 2) {
        // tile i lives in ra; start tile i+1 into rb, then finish tile i
        if (i + 1 < n_mine) issue_loads(rb, phys_next);
        long long phys_n2 = tc_physical_row(p, bi, idx_n2);
        int idx_n3 = load_idx(i + 3);
        ok = finish_tile(i, ra);
        if (!ok || i + 1 >= n_mine) break;
        // tile i+1 lives in rb; start tile i+2 into ra, then finish tile i+1
        if (i + 2 < n_mine) issue_loads(ra, phys_n2);
        phys_next = tc_physical_row(p, bi, idx_n3);
        idx_n2 = load_idx(i + 4);
        ok = finish_tile(i + 1, rb);
      }
    }
    if (!ok && lane == 0) {
      ctl->abort = 1;
      set_status(p.status, PTO_ST_WAIT_EXPIRED, blockIdx.x, 32);
    }
  }

  // ---- teardown -----------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemColsTc);
  }
}

}  // namespace

cudaError_t launch_sfa_tc(const SfaParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(sfa_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kTcSmemBytes));
  if (e != cudaSuccess) return e;
  const int t = p.b * p.s1;
  sfa_tc_kernel<<<t * 2 * p.n_split, kTcThreads, kTcSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pto
