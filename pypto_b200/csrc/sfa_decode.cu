// Sparse MLA attention over the rows selected by the indexer (decode and prefill entries).
//
// Per query token (b, i):  n = clamp(S_b - s1 + 1 + i, 0, topk); for the first n indices
//   r_j = block_table[b, idx_j / bs] * bs + idx_j % bs
//   kn  = bf16( fp32(int8 latent[r_j]) * scale[r_j, c / 128] ),   K = [kn | rope[r_j]]  (576 wide)
//   s   = fp32(q . K^T) * softmax_scale;  P = softmax(s);  O = bf16( P . kn )           (512 wide)
// (reference: examples/models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:45-207; golden
// deepseekv32_sparse_flash_attention_quant.py:169-254; packed rows
// sparse_attention_antiquant_impl.py:45-243.)
//
// Kernel: one CTA per (token, block of 64 heads, split of the selected rows). Tiles of 64 rows are
// gathered with 16-byte cp.async into a staging buffer (raw 656-byte rows: 512 int8 | 64 bf16 |
// 4 f32, the same layout as the packed cache), dequantised into a bf16 K tile in shared memory, and
// consumed by bf16 mma.sync (m16n8k16, fp32 accumulate) for both q.K^T and P.V with an online
// softmax: P = bf16(exp(s - running max)) un-normalised, (m, l, O) in fp32, one rounding of P and
// one of the output. Splits are merged by `sfa_combine_kernel`.

#include "common.cuh"

namespace pto {

namespace {

constexpr int kHB = 64;        // heads per CTA
constexpr int kTile = 64;      // selected rows per tile
constexpr int kD = 576;        // q/k width
constexpr int kDV = 512;       // v width
constexpr int kSfaThreads = 256;
constexpr int kQStride = kD * 2 + 16;   // bytes, 73 * 16
constexpr int kKStride = kD * 2 + 16;
constexpr int kPStride = kTile * 2 + 16;  // 9 * 16
constexpr int kRawRow = 656;            // 41 * 16
constexpr int kChunksPerRow = kRawRow / 16;

struct SfaSmem {
  uint8_t q[kHB * kQStride];
  uint8_t k[kTile * kKStride];
  uint8_t raw[kTile * kRawRow];
  uint8_t p[kHB * kPStride];
  float red[4][kHB];
  long long rows[2][kTile];
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// physical cache row of selected entry j of this token, or -1 when it must be skipped
__device__ __forceinline__ long long physical_row(const SfaParams& p, int bi, const int32_t* idx_row, int j, int end) {
  if (j >= end) return -1;
  const int idx = idx_row[j];
  if (idx < 0) return -1;
  const int blk = idx / p.block_size;
  if (blk >= p.max_blocks) {
    set_status(p.status, PTO_ST_BAD_PAGE, idx, 10);
    return -1;
  }
  const int phys = p.block_table[static_cast<int64_t>(bi) * p.max_blocks + blk];
  const long long r = static_cast<long long>(phys) * p.block_size + idx % p.block_size;
  if (phys < 0 || r >= p.n_rows) {
    set_status(p.status, PTO_ST_BAD_PAGE, phys, 11);
    return -1;
  }
  return r;
}

__device__ __forceinline__ void issue_gather(const SfaParams& p, SfaSmem* sm, const long long* rows) {
  const uint32_t raw_base = smem_u32(sm->raw);
  for (int g = threadIdx.x; g < kTile * kChunksPerRow; g += kSfaThreads) {
    const int lr = g / kChunksPerRow;
    const int c = g - lr * kChunksPerRow;
    const long long r = rows[lr];
    if (r < 0) continue;
    const uint8_t* src;
    if (p.packed) {
      src = reinterpret_cast<const uint8_t*>(p.kn) + r * kRawRow + c * 16;
    } else if (c < 32) {
      src = reinterpret_cast<const uint8_t*>(p.kn) + r * 512 + c * 16;
    } else if (c < 40) {
      src = reinterpret_cast<const uint8_t*>(p.kr) + r * 128 + (c - 32) * 16;
    } else {
      src = reinterpret_cast<const uint8_t*>(p.kn_scales) + r * 16;
    }
    cp_async16(raw_base + lr * kRawRow + c * 16, src);
  }
  cp_async_commit();
}

// raw staging rows -> bf16 K tile. Thread (lr = tid % 64, qd = tid / 64) converts dims
// [qd*128, qd*128+128) of the latent part (one scale) and 16 of the 64 rope values.
__device__ __forceinline__ void convert_tile(SfaSmem* sm, const long long* rows) {
  const int lr = threadIdx.x & (kTile - 1);
  const int qd = threadIdx.x >> 6;
  uint8_t* kdst = sm->k + lr * kKStride;
  if (rows[lr] < 0) {
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(kdst + qd * 256 + c * 16) = z;
    *reinterpret_cast<uint4*>(kdst + 1024 + qd * 32) = z;
    *reinterpret_cast<uint4*>(kdst + 1024 + qd * 32 + 16) = z;
    return;
  }
  const uint8_t* src = sm->raw + lr * kRawRow;
  const float scale = *reinterpret_cast<const float*>(src + 640 + qd * 4);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + qd * 128 + c * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float f0 = static_cast<float>(static_cast<int8_t>(w[e] & 0xff)) * scale;
      const float f1 = static_cast<float>(static_cast<int8_t>((w[e] >> 8) & 0xff)) * scale;
      const float f2 = static_cast<float>(static_cast<int8_t>((w[e] >> 16) & 0xff)) * scale;
      const float f3 = static_cast<float>(static_cast<int8_t>((w[e] >> 24) & 0xff)) * scale;
      o[2 * e] = pack_bf16x2(f0, f1);
      o[2 * e + 1] = pack_bf16x2(f2, f3);
    }
    *reinterpret_cast<uint4*>(kdst + qd * 256 + c * 32) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(kdst + qd * 256 + c * 32 + 16) = make_uint4(o[4], o[5], o[6], o[7]);
  }
  *reinterpret_cast<uint4*>(kdst + 1024 + qd * 32) = *reinterpret_cast<const uint4*>(src + 512 + qd * 32);
  *reinterpret_cast<uint4*>(kdst + 1024 + qd * 32 + 16) = *reinterpret_cast<const uint4*>(src + 512 + qd * 32 + 16);
}

__global__ void __launch_bounds__(kSfaThreads, 1)
sfa_mma_kernel(SfaParams p) {
  extern __shared__ __align__(16) uint8_t sfa_smem_raw[];
  SfaSmem* sm = reinterpret_cast<SfaSmem*>(sfa_smem_raw);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int n_hb = (p.nq + kHB - 1) / kHB;
  int bid = blockIdx.x;
  const int sp = bid % p.n_split;
  bid /= p.n_split;
  const int hb = bid % n_hb;
  const int ti = bid / n_hb;
  const int bi = ti / p.s1;
  const int si = ti % p.s1;

  int n = p.act_seq[bi] - p.s1 + 1 + si;
  n = max(0, min(n, p.topk_k));
  const int tiles_total = (n + kTile - 1) / kTile;
  const int tiles_per_split = (tiles_total + p.n_split - 1) / p.n_split;
  const int begin = min(n, sp * tiles_per_split * kTile);
  const int end = min(n, (sp + 1) * tiles_per_split * kTile);
  const int ntiles = (end - begin + kTile - 1) / kTile;
  const int32_t* idx_row = p.topk + static_cast<int64_t>(ti) * p.topk_k;

  const int hh = warp >> 2;  // head half (32 heads)
  const int wq = warp & 3;   // column quarter for q.K^T, dim quarter for P.V
  const int r0 = lane >> 2;
  const int cpair = (lane & 3) * 2;

  // ---- empty range -----------------------------------------------------------------------------
  if (ntiles == 0) {
    if (p.n_split == 1) {
      for (int e = tid; e < kHB * (kDV / 8); e += kSfaThreads) {
        const int row = e / (kDV / 8), c = e % (kDV / 8);
        const int head = hb * kHB + row;
        if (head < p.nq) {
          *reinterpret_cast<uint4*>(p.out + (static_cast<int64_t>(ti) * p.nq_total + p.head_begin + head) * kDV + c * 8) =
              make_uint4(0, 0, 0, 0);
        }
      }
    } else {
      for (int row = tid; row < kHB; row += kSfaThreads) {
        const int head = hb * kHB + row;
        if (head < p.nq) {
          float* ml = p.part_ml + ((static_cast<int64_t>(ti) * p.n_split + sp) * p.nq + head) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        }
      }
    }
    return;
  }

  // ---- prologue: rows of tiles 0 and 1, gather of tile 0, Q tile --------------------------------
  if (tid < kTile) sm->rows[0][tid] = physical_row(p, bi, idx_row, begin + tid, end);
  else if (tid < 2 * kTile) sm->rows[1][tid - kTile] = physical_row(p, bi, idx_row, begin + kTile + (tid - kTile), end);
  for (int e = tid; e < kHB * (kD / 8); e += kSfaThreads) {
    const int row = e / (kD / 8), c = e % (kD / 8);
    const int head = hb * kHB + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head < p.nq) {
      const int64_t qrow = static_cast<int64_t>(ti) * p.nq_total + p.head_begin + head;
      v = (c < 64) ? *reinterpret_cast<const uint4*>(p.q_nope + qrow * kDV + c * 8)
                   : *reinterpret_cast<const uint4*>(p.q_rope + qrow * 64 + (c - 64) * 8);
    }
    *reinterpret_cast<uint4*>(sm->q + row * kQStride + c * 16) = v;
  }
  __syncthreads();
  issue_gather(p, sm, sm->rows[0]);

  float o[2][16][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 16; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[a][b][c] = 0.f;
  float m_run[4], l_run[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
  }

  const uint32_t q_base = smem_u32(sm->q);
  const uint32_t k_base = smem_u32(sm->k);
  const uint32_t p_base = smem_u32(sm->p);

  for (int jt = 0; jt < ntiles; ++jt) {
    const long long* rows_cur = sm->rows[jt & 1];
    cp_async_wait_all();
    __syncthreads();  // staging of tile jt landed; previous tile's K/P no longer read
    convert_tile(sm, rows_cur);
    __syncthreads();  // K tile ready, staging free
    if (jt + 1 < ntiles) issue_gather(p, sm, sm->rows[(jt + 1) & 1]);

    // ---- S = Q . K^T : warp tile 32 heads x 16 rows --------------------------------------------
    float s[2][2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[a][b][c] = 0.f;
    {
      const uint32_t a_addr0 = q_base + (hh * 32 + (lane & 15)) * kQStride + (lane >> 4) * 16;
      const uint32_t b_addr = k_base + (wq * 16 + (lane & 7) + ((lane >> 4) << 3)) * kKStride + ((lane >> 3) & 1) * 16;
#pragma unroll 4
      for (int kk = 0; kk < kD / 16; ++kk) {
        uint32_t a0[4], a1[4], b[4];
        ldsm_x4(a_addr0 + kk * 32, a0[0], a0[1], a0[2], a0[3]);
        ldsm_x4(a_addr0 + 16 * kQStride + kk * 32, a1[0], a1[1], a1[2], a1[3]);
        ldsm_x4(b_addr + kk * 32, b[0], b[1], b[2], b[3]);
        mma_bf16(s[0][0], a0, b[0], b[1]);
        mma_bf16(s[0][1], a0, b[2], b[3]);
        mma_bf16(s[1][0], a1, b[0], b[1]);
        mma_bf16(s[1][1], a1, b[2], b[3]);
      }
    }
    // ---- scale, mask, row max --------------------------------------------------------------------
    float mt_part[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) mt_part[r] = -INFINITY;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int col = wq * 16 + b * 8 + cpair + (c & 1);
          const bool valid = rows_cur[col] >= 0;
          const float v = valid ? s[a][b][c] * p.scale_log2 : -INFINITY;
          s[a][b][c] = v;
          const int r = a * 2 + (c >> 1);
          mt_part[r] = fmaxf(mt_part[r], v);
        }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      mt_part[r] = fmaxf(mt_part[r], __shfl_xor_sync(0xffffffffu, mt_part[r], 1));
      mt_part[r] = fmaxf(mt_part[r], __shfl_xor_sync(0xffffffffu, mt_part[r], 2));
    }
    if ((lane & 3) == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r) sm->red[wq][hh * 32 + (r >> 1) * 16 + (r & 1) * 8 + r0] = mt_part[r];
    }
    __syncthreads();
    float alpha[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = hh * 32 + (r >> 1) * 16 + (r & 1) * 8 + r0;
      const float mt = fmaxf(fmaxf(sm->red[0][row], sm->red[1][row]), fmaxf(sm->red[2][row], sm->red[3][row]));
      const float m_new = fmaxf(m_run[r], mt);
      alpha[r] = (m_new == -INFINITY) ? 1.f : ex2(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
    // ---- P = exp2(s - m), bf16, to shared; partial row sums in fp32 ------------------------------
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int rA = a * 2, rB = a * 2 + 1;
        const float mA = (m_run[rA] == -INFINITY) ? 0.f : m_run[rA];
        const float mB = (m_run[rB] == -INFINITY) ? 0.f : m_run[rB];
        const float p0 = ex2(s[a][b][0] - mA), p1 = ex2(s[a][b][1] - mA);
        const float p2 = ex2(s[a][b][2] - mB), p3 = ex2(s[a][b][3] - mB);
        l_run[rA] += p0 + p1;
        l_run[rB] += p2 + p3;
        const int col = wq * 16 + b * 8 + cpair;
        const int rowA = hh * 32 + a * 16 + r0;
        *reinterpret_cast<uint32_t*>(sm->p + rowA * kPStride + col * 2) = pack_bf16x2(p0, p1);
        *reinterpret_cast<uint32_t*>(sm->p + (rowA + 8) * kPStride + col * 2) = pack_bf16x2(p2, p3);
      }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 16; ++b) {
        o[a][b][0] *= alpha[a * 2];
        o[a][b][1] *= alpha[a * 2];
        o[a][b][2] *= alpha[a * 2 + 1];
        o[a][b][3] *= alpha[a * 2 + 1];
      }
    __syncthreads();  // P tile complete; nobody reads this tile's row list any more
    if (jt + 2 < ntiles && tid < kTile) {
      // rows of tile jt+2 reuse the buffer of tile jt; consumed after the barriers of iteration jt+1
      sm->rows[jt & 1][tid] = physical_row(p, bi, idx_row, begin + (jt + 2) * kTile + tid, end);
    }

    // ---- O += P . V : warp tile 32 heads x 128 dims ---------------------------------------------
    {
      const uint32_t a_addr0 = p_base + (hh * 32 + (lane & 15)) * kPStride + (lane >> 4) * 16;
      const uint32_t v_addr = k_base + ((lane & 7) + ((lane >> 3) & 1) * 8) * kKStride + (wq * 128 + (lane >> 4) * 8) * 2;
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk) {
        uint32_t a0[4], a1[4];
        ldsm_x4(a_addr0 + kk * 32, a0[0], a0[1], a0[2], a0[3]);
        ldsm_x4(a_addr0 + 16 * kPStride + kk * 32, a1[0], a1[1], a1[2], a1[3]);
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t b[4];
          ldsm_x4_trans(v_addr + kk * 16 * kKStride + np * 32, b[0], b[1], b[2], b[3]);
          mma_bf16(o[0][2 * np], a0, b[0], b[1]);
          mma_bf16(o[0][2 * np + 1], a0, b[2], b[3]);
          mma_bf16(o[1][2 * np], a1, b[0], b[1]);
          mma_bf16(o[1][2 * np + 1], a1, b[2], b[3]);
        }
      }
    }
  }

  // ---- row sums over the quad and the four column-quarter warps ------------------------------------
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if ((lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 4; ++r) sm->red[wq][hh * 32 + (r >> 1) * 16 + (r & 1) * 8 + r0] = l_run[r];
  }
  __syncthreads();
  float l_tot[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = hh * 32 + (r >> 1) * 16 + (r & 1) * 8 + r0;
    l_tot[r] = (sm->red[0][row] + sm->red[1][row]) + (sm->red[2][row] + sm->red[3][row]);
  }

  // ---- write ------------------------------------------------------------------------------------------
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = a * 2 + half;
      const int row = hh * 32 + a * 16 + half * 8 + r0;
      const int head = hb * kHB + row;
      if (head >= p.nq) continue;
      if (p.n_split == 1) {
        const float inv = l_tot[r] > 0.f ? 1.f / l_tot[r] : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(ti) * p.nq_total + p.head_begin + head) * kDV + wq * 128 + cpair;
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          *reinterpret_cast<uint32_t*>(dst + b * 8) = pack_bf16x2(o[a][b][half * 2] * inv, o[a][b][half * 2 + 1] * inv);
        }
      } else {
        const int64_t prow = (static_cast<int64_t>(ti) * p.n_split + sp) * p.nq + head;
        float* dst = p.part_o + prow * kDV + wq * 128 + cpair;
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          *reinterpret_cast<float2*>(dst + b * 8) = make_float2(o[a][b][half * 2], o[a][b][half * 2 + 1]);
        }
        if (wq == 0 && (lane & 3) == 0) {
          p.part_ml[prow * 2] = m_run[r];
          p.part_ml[prow * 2 + 1] = l_tot[r];
        }
      }
    }
}

// Merge of the split partials: O = sum_i O_i 2^(m_i - m) / sum_i l_i 2^(m_i - m), rounded once to bf16.
// One CTA per (token, head). The splits' maxima and sums are fetched by one lane each and reduced by shuffles,
// the output rows of up to eight splits are requested together: two trips to memory instead of one per split.
constexpr int kMaxSplit = 32;
__global__ void __launch_bounds__(128)
sfa_combine_kernel(SfaParams p) {
  __shared__ float wgt[kMaxSplit];
  __shared__ float inv_l;
  pdl_wait();  // launched with programmatic serialization behind the kernel that writes the partials
  const int64_t th = blockIdx.x;  // token * nq + head
  const int ti = static_cast<int>(th / p.nq);
  const int head = static_cast<int>(th % p.nq);
  const int tid = threadIdx.x;
  const int64_t prow0 = static_cast<int64_t>(ti) * p.n_split * p.nq + head;  // row of split 0; splits are nq rows apart
  if (tid < 32) {
    float mi = -INFINITY, li = 0.f;
    if (tid < p.n_split) {
      const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + (prow0 + static_cast<int64_t>(tid) * p.nq) * 2);
      mi = ml.x;
      li = ml.y;
    }
    float m = mi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float w = (li > 0.f && m != -INFINITY) ? ex2(mi - m) : 0.f;
    float l = li * w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    wgt[tid] = w;
    if (tid == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < p.n_split; s0 += 8) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sp = s0 + u;
      v[u] = (sp < p.n_split && wgt[sp] != 0.f)
                 ? *reinterpret_cast<const float4*>(p.part_o + (prow0 + static_cast<int64_t>(sp) * p.nq) * kDV + tid * 4)
                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float w = s0 + u < p.n_split ? wgt[s0 + u] : 0.f;
      acc.x += v[u].x * w;
      acc.y += v[u].y * w;
      acc.z += v[u].z * w;
      acc.w += v[u].w * w;
    }
  }
  const float inv = inv_l;
  __nv_bfloat16* dst = p.out + (static_cast<int64_t>(ti) * p.nq_total + p.head_begin + head) * kDV + tid * 4;
  uint2 pk;
  pk.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  pk.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(dst) = pk;
}

}  // namespace

cudaError_t launch_sfa(const SfaParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(sfa_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(SfaSmem)));
  if (e != cudaSuccess) return e;
  const int t = p.b * p.s1;
  const int n_hb = (p.nq + kHB - 1) / kHB;
  if (p.nq == 128) {
    // all 128 heads of a token: the tcgen05 kernel on a pair of SMs that shares every MMA (sfa_pair.cu; int8, packed
    // and bf16 caches); narrower head slices use mma.sync below
    e = launch_sfa_pair(p, stream);
  } else {
    count_launch();
    sfa_mma_kernel<<<t * n_hb * p.n_split, kSfaThreads, sizeof(SfaSmem), stream>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return e;
  if (p.n_split > 1) {
    if (p.n_split > kMaxSplit) return cudaErrorInvalidValue;
    count_launch();
    // may be scheduled while the attention kernel drains; its first instruction waits for that grid
    e = launch_maybe_pdl(sfa_combine_kernel, dim3(static_cast<unsigned>(t * p.nq)), dim3(128), 0, stream, true, p);
  }
  return e;
}

}  // namespace pto
