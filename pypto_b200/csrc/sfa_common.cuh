// Helpers shared by the tcgen05 sparse-attention kernels: descriptors for the 64-byte-swizzled and
// MN-major operands, TMEM store, int8 -> bf16 dequantisation, paged row lookup.
#pragma once
#include <climits>

#include "common.cuh"

namespace pto {

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint64_t desc_kmajor_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;  // 8 rows * 64 B
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;  // SWIZZLE_64B
  return d;
}

// MN-major operand, 128-byte swizzle: 64 elements (128 B) contiguous along MN, 8 K-rows per 1024-byte
// atom; `lbo` = bytes between 64-element groups along MN, `sbo` = bytes between 8-row groups along K
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// 16 int8 -> 16 bf16 of (value * scale): byte b^0x80 placed in the mantissa of 2^23 gives
// 2^23 + 128 + x exactly; subtracting 8388736 leaves x; one fp32 multiply and one rounding to bf16,
// i.e. bf16(fp32(x) * scale) as the golden computes it.
__device__ __forceinline__ void dequant16(const uint4 v, const float scale, uint4& o0, uint4& o1) {
  const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
  uint32_t o[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float f0 = (__uint_as_float(__byte_perm(w[e], 0x4B000000u, 0x7540)) - 8388736.0f) * scale;
    const float f1 = (__uint_as_float(__byte_perm(w[e], 0x4B000000u, 0x7541)) - 8388736.0f) * scale;
    const float f2 = (__uint_as_float(__byte_perm(w[e], 0x4B000000u, 0x7542)) - 8388736.0f) * scale;
    const float f3 = (__uint_as_float(__byte_perm(w[e], 0x4B000000u, 0x7543)) - 8388736.0f) * scale;
    o[2 * e] = pack_bf16x2(f0, f1);
    o[2 * e + 1] = pack_bf16x2(f2, f3);
  }
  o0 = make_uint4(o[0], o[1], o[2], o[3]);
  o1 = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ long long tc_physical_row(const SfaParams& p, int bi, int idx) {
  if (idx < 0) return -1;
  const int blk = idx / p.block_size;
  if (blk >= p.max_blocks) {
    set_status(p.status, PTO_ST_BAD_PAGE, idx, 20);
    return -1;
  }
  const int phys = p.block_table[static_cast<int64_t>(bi) * p.max_blocks + blk];
  const long long r = static_cast<long long>(phys) * p.block_size + idx % p.block_size;
  if (phys < 0 || r >= p.n_rows) {
    set_status(p.status, PTO_ST_BAD_PAGE, phys, 21);
    return -1;
  }
  return r;
}

// tcgen05.mma with the A operand in tensor memory (row m of A = TMEM lane m, 32-bit column c holds the
// K elements 2c and 2c+1 of a 16-bit type), B in shared memory.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory accesses by 32-bit shared-window address: a generic pointer costs two registers and an
// address conversion per access, and the softmax and producer loops have no register to spare.
__device__ __forceinline__ float4 lds_v4f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds_v4u(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts_v4f(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void sts_v4u(uint32_t a, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ void sts_u8(uint32_t a, uint32_t v) { asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }

// Read-only global loads that stay where they are written. The compiler treats `__ldg` as a load of
// invariant memory and is free to sink it to its first use, across waits and barriers, which turns a
// software prefetch into a load-then-stall; volatile asm keeps the issue point. The gathers do not
// allocate in L1: beside ~220 KB of shared memory the L1 is a few KB, and it is needed for the stack
// (a spilled register or a by-value argument re-read in a loop otherwise costs a trip to L2).
__device__ __forceinline__ uint4 ldg_pinned_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float2 ldg_pinned_v2f(const void* p) {
  float2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ int ldg_pinned_i32(const void* p) {
  int v;
  asm volatile("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// 16 bytes global -> shared without a register in between (L2 only); `src_bytes` 0 writes zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}

// The same lookup in two steps, so that a caller can fetch the block-table entry a tile ahead and
// only branch on it once it has arrived.
constexpr int kTableSkip = INT_MIN;  // nothing to fetch: padding index, or an index already reported
__device__ __forceinline__ int tc_table_entry(const SfaParams& p, int bi, int idx) {
  if (idx < 0) return kTableSkip;
  const int blk = idx / p.block_size;
  if (blk >= p.max_blocks) {
    set_status(p.status, PTO_ST_BAD_PAGE, idx, 20);
    return kTableSkip;
  }
  return ldg_pinned_i32(p.block_table + static_cast<int64_t>(bi) * p.max_blocks + blk);
}
__device__ __forceinline__ long long tc_row_from_entry(const SfaParams& p, int idx, int entry) {
  if (entry == kTableSkip) return -1;
  const long long r = static_cast<long long>(entry) * p.block_size + idx % p.block_size;
  if (entry < 0 || r >= p.n_rows) {
    set_status(p.status, PTO_ST_BAD_PAGE, entry, 21);
    return -1;
  }
  return r;
}

}  // namespace pto
