// MLA + lightning-indexer prolog: everything between the projections (the weight-streaming products of
// prolog_gemm.cu and prolog_sgemm.cu, issued by the C entry point) — RMSNorm / LayerNorm, rope, Hadamard rotation, dynamic int8 quantisation, dequantisation of
// the int32 products, and the scatter of the new token's rows into the paged caches.
//
// Arithmetic follows the reference's torch goldens step by step, including every intermediate rounding to
// bf16 (examples/models/deepseek_v32_exp/deepseekv32_mla_indexer_prolog_quant.py: `quant` :35-53,
// `rms_norm` :56-73, `apply_rotary_pos_emb_v2` :106-131, `single_rope` :140-152, `layer_norm` :155-162,
// `mla_prolog_quant_v32_compute` :409-541, `indexer_prolog` :544-614). Products and sums that the goldens
// round separately are kept separate here (`__fmul_rn` / `__fadd_rn`, no contraction into FMAs).
#include "common.cuh"

namespace pto {

namespace {

constexpr int kHeads = 128;     // attention heads
constexpr int kNope = 128;      // per-head query width before absorption
constexpr int kRope = 64;       // rope width (attention and indexer)
constexpr int kLora = 512;      // latent KV width
constexpr int kIdxHeads = 64;   // indexer heads
constexpr int kIdxDim = 128;    // indexer head width
constexpr int kQHead = kNope + kRope;
constexpr int kPackedRow = kLora + 2 * kRope + 16;  // 656 bytes: int8 latent | bf16 rope | 4 fp32 scales

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float ld_bf16(const __nv_bfloat16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions over up to 32 warps; `red` holds 32 floats. The result is returned to every thread.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // `red` may still be read from a previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;  // maxima of absolute values: 0 is neutral
  return warp_max(r);
}

// round(x * 127/max) -> int32 -> fp16 -> trunc -> int8: integers up to 127 are exact in fp16, so the chain
// after the round-half-even is the identity
__device__ __forceinline__ int8_t quant_one(float v, float scale_q) {
  return static_cast<int8_t>(__float2int_rn(__fmul_rn(v, scale_q)));
}

// ---- query down-projection: bf16 rounding, RMSNorm, then per-token int8 (kQuant) or the bf16 row itself ----
// grid = tokens, 512 threads, dynamic shared memory = q_lora floats (16-byte aligned rows: ld and q_lora multiples of 4)
template <bool kQuant>
__global__ void __launch_bounds__(512)
prolog_qnorm_kernel(const float* __restrict__ qa, int ld, int n_split, long long split_stride,
                    const __nv_bfloat16* __restrict__ gamma, int q_lora, float eps, int8_t* __restrict__ q_norm,
                    float* __restrict__ q_norm_scale, __nv_bfloat16* __restrict__ q_norm_bf16) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  pdl_wait();  // the projection before it may still be running when this grid is scheduled
  if (threadIdx.x == 0) pdl_trigger();
  const int ti = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(qa + static_cast<int64_t>(ti) * ld);
  float4* row4 = reinterpret_cast<float4*>(row);
  const int groups = q_lora >> 2;  // four values per step: at q_lora = 1536 every thread makes one trip to memory
  const float inv_n = 1.0f / static_cast<float>(q_lora);
  float ss = 0.f;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float4 part[8];  // K-split partials of the projection (n_split <= 8): requested together, added in split order
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) {
      part[sp] = sp < n_split ? __ldg(src + g + sp * (split_stride >> 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 v = part[0];
#pragma unroll
    for (int sp = 1; sp < 8; ++sp) {
      if (sp < n_split) {
        v.x = __fadd_rn(v.x, part[sp].x);
        v.y = __fadd_rn(v.y, part[sp].y);
        v.z = __fadd_rn(v.z, part[sp].z);
        v.w = __fadd_rn(v.w, part[sp].w);
      }
    }
    v.x = bf16_round(v.x);
    v.y = bf16_round(v.y);
    v.z = bf16_round(v.z);
    v.w = bf16_round(v.w);
    row4[g] = v;
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v.x, v.x), inv_n));
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v.y, v.y), inv_n));
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v.z, v.z), inv_n));
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v.w, v.w), inv_n));
  }
  const float rms = sqrtf(block_sum(ss, red) + eps);
  float amax = 0.f;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float4 v = row4[g];
    const uint2 gm = __ldg(reinterpret_cast<const uint2*>(gamma) + g);  // four bf16
    v.x = bf16_round(__fmul_rn(__fdiv_rn(v.x, rms), __uint_as_float(gm.x << 16)));
    v.y = bf16_round(__fmul_rn(__fdiv_rn(v.y, rms), __uint_as_float(gm.x & 0xffff0000u)));
    v.z = bf16_round(__fmul_rn(__fdiv_rn(v.z, rms), __uint_as_float(gm.y << 16)));
    v.w = bf16_round(__fmul_rn(__fdiv_rn(v.w, rms), __uint_as_float(gm.y & 0xffff0000u)));
    if constexpr (kQuant) {
      row4[g] = v;
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    } else {
      uint2 o;  // the values are bf16 already: their upper halves are the row
      o.x = (__float_as_uint(v.x) >> 16) | (__float_as_uint(v.y) & 0xffff0000u);
      o.y = (__float_as_uint(v.z) >> 16) | (__float_as_uint(v.w) & 0xffff0000u);
      reinterpret_cast<uint2*>(q_norm_bf16 + static_cast<int64_t>(ti) * q_lora)[g] = o;
    }
  }
  if constexpr (!kQuant) return;
  amax = block_max(amax, red);
  const float scale_q = __fdiv_rn(127.0f, amax);
  char4* dst = reinterpret_cast<char4*>(q_norm + static_cast<int64_t>(ti) * q_lora);
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    const float4 v = row4[g];
    char4 q;
    q.x = quant_one(v.x, scale_q);
    q.y = quant_one(v.y, scale_q);
    q.z = quant_one(v.z, scale_q);
    q.w = quant_one(v.w, scale_q);
    dst[g] = q;
  }
  if (threadIdx.x == 0) q_norm_scale[ti] = __fdiv_rn(1.0f, scale_q);
}

// ---- query up-projection: int32 -> bf16, rope of the 64-wide tail ----------------------------------------
// grid = (16 head groups, tokens), block = 256: eight heads (1536 values) per block
constexpr int kQbHeadsPerBlock = 8;
__global__ void __launch_bounds__(256)
prolog_qb_dequant_rope_kernel(const int32_t* __restrict__ qb_i32, const float* __restrict__ q_norm_scale,
                              const float* __restrict__ w_scale, const __nv_bfloat16* __restrict__ cos,
                              const __nv_bfloat16* __restrict__ sin, __nv_bfloat16* __restrict__ q_b,
                              __nv_bfloat16* __restrict__ q_rope) {
  __shared__ float pe[kQbHeadsPerBlock][kRope];
  pdl_wait();
  if (threadIdx.x == 0) pdl_trigger();
  const int hg = blockIdx.x, ti = blockIdx.y;
  const float rs = q_norm_scale[ti];
  const int64_t col0 = static_cast<int64_t>(hg) * kQbHeadsPerBlock * kQHead;
  const int64_t row0 = static_cast<int64_t>(ti) * kHeads * kQHead;
#pragma unroll
  for (int u = 0; u < kQbHeadsPerBlock * kQHead / 256; ++u) {
    const int e = u * 256 + threadIdx.x;  // element of the block's 8 x 192 slice
    const int64_t col = col0 + e;
    const float v = bf16_round(__fmul_rn(__fmul_rn(static_cast<float>(qb_i32[row0 + col]), rs), w_scale[col]));
    q_b[row0 + col] = __float2bfloat16_rn(v);
    const int hh = e / kQHead, c = e % kQHead;
    if (c >= kNope) pe[hh][c - kNope] = v;
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < kQbHeadsPerBlock * kRope / 256; ++u) {
    const int e = u * 256 + threadIdx.x;
    const int hh = e / kRope, c = e % kRope;
    // de-interleaved layout: first half = even dims, second half = odd dims; rotate_half = (-second, first)
    const int j = c & 31;
    const float even = pe[hh][2 * j], odd = pe[hh][2 * j + 1];
    const float cs = ld_bf16(cos + ti * kRope + c), sn = ld_bf16(sin + ti * kRope + c);
    const float x = c < 32 ? even : odd;
    const float rot = c < 32 ? -odd : even;
    q_rope[(static_cast<int64_t>(ti) * kHeads + hg * kQbHeadsPerBlock + hh) * kRope + c] =
        __float2bfloat16_rn(__fadd_rn(__fmul_rn(x, cs), __fmul_rn(rot, sn)));
  }
}

// ---- per token: latent KV row, rope key, indexer key, indexer weights; scatter into the caches ---------
// grid = tokens, block = 128 (thread i owns latent dims 4i..4i+3: warp w = 128-wide quantisation tile w)
__global__ void __launch_bounds__(128)
prolog_kv_kernel(const float* __restrict__ kv, const float* __restrict__ ki, const float* __restrict__ wp, int ld,
                 int n_split, long long split_stride, const __nv_bfloat16* __restrict__ gamma_ckv, const __nv_bfloat16* __restrict__ cos,
                 const __nv_bfloat16* __restrict__ sin, const __nv_bfloat16* __restrict__ ln_gamma,
                 const __nv_bfloat16* __restrict__ ln_beta, const __nv_bfloat16* __restrict__ hadamard_k,
                 const int64_t* __restrict__ cache_index, int64_t cache_rows, float eps_ckv, float ln_eps,
                 int8_t* __restrict__ kv_cache, __nv_bfloat16* __restrict__ kr_cache, float* __restrict__ kv_scale_cache,
                 int8_t* __restrict__ idx_k_cache, __half* __restrict__ idx_k_scale_cache, __half* __restrict__ weights,
                 int8_t* __restrict__ packed_cache, int32_t* status) {
  __shared__ float red[32];
  __shared__ float pe[kRope];
  __shared__ float kvec[kIdxDim];
  __shared__ __align__(16) __nv_bfloat16 had[kIdxDim * kIdxDim];  // 32 KB, fetched while the norms are computed
  const int ti = blockIdx.x, i = threadIdx.x, lane = i & 31, warp = i >> 5;
  {
    const uint4* hsrc = reinterpret_cast<const uint4*>(hadamard_k);
    uint4* hdst = reinterpret_cast<uint4*>(had);
#pragma unroll 4
    for (int u = i; u < kIdxDim * kIdxDim / 8; u += 128) hdst[u] = __ldg(hsrc + u);
  }
  const int64_t row = cache_index[ti];
  const bool row_ok = row >= 0 && row < cache_rows;
  if (!row_ok && i == 0) set_status(status, PTO_ST_BAD_PAGE, static_cast<int>(row), 60);

  // a projection value: its K-split partials added in split order
  auto proj = [&](const float* p) {
    float part[8];  // all partials requested before the first is used (n_split <= 8)
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) part[sp] = sp < n_split ? __ldg(p + sp * split_stride) : 0.f;
    float a = part[0];
#pragma unroll
    for (int sp = 1; sp < 8; ++sp) {
      if (sp < n_split) a = __fadd_rn(a, part[sp]);
    }
    return a;
  };
  // latent part: bf16 rounding, RMSNorm, int8 per 128-wide tile
  const float* src = kv + static_cast<int64_t>(ti) * ld;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[e] = bf16_round(proj(src + 4 * i + e));
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v[e], v[e]), 1.0f / kLora));
  }
  const float rms = sqrtf(block_sum(ss, red) + eps_ckv);
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[e] = bf16_round(__fmul_rn(__fdiv_rn(v[e], rms), ld_bf16(gamma_ckv + 4 * i + e)));
    amax = fmaxf(amax, fabsf(v[e]));
  }
  amax = warp_max(amax);
  const float scale_q = __fdiv_rn(127.0f, amax);
  if (row_ok) {
    char4 q;
    q.x = quant_one(v[0], scale_q);
    q.y = quant_one(v[1], scale_q);
    q.z = quant_one(v[2], scale_q);
    q.w = quant_one(v[3], scale_q);
    *reinterpret_cast<char4*>(kv_cache + row * kLora + 4 * i) = q;
    const float dq = __fdiv_rn(1.0f, scale_q);
    if (lane == 0) kv_scale_cache[row * 4 + warp] = dq;
    if (packed_cache != nullptr) {  // the same row in the packed layout: 512 int8 | 64 bf16 | 4 f32
      *reinterpret_cast<char4*>(packed_cache + row * kPackedRow + 4 * i) = q;
      if (lane == 0) *reinterpret_cast<float*>(packed_cache + row * kPackedRow + kLora + 2 * kRope + 4 * warp) = dq;
    }
  }

  // rope key: the 64 values after the latent part, de-interleaved rope
  if (i < kRope) pe[i] = bf16_round(proj(src + kLora + i));
  __syncthreads();
  if (i < kRope && row_ok) {
    const int j = i & 31;
    const float even = pe[2 * j], odd = pe[2 * j + 1];
    const float cs = ld_bf16(cos + ti * kRope + i), sn = ld_bf16(sin + ti * kRope + i);
    const float x = i < 32 ? even : odd;
    const float rot = i < 32 ? -odd : even;
    const __nv_bfloat16 kr = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x, cs), __fmul_rn(rot, sn)));
    kr_cache[row * kRope + i] = kr;
    if (packed_cache != nullptr) *reinterpret_cast<__nv_bfloat16*>(packed_cache + row * kPackedRow + kLora + 2 * i) = kr;
  }

  // indexer key: LayerNorm in fp32 -> bf16, rope on the first 64 dims (halves, no de-interleave), Hadamard, int8
  const float x = proj(ki + static_cast<int64_t>(ti) * ld + i);
  const float mean = block_sum(x, red) * (1.0f / kIdxDim);
  const float dx = x - mean;
  const float var = block_sum(__fmul_rn(dx, dx), red) * (1.0f / kIdxDim);
  const float y = __fdiv_rn(dx, sqrtf(var + ln_eps));
  kvec[i] = bf16_round(__fadd_rn(__fmul_rn(y, ld_bf16(ln_gamma + i)), ld_bf16(ln_beta + i)));
  __syncthreads();
  float k = kvec[i];
  if (i < kRope) {
    const float cs = ld_bf16(cos + ti * kRope + i), sn = ld_bf16(sin + ti * kRope + i);
    const float rot = i < 32 ? -kvec[i + 32] : kvec[i - 32];
    k = bf16_round(__fadd_rn(__fmul_rn(k, cs), __fmul_rn(rot, sn)));
  }
  __syncthreads();
  kvec[i] = k;
  __syncthreads();
  float acc = 0.f;
#pragma unroll 8
  for (int r = 0; r < kIdxDim; ++r) acc = fmaf(kvec[r], __bfloat162float(had[r * kIdxDim + i]), acc);
  const float hk = bf16_round(acc);
  const float kmax = block_max(fabsf(hk), red);
  const float ksq = __fdiv_rn(127.0f, kmax);
  if (row_ok) {
    idx_k_cache[row * kIdxDim + i] = quant_one(hk, ksq);
    if (i == 0) idx_k_scale_cache[row] = __float2half_rn(__fdiv_rn(1.0f, ksq));
  }

  // indexer weights: bf16 rounding, then heads^-1/2 and dim^-1/2 in fp32, fp16 out
  if (i < kIdxHeads) {
    const float w = bf16_round(proj(wp + static_cast<int64_t>(ti) * ld + i));
    weights[static_cast<int64_t>(ti) * kIdxHeads + i] =
        __float2half_rn(__fmul_rn(__fmul_rn(w, 0.125f), 0.08838834764831845f));
  }
}

// ---- indexer query: int32 -> bf16, rope, Hadamard, per-head int8 ------------------------------------------
// grid = (8 head groups, tokens), block = 128: eight heads per block share the Hadamard matrix, staged in
// shared memory while the products are dequantised
constexpr int kHeadsPerBlock = 8;
__global__ void __launch_bounds__(128)
prolog_idxq_kernel(const int32_t* __restrict__ qi_i32, const float* __restrict__ q_norm_scale,
                   const float* __restrict__ w_scale, const __nv_bfloat16* __restrict__ cos,
                   const __nv_bfloat16* __restrict__ sin, const __nv_bfloat16* __restrict__ hadamard_q,
                   int8_t* __restrict__ q_int8, __half* __restrict__ q_scale) {
  __shared__ float red8[4][kHeadsPerBlock];
  __shared__ float qv[kHeadsPerBlock][kIdxDim];
  __shared__ __align__(16) float qt[kIdxDim][kHeadsPerBlock];  // the roped rows, dim-major: 8 heads of a dim in 32 B
  __shared__ __align__(16) __nv_bfloat16 had[kIdxDim * kIdxDim];
  const int hg = blockIdx.x, ti = blockIdx.y, i = threadIdx.x;
  {
    const uint4* hsrc = reinterpret_cast<const uint4*>(hadamard_q);
    uint4* hdst = reinterpret_cast<uint4*>(had);
#pragma unroll 4
    for (int u = i; u < kIdxDim * kIdxDim / 8; u += 128) hdst[u] = __ldg(hsrc + u);
  }
  const float rs = q_norm_scale[ti];
  const float cs = i < kRope ? ld_bf16(cos + ti * kRope + i) : 0.f;
  const float sn = i < kRope ? ld_bf16(sin + ti * kRope + i) : 0.f;
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) {
    const int64_t col = static_cast<int64_t>(hg * kHeadsPerBlock + hh) * kIdxDim + i;
    const float v = __fmul_rn(__fmul_rn(static_cast<float>(qi_i32[static_cast<int64_t>(ti) * kIdxHeads * kIdxDim + col]), rs),
                              w_scale[col]);
    qv[hh][i] = bf16_round(v);
  }
  __syncthreads();
  float q[kHeadsPerBlock];
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) {
    q[hh] = qv[hh][i];
    if (i < kRope) {
      const float rot = i < 32 ? -qv[hh][i + 32] : qv[hh][i - 32];
      q[hh] = bf16_round(__fadd_rn(__fmul_rn(q[hh], cs), __fmul_rn(rot, sn)));
    }
  }
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) qt[i][hh] = q[hh];
  __syncthreads();
  float acc[kHeadsPerBlock];
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) acc[hh] = 0.f;
#pragma unroll 4
  for (int r = 0; r < kIdxDim; ++r) {  // per dim: one Hadamard element and two broadcast 16-byte reads of the 8 heads
    const float hv = __bfloat162float(had[r * kIdxDim + i]);
    const float4 a = *reinterpret_cast<const float4*>(&qt[r][0]);
    const float4 b = *reinterpret_cast<const float4*>(&qt[r][4]);
    acc[0] = fmaf(a.x, hv, acc[0]);
    acc[1] = fmaf(a.y, hv, acc[1]);
    acc[2] = fmaf(a.z, hv, acc[2]);
    acc[3] = fmaf(a.w, hv, acc[3]);
    acc[4] = fmaf(b.x, hv, acc[4]);
    acc[5] = fmaf(b.y, hv, acc[5]);
    acc[6] = fmaf(b.z, hv, acc[6]);
    acc[7] = fmaf(b.w, hv, acc[7]);
  }
  // the eight row maxima with one hand-over through shared memory
  float hq[kHeadsPerBlock];
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) {
    hq[hh] = bf16_round(acc[hh]);
    const float m = warp_max(fabsf(hq[hh]));
    if ((i & 31) == 0) red8[i >> 5][hh] = m;
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < kHeadsPerBlock; ++hh) {
    const float amax = fmaxf(fmaxf(red8[0][hh], red8[1][hh]), fmaxf(red8[2][hh], red8[3][hh]));
    const float sq = __fdiv_rn(127.0f, amax);
    const int64_t head = static_cast<int64_t>(ti) * kIdxHeads + hg * kHeadsPerBlock + hh;
    q_int8[head * kIdxDim + i] = quant_one(hq[hh], sq);
    if (i == 0) q_scale[head] = __float2half_rn(__fdiv_rn(1.0f, sq));
  }
}

// ==== the two prologs of the non-quantised chain ===========================================================
// Arithmetic of the system tests' goldens: `mla_prolog_compute` without quantisation
// (framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_mla_prolog_golden_v32.py:176-303) and the
// non-quantised `indexer_prolog` (.../gen_lightning_indexer_prolog.py:253-293); operators
// `MlaPrologComputeV32` (framework/src/operator/models/deepseek_v3.2_exp/dynamic_mla_v32.cpp:187-345) and
// `LightningIndexerPrologCompute` (.../lightning_indexer_prolog.cpp:129-227). Every rope here de-interleaves
// (even dims first), the indexer's too; there is no Hadamard rotation and the weights are not scaled.

// de-interleaving rope of 64 values held in shared memory: output element c
__device__ __forceinline__ float rope_deinterleaved(const float* pe, int c, float cs, float sn) {
  const int j = c & 31;
  const float even = pe[2 * j], odd = pe[2 * j + 1];
  const float x = c < 32 ? even : odd;
  const float rot = c < 32 ? -odd : even;
  return __fadd_rn(__fmul_rn(x, cs), __fmul_rn(rot, sn));
}

// ---- per token: bf16 latent row, rope key, indexer key, indexer weights; scatter into the bf16 caches -----
// grid = tokens, block = 128 (thread i owns latent dims 4i..4i+3 and indexer-key dim i)
__global__ void __launch_bounds__(128)
prolog_kv_bf16_kernel(const float* __restrict__ kv, const float* __restrict__ ki, const float* __restrict__ wp, int ld,
                      int n_split, long long split_stride, const __nv_bfloat16* __restrict__ gamma_ckv,
                      const __nv_bfloat16* __restrict__ cos, const __nv_bfloat16* __restrict__ sin,
                      const __nv_bfloat16* __restrict__ ln_gamma, const __nv_bfloat16* __restrict__ ln_beta,
                      const int64_t* __restrict__ cache_index, int64_t cache_rows, float eps_ckv, float ln_eps,
                      __nv_bfloat16* __restrict__ kv_cache, __nv_bfloat16* __restrict__ kr_cache,
                      __nv_bfloat16* __restrict__ idx_k_cache, __nv_bfloat16* __restrict__ weights, int32_t* status) {
  __shared__ float red[32];
  __shared__ float pe[kRope];
  __shared__ float kpe[kRope];
  const int ti = blockIdx.x, i = threadIdx.x;
  const int64_t row = cache_index[ti];
  const bool row_ok = row >= 0 && row < cache_rows;
  if (!row_ok && i == 0) set_status(status, PTO_ST_BAD_PAGE, static_cast<int>(row), 61);
  auto proj = [&](const float* p) {
    float part[8];
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) part[sp] = sp < n_split ? __ldg(p + sp * split_stride) : 0.f;
    float a = part[0];
#pragma unroll
    for (int sp = 1; sp < 8; ++sp) {
      if (sp < n_split) a = __fadd_rn(a, part[sp]);
    }
    return a;
  };
  // latent part: bf16 rounding, RMSNorm, bf16
  const float* src = kv + static_cast<int64_t>(ti) * ld;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[e] = bf16_round(proj(src + 4 * i + e));
    ss = __fadd_rn(ss, __fmul_rn(__fmul_rn(v[e], v[e]), 1.0f / kLora));
  }
  const float rms = sqrtf(block_sum(ss, red) + eps_ckv);
  if (row_ok) {
    __nv_bfloat16 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[e] = __float2bfloat16_rn(__fmul_rn(__fdiv_rn(v[e], rms), ld_bf16(gamma_ckv + 4 * i + e)));
    }
    *reinterpret_cast<uint2*>(kv_cache + row * kLora + 4 * i) = *reinterpret_cast<const uint2*>(o);
  }
  // rope key and indexer key: the values to rotate go through shared memory
  if (i < kRope) pe[i] = bf16_round(proj(src + kLora + i));
  const float x = proj(ki + static_cast<int64_t>(ti) * ld + i);
  const float mean = block_sum(x, red) * (1.0f / kIdxDim);
  const float dx = x - mean;
  const float var = block_sum(__fmul_rn(dx, dx), red) * (1.0f / kIdxDim);
  const float y = __fdiv_rn(dx, sqrtf(var + ln_eps));
  const float k = bf16_round(__fadd_rn(__fmul_rn(y, ld_bf16(ln_gamma + i)), ld_bf16(ln_beta + i)));
  if (i < kRope) kpe[i] = k;
  __syncthreads();
  if (row_ok) {
    float ko = k;
    if (i < kRope) {
      const float cs = ld_bf16(cos + ti * kRope + i), sn = ld_bf16(sin + ti * kRope + i);
      kr_cache[row * kRope + i] = __float2bfloat16_rn(rope_deinterleaved(pe, i, cs, sn));
      ko = rope_deinterleaved(kpe, i, cs, sn);
    }
    idx_k_cache[row * kIdxDim + i] = __float2bfloat16_rn(ko);
  }
  if (i < kIdxHeads) {
    weights[static_cast<int64_t>(ti) * kIdxHeads + i] = __float2bfloat16_rn(proj(wp + static_cast<int64_t>(ti) * ld + i));
  }
}

// ---- ropes of the two up-projections -----------------------------------------------------------------
// grid = (24 head groups, tokens), block = 256, two values per thread: groups 0..15 take eight attention heads
// each (q_b[t, head, 128:192] -> q_rope[t, head, :]), groups 16..23 eight indexer heads each
// (idx_query[t, head, 0:64] rotated in place; the other 64 dims of a head stay as the product wrote them)
__global__ void __launch_bounds__(256)
prolog_rope_bf16_kernel(const __nv_bfloat16* __restrict__ q_b, const __nv_bfloat16* __restrict__ cos,
                        const __nv_bfloat16* __restrict__ sin, __nv_bfloat16* __restrict__ q_rope,
                        __nv_bfloat16* __restrict__ idx_query) {
  __shared__ float pe[8][kRope];
  pdl_wait();
  if (threadIdx.x == 0) pdl_trigger();
  const int g = blockIdx.x, ti = blockIdx.y;
  const bool att = g < kHeads / 8;
  const int head0 = att ? g * 8 : (g - kHeads / 8) * 8;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int e = u * 256 + threadIdx.x;
    const int hh = e >> 6, c = e & 63;
    const __nv_bfloat16* src = att ? q_b + (static_cast<int64_t>(ti) * kHeads + head0 + hh) * kQHead + kNope + c
                                   : idx_query + (static_cast<int64_t>(ti) * kIdxHeads + head0 + hh) * kIdxDim + c;
    pe[hh][c] = __bfloat162float(*src);
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int e = u * 256 + threadIdx.x;
    const int hh = e >> 6, c = e & 63;
    const float cs = ld_bf16(cos + ti * kRope + c), sn = ld_bf16(sin + ti * kRope + c);
    const __nv_bfloat16 o = __float2bfloat16_rn(rope_deinterleaved(pe[hh], c, cs, sn));
    if (att) {
      q_rope[(static_cast<int64_t>(ti) * kHeads + head0 + hh) * kRope + c] = o;
    } else {
      idx_query[(static_cast<int64_t>(ti) * kIdxHeads + head0 + hh) * kIdxDim + c] = o;
    }
  }
}

// ---- split caches -> packed 656-byte rows: one warp per row, 41 16-byte pieces ----------------------------
__global__ void __launch_bounds__(256)
kv_pack_rows_kernel(const int8_t* __restrict__ kv, const __nv_bfloat16* __restrict__ kr, const float* __restrict__ sc,
                    int64_t rows, int8_t* __restrict__ packed) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    uint4* dst = reinterpret_cast<uint4*>(packed + r * kPackedRow);
    dst[lane] = __ldg(reinterpret_cast<const uint4*>(kv + r * kLora) + lane);
    if (lane < 8) dst[32 + lane] = __ldg(reinterpret_cast<const uint4*>(kr + r * kRope) + lane);
    if (lane == 8) dst[40] = __ldg(reinterpret_cast<const uint4*>(sc + r * 4));
  }
}

}  // namespace

cudaError_t launch_kv_pack_rows(const int8_t* kv, const void* kr, const float* sc, int64_t rows, int8_t* packed,
                                int num_sms, cudaStream_t stream) {
  const int64_t want = (rows + 7) / 8;
  const int grid = static_cast<int>(want < static_cast<int64_t>(num_sms) * 8 ? (want < 1 ? 1 : want) : num_sms * 8);
  count_launch();
  kv_pack_rows_kernel<<<grid, 256, 0, stream>>>(kv, reinterpret_cast<const __nv_bfloat16*>(kr), sc, rows, packed);
  return cudaGetLastError();
}

cudaError_t launch_prolog_qnorm_quant(const float* qa, int ld, int n_split, long long split_stride, const void* gamma_cq,
                                      int t, int q_lora, float eps, int8_t* q_norm, float* q_norm_scale,
                                      cudaStream_t stream, bool pdl) {
  const size_t dyn = static_cast<size_t>(q_lora) * sizeof(float);
  if (dyn > 40 * 1024) {  // beyond what fits the default 48 KB next to the kernel's static shared memory
    cudaError_t e = cudaFuncSetAttribute(prolog_qnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dyn));
    if (e != cudaSuccess) return e;
  }
  count_launch();
  return launch_maybe_pdl(prolog_qnorm_kernel<true>, dim3(t), dim3(512), dyn, stream, pdl, qa, ld, n_split, split_stride,
                          reinterpret_cast<const __nv_bfloat16*>(gamma_cq), q_lora, eps, q_norm, q_norm_scale,
                          static_cast<__nv_bfloat16*>(nullptr));
}

cudaError_t launch_prolog_qnorm_bf16(const float* qa, int ld, int n_split, long long split_stride, const void* gamma_cq,
                                     int t, int q_lora, float eps, void* q_norm, cudaStream_t stream, bool pdl) {
  const size_t dyn = static_cast<size_t>(q_lora) * sizeof(float);
  if (dyn > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(prolog_qnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dyn));
    if (e != cudaSuccess) return e;
  }
  count_launch();
  return launch_maybe_pdl(prolog_qnorm_kernel<false>, dim3(t), dim3(512), dyn, stream, pdl, qa, ld, n_split,
                          split_stride, reinterpret_cast<const __nv_bfloat16*>(gamma_cq), q_lora, eps,
                          static_cast<int8_t*>(nullptr), static_cast<float*>(nullptr),
                          reinterpret_cast<__nv_bfloat16*>(q_norm));
}

cudaError_t launch_prolog_qb_dequant_rope(const int32_t* qb_i32, const float* q_norm_scale, const float* w_scale,
                                          const void* cos, const void* sin, int t, void* q_b, void* q_rope,
                                          cudaStream_t stream, bool pdl) {
  count_launch();
  return launch_maybe_pdl(prolog_qb_dequant_rope_kernel, dim3(kHeads / kQbHeadsPerBlock, t), dim3(256), 0, stream, pdl,
                          qb_i32, q_norm_scale, w_scale, reinterpret_cast<const __nv_bfloat16*>(cos),
                          reinterpret_cast<const __nv_bfloat16*>(sin), reinterpret_cast<__nv_bfloat16*>(q_b),
                          reinterpret_cast<__nv_bfloat16*>(q_rope));
}

cudaError_t launch_prolog_kv(const float* kv, const float* ki, const float* wp, int ld, int n_split,
                             long long split_stride, const void* gamma_ckv, const void* cos,
                             const void* sin, const void* ln_gamma, const void* ln_beta, const void* hadamard_k,
                             const int64_t* cache_index, int64_t cache_rows, int t, float eps_ckv, float ln_eps,
                             int8_t* kv_cache, void* kr_cache, float* kv_scale_cache, int8_t* idx_k_cache,
                             void* idx_k_scale_cache, void* weights, int8_t* packed_cache, int32_t* status,
                             cudaStream_t stream) {
  count_launch();
  prolog_kv_kernel<<<t, 128, 0, stream>>>(
      kv, ki, wp, ld, n_split, split_stride, reinterpret_cast<const __nv_bfloat16*>(gamma_ckv),
      reinterpret_cast<const __nv_bfloat16*>(cos),
      reinterpret_cast<const __nv_bfloat16*>(sin), reinterpret_cast<const __nv_bfloat16*>(ln_gamma),
      reinterpret_cast<const __nv_bfloat16*>(ln_beta), reinterpret_cast<const __nv_bfloat16*>(hadamard_k), cache_index,
      cache_rows, eps_ckv, ln_eps, kv_cache, reinterpret_cast<__nv_bfloat16*>(kr_cache), kv_scale_cache, idx_k_cache,
      reinterpret_cast<__half*>(idx_k_scale_cache), reinterpret_cast<__half*>(weights), packed_cache, status);
  return cudaGetLastError();
}

cudaError_t launch_prolog_kv_bf16(const float* kv, const float* ki, const float* wp, int ld, int n_split,
                                  long long split_stride, const void* gamma_ckv, const void* cos, const void* sin,
                                  const void* ln_gamma, const void* ln_beta, const int64_t* cache_index,
                                  int64_t cache_rows, int t, float eps_ckv, float ln_eps, void* kv_cache, void* kr_cache,
                                  void* idx_k_cache, void* weights, int32_t* status, cudaStream_t stream) {
  count_launch();
  prolog_kv_bf16_kernel<<<t, 128, 0, stream>>>(
      kv, ki, wp, ld, n_split, split_stride, reinterpret_cast<const __nv_bfloat16*>(gamma_ckv),
      reinterpret_cast<const __nv_bfloat16*>(cos), reinterpret_cast<const __nv_bfloat16*>(sin),
      reinterpret_cast<const __nv_bfloat16*>(ln_gamma), reinterpret_cast<const __nv_bfloat16*>(ln_beta), cache_index,
      cache_rows, eps_ckv, ln_eps, reinterpret_cast<__nv_bfloat16*>(kv_cache), reinterpret_cast<__nv_bfloat16*>(kr_cache),
      reinterpret_cast<__nv_bfloat16*>(idx_k_cache), reinterpret_cast<__nv_bfloat16*>(weights), status);
  return cudaGetLastError();
}

cudaError_t launch_prolog_rope_bf16(const void* q_b, const void* cos, const void* sin, int t, void* q_rope,
                                    void* idx_query, cudaStream_t stream, bool pdl) {
  count_launch();
  return launch_maybe_pdl(prolog_rope_bf16_kernel, dim3((kHeads + kIdxHeads) / 8, t), dim3(256), 0, stream, pdl,
                          reinterpret_cast<const __nv_bfloat16*>(q_b), reinterpret_cast<const __nv_bfloat16*>(cos),
                          reinterpret_cast<const __nv_bfloat16*>(sin), reinterpret_cast<__nv_bfloat16*>(q_rope),
                          reinterpret_cast<__nv_bfloat16*>(idx_query));
}

cudaError_t launch_prolog_idxq(const int32_t* qi_i32, const float* q_norm_scale, const float* w_scale, const void* cos,
                               const void* sin, const void* hadamard_q, int t, int8_t* q_int8, void* q_scale,
                               cudaStream_t stream) {
  count_launch();
  prolog_idxq_kernel<<<dim3(kIdxHeads / kHeadsPerBlock, t), 128, 0, stream>>>(
      qi_i32, q_norm_scale, w_scale, reinterpret_cast<const __nv_bfloat16*>(cos),
      reinterpret_cast<const __nv_bfloat16*>(sin), reinterpret_cast<const __nv_bfloat16*>(hadamard_q), q_int8,
      reinterpret_cast<__half*>(q_scale));
  return cudaGetLastError();
}

}  // namespace pto
