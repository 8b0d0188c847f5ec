// Tensor-core attention for the encoder graphs: softmax(Q K^T * scale) V per
// (batch, head), fp32 in and out, with the matrix products on the warp-level
// tensor-core path (mma.sync m16n8k16, bf16 operands, fp32 accumulators).
//
// It replaces, for head sizes that are multiples of 16 up to 128, the chain the
// reference lowers with CPU loops: two batched fp32 MatMuls
// (src/Conversion/ONNXToKrnl/Math/MatMul.cpp:488-507), a Mul by a constant and
// a Softmax over the last axis (src/Conversion/ONNXToKrnl/Math/Softmax.cpp:25-134).
//
// Accuracy: every fp32 operand a is split as a = hi + lo with hi = bf16(a),
// lo = bf16(a - hi), and each product block is computed as
// hi*hi + lo*hi + hi*lo, which leaves a relative error of about 2^-16 per
// product -- far inside the 1e-3 parity tolerance of the fp32 ops -- while the
// accumulation stays in fp32.  The softmax is computed online over key blocks
// (running maximum and sum, rescaling the accumulator), which is the same
// function as the reference's three-loop form up to fp32 rounding.
//
// Layout: Q, K, V, out are [B, S, *] row-major with row pitches ld_in / ld_out
// (so a fused [T, 3H] QKV buffer is read in place); head h owns columns
// [h*DH, (h+1)*DH).  One CTA = 64 query rows of one (b, h) (4 warps x 16 rows);
// K and V stream through shared memory in blocks of 64 keys as bf16 hi/lo
// pairs.  Scores never leave registers.
#include <cuda_bf16.h>

#include "../common.cuh"
#include "../runtime/internal.h"

namespace omcuda {

namespace {

constexpr int kQRows = 64;  // query rows per CTA
constexpr int kKeys = 64;   // keys per block
constexpr int kPad = 8;     // bf16 elements of row padding (bank spread)

__device__ __forceinline__ void split_bf16(float a, __nv_bfloat16 &hi,
    __nv_bfloat16 &lo) {
  hi = __float2bfloat16_rn(a);
  lo = __float2bfloat16_rn(__fsub_rn(a, __bfloat162float(hi)));
}

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) |
         ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

// Splits two floats into packed {hi0,hi1} and {lo0,lo1}.
__device__ __forceinline__ void split2(float x, float y, uint32_t &hi,
    uint32_t &lo) {
  __nv_bfloat16 xh, xl, yh, yl;
  split_bf16(x, xh, xl);
  split_bf16(y, yh, yl);
  hi = pack_bf16(xh, yh);
  lo = pack_bf16(xl, yl);
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4],
    uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0,
    uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile(
      "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
      : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
      : "r"(addr));
}

template <int DH>
__global__ void __launch_bounds__(128)
    attention_mma_kernel(const float *__restrict__ Q, const float *__restrict__ K,
        const float *__restrict__ V, int64_t S, int64_t heads, float scale,
        float *__restrict__ out, int64_t ld_in, int64_t ld_out,
        uint32_t *__restrict__ out_range) {
  constexpr int LD = DH + kPad;  // smem row pitch in bf16 elements
  constexpr int KS = DH / 16;    // k-steps over the head dimension
  constexpr int NT_O = DH / 8;   // n-tiles of the output
  constexpr int NT_S = kKeys / 8;

  extern __shared__ __align__(16) __nv_bfloat16 att_smem[];
  // [hi|lo][key][dh] for K, then the same for V
  __nv_bfloat16 (*sK)[kKeys * LD] =
      reinterpret_cast<__nv_bfloat16 (*)[kKeys * LD]>(att_smem);
  __nv_bfloat16 (*sV)[kKeys * LD] =
      reinterpret_cast<__nv_bfloat16 (*)[kKeys * LD]>(att_smem + 2 * kKeys * LD);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / heads, h = bh % heads;
  const int64_t q0 = (int64_t)blockIdx.x * kQRows + warp * 16;
  const float *Qb = Q + (b * S) * ld_in + h * DH;
  const float *Kb = K + (b * S) * ld_in + h * DH;
  const float *Vb = V + (b * S) * ld_in + h * DH;

  // Q fragments (A operand), split once: rows q0+g and q0+g+8.
  uint32_t qh[KS][4], ql[KS][4];
  {
    const int64_t r0 = q0 + g, r1 = q0 + g + 8;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + 2 * t;
      float2 v00 = make_float2(0.f, 0.f), v10 = v00, v01 = v00, v11 = v00;
      if (r0 < S) {
        v00 = *reinterpret_cast<const float2 *>(Qb + r0 * ld_in + c);
        v01 = *reinterpret_cast<const float2 *>(Qb + r0 * ld_in + c + 8);
      }
      if (r1 < S) {
        v10 = *reinterpret_cast<const float2 *>(Qb + r1 * ld_in + c);
        v11 = *reinterpret_cast<const float2 *>(Qb + r1 * ld_in + c + 8);
      }
      split2(v00.x, v00.y, qh[ks][0], ql[ks][0]);
      split2(v10.x, v10.y, qh[ks][1], ql[ks][1]);
      split2(v01.x, v01.y, qh[ks][2], ql[ks][2]);
      split2(v11.x, v11.y, qh[ks][3], ql[ks][3]);
    }
  }

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i)
    o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY; // running max of rows g and g+8
  float l0 = 0.0f, l1 = 0.0f;           // running sums

  for (int64_t j0 = 0; j0 < S; j0 += kKeys) {
    __syncthreads(); // previous block's fragments are no longer read
    // Stage K and V rows j0..j0+63 as bf16 hi/lo.
    for (int i = threadIdx.x; i < kKeys * (DH / 4); i += 128) {
      const int key = i / (DH / 4), c4 = (i % (DH / 4)) * 4;
      float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
      if (j0 + key < S) {
        kv = *reinterpret_cast<const float4 *>(Kb + (j0 + key) * ld_in + c4);
        vv = *reinterpret_cast<const float4 *>(Vb + (j0 + key) * ld_in + c4);
      }
      uint32_t h0, l0w, h1, l1w;
      split2(kv.x, kv.y, h0, l0w);
      split2(kv.z, kv.w, h1, l1w);
      *reinterpret_cast<uint2 *>(&sK[0][key * LD + c4]) = make_uint2(h0, h1);
      *reinterpret_cast<uint2 *>(&sK[1][key * LD + c4]) = make_uint2(l0w, l1w);
      split2(vv.x, vv.y, h0, l0w);
      split2(vv.z, vv.w, h1, l1w);
      *reinterpret_cast<uint2 *>(&sV[0][key * LD + c4]) = make_uint2(h0, h1);
      *reinterpret_cast<uint2 *>(&sV[1][key * LD + c4]) = make_uint2(l0w, l1w);
    }
    __syncthreads();

    // S = Q K^T for this warp's 16 rows x 64 keys.
    float s[NT_S][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt)
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) {
        const int off = (nt * 8 + g) * LD + ks * 16 + 2 * t;
        const uint32_t bh0 = *reinterpret_cast<const uint32_t *>(&sK[0][off]);
        const uint32_t bh1 = *reinterpret_cast<const uint32_t *>(&sK[0][off + 8]);
        const uint32_t bl0 = *reinterpret_cast<const uint32_t *>(&sK[1][off]);
        const uint32_t bl1 = *reinterpret_cast<const uint32_t *>(&sK[1][off + 8]);
        mma_bf16(s[nt], ql[ks], bh0, bh1); // small terms first
        mma_bf16(s[nt], qh[ks], bl0, bl1);
        mma_bf16(s[nt], qh[ks], bh0, bh1);
      }
    }
    // Scale (the graph's Mul by a constant), mask keys past S, block maxima.
    float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      const int64_t key = j0 + nt * 8 + 2 * t;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = __fmul_rn(s[nt][e], scale);
        if (key + (e & 1) >= S)
          v = -INFINITY;
        s[nt][e] = v;
      }
      bm0 = fmaxf(bm0, fmaxf(s[nt][0], s[nt][1]));
      bm1 = fmaxf(bm1, fmaxf(s[nt][2], s[nt][3]));
    }
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
    const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
    // exp(-inf - finite) = 0 covers the first block; every block holds at
    // least one unmasked key, so mn0 / mn1 are finite.
    const float r0 = expf(m0 - mn0), r1 = expf(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      s[nt][0] = expf(s[nt][0] - mn0);
      s[nt][1] = expf(s[nt][1] - mn0);
      s[nt][2] = expf(s[nt][2] - mn1);
      s[nt][3] = expf(s[nt][3] - mn1);
      ps0 += s[nt][0] + s[nt][1];
      ps1 += s[nt][2] + s[nt][3];
    }
    ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
    ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
    ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
    ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
    l0 = l0 * r0 + ps0;
    l1 = l1 * r1 + ps1;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= r0;
      o[i][1] *= r0;
      o[i][2] *= r1;
      o[i][3] *= r1;
    }
    // O += P V.  The accumulator layout of two adjacent score tiles is the A
    // operand layout of one 16-key step.
#pragma unroll
    for (int kk = 0; kk < kKeys / 16; ++kk) {
      uint32_t ph[4], pl[4];
      split2(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);
      split2(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);
      split2(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);
      split2(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
      // ldmatrix.trans: lane supplies the row (key) address of one 8x8 block:
      // blocks 0,1 = keys kk*16 + {0..7, 8..15} at dh tile d, blocks 2,3 the
      // same keys at dh tile d+1.
      const int mrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int mcol = (lane >> 4) * 8;
#pragma unroll
      for (int d = 0; d < NT_O; d += 2) {
        uint32_t vh0, vh1, vh2, vh3, vl0, vl1, vl2, vl3;
        const int off = mrow * LD + d * 8 + mcol;
        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(&sV[0][off]), vh0,
            vh1, vh2, vh3);
        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(&sV[1][off]), vl0,
            vl1, vl2, vl3);
        mma_bf16(o[d], pl, vh0, vh1);
        mma_bf16(o[d], ph, vl0, vl1);
        mma_bf16(o[d], ph, vh0, vh1);
        mma_bf16(o[d + 1], pl, vh2, vh3);
        mma_bf16(o[d + 1], ph, vl2, vl3);
        mma_bf16(o[d + 1], ph, vh2, vh3);
      }
    }
  }

  // Normalise and store; fold the outputs into the running range.
  float lo = INFINITY, hi = -INFINITY;
  const float inv0 = __fdiv_rn(1.0f, l0), inv1 = __fdiv_rn(1.0f, l1);
  const int64_t r0 = q0 + g, r1 = q0 + g + 8;
  float *ob = out + (b * S) * ld_out + h * DH;
#pragma unroll
  for (int i = 0; i < NT_O; ++i) {
    const int c = i * 8 + 2 * t;
    if (r0 < S) {
      float2 v = make_float2(o[i][0] * inv0, o[i][1] * inv0);
      *reinterpret_cast<float2 *>(ob + r0 * ld_out + c) = v;
      lo = fminf(lo, fminf(v.x, v.y));
      hi = fmaxf(hi, fmaxf(v.x, v.y));
    }
    if (r1 < S) {
      float2 v = make_float2(o[i][2] * inv1, o[i][3] * inv1);
      *reinterpret_cast<float2 *>(ob + r1 * ld_out + c) = v;
      lo = fminf(lo, fminf(v.x, v.y));
      hi = fmaxf(hi, fmaxf(v.x, v.y));
    }
  }
  if (out_range)
    range_commit_warp(out_range, lo, hi);
}

} // namespace

// True when the tensor-core kernel can take the problem: head size 32, 64 or
// 128 and 8-byte aligned rows.
bool attention_mma_supported(const float *Q, const float *K, const float *V,
    const float *out, int64_t dh, int64_t ld_in, int64_t ld_out) {
  return (dh == 32 || dh == 64 || dh == 128) && (ld_in % 4 == 0) &&
         (ld_out % 2 == 0) &&
         ((((uintptr_t)Q | (uintptr_t)K | (uintptr_t)V) & 15u) == 0) &&
         (((uintptr_t)out & 7u) == 0);
}

int launch_attention_mma(const float *Q, const float *K, const float *V,
    int64_t B, int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    int64_t ld_in, int64_t ld_out, void *out_range, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(S, kQRows), (unsigned)(B * heads));
  uint32_t *rng = (uint32_t *)out_range;
  const size_t smem = (size_t)4 * kKeys * (dh + kPad) * sizeof(__nv_bfloat16);
  if (dh == 64) {
    attention_mma_kernel<64><<<grid, 128, smem, st>>>(
        Q, K, V, S, heads, scale, out, ld_in, ld_out, rng);
  } else if (dh == 32) {
    attention_mma_kernel<32><<<grid, 128, smem, st>>>(
        Q, K, V, S, heads, scale, out, ld_in, ld_out, rng);
  } else {
    static PerDeviceInt attr_set;
    if (!attr_set.get()) {
      OMCUDA_CHECK(cudaFuncSetAttribute(attention_mma_kernel<128>,
          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      attr_set.set(1);
    }
    attention_mma_kernel<128><<<grid, 128, smem, st>>>(
        Q, K, V, S, heads, scale, out, ld_in, ld_out, rng);
  }
  OMCUDA_CHECK_LAUNCH("attention_mma_kernel");
  return OMCUDA_OK;
}

} // namespace omcuda
