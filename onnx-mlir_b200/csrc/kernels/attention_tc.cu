// Attention on the Blackwell tensor cores (tcgen05.mma kind::f16, bf16
// operands, fp32 accumulators in tensor memory) for the encoder graphs:
// softmax(Q K^T * scale) V per (batch, head), head size 64, sequence length a
// multiple of 128.
//
// It stands for the chain the reference lowers with CPU loops: two batched
// fp32 MatMuls (src/Conversion/ONNXToKrnl/Math/MatMul.cpp:488-507), a Mul by a
// constant and a Softmax over the last axis
// (src/Conversion/ONNXToKrnl/Math/Softmax.cpp:25-134).
//
// Accuracy.  Every fp32 operand a arrives already split as a = hi + lo with
// hi = bf16(a), lo = bf16(a - hi) (two bf16 planes, written by the QKV GEMM's
// epilogue or by split_bf16_kernel below), and each product is evaluated as
// lo*hi + hi*lo + hi*hi, which leaves a relative error of about 2^-16 per
// product, far inside the 1e-3 tolerance of the fp32 ops; accumulation is
// fp32.  The softmax runs online over key blocks (an exponent offset that
// tracks the running maximum, and the running sum), the same function as the
// reference's three-loop form up to fp32 rounding.
//
// Layout in HBM: the planes are [T, ld] bf16 row-major (T = batch*seq tokens);
// head h of Q / K / V owns columns [col + 64 h, col + 64 h + 64) of its rows.
// out is [T, ld_out] fp32.
//
// A work item = 128 query rows of one (batch, head).  Two persistent CTAs
// share an SM, so that one's softmax (CUDA cores) overlaps the other's matrix
// products (tensor pipe); each walks its share of the items and requests the
// Q and first K tiles of its next item while the current one is in its last
// key block.  Per block of 128 keys:
//   thread 0   waits for the K tiles (TMA, 128-byte swizzle), issues
//              S = Q K^T as 12 MMAs (3 split terms x 4 k-steps) into tensor
//              memory, commits to an mbarrier, refills the K buffers;
//   8 warps    two threads per query row (its TMEM lane), 64 keys each: row
//              maximum (exchanged through shared memory), p = 2^(s*c - m),
//              running sum, p split into bf16 hi/lo and stored back over the
//              scores in tensor memory;
//   thread 0   issues O_j = P V as 16 MMAs with P read from tensor memory and
//              V (keys x 64, MN-major) from shared memory: P_hi against
//              [V_hi | V_lo] as one N = 128 product per 16-key slice (into
//              128 columns of tensor memory), P_lo V_hi on top of the first
//              64 columns; refills V;
// O accumulates in tensor memory over the key blocks of an item (the P V MMAs
// add to it); the exponent offset of a row follows its running maximum lazily,
// moving only when a block's maximum exceeds it by more than 2^8, and only
// then are O and the row sum rescaled (a tensor-memory load / multiply /
// store pass): on typical data one pass or none per item instead of one
// register fold per block.  At the end of the item the 8 warps read O (the sum
// of its two 64-column halves), normalise and store.
// The normalised 128 x 64 result of an item is staged in the (then free) V
// buffers and leaves with two TMA stores of whole 128-byte lines.
// Every wait on an mbarrier is bounded (tc_ptx.cuh); a timeout raises the
// CTA's abort flag, the CTA frees its tensor memory, writes the status word
// and returns.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "../common.cuh"
#include "../runtime/internal.h"
#include "tc_ptx.cuh"

namespace omcuda {

namespace {

constexpr int kTQ = 128;            // query rows per CTA
constexpr int kTK = 128;            // keys per block
constexpr int kTDh = 64;            // head size
constexpr int kTile = 128 * 128;    // bytes of one 128-row x 64-bf16 tile
constexpr int kTcAttSmem = 6 * kTile + 1024;
constexpr uint32_t kTmemColsAtt = 256; // S/P: 0..127, O_j: 128..255
constexpr int kTcAttThreads = 256;     // two threads per query row

// Four MMAs over the four 16-element K slices of a 64-wide K-major operand
// pair, issued back to back from one asm block (descriptor + 2 per 32-byte
// slice): instructions between two tcgen05.mma of the lone issuing thread
// would each delay the next issue.
__device__ __forceinline__ void umma_bf16_ss_x4(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile("{\n\t"
               ".reg .pred p, t;\n\t"
               ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "setp.eq.b32 t, 0, 0;\n\t"
               "add.u64 a1, %1, 2;\n\t"
               "add.u64 a2, %1, 4;\n\t"
               "add.u64 a3, %1, 6;\n\t"
               "add.u64 b1, %2, 2;\n\t"
               "add.u64 b2, %2, 4;\n\t"
               "add.u64 b3, %2, 6;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, t;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
               : "memory");
}

// Four P V MMAs over 64 keys (two 32-key chunks): A (P) from tensor memory at
// columns a, a + 8, a + 32, a + 40; B (V, MN-major) advances 16 keys = 2048
// bytes (descriptor + 128) per slice.
__device__ __forceinline__ void umma_bf16_ts_x4(uint32_t d_tmem, uint32_t a_tmem,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile("{\n\t"
               ".reg .pred p, t;\n\t"
               ".reg .b32 a1, a2, a3;\n\t"
               ".reg .b64 b1, b2, b3;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "setp.eq.b32 t, 0, 0;\n\t"
               "add.u32 a1, %1, 8;\n\t"
               "add.u32 a2, %1, 32;\n\t"
               "add.u32 a3, %1, 40;\n\t"
               "add.u64 b1, %2, 128;\n\t"
               "add.u64 b2, %2, 256;\n\t"
               "add.u64 b3, %2, 384;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, t;\n\t"
               "}" ::"r"(d_tmem),
               "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
               : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(
          taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
      "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]),
      "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// {hi(b), hi(a)} as packed bf16 (a in the low half), round to nearest even.
__device__ __forceinline__ uint32_t cvt_bf16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// Barrier between the two warps (64 threads) that share a lane quadrant;
// named barriers 1..4, constant ids so that only those are reserved.
__device__ __forceinline__ void pair_barrier(int quad) {
  switch (quad) {
  case 0:
    asm volatile("bar.sync 1, 64;" ::: "memory");
    break;
  case 1:
    asm volatile("bar.sync 2, 64;" ::: "memory");
    break;
  case 2:
    asm volatile("bar.sync 3, 64;" ::: "memory");
    break;
  default:
    asm volatile("bar.sync 4, 64;" ::: "memory");
    break;
  }
}

// Instruction descriptor of tcgen05.mma kind::f16 with bf16 operands and an
// fp32 accumulator, M = 128; b_mn_major selects an MN-major (transposed) B.
__host__ __device__ constexpr uint32_t att_idesc(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// Coordinates of one work item: 128 query rows of one (batch, head).
struct AttItem {
  int32_t row_q, row_kv, cq, ck, cv, col_out;
};

__device__ __forceinline__ AttItem att_item(int64_t item, int nq, int64_t S,
    int64_t heads, int32_t q_col, int32_t k_col, int32_t v_col) {
  const int64_t bh = item / nq, qt = item % nq;
  const int64_t b = bh / heads, h = bh % heads;
  AttItem it;
  it.row_kv = (int32_t)(b * S);
  it.row_q = it.row_kv + (int32_t)qt * kTQ;
  it.col_out = (int32_t)h * kTDh;
  it.cq = q_col + it.col_out;
  it.ck = k_col + it.col_out;
  it.cv = v_col + it.col_out;
  return it;
}

__global__ void __launch_bounds__(kTcAttThreads, 2)
    attention_tc_kernel(const __grid_constant__ CUtensorMap map_hi,
        const __grid_constant__ CUtensorMap map_lo,
        const __grid_constant__ CUtensorMap map_out, int32_t q_col, int32_t k_col,
        int32_t v_col, int64_t S, int64_t heads, int64_t n_items, float scale_log2e,
        uint32_t *__restrict__ out_range, int *status, uint64_t wait_ns) {
  extern __shared__ uint8_t att_tc_smem[];
  __shared__ uint64_t bar_q, bar_k, bar_v, bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xch[2][kTQ]; // row maximum / row sum of each half of the keys

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Warps w and w + 4 share the 32 query rows (TMEM lanes) of quadrant w & 3:
  // `half` 0 takes keys 0..63 of every block and output columns 0..31, half 1
  // the rest.
  const int quad = warp & 3, half = warp >> 2;
  const int row = quad * 32 + lane;
  const int nkb = (int)(S / kTK);
  const int nq = (int)(S / kTQ);

  const uint32_t smem0 = (smem_u32(att_tc_smem) + 1023u) & ~1023u;
  const uint32_t s_qh = smem0, s_ql = smem0 + kTile, s_kh = smem0 + 2 * kTile,
                 s_kl = smem0 + 3 * kTile, s_vh = smem0 + 4 * kTile,
                 s_vl = smem0 + 5 * kTile;

  if (tid == 32) {
    prefetch_tensormap(&map_hi);
    prefetch_tensormap(&map_lo);
    prefetch_tensormap(&map_out);
  }
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar_q), 1);
    mbar_init(smem_u32(&bar_k), 1);
    mbar_init(smem_u32(&bar_v), 1);
    mbar_init(smem_u32(&bar_s), 1);
    mbar_init(smem_u32(&bar_o), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0)
    tmem_alloc(smem_u32(&tmem_slot), kTmemColsAtt);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t t_s = tmem;          // scores, then P, columns 0..127
  const uint32_t t_o = tmem + 128u;   // P V of the current key block
  const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
  const int kc0 = half * (kTK / 2); // first key column of this thread's share
  volatile int *abortp = &abort_flag;

  // The CTA walks the items blockIdx.x, blockIdx.x + gridDim.x, ...; the
  // operands of an item's first key block are requested while the item
  // before it is still in its last block, as soon as their buffers are free.
  if (tid == 0 && (int64_t)blockIdx.x < n_items) {
    const AttItem it = att_item(blockIdx.x, nq, S, heads, q_col, k_col, v_col);
    mbar_expect_tx(smem_u32(&bar_q), 2 * kTile);
    tma_load_2d(s_qh, &map_hi, it.cq, it.row_q, smem_u32(&bar_q));
    tma_load_2d(s_ql, &map_lo, it.cq, it.row_q, smem_u32(&bar_q));
    mbar_expect_tx(smem_u32(&bar_k), 2 * kTile);
    tma_load_2d(s_kh, &map_hi, it.ck, it.row_kv, smem_u32(&bar_k));
    tma_load_2d(s_kl, &map_lo, it.ck, it.row_kv, smem_u32(&bar_k));
    mbar_expect_tx(smem_u32(&bar_v), 2 * kTile);
    tma_load_2d(s_vh, &map_hi, it.cv, it.row_kv, smem_u32(&bar_v));
    tma_load_2d(s_vl, &map_lo, it.cv, it.row_kv, smem_u32(&bar_v));
  }

  constexpr uint32_t kIdescQK = att_idesc(kTK, 0);
  constexpr uint32_t kIdescPV = att_idesc(kTDh, 1);
  // P_hi against V_hi and V_lo in one MMA of N = 128: the B descriptor's
  // leading-dimension offset (stride between 64-element groups along N) is
  // the distance from the V_hi tile to the V_lo tile, so output columns
  // 0..63 hold P_hi V_hi and 64..127 hold P_hi V_lo.
  constexpr uint32_t kIdescPV2 = att_idesc(2 * kTDh, 1);
  constexpr uint64_t kLboField = (uint64_t)0x3fff << 16;

  bool ok = true;
  uint32_t nblk = 0;  // key blocks done by this CTA: parity of bar_k / s / v / o
  uint32_t nitem = 0; // items done by this CTA: parity of bar_q
  float lo_run = INFINITY, hi_run = -INFINITY; // range of this thread's outputs

  for (int64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++nitem) {
    const AttItem it = att_item(item, nq, S, heads, q_col, k_col, v_col);
    const bool has_next = item + gridDim.x < n_items;
    AttItem nx = it;
    if (tid == 0 && has_next)
      nx = att_item(item + gridDim.x, nq, S, heads, q_col, k_col, v_col);

    // O accumulates in tensor memory over the key blocks of the item.  The
    // exponent offset m_ref of a row follows its running maximum lazily: it
    // moves (and O and the row sum are rescaled) only when a block's maximum
    // exceeds it by more than 2^8, so p never exceeds 256 and most blocks
    // need no pass over O at all.  Any offset gives the same softmax once
    // the sum over the same p normalises the result.
    float m_ref = -INFINITY; // exponent offset, in units of s * scale * log2(e)
    float l_run = 0.0f;      // running sum of p

    for (int j = 0; j < nkb; ++j, ++nblk) {
      const uint32_t ph = nblk & 1u;
      // ---- S = Q K_j^T ----
      if (tid == 0) {
        if (j == 0)
          ok = mbar_wait(smem_u32(&bar_q), nitem & 1u, abortp, wait_ns);
        ok = ok && mbar_wait(smem_u32(&bar_k), ph, abortp, wait_ns);
        if (ok) {
          tcgen05_fence_after();
          // small terms first: Ql Kh, Qh Kl, then Qh Kh
          const uint32_t qa[3] = {s_ql, s_qh, s_qh};
          const uint32_t kb[3] = {s_kh, s_kl, s_kh};
          static_assert(kTDh == 64, "four K slices per operand row");
#pragma unroll
          for (int t = 0; t < 3; ++t)
            umma_bf16_ss_x4(t_s, make_smem_desc(qa[t]), make_smem_desc(kb[t]),
                kIdescQK, t != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bar_s));
          if (j == 0 && nitem != 0) {
            // The V buffers held the previous item's output for its TMA
            // store: refill them once the store has read them.
            tma_store_wait_read();
            mbar_expect_tx(smem_u32(&bar_v), 2 * kTile);
            tma_load_2d(s_vh, &map_hi, it.cv, it.row_kv, smem_u32(&bar_v));
            tma_load_2d(s_vl, &map_lo, it.cv, it.row_kv, smem_u32(&bar_v));
          }
          ok = mbar_wait(smem_u32(&bar_s), ph, abortp, wait_ns);
          if (ok && j + 1 < nkb) { // the K buffers are free again
            mbar_expect_tx(smem_u32(&bar_k), 2 * kTile);
            tma_load_2d(s_kh, &map_hi, it.ck, it.row_kv + (j + 1) * kTK, smem_u32(&bar_k));
            tma_load_2d(s_kl, &map_lo, it.ck, it.row_kv + (j + 1) * kTK, smem_u32(&bar_k));
          } else if (ok && has_next) { // so are the Q buffers: next item
            mbar_expect_tx(smem_u32(&bar_q), 2 * kTile);
            tma_load_2d(s_qh, &map_hi, nx.cq, nx.row_q, smem_u32(&bar_q));
            tma_load_2d(s_ql, &map_lo, nx.cq, nx.row_q, smem_u32(&bar_q));
            mbar_expect_tx(smem_u32(&bar_k), 2 * kTile);
            tma_load_2d(s_kh, &map_hi, nx.ck, nx.row_kv, smem_u32(&bar_k));
            tma_load_2d(s_kl, &map_lo, nx.ck, nx.row_kv, smem_u32(&bar_k));
          }
        }
      }
      ok = __syncthreads_and(ok) != 0;
      if (!ok)
        break;
      tcgen05_fence_after();

      // ---- online softmax: this thread's half of its row ----
      __syncwarp(); // tcgen05.ld / st are warp-collective: enter them converged
      // The thread's 64 scores are read from tensor memory once and stay in
      // registers for both passes (maximum, then exponentials).
      static_assert(kTK / 2 == 64, "two 32-column loads per thread");
      uint32_t sv[2][32];
      tmem_ld32(t_s + lane_base + (uint32_t)kc0, sv[0]);
      tmem_ld32(t_s + lane_base + (uint32_t)kc0 + 32u, sv[1]);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx = max3f(mx, __uint_as_float(sv[h2][i]), __uint_as_float(sv[h2][i + 1]));
      // Row maximum over both halves (the two threads of a row sit in warps w
      // and w + 4: a 64-thread named barrier per quadrant).
      xch[half][row] = mx;
      pair_barrier(quad);
      mx = fmaxf(mx, xch[half ^ 1][row]);
      const float m_blk = __fmul_rn(mx, scale_log2e);
      // (true for every row on the first block: m_ref is -inf)
      const bool move = m_blk > __fadd_rn(m_ref, 8.0f);
      // Both threads of a row and both warps of a quadrant see the same rows
      // and maxima, so they take this branch together.
      if (j > 0 && __any_sync(0xffffffffu, move)) {
        const float f = move ? ex2_approx(__fsub_rn(m_ref, m_blk)) : 1.0f;
        l_run = __fmul_rn(l_run, f);
        const uint64_t f2 = pack_f32x2(f, f);
#pragma unroll 1
        for (uint32_t part = 0; part < 2; ++part) { // P_hi V_hi + P_lo V_hi | P_hi V_lo
          const uint32_t ta = t_o + part * 64u + lane_base + (uint32_t)(half * 32);
          uint32_t v[32];
          tmem_ld32(ta, v);
          tmem_ld_wait();
          uint32_t w0[16], w1[16];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float a, b;
            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), f2), a, b);
            w0[i] = __float_as_uint(a);
            w0[i + 1] = __float_as_uint(b);
            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(v[16 + i]), __uint_as_float(v[17 + i])), f2), a, b);
            w1[i] = __float_as_uint(a);
            w1[i + 1] = __float_as_uint(b);
          }
          tmem_st16(ta, w0);
          tmem_st16(ta + 16u, w1);
        }
        tmem_st_wait();
      }
      if (move)
        m_ref = m_blk;
      // (packed fp32 below: two individually rounded operations per instruction)
      const uint64_t scale2 = pack_f32x2(scale_log2e, scale_log2e);
      const uint64_t neg_m2 = pack_f32x2(-m_ref, -m_ref);
      const uint64_t minus1 = pack_f32x2(-1.0f, -1.0f);
      uint64_t psum2 = pack_f32x2(0.0f, 0.0f);
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int c = kc0 + 32 * h2;
        const uint32_t(&v)[32] = sv[h2];
        uint32_t whi[16], wlo[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a0, a1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[2 * i]),
                                     __uint_as_float(v[2 * i + 1])),
                           scale2, neg_m2),
              a0, a1);
          const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
          const uint64_t p2 = pack_f32x2(p0, p1);
          psum2 = add_f32x2(psum2, p2);
          const uint32_t hi = cvt_bf16x2(p0, p1);
          // p - hi: one rounding, as the subtraction has
          float r0, r1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(hi << 16),
                                     __uint_as_float(hi & 0xffff0000u)),
                           minus1, p2),
              r0, r1);
          whi[i] = hi;
          wlo[i] = cvt_bf16x2(r0, r1);
        }
        // P of keys c..c+31: hi in columns c..c+15, lo in c+16..c+31 (the
        // scores of those columns are already consumed).
        tmem_st16(t_s + lane_base + (uint32_t)c, whi);
        tmem_st16(t_s + lane_base + (uint32_t)c + 16u, wlo);
      }
      float ps0, ps1;
      unpack_f32x2(psum2, ps0, ps1);
      l_run = __fadd_rn(l_run, __fadd_rn(ps0, ps1));
      tmem_st_wait();
      tcgen05_fence_before();
      __syncthreads(); // every row of P is in tensor memory

      // ---- O_j = P V_j ----
      if (tid == 0) {
        tcgen05_fence_after();
        ok = mbar_wait(smem_u32(&bar_v), ph, abortp, wait_ns);
        if (ok) {
          tcgen05_fence_after();
          static_assert(kTK == 128, "two groups of four 16-key slices per block");
          const uint64_t dvh = make_smem_desc(s_vh);
          const uint64_t dv2 = (dvh & ~kLboField) | ((uint64_t)((s_vl - s_vh) >> 4) << 16);
          // P_hi [V_hi | V_lo] into columns 0..127 of O_j, then P_lo V_hi on
          // top of columns 0..63 (hi parts at column offset 0, lo at 16)
          umma_bf16_ts_x4(t_o, t_s, dv2, kIdescPV2, j != 0 ? 1u : 0u);
          umma_bf16_ts_x4(t_o, t_s + 64u, dv2 + 512, kIdescPV2, 1u);
          umma_bf16_ts_x4(t_o, t_s + 16u, dvh, kIdescPV, 1u);
          umma_bf16_ts_x4(t_o, t_s + 64u + 16u, dvh + 512, kIdescPV, 1u);
          umma_commit(smem_u32(&bar_o));
          ok = mbar_wait(smem_u32(&bar_o), ph, abortp, wait_ns);
          if (ok && j + 1 < nkb) { // the V buffers are free again
            mbar_expect_tx(smem_u32(&bar_v), 2 * kTile);
            tma_load_2d(s_vh, &map_hi, it.cv, it.row_kv + (j + 1) * kTK, smem_u32(&bar_v));
            tma_load_2d(s_vl, &map_lo, it.cv, it.row_kv + (j + 1) * kTK, smem_u32(&bar_v));
          }
        }
      }
      // No CTA barrier here: the other threads go on to wait for the next
      // block's scores, which thread 0 requests only once this P V is done.
    }
    ok = __syncthreads_and(ok) != 0; // the item's last P V is complete
    if (!ok)
      break;
    tcgen05_fence_after();
    __syncwarp();
    float o[kTDh / 2];
    {
      uint32_t v[32];
      tmem_ld32(t_o + lane_base + (uint32_t)(half * 32), v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        o[i] = __uint_as_float(v[i]);
      // ... plus the P_hi V_lo part from the upper 64 columns
      tmem_ld32(t_o + 64u + lane_base + (uint32_t)(half * 32), v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 2)
        unpack_f32x2(add_f32x2(pack_f32x2(o[i], o[i + 1]),
                         pack_f32x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]))),
            o[i], o[i + 1]);
    }
    tcgen05_fence_before();

    // Row sum over both halves, then normalise.  The 128 x 64 result leaves
    // through the V buffers (free after the last P V): half 0's 32 columns in
    // the first 16 KiB tile, half 1's in the second, rows of 128 bytes in the
    // 128-byte swizzle pattern, one TMA store per tile, which writes whole
    // lines.  The next item's V load waits for the store to have read them.
    xch[half][row] = l_run;
    pair_barrier(quad);
    const float inv = __fdiv_rn(1.0f, __fadd_rn(xch[0][row], xch[1][row]));
    const uint32_t my_row = (half ? s_vl : s_vh) + (uint32_t)row * 128u;
    const uint32_t swz = ((uint32_t)row & 7u) << 4;
#pragma unroll
    for (int i = 0; i < kTDh / 2; i += 4) {
      const float4 v = make_float4(__fmul_rn(o[i], inv), __fmul_rn(o[i + 1], inv),
          __fmul_rn(o[i + 2], inv), __fmul_rn(o[i + 3], inv));
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                       my_row + (((uint32_t)i * 4u) ^ swz)),
                   "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                   : "memory");
      lo_run = fminf(lo_run, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
      hi_run = fmaxf(hi_run, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    fence_proxy_async_smem(); // the tiles were written through the generic proxy
    __syncthreads();
    if (tid == 0) {
      tma_store_2d(&map_out, s_vh, it.col_out, it.row_q);
      tma_store_2d(&map_out, s_vl, it.col_out + 32, it.row_q);
      tma_store_commit();
    }
  }

  if (ok && out_range && (int64_t)blockIdx.x < n_items)
    range_commit_warp(out_range, lo_run, hi_run);
  if (tid == 0)
    tma_store_wait_all();

  // ---- teardown ----
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tcgen05_fence_after();
    tmem_dealloc(tmem, kTmemColsAtt);
  }
  if (tid == 0 && abort_flag)
    atomicExch(status, 1);
}

// x [rows, cols] fp32 with row pitch ld_x -> bf16 planes hi, lo [rows, ld_p]
// at column offset col0: hi = bf16(x), lo = bf16(x - hi).
__global__ void __launch_bounds__(256)
    split_bf16_kernel(const float *__restrict__ x, int64_t rows, int64_t cols,
        int64_t ld_x, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
        int64_t ld_p, int64_t col0) {
  const int64_t c4n = cols >> 2;
  const int64_t total = rows * c4n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / c4n, c = (i % c4n) * 4;
    const float4 v = *reinterpret_cast<const float4 *>(x + r * ld_x + c);
    const uint32_t h0 = cvt_bf16x2(v.x, v.y), h1 = cvt_bf16x2(v.z, v.w);
    const uint32_t l0 = cvt_bf16x2(__fsub_rn(v.x, __uint_as_float(h0 << 16)),
        __fsub_rn(v.y, __uint_as_float(h0 & 0xffff0000u)));
    const uint32_t l1 = cvt_bf16x2(__fsub_rn(v.z, __uint_as_float(h1 << 16)),
        __fsub_rn(v.w, __uint_as_float(h1 & 0xffff0000u)));
    *reinterpret_cast<uint2 *>(hi + r * ld_p + col0 + c) = make_uint2(h0, h1);
    *reinterpret_cast<uint2 *>(lo + r * ld_p + col0 + c) = make_uint2(l0, l1);
  }
}

} // namespace

bool attention_tc_supported(int64_t B, int64_t S, int64_t heads, int64_t dh,
    int64_t ld_planes, int64_t ld_out, const void *hi, const void *lo,
    const float *out) {
  // OMCUDA_ATTENTION=mma|simt keeps the older kernels, to cross-check them.
  static const bool disabled = [] {
    const char *s = getenv("OMCUDA_ATTENTION");
    return s && (strcmp(s, "mma") == 0 || strcmp(s, "simt") == 0);
  }();
  if (disabled)
    return false;
  return dh == kTDh && S > 0 && S % kTK == 0 && B * heads > 0 &&
         B * S < (int64_t(1) << 31) && ld_planes % 8 == 0 && ld_out % 4 == 0 &&
         ((((uintptr_t)hi | (uintptr_t)lo | (uintptr_t)out) & 15u) == 0);
}

int launch_attention_tc(const void *hi, const void *lo, int64_t ld_planes,
    int64_t q_col, int64_t k_col, int64_t v_col, int64_t B, int64_t S,
    int64_t heads, float scale, float *out, int64_t ld_out, void *out_range,
    cudaStream_t st) {
  if ((q_col | k_col | v_col) % 8 != 0)
    return fail(OMCUDA_EINVAL, "Attention: column offsets must be multiples of 8");
  static PerDeviceInt attr_set;
  if (!attr_set.get()) {
    OMCUDA_CHECK(cudaFuncSetAttribute(attention_tc_kernel,
        cudaFuncAttributeMaxDynamicSharedMemorySize, kTcAttSmem));
    attr_set.set(1);
  }
  const int64_t T = B * S;
  CUtensorMap map_hi, map_lo, map_out;
  int rc = make_tma_map_2d(&map_hi, hi, T, ld_planes, ld_planes * 2, kTDh, kTK, 2, 128);
  if (rc != OMCUDA_OK)
    return rc;
  rc = make_tma_map_2d(&map_lo, lo, T, ld_planes, ld_planes * 2, kTDh, kTK, 2, 128);
  if (rc != OMCUDA_OK)
    return rc;
  // output: boxes of 128 rows x 32 fp32 columns (128-byte rows)
  rc = make_tma_map_2d(&map_out, out, T, heads * kTDh, ld_out * 4, 32, kTQ, 4, 128);
  if (rc != OMCUDA_OK)
    return rc;
  int *status = tc_status_word();
  if (!status)
    return fail(OMCUDA_ENOMEM, "Attention: cannot allocate the status word");
  const int64_t n_items = (S / kTQ) * B * heads;
  const float scale_log2e = scale * 1.4426950408889634f;
  // Persistent CTAs, two per SM, each walking its share of the
  // (batch, head, 128-query-row) items.
  const int64_t resident = (int64_t)sm_count() * 2;
  const unsigned grid = (unsigned)(n_items < resident ? n_items : resident);
  attention_tc_kernel<<<grid, kTcAttThreads, kTcAttSmem, st>>>(map_hi, map_lo, map_out,
      (int32_t)q_col, (int32_t)k_col, (int32_t)v_col, S, heads, n_items, scale_log2e,
      (uint32_t *)out_range, status, tc_wait_limit_ns());
  OMCUDA_CHECK_LAUNCH("attention_tc_kernel");
  return OMCUDA_OK;
}

int launch_split_bf16(const float *x, int64_t rows, int64_t cols, int64_t ld_x,
    void *hi, void *lo, int64_t ld_p, int64_t col0, cudaStream_t st) {
  if (cols % 4 != 0 || ld_x % 4 != 0 || ld_p % 4 != 0 || col0 % 4 != 0 ||
      (((uintptr_t)x & 15u) != 0) || ((((uintptr_t)hi | (uintptr_t)lo) & 7u) != 0))
    return fail(OMCUDA_EINVAL, "SplitBf16: rows must be 16-byte aligned");
  const int64_t total = rows * (cols >> 2);
  if (total == 0)
    return OMCUDA_OK;
  int64_t want = ceil_div(total, 256 * 4);
  const int64_t cap = (int64_t)sm_count() * 8;
  split_bf16_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(x, rows,
      cols, ld_x, (__nv_bfloat16 *)hi, (__nv_bfloat16 *)lo, ld_p, col0);
  OMCUDA_CHECK_LAUNCH("split_bf16_kernel");
  return OMCUDA_OK;
}

} // namespace omcuda

using namespace omcuda;

extern "C" int omcudaDevSplitBf16(const float *x, int64_t rows, int64_t cols,
    int64_t ld_x, void *hi, void *lo, int64_t ld_planes, int64_t col0,
    void *stream) {
  if (rows < 0 || cols < 0 || ld_x < cols || ld_planes < col0 + cols ||
      (rows > 0 && cols > 0 && (!x || !hi || !lo)))
    return fail(OMCUDA_EINVAL, "SplitBf16: bad argument");
  return launch_split_bf16(x, rows, cols, ld_x, hi, lo, ld_planes, col0,
      (cudaStream_t)stream);
}

extern "C" int omcudaDevAttentionBf16Supported(int64_t B, int64_t S,
    int64_t heads, int64_t dh, int64_t ld_planes, int64_t ld_out) {
  return attention_tc_supported(B, S, heads, dh, ld_planes, ld_out, nullptr,
             nullptr, nullptr)
             ? 1
             : 0;
}

extern "C" int omcudaDevAttentionBf16(const void *hi, const void *lo,
    int64_t ld_planes, int64_t q_col, int64_t k_col, int64_t v_col, int64_t B,
    int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    int64_t ld_out, void *out_range, void *stream) {
  if (B < 0 || S <= 0 || heads <= 0 || !hi || !lo || !out || q_col < 0 ||
      k_col < 0 || v_col < 0 || ld_out < heads * dh ||
      ld_planes < heads * dh + (q_col > k_col ? (q_col > v_col ? q_col : v_col)
                                               : (k_col > v_col ? k_col : v_col)))
    return fail(OMCUDA_EINVAL, "AttentionBf16: bad argument");
  // The kernel takes the row maximum of the raw scores and scales it
  // afterwards, which equals the maximum of the scaled scores only for a
  // positive scale.
  if (!(scale > 0.0f) || !(scale < INFINITY))
    return fail(OMCUDA_EINVAL,
        "AttentionBf16: the scale must be positive and finite (got %g); "
        "omcudaDevAttention takes any scale", (double)scale);
  if (B == 0)
    return OMCUDA_OK;
  if (!attention_tc_supported(B, S, heads, dh, ld_planes, ld_out, hi, lo, out))
    return fail(OMCUDA_ENOTSUP,
        "AttentionBf16: needs head size 64, a sequence length that is a "
        "multiple of 128 and 16-byte aligned rows");
  return launch_attention_tc(hi, lo, ld_planes, q_col, k_col, v_col, B, S, heads,
      scale, out, ld_out, out_range, (cudaStream_t)stream);
}
