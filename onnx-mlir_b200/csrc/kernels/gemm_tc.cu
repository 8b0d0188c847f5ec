// int8 x int8 -> int32 GEMM on Blackwell tensor cores (tcgen05.mma kind::i8)
// with the zero-point / dequantize / requantize epilogues of
// gemm_epilogue.cuh.  It computes what onnx-mlir's MatMulInteger and
// QLinearMatMul lowerings compute with CPU loops
// (src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:59-90,
//  src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:89-138,
//  src/Conversion/ONNXToKrnl/Math/MatMul.cpp:278-327).
//
// Data layout in HBM: A is [M,K] row-major 8-bit (K-major, as ONNX gives it);
// B is the prepared K-major copy Bt[N][kp] (gemm_simt.cu); Y is [M,N]
// row-major i32 / f32 / 8-bit.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of a 128x128-byte A
//              tile and a BNx128-byte Bt tile per pipeline stage, 128-byte
//              swizzle, completion on an mbarrier.  Plain (non-multicast)
//              loads only.
//   warp 1     allocates tensor memory; its lane 0 issues tcgen05.mma
//              (M=128, N=BN, K=32 per instruction, four per stage) into one of
//              two TMEM accumulator buffers and commits to mbarriers to free
//              the smem stage / publish the accumulator.
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp owns the 32
//              TMEM lanes its id modulo 4 selects), apply the epilogue, store.
// The two accumulator buffers let the epilogue of tile i overlap the MMAs of
// tile i+1.
//
// Every wait on an mbarrier is bounded: after about two seconds without
// progress the waiting thread raises a CTA-wide abort flag, the kernel writes
// a non-zero word to *status, releases its tensor memory and returns.
#include <cuda.h>

#include "../runtime/internal.h"
#include "gemm_epilogue.cuh"

namespace omcuda {

namespace {

constexpr int kBM = 128;       // rows of A per tile
constexpr int kBK = 128;       // bytes (= int8 elements) of K per stage
constexpr int kUmmaK = 32;     // K of one tcgen05.mma kind::i8
constexpr int kThreads = 192;  // 6 warps
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// ---- PTX wrappers -------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(
    uint32_t bar, uint32_t parity, volatile int *abort_flag, uint64_t t0) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag)
        return false;
      if (global_timer() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map,
    int32_t x, int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_dst),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                   : "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread
// has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
        "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128
// bytes with the 128-byte swizzle (what the TMA loads above write): eight rows
// form one 1024-byte swizzle atom, so the stride between 8-row groups is 1024
// bytes; the leading-dimension offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused)
  d |= (uint64_t)(1024u >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                    // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                    // layout: 128-byte swizzle
  return d;
}

template <int BN>
struct TcConfig {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN; // two accumulator buffers
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024; // + align slack
};

// ---- epilogue store helpers -----------------------------------------------------

template <typename T>
__device__ __forceinline__ void store_chunk32(T *dst, const uint32_t (&w)[32],
    int valid, bool vec_ok) {
  // dst points at 32 consecutive 4-byte outputs of one row.
  if (vec_ok && valid == 32) {
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      d4[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  } else {
    uint32_t *d = reinterpret_cast<uint32_t *>(dst);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid)
        d[j] = w[j];
  }
}

} // namespace

// ---- the kernel -------------------------------------------------------------------

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap map_a,
        const __grid_constant__ CUtensorMap map_b, EpiParams p, uint32_t idesc,
        int *status) {
  using Cfg = TcConfig<BN>;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kStages];
  __shared__ uint64_t bar_empty[kStages];
  __shared__ uint64_t bar_acc_full[2];
  __shared__ uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t t0 = global_timer();

  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int64_t tiles_m = ceil_div(p.M, kBM);
  const int64_t tiles_n = ceil_div(p.N, BN);
  const int64_t num_tiles = tiles_m * tiles_n;
  const int num_kb = (int)ceil_div(p.K, kBK);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), 4); // one arrive per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1)
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int *abortp = &abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int32_t m0 = (int32_t)((t / tiles_n) * kBM);
        const int32_t n0 = (int32_t)((t % tiles_n) * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, t0)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[stage]);
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          mbar_expect_tx(full, Cfg::kStageBytes);
          tma_load_2d(sa, &map_a, kb * kBK, m0, full);
          tma_load_2d(sb, &map_b, kb * kBK, n0, full);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t it = 0;
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_phase ^ 1u, abortp, t0)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, t0)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t adesc = make_smem_desc(sa + kk * kUmmaK);
            const uint64_t bdesc = make_smem_desc(sb + kk * kUmmaK);
            umma_i8(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_empty[stage]));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok)
          umma_commit(smem_u32(&bar_acc_full[buf]));
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32)
    const EpiScalars sc = epi_scalars(p);
    const bool y4_ok = ((p.N & 3) == 0) && (((uintptr_t)p.Y & 15u) == 0);
    const bool y1_ok = ((p.N & 15) == 0) && (((uintptr_t)p.Y & 15u) == 0);
    bool ok = true;
    int64_t it = 0;
    for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int buf = (int)(it & 1);
      const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
      const int64_t m = (t / tiles_n) * kBM + quad * 32 + lane;
      const int64_t n0 = (t % tiles_n) * BN;
      if (!mbar_wait(smem_u32(&bar_acc_full[buf]), acc_phase, abortp, t0)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const bool row_ok = m < p.M;
      EpiRow row;
      row.az = 0;
      row.rs = 0;
      if (row_ok)
        row = epi_row(p, m);
      float lo = INFINITY, hi = -INFINITY;
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld is warp-collective: enter it converged
        tmem_ld32(taddr + (uint32_t)c, v);
        tmem_ld_wait();
        const int64_t nc = n0 + c;
        int valid = (int)((p.N - nc) < 32 ? (p.N - nc) : 32);
        if (!row_ok || valid <= 0) {
          // rows / columns past the edge of Y: nothing to store
        } else if (p.kind == OMCUDA_EPI_I32) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid)
              v[j] = (uint32_t)epi_int(p, row, (int32_t)v[j], nc + j);
          store_chunk32(reinterpret_cast<int32_t *>(p.Y) + m * p.N + nc, v,
              valid, y4_ok);
        } else if (p.kind == OMCUDA_EPI_DEQUANT) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < valid) {
              int32_t a = epi_int(p, row, (int32_t)v[j], nc + j);
              float y = epi_dequant(p, sc, a, nc + j);
              lo = fminf(lo, y);
              hi = fmaxf(hi, y);
              v[j] = __float_as_uint(y);
            }
          }
          store_chunk32(reinterpret_cast<float *>(p.Y) + m * p.N + nc, v,
              valid, y4_ok);
        } else {
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            packed[j] = 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < valid) {
              int32_t a = epi_int(p, row, (int32_t)v[j], nc + j);
              packed[j >> 2] |= epi_requant(p, sc, a, nc + j) << (8 * (j & 3));
            }
          }
          uint8_t *dst = reinterpret_cast<uint8_t *>(p.Y) + m * p.N + nc;
          if (y1_ok && valid == 32) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst);
            d4[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            d4[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
            for (int j = 0; j < valid; ++j)
              dst[j] = (uint8_t)(packed[j >> 2] >> (8 * (j & 3)));
          }
        }
      }
      // The accumulator buffer may be overwritten once all four warps are done.
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(smem_u32(&bar_acc_empty[buf]));
      if (p.out_range && p.kind == OMCUDA_EPI_DEQUANT)
        epi_range_commit(p.out_range, lo, hi);
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && abort_flag)
    atomicExch(status, 1);
}

// ---- host side ----------------------------------------------------------------------

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
    void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault,
            &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  }
  return fn;
}

// 2-D map over a row-major [rows, cols_bytes] byte matrix whose row pitch is
// pitch bytes; box = 128 bytes x box_rows, 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t cols,
    int64_t pitch, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn)
    return fail(OMCUDA_ECUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base),
      dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(OMCUDA_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return OMCUDA_OK;
}

// Instruction descriptor of tcgen05.mma kind::i8: s32 accumulator, operand
// signedness per operand, both operands K-major, N and M of the instruction.
uint32_t make_idesc(int a_signed, int b_signed, int n) {
  uint32_t d = 0;
  d |= 2u << 4;                        // accumulator format: s32
  d |= (a_signed ? 1u : 0u) << 7;      // A: 0 = u8, 1 = s8
  d |= (b_signed ? 1u : 0u) << 10;     // B: 0 = u8, 1 = s8
  d |= (uint32_t)(n >> 3) << 17;       // N / 8
  d |= (uint32_t)(kBM >> 4) << 24;     // M / 16
  return d;
}

int *g_status_word = nullptr;

int *status_word() {
  if (!g_status_word) {
    if (cudaMalloc(&g_status_word, sizeof(int)) != cudaSuccess)
      return nullptr;
    cudaMemset(g_status_word, 0, sizeof(int));
  }
  return g_status_word;
}

template <int BN>
int launch_bn(const omcudaGemmArgs &a, cudaStream_t st) {
  using Cfg = TcConfig<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    OMCUDA_CHECK(cudaFuncSetAttribute(gemm_i8_tc_kernel<BN>,
        cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, a.A, a.M, a.K, a.K, kBM);
  if (rc != OMCUDA_OK)
    return rc;
  rc = make_map(&map_b, a.B.bt, a.N, a.B.kp, a.B.kp, BN);
  if (rc != OMCUDA_OK)
    return rc;
  int *status = status_word();
  if (!status)
    return fail(OMCUDA_ENOMEM, "GemmI8: cannot allocate the status word");
  EpiParams p = make_epi_params(a);
  int64_t tiles = ceil_div(a.M, kBM) * ceil_div(a.N, BN);
  int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  uint32_t idesc = make_idesc(a.a_signed, a.B.b_signed, BN);
  gemm_i8_tc_kernel<BN><<<grid, kThreads, Cfg::kSmemBytes, st>>>(
      map_a, map_b, p, idesc, status);
  OMCUDA_CHECK_LAUNCH("gemm_i8_tc_kernel");
  return OMCUDA_OK;
}

} // namespace

bool gemm_tc_supported(const omcudaGemmArgs &a) {
  return (a.K % 16 == 0) && (((uintptr_t)a.A & 15u) == 0) &&
         (((uintptr_t)a.B.bt & 15u) == 0) && a.M < (int64_t(1) << 31) &&
         a.N < (int64_t(1) << 31);
}

int launch_gemm_tc(const omcudaGemmArgs &a, cudaStream_t st) {
  // Tile width: the widest tile that still gives every SM work.
  const int64_t tm = ceil_div(a.M, kBM);
  const int sms = sm_count();
  if (a.N > 128 && tm * ceil_div(a.N, 256) >= sms)
    return launch_bn<256>(a, st);
  if (a.N > 64 && tm * ceil_div(a.N, 128) >= sms / 2)
    return launch_bn<128>(a, st);
  return launch_bn<64>(a, st);
}

// Reads (and clears) the word the GEMM kernels raise when a bounded wait gave
// up.  Synchronises the stream.
int gemm_tc_check_status(cudaStream_t st) {
  if (!g_status_word)
    return OMCUDA_OK;
  int h = 0;
  OMCUDA_CHECK(cudaMemcpyAsync(&h, g_status_word, sizeof(int),
      cudaMemcpyDeviceToHost, st));
  OMCUDA_CHECK(cudaStreamSynchronize(st));
  if (h != 0) {
    cudaMemsetAsync(g_status_word, 0, sizeof(int), st);
    return fail(OMCUDA_ETIMEDOUT,
        "int8 GEMM: a device-side wait on the TMA/MMA pipeline timed out");
  }
  return OMCUDA_OK;
}

} // namespace omcuda
