// Persistent, warp-specialised bf16 GEMM for sm_100a:  C[M,N] = op(A) * op(B)^T
//
//   warp 0      : TMA producer (cp.async.bulk.tensor, 128-byte swizzle, mbarrier tx)
//   warp 1      : tcgen05.mma issuer (one thread), accumulators in TMEM, double buffered
//   warps 2..5  : epilogue, tcgen05.ld -> bias / ReLU / per-column statistics -> global
//
// Operands may be K-major (rows of the matrix are contiguous along K) or MN-major
// (stored [K][MN]); the latter is what weight-gradient GEMMs need, where K is the
// pixel dimension of NHWC activations.  Split-K with fp32 atomic accumulation
// covers the few-tiles / long-K shape of those GEMMs.  Used for dense layers,
// 1x1 convolutions (NHWC makes them plain GEMMs) and the LSTM projections; the
// reference reaches cuBLAS / cuDNN through TensorFlow for the same ops
// (official/resnet/resnet_model.py:97-101,552) and has a naive CPU GEMM
// (deep500 .../cpp/utility/gemm.hpp:9-64) that serves as the oracle.
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_count.cuh"
#include "sm100_primitives.cuh"
#include "tensormap.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ATOMIC = 2 };

struct GemmParams {
  int M, N, K;
  int ldc;
  int out_mode;
  int relu;
  int splits;
  int kb_per_split;
  void* C;
  const float* bias;       // per output column, may be null
  float* col_sum;          // optional per-column sum of the (pre-activation) output
  float* col_sqsum;        // optional per-column sum of squares
  int* error_flag;
};

template <int BN>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 + 256;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * C::B_STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles * p.splits;
  const int kb_total = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int split = t / (m_tiles * n_tiles), rem = t % (m_tiles * n_tiles);
        const int m0 = (rem / n_tiles) * BM, n0 = (rem % n_tiles) * BN;
        const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[stage], A_STAGE_BYTES + C::B_STAGE_BYTES);
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * C::B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(a_dst + i * 8192, &tmA, &full[stage], m0 + 64 * i, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
          }
          if (B_MN) {
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(b_dst + i * 8192, &tmB, &full[stage], n0 + 64 * i, k0);
          } else {
            tma_load_2d(b_dst, &tmB, &full[stage], k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int split = t / (m_tiles * n_tiles);
        const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, kb_total);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const uint64_t adesc = A_MN ? umma_smem_desc(a_addr + j * 2048, 8192, 1024)
                                        : umma_smem_desc(a_addr + j * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_addr + j * 2048, 8192, 1024)
                                        : umma_smem_desc(b_addr + j * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // smem stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps = 128 TMEM lanes)
    const int q = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int rem = t % (m_tiles * n_tiles);
      const int m0 = (rem / n_tiles) * BM, n0 = (rem % n_tiles) * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
        }
        if (p.col_sum != nullptr) {
          // per-column statistics of this tile: reduce over the warp's 32 rows, one atomic per column
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float s = row_ok ? v[j] : 0.0f, s2 = s * s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              s += __shfl_xor_sync(0xffffffffu, s, o);
              s2 += __shfl_xor_sync(0xffffffffu, s2, o);
            }
            if (lane == 0 && col0 + j < p.N) {
              atomicAdd(p.col_sum + col0 + j, s);
              atomicAdd(p.col_sqsum + col0 + j, s2);
            }
          }
        }
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        }
        if (row_ok) {
          if (p.out_mode == OUT_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (col0 + g * 8 < p.N) {
                uint4 pk;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dst + g * 8) = pk;
              }
            }
          } else if (p.out_mode == OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (col0 + g * 4 < p.N)
                *reinterpret_cast<float4*>(dst + g * 4) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          } else {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) atomicAdd(dst + j, v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {  // a bounded wait ran out: let copies in flight land before the CTA exits
    __nanosleep(1000000);
    if (threadIdx.x == 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 1);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, A_MN, B_MN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total = m_tiles * n_tiles * p.splits;
  const int grid = total < sms ? total : sms;
  gemm_bf16_kernel<BN, A_MN, B_MN><<<grid, 192, C::SMEM_BYTES, stream>>>(ta, tb, p);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

template <int BN>
int launch_major(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms,
                 cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, false, false>(ta, tb, p, sms, s);
  if (!a_mn && b_mn) return launch<BN, false, true>(ta, tb, p, sms, s);
  if (a_mn && b_mn) return launch<BN, true, true>(ta, tb, p, sms, s);
  return launch<BN, true, false>(ta, tb, p, sms, s);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace

extern "C" {

// C[M,N] = A * B^T (+bias, ReLU, column statistics).  A is [M][K] (a_mn=0, row stride lda)
// or stored [K][M] (a_mn=1); B is [N][K] (b_mn=0, row stride ldb) or stored [K][N] (b_mn=1).
// out_mode: 0 bf16, 1 fp32, 2 fp32 atomic accumulate (split-K; C must be zeroed by the caller).
// Requirements: 16-byte aligned bases, lda/ldb multiples of 8, ldc multiple of 8, N multiple of 8.
int esgd_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                   int b_mn, int out_mode, const float* bias, int relu, int splits, float* col_sum,
                   float* col_sqsum, int* error_flag, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N % 8) || (lda % 8) || (ldb % 8) || (ldc % 8)) return -1;
  const int BN = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
  CUtensorMap ta, tb;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = 128; }
    strides[0] = (uint64_t)lda * 2;
    int r = esgd::make_tensormap_bf16(&ta, A, 2, dims, strides, box, nullptr);
    if (r != 0) return 1000 + r;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = 64; }
    else { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = (uint32_t)BN; }
    strides[0] = (uint64_t)ldb * 2;
    r = esgd::make_tensormap_bf16(&tb, B, 2, dims, strides, box, nullptr);
    if (r != 0) return 2000 + r;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.out_mode = out_mode; p.relu = relu;
  const int kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  p.kb_per_split = (kb_total + splits - 1) / splits;
  p.splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  if (p.splits > 1 && out_mode != OUT_F32_ATOMIC) return -2;
  p.C = C; p.bias = bias; p.col_sum = col_sum; p.col_sqsum = col_sqsum; p.error_flag = error_flag;
  cudaStream_t s = (cudaStream_t)stream;
  const int sms = sm_count();
  if (BN == 64) return launch_major<64>(a_mn, b_mn, ta, tb, p, sms, s);
  if (BN == 128) return launch_major<128>(a_mn, b_mn, ta, tb, p, sms, s);
  return launch_major<256>(a_mn, b_mn, ta, tb, p, sms, s);
}

}  // extern "C"
