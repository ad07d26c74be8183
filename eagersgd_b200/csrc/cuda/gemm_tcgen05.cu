// bf16 GEMM on tcgen05 / TMEM / TMA for sm_100a:  C[M,N] = op(A) * op(B)^T
//
// Operands may be K-major (rows contiguous along K) or MN-major (stored [K][MN]);
// the latter is what weight-gradient GEMMs over NHWC activations need, where K is
// the pixel dimension.  Split-K with fp32 atomic accumulation covers their
// few-tiles / long-K shape.  Used for dense layers, 1x1 convolutions (NHWC makes
// them plain GEMMs) and the LSTM projections; the reference reaches cuBLAS / cuDNN
// through TensorFlow for the same ops (official/resnet/resnet_model.py:97-101,552)
// and has a naive CPU GEMM (deep500 .../cpp/utility/gemm.hpp:9-64), the oracle.
// The pipeline itself (producer / MMA / epilogue warps) lives in umma_pipeline.cuh.
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_count.cuh"
#include "tensormap.cuh"
#include "umma_pipeline.cuh"

using namespace umma;

namespace {

template <int BN_, bool A_MN_, bool B_MN_>
struct GemmProblem {
  static constexpr int BN = BN_;
  static constexpr bool A_MN = A_MN_, B_MN = B_MN_, kZeroStages = false, kHalo = false;
  CUtensorMap tmA, tmB, tmC, tmR;   // tmR: optional residual, same geometry as the output
  int M, N, K;
  int m_tiles, n_tiles, splits, kb_total, kb_per_split;
  int fixed_n;        // every CTA keeps one column range (needed for the per-CTA statistics flush)
  int res_kb;         // > 0: all k-blocks of B for the CTA's column range stay in shared memory
  float* c_f32;       // fp32 output (direct modes)
  int ldc;
  int chained;        // launched with programmatic stream serialization: wait for the previous kernel in the kernel

  struct Tile { int kb0, kb1, n0, m0; };

  __device__ __forceinline__ bool tile(int it, Tile& t) const {
    int m_idx, n_idx, split = 0;
    if (fixed_n) {
      n_idx = blockIdx.x % n_tiles;
      m_idx = blockIdx.x / n_tiles + it * (gridDim.x / n_tiles);
      if (m_idx >= m_tiles) return false;
    } else {
      const int id = blockIdx.x + it * gridDim.x;
      if (id >= m_tiles * n_tiles * splits) return false;
      split = id / (m_tiles * n_tiles);
      const int rem = id % (m_tiles * n_tiles);
      m_idx = rem / n_tiles;
      n_idx = rem % n_tiles;
    }
    t.m0 = m_idx * BM;
    t.n0 = n_idx * BN;
    t.kb0 = split * kb_per_split;
    t.kb1 = min(t.kb0 + kb_per_split, kb_total);
    return true;
  }
  __device__ __forceinline__ void load_a(const Tile& t, int kb, uint8_t* a, uint64_t* bar) const {
    const int k0 = kb * BK;
    if (A_MN) {
#pragma unroll
      for (int i = 0; i < BM / 64; ++i) tma_load_2d(a + i * 8192, &tmA, bar, t.m0 + 64 * i, k0);
    } else {
      tma_load_2d(a, &tmA, bar, k0, t.m0);
    }
  }
  __device__ __forceinline__ void load_b(const Tile& t, int kb, uint8_t* b, uint64_t* bar) const {
    const int k0 = kb * BK;
    if (B_MN) {
#pragma unroll
      for (int i = 0; i < BN / 64; ++i) tma_load_2d(b + i * 8192, &tmB, bar, t.n0 + 64 * i, k0);
    } else {
      tma_load_2d(b, &tmB, bar, k0, t.n0);
    }
  }
  __device__ __forceinline__ void load(const Tile& t, int kb, uint8_t* a, uint8_t* b, uint64_t* bar) const {
    load_a(t, kb, a, bar);
    load_b(t, kb, b, bar);
  }
  __device__ __forceinline__ void store_panel(const Tile& t, int panel, const void* smem) const {
    tma_store_2d(&tmC, smem, t.n0 + panel * 64, t.m0);
  }
  __device__ __forceinline__ bool row_valid(const Tile& t, int row) const { return t.m0 + row < M; }
  __device__ __forceinline__ int out_row(int row) const { return row; }
  __device__ __forceinline__ int valid_prefix(const Tile& t) const { return min(BM, M - t.m0); }
  __device__ __forceinline__ void load_res_panel(const Tile& t, int panel, void* smem, uint64_t* bar) const {
    tma_load_2d(smem, &tmR, bar, t.n0 + panel * 64, t.m0);
  }
  __device__ __forceinline__ void* row_ptr(const Tile& t, int row) const {
    return (t.m0 + row < M) ? (void*)(c_f32 + (size_t)(t.m0 + row) * ldc) : nullptr;
  }
};

template <class P>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_kernel(const __grid_constant__ P prob, const Epilogue ep) {
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&prob.tmA);
    tma_prefetch_desc(&prob.tmB);
  }
  if (prob.chained) {
    // This grid was allowed to start while the kernel before it in the stream was still running (its launch
    // latency is hidden that way): nothing of that kernel's output may be touched before this returns.  The
    // kernel after this one may be scheduled now; it waits for this grid in the same way.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  run(prob, ep);
}

// Set by callers that issue a chain of dependent launches (the LSTM time loop) around their calls.
thread_local int g_chained = 0;

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

struct GemmArgs {
  const void *A, *B;
  void* C;
  int M, N, K, lda, ldb, ldc, out_mode, splits;
};

template <int BN, bool A_MN, bool B_MN>
int launch(const GemmArgs& g, Epilogue ep, cudaStream_t stream) {
  using P = GemmProblem<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  P p;
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (A_MN) { dims[0] = (uint64_t)g.M; dims[1] = (uint64_t)g.K; box[0] = 64; box[1] = 64; }
  else { dims[0] = (uint64_t)g.K; dims[1] = (uint64_t)g.M; box[0] = 64; box[1] = 128; }
  strides[0] = (uint64_t)g.lda * 2;
  int r = esgd::make_tensormap_bf16(&p.tmA, g.A, 2, dims, strides, box, nullptr);
  if (r != 0) return 1000 + r;
  if (B_MN) { dims[0] = (uint64_t)g.N; dims[1] = (uint64_t)g.K; box[0] = 64; box[1] = 64; }
  else { dims[0] = (uint64_t)g.K; dims[1] = (uint64_t)g.N; box[0] = 64; box[1] = (uint32_t)BN; }
  strides[0] = (uint64_t)g.ldb * 2;
  r = esgd::make_tensormap_bf16(&p.tmB, g.B, 2, dims, strides, box, nullptr);
  if (r != 0) return 2000 + r;
  if (g.out_mode == OUT_BF16) {
    dims[0] = (uint64_t)g.N; dims[1] = (uint64_t)g.M; box[0] = 64; box[1] = 128;
    strides[0] = (uint64_t)g.ldc * 2;
    r = esgd::make_tensormap_bf16(&p.tmC, g.C, 2, dims, strides, box, nullptr);
    if (r != 0) return 3000 + r;
  } else {
    p.tmC = p.tmA;  // unused
  }
  p.tmR = p.tmC;
  if (ep.residual != nullptr) {
    dims[0] = (uint64_t)g.N; dims[1] = (uint64_t)g.M; box[0] = 64; box[1] = 128;
    strides[0] = (uint64_t)ep.ldr * 2;
    r = esgd::make_tensormap_bf16(&p.tmR, ep.residual, 2, dims, strides, box, nullptr);
    if (r != 0) return 4000 + r;
  }
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.m_tiles = (g.M + BM - 1) / BM;
  p.n_tiles = (g.N + BN - 1) / BN;
  p.kb_total = (g.K + BK - 1) / BK;
  int splits = g.splits < 1 ? 1 : g.splits;
  if (splits > p.kb_total) splits = p.kb_total;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  if (p.splits > 1 && g.out_mode != OUT_F32_ATOMIC) return -2;
  p.c_f32 = (float*)g.C;
  p.ldc = g.ldc;
  const int sms = sm_count();
  int grid;
  // B stays in shared memory when its whole K extent fits beside four A stages and every CTA has several
  // tiles of one column range to amortise the load over
  const bool resident = resident_enabled() && p.splits == 1 && p.kb_total <= Cfg<BN>::MAX_RES_KB &&
                        p.n_tiles <= sms / 2 && p.m_tiles >= 2 * (sms / p.n_tiles);
  p.res_kb = resident ? p.kb_total : 0;
  p.fixed_n = (ep.col_sum != nullptr || resident) ? 1 : 0;
  if (p.fixed_n) {
    if (p.splits != 1 || p.n_tiles > sms) return -3;
    const int total = p.m_tiles * p.n_tiles;
    grid = (sms / p.n_tiles) * p.n_tiles;
    if (grid > total) grid = total;
  } else {
    const int total = p.m_tiles * p.n_tiles * p.splits;
    grid = total < sms ? total : sms;
  }
  p.chained = g_chained;
  esgd::count_launch();
  if (p.chained) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg<BN>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_kernel<P>, p, ep);
  }
  gemm_kernel<P><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(p, ep);
  return (int)cudaGetLastError();
}

template <int BN>
int launch_major(int a_mn, int b_mn, const GemmArgs& g, const Epilogue& ep, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, false, false>(g, ep, s);
  if (!a_mn && b_mn) return launch<BN, false, true>(g, ep, s);
  if (a_mn && b_mn) return launch<BN, true, true>(g, ep, s);
  return launch<BN, true, false>(g, ep, s);
}

}  // namespace

extern "C" {

// C[M,N] = A * B^T (+bias, ReLU, column statistics).  A is [M][K] (a_mn=0, row stride lda)
// or stored [K][M] (a_mn=1); B is [N][K] (b_mn=0, row stride ldb) or stored [K][N] (b_mn=1).
// out_mode: 0 bf16, 1 fp32, 2 fp32 atomic accumulate (split-K; C must be zeroed by the caller).
// Requirements: 16-byte aligned bases, lda/ldb/ldc multiples of 8, N multiple of 8.
// col_sum / col_sqsum (bf16 output only) accumulate into caller-zeroed fp32 arrays of N.
// residual (bf16 output only): a bf16 [M][N] tensor with row stride ldr (multiple of 8), added before rounding.
int esgd_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                   int b_mn, int out_mode, const float* bias, int relu, int splits, float* col_sum,
                   float* col_sqsum, const void* residual, int ldr, int* error_flag, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N % 8) || (lda % 8) || (ldb % 8) || (ldc % 8)) return -1;
  if (col_sum != nullptr && out_mode != OUT_BF16) return -4;
  if (residual != nullptr && (out_mode != OUT_BF16 || (ldr % 8) || ((uintptr_t)residual & 15))) return -5;
  if (out_mode != OUT_BF16 && (((uintptr_t)C & 15) || ((uintptr_t)bias & 15))) return -6;   // 16-byte fp32 accesses
  GemmArgs g{A, B, C, M, N, K, lda, ldb, ldc, out_mode, splits};
  Epilogue ep;
  ep.out_mode = out_mode; ep.relu = relu; ep.n_total = N; ep.bias = bias;
  ep.col_sum = col_sum; ep.col_sqsum = col_sqsum; ep.error_flag = error_flag;
  ep.tx_bytes = 0; ep.tx_bytes_a = 0;
  ep.residual = residual; ep.ldr = ldr;
  cudaStream_t s = (cudaStream_t)stream;
  const int BN = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
  if (BN == 64) return launch_major<64>(a_mn, b_mn, g, ep, s);
  if (BN == 128) return launch_major<128>(a_mn, b_mn, g, ep, s);
  return launch_major<256>(a_mn, b_mn, g, ep, s);
}

// Launches of this thread from now on are links of a chain of dependent kernels (1) or ordinary launches (0).
void esgd_gemm_set_chained(int on) { g_chained = on; }

}  // extern "C"
