// Implicit-GEMM convolution (forward and data gradient) for NHWC bf16 on sm_100a.
//
//   y[n, p, q, k] = sum_{r, s, c} x[n, p*stride + r - pad, q*stride + s - pad, c] * w[k, r, s, c]
//
// GEMM view: M = output pixels, N = Cout, K = R*S*Cin.  One k-block is one filter
// tap (r, s) and 64 input channels: the A tile is fetched by ONE 4-D TMA load over
// the NHWC tensor — a box of BW x BH x BI output pixels shifted by the tap, with the
// hardware zero-filling everything outside the image (that is the padding) and
// element strides 2 for strided convolutions — and lands in shared memory already in
// the 128-byte-swizzled K-major layout tcgen05.mma reads.  Weights are used in their
// channels_last storage [Cout][R][S][Cin], which is the K-major B matrix as is.  The
// output tile goes back with a 4-D TMA store (clipped at the image edge) and the
// batch-norm statistics of the stored values are taken in the epilogue.
//
// The data gradient of a stride-1 convolution is the same kernel run on dy with the
// filter rotated by 180 degrees and its channel axes swapped.  The reference gets
// these ops from cuDNN through TensorFlow (official/resnet/resnet_model.py:97-101);
// its CPU restatements are deep500 .../cpp/utility/crosscorrelation.hpp:14-129 and
// conv_op.cpp:291-321.
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_count.cuh"
#include "tensormap.cuh"
#include "umma_pipeline.cuh"

using namespace umma;

namespace {

template <int BN_>
struct ConvProblem {
  static constexpr int BN = BN_;
  static constexpr bool A_MN = false, B_MN = false;
  CUtensorMap tmX, tmW, tmY;
  int N, Ho, Wo, Cout;
  int R, S, stride, pad;
  int cblks;                 // Cin / 64
  int BW, BH, BI;            // output-pixel box of a tile (BW*BH*BI <= 128)
  int w_tiles, h_tiles, i_tiles, n_tiles;
  int fixed_n;

  struct Tile { int kb0, kb1, n0, w0, h0, i0; };

  __device__ __forceinline__ bool tile(int it, Tile& t) const {
    const int m_tiles = w_tiles * h_tiles * i_tiles;
    int m_idx, n_idx;
    if (fixed_n) {
      n_idx = blockIdx.x % n_tiles;
      m_idx = blockIdx.x / n_tiles + it * (gridDim.x / n_tiles);
      if (m_idx >= m_tiles) return false;
    } else {
      const int id = blockIdx.x + it * gridDim.x;
      if (id >= m_tiles * n_tiles) return false;
      m_idx = id / n_tiles;
      n_idx = id % n_tiles;
    }
    t.w0 = (m_idx % w_tiles) * BW;
    t.h0 = ((m_idx / w_tiles) % h_tiles) * BH;
    t.i0 = (m_idx / (w_tiles * h_tiles)) * BI;
    t.n0 = n_idx * BN;
    t.kb0 = 0;
    t.kb1 = R * S * cblks;
    return true;
  }
  __device__ __forceinline__ void load(const Tile& t, int kb, uint8_t* a, uint8_t* b, uint64_t* bar) const {
    const int tap = kb / cblks, cb = kb - tap * cblks;
    const int r = tap / S, s = tap - r * S;
    tma_load_4d(a, &tmX, bar, cb * 64, t.w0 * stride + s - pad, t.h0 * stride + r - pad, t.i0);
    tma_load_2d(b, &tmW, bar, kb * 64, t.n0);
  }
  __device__ __forceinline__ void store_panel(const Tile& t, int panel, const void* smem) const {
    tma_store_4d(&tmY, smem, t.n0 + panel * 64, t.w0, t.h0, t.i0);
  }
  __device__ __forceinline__ bool row_valid(const Tile& t, int row) const {
    const int wi = row % BW, hi = (row / BW) % BH, ni = row / (BW * BH);
    return ni < BI && t.w0 + wi < Wo && t.h0 + hi < Ho && t.i0 + ni < N;
  }
  __device__ __forceinline__ void* row_ptr(const Tile&, int) const { return nullptr; }
};

template <class P>
__global__ void __launch_bounds__(NUM_THREADS, 1) conv_kernel(const __grid_constant__ P prob, const Epilogue ep) {
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&prob.tmX);
    tma_prefetch_desc(&prob.tmW);
    tma_prefetch_desc(&prob.tmY);
  }
  run(prob, ep);
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

struct ConvArgs {
  const void *x, *w;
  void* y;
  int N, H, W, Cin, Cout, R, S, stride, pad;
};

template <int BN>
int launch(const ConvArgs& a, Epilogue ep, cudaStream_t stream) {
  using P = ConvProblem<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  P p;
  p.N = a.N; p.Cout = a.Cout; p.R = a.R; p.S = a.S; p.stride = a.stride; p.pad = a.pad;
  p.Ho = (a.H + 2 * a.pad - a.R) / a.stride + 1;
  p.Wo = (a.W + 2 * a.pad - a.S) / a.stride + 1;
  p.cblks = a.Cin / 64;
  // output-pixel box: whole rows when they fit, as many rows / images as 128 GEMM rows allow
  if (p.Wo >= 128) { p.BW = 128; p.BH = 1; p.BI = 1; }
  else {
    p.BW = p.Wo;
    int max_h = 128 / p.BW;
    p.BH = 1;
    for (int d = 1; d <= max_h && d <= p.Ho; ++d) if (p.Ho % d == 0) p.BH = d;   // largest divisor of Ho that fits
    p.BI = 1;
    if (p.BH == p.Ho) { p.BI = 128 / (p.BW * p.BH); if (p.BI > a.N) p.BI = a.N; if (p.BI < 1) p.BI = 1; }
  }
  p.w_tiles = (p.Wo + p.BW - 1) / p.BW;
  p.h_tiles = (p.Ho + p.BH - 1) / p.BH;
  p.i_tiles = (a.N + p.BI - 1) / p.BI;
  p.n_tiles = (a.Cout + BN - 1) / BN;
  {
    // input: dims (C, W, H, N); box in INPUT elements = output box * stride (element strides pick every stride-th)
    uint64_t dims[4] = {(uint64_t)a.Cin, (uint64_t)a.W, (uint64_t)a.H, (uint64_t)a.N};
    uint64_t strides[3] = {(uint64_t)a.Cin * 2, (uint64_t)a.W * a.Cin * 2, (uint64_t)a.H * a.W * a.Cin * 2};
    uint32_t box[4] = {64, (uint32_t)(p.BW * a.stride), (uint32_t)(p.BH * a.stride), (uint32_t)p.BI};
    uint32_t es[4] = {1, (uint32_t)a.stride, (uint32_t)a.stride, 1};
    if (box[1] > 256 || box[2] > 256) return -5;
    int r = esgd::make_tensormap_bf16(&p.tmX, a.x, 4, dims, strides, box, es);
    if (r != 0) return 1000 + r;
  }
  {
    uint64_t dims[2] = {(uint64_t)a.R * a.S * a.Cin, (uint64_t)a.Cout};
    uint64_t strides[1] = {(uint64_t)a.R * a.S * a.Cin * 2};
    uint32_t box[2] = {64, (uint32_t)BN};
    int r = esgd::make_tensormap_bf16(&p.tmW, a.w, 2, dims, strides, box, nullptr);
    if (r != 0) return 2000 + r;
  }
  {
    uint64_t dims[4] = {(uint64_t)a.Cout, (uint64_t)p.Wo, (uint64_t)p.Ho, (uint64_t)a.N};
    uint64_t strides[3] = {(uint64_t)a.Cout * 2, (uint64_t)p.Wo * a.Cout * 2, (uint64_t)p.Ho * p.Wo * a.Cout * 2};
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    int r = esgd::make_tensormap_bf16(&p.tmY, a.y, 4, dims, strides, box, nullptr);
    if (r != 0) return 3000 + r;
  }
  const int sms = sm_count();
  const int total = p.w_tiles * p.h_tiles * p.i_tiles * p.n_tiles;
  int grid;
  p.fixed_n = (ep.col_sum != nullptr) ? 1 : 0;
  if (p.fixed_n) {
    if (p.n_tiles > sms) return -3;
    grid = (sms / p.n_tiles) * p.n_tiles;
    if (grid > total) grid = total;
  } else {
    grid = total < sms ? total : sms;
  }
  ep.a_tx_bytes = (uint32_t)(p.BW * p.BH * p.BI * 128);
  conv_kernel<P><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(p, ep);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// x: [N,H,W,Cin] bf16, w: [Cout,R,S,Cin] bf16, y: [N,Ho,Wo,Cout] bf16.  Cin % 64 == 0, Cout % 8 == 0.
// col_sum / col_sqsum (optional, caller-zeroed fp32[Cout]) receive the statistics of the stored y.
int esgd_conv2d_fwd(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S,
                    int stride, int pad, int relu, float* col_sum, float* col_sqsum, int* error_flag, void* stream) {
  if (Cin % 64 || Cout % 8 || stride < 1 || stride > 2) return -1;
  ConvArgs a{x, w, y, N, H, W, Cin, Cout, R, S, stride, pad};
  Epilogue ep;
  ep.out_mode = OUT_BF16; ep.relu = relu; ep.n_total = Cout; ep.bias = nullptr;
  ep.col_sum = col_sum; ep.col_sqsum = col_sqsum; ep.error_flag = error_flag;
  ep.a_tx_bytes = 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int BN = Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256);
  if (BN == 64) return launch<64>(a, ep, s);
  if (BN == 128) return launch<128>(a, ep, s);
  return launch<256>(a, ep, s);
}

}  // extern "C"
