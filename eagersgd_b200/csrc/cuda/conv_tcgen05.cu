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
#include <stdlib.h>
#include "launch_count.cuh"
#include "tensormap.cuh"
#include "umma_pipeline.cuh"

using namespace umma;

namespace {

template <int BN_>
struct ConvProblem {
  static constexpr int BN = BN_;
  static constexpr bool A_MN = false, B_MN = false, kZeroStages = false, kHalo = false;
  CUtensorMap tmX, tmW, tmY;
  int N, Ho, Wo, Cout;
  int R, S, stride, pad;
  int cblks;                 // Cin / 64
  int BW, BH, BI;            // output-pixel box of a tile (BW*BH*BI <= 128)
  int w_tiles, h_tiles, i_tiles, n_tiles;
  int fixed_n;
  int res_kb;                // > 0: the whole filter bank of the CTA's channel range stays in shared memory

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
  __device__ __forceinline__ void load_a(const Tile& t, int kb, uint8_t* a, uint64_t* bar) const {
    const int tap = kb / cblks, cb = kb - tap * cblks;
    const int r = tap / S, s = tap - r * S;
    tma_load_4d(a, &tmX, bar, cb * 64, t.w0 * stride + s - pad, t.h0 * stride + r - pad, t.i0);
  }
  __device__ __forceinline__ void load_b(const Tile& t, int kb, uint8_t* b, uint64_t* bar) const {
    tma_load_2d(b, &tmW, bar, kb * 64, t.n0);
  }
  __device__ __forceinline__ void load(const Tile& t, int kb, uint8_t* a, uint8_t* b, uint64_t* bar) const {
    load_a(t, kb, a, bar);
    load_b(t, kb, b, bar);
  }
  __device__ __forceinline__ void store_panel(const Tile& t, int panel, const void* smem) const {
    tma_store_4d(&tmY, smem, t.n0 + panel * 64, t.w0, t.h0, t.i0);
  }
  __device__ __forceinline__ bool row_valid(const Tile& t, int row) const {
    const int wi = row % BW, hi = (row / BW) % BH, ni = row / (BW * BH);
    return ni < BI && t.w0 + wi < Wo && t.h0 + hi < Ho && t.i0 + ni < N;
  }
  __device__ __forceinline__ int valid_prefix(const Tile& t) const {   // box inside the tensor: its pixels, in order
    return (t.w0 + BW <= Wo && t.h0 + BH <= Ho && t.i0 + BI <= N) ? BW * BH * BI : -1;
  }
  __device__ __forceinline__ void* row_ptr(const Tile&, int) const { return nullptr; }
  __device__ __forceinline__ void load_res_panel(const Tile&, int, void*, uint64_t*) const {}
  __device__ __forceinline__ int out_row(int row) const { return row; }
};

// Stride-1 convolution whose taps are shifted views of one input box per 64-channel block (halo mode of the
// pipeline).  A tile is BH full output rows of one image; GEMM row m stands for the pixel (m / PW, m % PW) of
// the box pitch PW = Wo + S - 1, so the S - 1 margin columns of every row (and the rows past BH * PW) compute
// values that are dropped: out_row() gives a GEMM row its place in the dense [BH][Wo] tile that is stored.
template <int BN_>
struct ConvHaloProblem {
  static constexpr int BN = BN_;
  static constexpr bool A_MN = false, B_MN = false, kZeroStages = false, kHalo = true;
  CUtensorMap tmX, tmW, tmY;
  int N, Ho, Wo, Cout;
  int R, S, pad;
  int cblks;                 // Cin / 64
  int BH, PW;                // output rows per tile, pixel pitch of the input box
  int h_tiles, n_tiles;
  int res_kb;                // > 0: the filter bank of the CTA's channel range is resident

  struct Tile { int kb0, kb1, n0, h0, i0; };

  __device__ __forceinline__ bool tile(int it, Tile& t) const {
    const int n_idx = blockIdx.x % n_tiles;
    const int m_idx = blockIdx.x / n_tiles + it * (gridDim.x / n_tiles);
    if (m_idx >= h_tiles * N) return false;
    t.h0 = (m_idx % h_tiles) * BH;
    t.i0 = m_idx / h_tiles;
    t.n0 = n_idx * BN;
    t.kb0 = 0;
    t.kb1 = R * S * cblks;
    return true;
  }
  __device__ __forceinline__ void load_halo(const Tile& t, int cb, void* smem, uint64_t* bar) const {
    tma_load_4d(smem, &tmX, bar, cb * 64, -pad, t.h0 - pad, t.i0);
  }
  __device__ __forceinline__ void load_b(const Tile& t, int kb, uint8_t* b, uint64_t* bar) const {
    tma_load_2d(b, &tmW, bar, kb * 64, t.n0);
  }
  __device__ __forceinline__ void load_a(const Tile&, int, uint8_t*, uint64_t*) const {}
  __device__ __forceinline__ void load(const Tile&, int, uint8_t*, uint8_t*, uint64_t*) const {}
  __device__ __forceinline__ void store_panel(const Tile& t, int panel, const void* smem) const {
    tma_store_4d(&tmY, smem, t.n0 + panel * 64, 0, t.h0, t.i0);
  }
  __device__ __forceinline__ int out_row(int row) const {
    const int hl = row / PW, wl = row - hl * PW;
    return (hl < BH && wl < Wo) ? hl * Wo + wl : -1;
  }
  __device__ __forceinline__ bool row_valid(const Tile&, int row) const { return row < BH * Wo; }
  __device__ __forceinline__ int valid_prefix(const Tile&) const { return BH * Wo; }
  __device__ __forceinline__ void* row_ptr(const Tile&, int) const { return nullptr; }
  __device__ __forceinline__ void load_res_panel(const Tile&, int, void*, uint64_t*) const {}
};


// Weight gradient:  dw[k, r, s, c] = sum over output pixels of dy[pixel, k] * x[pixel shifted by tap (r, s), c].
// GEMM view per tap: M = Cout, N = Cin, K = pixels.  Both operands are "MN-major" (the pixel dimension is the
// row of the NHWC storage): a k-block is a box of up to 64 output pixels, loaded once from dy (two 64-channel
// atoms for the 128 MMA rows) and once from x at the tap's offset (zero-filled outside the image, element
// strides for stride 2).  Boxes smaller than 64 pixels leave the tail rows of the stage at their initial
// zeros.  Work is split over taps, channel tiles and pixel ranges (split-K) and meets in fp32 atomics.
template <int BN_>
struct ConvWgradProblem {
  static constexpr int BN = BN_;
  static constexpr bool A_MN = true, B_MN = true, kZeroStages = true;
  CUtensorMap tmDY, tmX;
  int N, Ho, Wo, Cout, Cin;
  int R, S, stride, pad;
  int BW, BH, BI, w_tiles, h_tiles, i_tiles;
  int m_tiles, n_tiles, splits, boxes_total, boxes_per_split;
  float* dw;   // [Cout][R*S][Cin]
  static constexpr int res_kb = 0;   // both operands change with every k-block

  struct Tile { int kb0, kb1, n0, m0, tap; };

  __device__ __forceinline__ bool tile(int it, Tile& t) const {
    const int taps = R * S;
    const int per_split = taps * m_tiles * n_tiles;
    const int id = blockIdx.x + it * gridDim.x;
    if (id >= per_split * splits) return false;
    const int split = id / per_split;       // neighbouring CTAs share a pixel range: the boxes are reused out of L2
    int rem = id - split * per_split;
    t.tap = rem % taps; rem /= taps;
    t.n0 = (rem % n_tiles) * BN;
    t.m0 = (rem / n_tiles) * BM;
    t.kb0 = split * boxes_per_split;
    t.kb1 = min(t.kb0 + boxes_per_split, boxes_total);
    return true;
  }
  __device__ __forceinline__ void load(const Tile& t, int kb, uint8_t* a, uint8_t* b, uint64_t* bar) const {
    const int w0 = (kb % w_tiles) * BW, h0 = ((kb / w_tiles) % h_tiles) * BH, i0 = (kb / (w_tiles * h_tiles)) * BI;
    const int r = t.tap / S, s = t.tap - r * S;
#pragma unroll
    for (int i = 0; i < BM / 64; ++i) tma_load_4d(a + i * 8192, &tmDY, bar, t.m0 + 64 * i, w0, h0, i0);
#pragma unroll
    for (int i = 0; i < BN / 64; ++i)
      tma_load_4d(b + i * 8192, &tmX, bar, t.n0 + 64 * i, w0 * stride + s - pad, h0 * stride + r - pad, i0);
  }
  __device__ __forceinline__ void load_a(const Tile&, int, uint8_t*, uint64_t*) const {}
  __device__ __forceinline__ void load_b(const Tile&, int, uint8_t*, uint64_t*) const {}
  __device__ __forceinline__ void store_panel(const Tile&, int, const void*) const {}
  __device__ __forceinline__ bool row_valid(const Tile& t, int row) const { return t.m0 + row < Cout; }
  __device__ __forceinline__ int valid_prefix(const Tile& t) const { return min(BM, Cout - t.m0); }
  __device__ __forceinline__ void load_res_panel(const Tile&, int, void*, uint64_t*) const {}
  __device__ __forceinline__ int out_row(int row) const { return row; }
  static constexpr bool kHalo = false;
  __device__ __forceinline__ void* row_ptr(const Tile& t, int row) const {
    const int k = t.m0 + row;
    return k < Cout ? (void*)(dw + ((size_t)k * (R * S) + t.tap) * Cin) : nullptr;
  }
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

template <class P>
__global__ void __launch_bounds__(NUM_THREADS, 1) conv_wgrad_kernel(const __grid_constant__ P prob, const Epilogue ep) {
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&prob.tmX);
    tma_prefetch_desc(&prob.tmDY);
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
  int out_h = 0, out_w = 0;                 // output extent override (0: from the usual formula)
  int64_t ys_w = 0, ys_h = 0, ys_n = 0;     // output strides in elements (0: dense NHWC)
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
  p.Ho = a.out_h ? a.out_h : (a.H + 2 * a.pad - a.R) / a.stride + 1;
  p.Wo = a.out_w ? a.out_w : (a.W + 2 * a.pad - a.S) / a.stride + 1;
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
    if (a.ys_w) { strides[0] = (uint64_t)a.ys_w * 2; strides[1] = (uint64_t)a.ys_h * 2; strides[2] = (uint64_t)a.ys_n * 2; }
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    int r = esgd::make_tensormap_bf16(&p.tmY, a.y, 4, dims, strides, box, nullptr);
    if (r != 0) return 3000 + r;
  }
  const int sms = sm_count();
  const int total = p.w_tiles * p.h_tiles * p.i_tiles * p.n_tiles;
  int grid;
  // the filter bank of the CTA's channel range stays in shared memory when it fits beside four input stages
  const int kb_total = a.R * a.S * p.cblks;
  const bool resident = resident_enabled() && kb_total <= Cfg<BN>::MAX_RES_KB && p.n_tiles <= sms / 2 &&
                        total / p.n_tiles >= 2 * (sms / p.n_tiles);
  p.res_kb = resident ? kb_total : 0;
  p.fixed_n = (ep.col_sum != nullptr || resident) ? 1 : 0;
  if (p.fixed_n) {
    if (p.n_tiles > sms) return -3;
    grid = (sms / p.n_tiles) * p.n_tiles;
    if (grid > total) grid = total;
  } else {
    grid = total < sms ? total : sms;
  }
  ep.tx_bytes_a = (uint32_t)(p.BW * p.BH * p.BI * 128);
  ep.residual = nullptr; ep.ldr = 0;
  ep.tx_bytes = ep.tx_bytes_a + (uint32_t)Cfg<BN>::B_STAGE_BYTES;
  conv_kernel<P><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(p, ep);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

// Halo mode applies to stride-1 convolutions with full-width tiles: the box (output rows + filter margin, full
// width + margin, 64 channels) and the rows its most shifted view reaches must fit in one HALO_BYTES slot.
bool halo_applicable(const ConvArgs& a, int Ho, int Wo, int* bh_out) {
  if (a.stride != 1 || a.R * a.S < 2 || a.out_h || a.out_w || a.ys_w) return false;
  const char* e = getenv("ESGD_CONV_HALO");
  if (e != nullptr && e[0] == '0') return false;
  const int PW = Wo + a.S - 1;
  if (PW > 128 || PW != a.W + 2 * a.pad || Ho + a.R - 1 != a.H + 2 * a.pad) return false;
  int bh = 0;
  for (int d = 1; d * PW <= BM && d <= Ho; ++d) if (Ho % d == 0) bh = d;
  if (bh == 0) return false;
  if (bh * Wo < 64) return false;                                   // too few real rows per tile: keep multi-image tiles
  const int view_rows = (a.R - 1) * PW + (a.S - 1) + BM;            // rows the last tap's view may touch
  if (view_rows * 128 > HALO_BYTES || (bh + a.R - 1) * PW * 128 > HALO_BYTES) return false;
  *bh_out = bh;
  return true;
}

template <int BN>
int launch_halo(const ConvArgs& a, Epilogue ep, int bh, cudaStream_t stream) {
  using P = ConvHaloProblem<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  P p;
  p.N = a.N; p.Cout = a.Cout; p.R = a.R; p.S = a.S; p.pad = a.pad;
  p.Ho = a.H + 2 * a.pad - a.R + 1;
  p.Wo = a.W + 2 * a.pad - a.S + 1;
  p.cblks = a.Cin / 64;
  p.BH = bh;
  p.PW = p.Wo + a.S - 1;
  p.h_tiles = p.Ho / bh;
  p.n_tiles = (a.Cout + BN - 1) / BN;
  {
    uint64_t dims[4] = {(uint64_t)a.Cin, (uint64_t)a.W, (uint64_t)a.H, (uint64_t)a.N};
    uint64_t strides[3] = {(uint64_t)a.Cin * 2, (uint64_t)a.W * a.Cin * 2, (uint64_t)a.H * a.W * a.Cin * 2};
    uint32_t box[4] = {64, (uint32_t)p.PW, (uint32_t)(bh + a.R - 1), 1};
    int r = esgd::make_tensormap_bf16(&p.tmX, a.x, 4, dims, strides, box, nullptr);
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
    uint32_t box[4] = {64, (uint32_t)p.Wo, (uint32_t)bh, 1};
    int r = esgd::make_tensormap_bf16(&p.tmY, a.y, 4, dims, strides, box, nullptr);
    if (r != 0) return 3000 + r;
  }
  const int sms = sm_count();
  if (p.n_tiles > sms) return -3;
  const int kb_total = a.R * a.S * p.cblks;
  // resident filter bank: beside two input boxes
  p.res_kb = (kb_total * Cfg<BN>::B_STAGE_BYTES + 2 * HALO_BYTES <= Cfg<BN>::STAGE_AREA) ? kb_total : 0;
  const int total = p.h_tiles * a.N * p.n_tiles;
  int grid = (sms / p.n_tiles) * p.n_tiles;
  if (grid > total) grid = total;
  ep.tx_bytes_a = (uint32_t)(p.PW * (bh + a.R - 1) * 128);
  ep.tx_bytes = 0;
  ep.residual = nullptr; ep.ldr = 0;
  conv_kernel<P><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(p, ep);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

template <int BN>
int launch_wgrad(const ConvArgs& a, const void* dy, float* dw, int* error_flag, cudaStream_t stream) {
  using P = ConvWgradProblem<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  P p;
  p.N = a.N; p.Cout = a.Cout; p.Cin = a.Cin; p.R = a.R; p.S = a.S; p.stride = a.stride; p.pad = a.pad;
  p.Ho = (a.H + 2 * a.pad - a.R) / a.stride + 1;
  p.Wo = (a.W + 2 * a.pad - a.S) / a.stride + 1;
  // pixel box of at most 64 rows (one k-block)
  if (p.Wo >= 64) { p.BW = 64; p.BH = 1; }
  else {
    p.BW = p.Wo;
    p.BH = 1;
    for (int d = 1; d <= 64 / p.BW && d <= p.Ho; ++d) if (p.Ho % d == 0) p.BH = d;
  }
  p.BI = 1;
  p.w_tiles = (p.Wo + p.BW - 1) / p.BW;
  p.h_tiles = (p.Ho + p.BH - 1) / p.BH;
  p.i_tiles = a.N;
  p.boxes_total = p.w_tiles * p.h_tiles * p.i_tiles;
  p.m_tiles = (a.Cout + BM - 1) / BM;
  p.n_tiles = (a.Cin + BN - 1) / BN;
  const int sms = sm_count();
  const int base_tiles = a.R * a.S * p.m_tiles * p.n_tiles;
  // Every split adds its partial sums with atomics: two waves of tiles when the filter bank is small, one
  // wave when it is large (the atomics of a 512 x 512 x 9 bank already outnumber its loads).
  const int waves = base_tiles < 32 ? 2 : 1;
  int splits = (waves * sms + base_tiles - 1) / base_tiles;
  if (splits < 1) splits = 1;
  if (splits > p.boxes_total) splits = p.boxes_total;
  p.boxes_per_split = (p.boxes_total + splits - 1) / splits;
  p.splits = (p.boxes_total + p.boxes_per_split - 1) / p.boxes_per_split;
  p.dw = dw;
  {
    uint64_t dims[4] = {(uint64_t)a.Cout, (uint64_t)p.Wo, (uint64_t)p.Ho, (uint64_t)a.N};
    uint64_t strides[3] = {(uint64_t)a.Cout * 2, (uint64_t)p.Wo * a.Cout * 2, (uint64_t)p.Ho * p.Wo * a.Cout * 2};
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, 1};
    int r = esgd::make_tensormap_bf16(&p.tmDY, dy, 4, dims, strides, box, nullptr);
    if (r != 0) return 1000 + r;
  }
  {
    uint64_t dims[4] = {(uint64_t)a.Cin, (uint64_t)a.W, (uint64_t)a.H, (uint64_t)a.N};
    uint64_t strides[3] = {(uint64_t)a.Cin * 2, (uint64_t)a.W * a.Cin * 2, (uint64_t)a.H * a.W * a.Cin * 2};
    uint32_t box[4] = {64, (uint32_t)(p.BW * a.stride), (uint32_t)(p.BH * a.stride), 1};
    uint32_t es[4] = {1, (uint32_t)a.stride, (uint32_t)a.stride, 1};
    int r = esgd::make_tensormap_bf16(&p.tmX, a.x, 4, dims, strides, box, es);
    if (r != 0) return 2000 + r;
  }
  Epilogue ep;
  ep.out_mode = OUT_F32_ATOMIC; ep.relu = 0; ep.n_total = a.Cin; ep.bias = nullptr;
  ep.col_sum = nullptr; ep.col_sqsum = nullptr; ep.error_flag = error_flag;
  ep.tx_bytes = (uint32_t)(p.BW * p.BH * 128 * (BM / 64 + BN / 64));
  ep.tx_bytes_a = 0; ep.residual = nullptr; ep.ldr = 0;
  const int total = base_tiles * p.splits;
  const int grid = total < sms ? total : sms;
  conv_wgrad_kernel<P><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(p, ep);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// dw: fp32 [Cout][R][S][Cin], zeroed by the caller (split-K partial sums are added atomically).
// x: [N,H,W,Cin] bf16, dy: [N,Ho,Wo,Cout] bf16.  Cin % 8 == 0, Cout % 8 == 0.
int esgd_conv2d_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, int Cout, int R, int S,
                      int stride, int pad, int* error_flag, void* stream) {
  if (Cin % 8 || Cout % 8 || stride < 1 || stride > 2) return -1;
  ConvArgs a{x, nullptr, nullptr, N, H, W, Cin, Cout, R, S, stride, pad};
  cudaStream_t s = (cudaStream_t)stream;
  const int BN = Cin <= 64 ? 64 : (Cin <= 128 ? 128 : 256);
  if (BN == 64) return launch_wgrad<64>(a, dy, dw, error_flag, s);
  if (BN == 128) return launch_wgrad<128>(a, dy, dw, error_flag, s);
  return launch_wgrad<256>(a, dy, dw, error_flag, s);
}

// x: [N,H,W,Cin] bf16, w: [Cout,R,S,Cin] bf16, y: [N,Ho,Wo,Cout] bf16.  Cin % 64 == 0, Cout % 8 == 0.
// col_sum / col_sqsum (optional, caller-zeroed fp32[Cout]) receive the statistics of the stored y.
// out_h / out_w override the output extent (taps that fall outside the input read zeros); ys_w / ys_h / ys_n
// (elements, 0 = dense) let y be a strided view, e.g. every second pixel of a larger tensor.
int esgd_conv2d_fwd_ex(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S,
                       int stride, int pad, int out_h, int out_w, int64_t ys_w, int64_t ys_h, int64_t ys_n, int relu,
                       float* col_sum, float* col_sqsum, int* error_flag, void* stream);

int esgd_conv2d_fwd(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S,
                    int stride, int pad, int relu, float* col_sum, float* col_sqsum, int* error_flag, void* stream) {
  return esgd_conv2d_fwd_ex(x, w, y, N, H, W, Cin, Cout, R, S, stride, pad, 0, 0, 0, 0, 0, relu, col_sum, col_sqsum,
                            error_flag, stream);
}

int esgd_conv2d_fwd_ex(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S,
                       int stride, int pad, int out_h, int out_w, int64_t ys_w, int64_t ys_h, int64_t ys_n, int relu,
                       float* col_sum, float* col_sqsum, int* error_flag, void* stream) {
  if (Cin % 64 || Cout % 8 || stride < 1 || stride > 2) return -1;
  if (ys_w && ((ys_w % 8) || (ys_h % 8) || (ys_n % 8))) return -6;
  ConvArgs a{x, w, y, N, H, W, Cin, Cout, R, S, stride, pad};
  a.out_h = out_h; a.out_w = out_w; a.ys_w = ys_w; a.ys_h = ys_h; a.ys_n = ys_n;
  Epilogue ep;
  ep.out_mode = OUT_BF16; ep.relu = relu; ep.n_total = Cout; ep.bias = nullptr;
  ep.col_sum = col_sum; ep.col_sqsum = col_sqsum; ep.error_flag = error_flag;
  ep.tx_bytes = 0; ep.tx_bytes_a = 0; ep.residual = nullptr; ep.ldr = 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int BN = Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256);
  int bh = 0;
  if (BN <= 128 && halo_applicable(a, (H + 2 * pad - R) / stride + 1, (W + 2 * pad - S) / stride + 1, &bh))
    return BN == 64 ? launch_halo<64>(a, ep, bh, s) : launch_halo<128>(a, ep, bh, s);
  if (BN == 64) return launch<64>(a, ep, s);
  if (BN == 128) return launch<128>(a, ep, s);
  return launch<256>(a, ep, s);
}

// Host arithmetic of the halo-mode forward / data-gradient launch, without launching (no device needed).
// out[0..9]: applicable (0/1), BH, PW, BN, resident filter k-blocks (0: streamed), input-box slots, filter stages,
// bytes of one input box, bytes the most shifted view reaches, stage area used.
void esgd_conv2d_halo_plan(int N, int H, int W, int Cin, int Cout, int R, int S, int stride, int pad, int* out) {
  for (int i = 0; i < 10; ++i) out[i] = 0;
  if (Cin % 64 || Cout % 8) return;
  ConvArgs a{nullptr, nullptr, nullptr, N, H, W, Cin, Cout, R, S, stride, pad};
  const int BN = Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256);
  int bh = 0;
  if (BN > 128 || stride != 1 || !halo_applicable(a, H + 2 * pad - R + 1, W + 2 * pad - S + 1, &bh)) return;
  const int PW = W + 2 * pad;
  const int b_stage = BN * 128, stage_area = BN == 64 ? Cfg<64>::STAGE_AREA : Cfg<128>::STAGE_AREA;
  const int kb_total = R * S * (Cin / 64);
  const int res_kb = (kb_total * b_stage + 2 * HALO_BYTES <= stage_area) ? kb_total : 0;
  const int nhalo = res_kb > 0 ? 2 : MAX_HALOS;
  int nstages = 1;
  if (res_kb == 0) {
    nstages = (stage_area - nhalo * HALO_BYTES) / b_stage;
    if (nstages > 8) nstages = 8;
  }
  out[0] = 1; out[1] = bh; out[2] = PW; out[3] = BN; out[4] = res_kb; out[5] = nhalo; out[6] = nstages;
  out[7] = PW * (bh + R - 1) * 128;
  out[8] = ((R - 1) * PW + (S - 1) + BM) * 128;
  out[9] = nhalo * HALO_BYTES + (res_kb > 0 ? res_kb : nstages) * b_stage;
}

}  // extern "C"
