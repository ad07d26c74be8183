// Softmax cross-entropy (forward + backward in one pass), 3x3/2 max pooling and
// global average pooling for NHWC bf16 activations.
//
// Reference semantics: sparse softmax cross-entropy averaged over the batch
// (official/resnet/resnet_run_loop_solo_imagenet_300.py:321-322; CPU restatements
// deep500 .../cpp/operators/softmax_op.cpp:53-96, python/softmax_crossentropy_op.py:11-49),
// max_pooling2d 3x3 stride 2 'SAME' and reduce_mean over H,W (resnet_model.py:521-549;
// maxpool_op.cpp, globalaveragepool_op.cpp).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include "launch_count.cuh"

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = sh[0];
  for (int w = 1; w < nw; ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
  __syncthreads();
  return r;
}

// One block per sample.  loss_sum accumulates sum_i loss_i * inv_batch; dlogits = (softmax - onehot) * grad_scale.
// A label outside [0, classes) is never used as an index: that sample gets zero loss and a zero gradient row.
template <typename T>
__global__ void __launch_bounds__(256) softmax_ce_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels,
                                                         int classes, int ld, float inv_batch, float grad_scale,
                                                         float* __restrict__ loss_sum, float* __restrict__ per_sample,
                                                         T* __restrict__ dlogits) {
  __shared__ float sh[8];
  const int row = blockIdx.x;
  const T* x = logits + (size_t)row * ld;
  float mx = -FLT_MAX;
  for (int c = threadIdx.x; c < classes; c += blockDim.x) mx = fmaxf(mx, to_f(x[c]));
  mx = block_reduce(mx, true, sh);
  float se = 0.0f;
  for (int c = threadIdx.x; c < classes; c += blockDim.x) se += __expf(to_f(x[c]) - mx);
  se = block_reduce(se, false, sh);
  const int64_t raw_label = labels[row];
  const bool valid = raw_label >= 0 && raw_label < (int64_t)classes;
  const int label = valid ? (int)raw_label : 0;
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) {
    float li = valid ? lse - to_f(x[label]) : 0.0f;
    if (per_sample != nullptr) per_sample[row] = li;
    atomicAdd(loss_sum, li * inv_batch);
  }
  if (dlogits != nullptr) {
    T* d = dlogits + (size_t)row * ld;
    const float inv_se = 1.0f / se;
    for (int c = threadIdx.x; c < classes; c += blockDim.x) {
      float p = __expf(to_f(x[c]) - mx) * inv_se;
      d[c] = from_f<T>(valid ? (p - (c == label ? 1.0f : 0.0f)) * grad_scale : 0.0f);
    }
  }
}

// ---- max pool 3x3 stride 2 pad 1, NHWC, vectors of 8 channels -----------------
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float v[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 f = __bfloat1622float2(h[q]);
    v[2 * q] = f.x;
    v[2 * q + 1] = f.y;
  }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float v[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ idx,
                                                          int N, int H, int W, int C, int OH, int OW) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * OH * OW * G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    int64_t t = i / G;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH);
    const int n = (int)(t / OH);
    float m[8];
    uint32_t first[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) { m[q] = -FLT_MAX; first[q] = 0; }
    for (int r = 0; r < 3; ++r) {
      const int h = oh * 2 - 1 + r;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < 3; ++s) {
        const int w = ow * 2 - 1 + s;
        if (w < 0 || w >= W) continue;
        float v[8];
        ld8(x + (((int64_t)n * H + h) * W + w) * C + g * 8, v);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (v[q] > m[q]) { m[q] = v[q]; first[q] = (uint32_t)(r * 3 + s); }   // first maximum in scan order
      }
    }
    st8(y + i * 8, m);
    if (idx != nullptr) {
      uint2 pk;
      pk.x = first[0] | (first[1] << 8) | (first[2] << 16) | (first[3] << 24);
      pk.y = first[4] | (first[5] << 8) | (first[6] << 16) | (first[7] << 24);
      *reinterpret_cast<uint2*>(idx + i * 8) = pk;
    }
  }
}

// Gather form: an input pixel receives dy of every window whose recorded arg-max it is.
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const uint8_t* __restrict__ idx,
                                                          const __nv_bfloat16* __restrict__ dy,
                                                          __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C,
                                                          int OH, int OW) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * H * W * G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    int64_t t = i / G;
    const int w = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // windows that contain row h: oh in {h/2, (h+1)/2} (one window when h is even); same for columns
    const int ohs[2] = {h / 2, (h + 1) / 2}, ows[2] = {w / 2, (w + 1) / 2};
    const int noh = ohs[0] == ohs[1] ? 1 : 2, now = ows[0] == ows[1] ? 1 : 2;
    for (int a = 0; a < noh; ++a) {
      const int oh = ohs[a];
      if (oh >= OH) continue;
      for (int b = 0; b < now; ++b) {
        const int ow = ows[b];
        if (ow >= OW) continue;
        const uint32_t my_pos = (uint32_t)((h - (oh * 2 - 1)) * 3 + (w - (ow * 2 - 1)));
        const int64_t o = (((int64_t)n * OH + oh) * OW + ow) * C + g * 8;
        const uint2 pk = *reinterpret_cast<const uint2*>(idx + o);
        float d[8];
        ld8(dy + o, d);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t word = q < 4 ? pk.x : pk.y;
          if (((word >> ((q & 3) * 8)) & 0xffu) == my_pos) acc[q] += d[q];
        }
      }
    }
    st8(dx + i * 8, acc);
  }
}

// ---- 2x spatial subsampling (the gather in front of a strided 1x1 convolution) ---------
__global__ void __launch_bounds__(256) subsample2_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                             __nv_bfloat16* __restrict__ y, int N, int H, int W,
                                                             int C, int OH, int OW) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * OH * OW * G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    int64_t t = i / G;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH);
    const int n = (int)(t / OH);
    *reinterpret_cast<uint4*>(y + i * 8) =
        *reinterpret_cast<const uint4*>(x + (((int64_t)n * H + oh * 2) * W + ow * 2) * C + g * 8);
  }
}
__global__ void __launch_bounds__(256) subsample2_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                             __nv_bfloat16* __restrict__ dx, int N, int H, int W,
                                                             int C, int OH, int OW) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * H * W * G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    int64_t t = i / G;
    const int w = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (!(h & 1) && !(w & 1))
      v = *reinterpret_cast<const uint4*>(dy + (((int64_t)n * OH + h / 2) * OW + w / 2) * C + g * 8);
    *reinterpret_cast<uint4*>(dx + i * 8) = v;
  }
}

// ---- global average pool: [N, HW, C] -> [N, C] -----------------------------------
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ y, int N, int HW, int C) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    const int n = (int)(i / G);
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < HW; ++p) {
      float v[8];
      ld8(x + ((int64_t)n * HW + p) * C + g * 8, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) a[q] += v[q];
    }
    const float inv = 1.0f / (float)HW;
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] *= inv;
    st8(y + i * 8, a);
  }
}

__global__ void __launch_bounds__(256) avgpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          __nv_bfloat16* __restrict__ dx, int N, int HW, int C) {
  const int G = C / 8;
  const int64_t total = (int64_t)N * HW * G;
  const float inv = 1.0f / (float)HW;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % G);
    const int n = (int)(i / ((int64_t)HW * G));
    float v[8];
    ld8(dy + ((int64_t)n * G + g) * 8, v);
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] *= inv;
    st8(dx + i * 8, v);
  }
}

// im2col for convolutions with very few input channels (the 7x7 / 2 stem on RGB images).
// Column layout per output pixel: R segments of SEG = roundup8(S*C) elements; segment r holds the
// S*C input values of filter row r — in NHWC they are contiguous in memory — followed by zeros, and the
// row is zero-padded to Kpad (a multiple of 64, so the product runs as a tensor-core GEMM).
// One thread per (pixel, segment): no divisions per element, 16-byte stores.
template <int MAXSEG>
__global__ void __launch_bounds__(256) im2col_small_c_kernel(const __nv_bfloat16* __restrict__ x,
                                                             __nv_bfloat16* __restrict__ col, int N, int H, int W,
                                                             int C, int R, int S, int stride, int pad, int Ho, int Wo,
                                                             int seg, int Kpad) {
  const int segs = Kpad / seg;              // R real segments + zero segments
  const int64_t total = (int64_t)N * Ho * Wo * segs;
  const int sc = S * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i % segs);
    int64_t t = i / segs;
    const int q = (int)(t % Wo); t /= Wo;
    const int p = (int)(t % Ho);
    const int n = (int)(t / Ho);
    __align__(16) __nv_bfloat16 v[MAXSEG];
#pragma unroll
    for (int j = 0; j < MAXSEG; ++j) v[j] = __float2bfloat16(0.0f);
    const int h = p * stride + r - pad;
    if (r < R && h >= 0 && h < H) {
      const int w0 = q * stride - pad;
      const __nv_bfloat16* src = x + (((int64_t)n * H + h) * W + w0) * C;
      const int lo = w0 < 0 ? -w0 * C : 0;                       // first valid element of the segment
      const int hi = (w0 + S > W) ? (W - w0) * C : sc;           // one past the last valid element
#pragma unroll
      for (int j = 0; j < MAXSEG; ++j)
        if (j >= lo && j < hi) v[j] = src[j];
    }
    __nv_bfloat16* dst = col + (t * 0 + (((int64_t)n * Ho + p) * Wo + q)) * Kpad + (int64_t)r * seg;
    for (int j = 0; j < seg; j += 8) *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(v + j);
  }
}

// The same columns, one output row of the image per block: the R input rows that the row's windows touch are
// staged in shared memory with 16-byte loads between zero guards (the horizontal padding), and every thread
// assembles 16-byte chunks of the column matrix from them with funnel shifts (a window starts on an even byte,
// not on a word).  Elements of a segment beyond S*C carry the neighbouring pixels instead of zeros; they meet
// zero weights.  Writes are the only large traffic (N*Ho*Wo*Kpad*2 bytes) and they are fully coalesced.
constexpr int kImLeftGuard = 32, kImRightGuard = 64;
__global__ void __launch_bounds__(256) im2col_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ col, int N, int H, int W, int C,
                                                          int R, int S, int stride, int pad, int Ho, int Wo, int seg,
                                                          int Kpad) {
  extern __shared__ __align__(16) uint8_t im_rows[];
  const int rowbytes = W * C * 2;
  const int pitch = kImLeftGuard + rowbytes + kImRightGuard;
  const int n = blockIdx.x / Ho, p = blockIdx.x % Ho;
  for (int r = 0; r < R; ++r) {
    const int h = p * stride + r - pad;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(x) + ((int64_t)n * H + h) * rowbytes;
    for (int i = threadIdx.x; i < pitch / 16; i += blockDim.x) {
      const int byte = i * 16 - kImLeftGuard;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h >= 0 && h < H && byte >= 0 && byte < rowbytes) v = __ldg(reinterpret_cast<const uint4*>(src + byte));
      *reinterpret_cast<uint4*>(im_rows + r * pitch + i * 16) = v;
    }
  }
  __syncthreads();
  const int chunks_per_seg = seg / 8, chunks_per_pixel = Kpad / 8;
  __nv_bfloat16* dst_row = col + ((int64_t)n * Ho + p) * Wo * Kpad;
  for (int ci = threadIdx.x; ci < Wo * chunks_per_pixel; ci += blockDim.x) {
    const int q = ci / chunks_per_pixel, k8 = ci - q * chunks_per_pixel;
    const int r = k8 / chunks_per_seg, c = k8 - r * chunks_per_seg;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (r < R) {
      const int off = kImLeftGuard + ((q * stride - pad) * C + 8 * c) * 2;
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(im_rows + r * pitch + (off & ~3));
      const int sh = (off & 3) * 8;
      const uint32_t w0 = wp[0], w1 = wp[1], w2 = wp[2], w3 = wp[3], w4 = wp[4];
      out.x = __funnelshift_r(w0, w1, sh);
      out.y = __funnelshift_r(w1, w2, sh);
      out.z = __funnelshift_r(w2, w3, sh);
      out.w = __funnelshift_r(w3, w4, sh);
    }
    *reinterpret_cast<uint4*>(dst_row + (int64_t)ci * 8) = out;
  }
}

int grid_for(int64_t items) {
  int64_t b = (items + 255) / 256;
  const int64_t cap = 148 * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

extern "C" {

// loss_sum (one float) must be zeroed by the caller.
int esgd_softmax_ce(const void* logits, int is_bf16, const int64_t* labels, int batch, int classes, int ld,
                    float grad_scale, float* loss_sum, float* per_sample, void* dlogits, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (is_bf16)
    softmax_ce_kernel<__nv_bfloat16><<<batch, 256, 0, s>>>((const __nv_bfloat16*)logits, labels, classes, ld,
                                                           1.0f / batch, grad_scale, loss_sum, per_sample,
                                                           (__nv_bfloat16*)dlogits);
  else
    softmax_ce_kernel<float><<<batch, 256, 0, s>>>((const float*)logits, labels, classes, ld, 1.0f / batch,
                                                   grad_scale, loss_sum, per_sample, (float*)dlogits);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

// idx (optional, one byte per output element) records the arg-max for the backward pass.
int esgd_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  maxpool_fwd_kernel<<<grid_for((int64_t)N * OH * OW * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, (uint8_t*)idx, N, H, W, C, OH, OW);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_maxpool3x3s2_bwd(const void* idx, const void* dy, void* dx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  maxpool_bwd_kernel<<<grid_for((int64_t)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)idx, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, H, W, C, OH, OW);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

// y[n, oh, ow, :] = x[n, 2*oh, 2*ow, :]   (OH = ceil(H/2), OW = ceil(W/2))
int esgd_subsample2_fwd(const void* x, void* y, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  subsample2_fwd_kernel<<<grid_for((int64_t)N * OH * OW * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, H, W, C, OH, OW);
  esgd::count_launch();
  return (int)cudaGetLastError();
}
int esgd_subsample2_bwd(const void* dy, void* dx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  subsample2_bwd_kernel<<<grid_for((int64_t)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, H, W, C, OH, OW);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

// col: [N*Ho*Wo, Kpad] bf16; seg = roundup8(S*C) <= 32; Kpad a multiple of seg with Kpad >= R*seg.
// Element (r, j) of a row is x[.., h+r, (w0*C + j)] for j < S*C: weights must be laid out the same way.
int esgd_im2col_small_c(const void* x, void* col, int N, int H, int W, int C, int R, int S, int stride, int pad,
                        int seg, int Kpad, void* stream) {
  if (seg % 8 || seg < S * C || seg > 32 || Kpad % seg || Kpad < R * seg) return -1;
  const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
  const int rowbytes = W * C * 2;
  const int smem = R * (kImLeftGuard + rowbytes + kImRightGuard);
  // staged-row kernel: rows must be 16-byte multiples on a 16-byte base, the guards must cover the padding and
  // the over-read of the last window, and the rows must fit in the default shared-memory budget
  if (rowbytes % 16 == 0 && ((uintptr_t)x & 15) == 0 && pad * C * 2 <= kImLeftGuard &&
      ((Wo - 1) * stride - pad) * C * 2 + seg * 2 + 8 <= rowbytes + kImRightGuard && smem <= 48 * 1024) {
    im2col_rows_kernel<<<N * Ho, 256, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)col, N, H, W, C, R, S, stride, pad, Ho, Wo, seg, Kpad);
    esgd::count_launch();
    return (int)cudaGetLastError();
  }
  im2col_small_c_kernel<32><<<grid_for((int64_t)N * Ho * Wo * (Kpad / seg)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)col, N, H, W, C, R, S, stride, pad, Ho, Wo, seg, Kpad);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream) {
  if (C % 8) return -1;
  avgpool_fwd_kernel<<<grid_for((int64_t)N * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, HW, C);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream) {
  if (C % 8) return -1;
  avgpool_bwd_kernel<<<grid_for((int64_t)N * HW * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, HW, C);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // extern "C"
