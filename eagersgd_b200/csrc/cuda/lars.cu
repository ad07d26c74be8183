// Fused LARS (layer-wise adaptive rate scaling) over flat buffers, sm_100a.
//
// Two launches per step, whatever the number of tensors:
//   norms kernel : per-tensor sum of squares of the fp32 master weights and of the gradient.  The flat buffers
//                  are cut into chunks that never straddle a tensor; one block per chunk, one atomic pair per block.
//   update kernel: per element, with its tensor's trust ratio eeta * |w| / (|g| + wd * |w| + eps) (1 for tensors
//                  that are not adapted and where a norm is zero):
//                      v = momentum * v + lr * trust * (g + wd * w);   w -= v;   bf16 copy of w
// which is the reference's LARS step (official/utils/lars_optimizer.py:101-115: scaled learning rate, then a
// momentum update) without a host round trip for the norms and without one small kernel per tensor.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_count.cuh"

namespace {

struct Chunk {
  int64_t start;    // first element (multiple of 8)
  int32_t len;      // elements (multiple of 8, at most kChunk)
  int32_t tensor;   // tensor index; negative: (-1 - index) of a tensor that is not adapted
};
constexpr int kChunk = 8192;

__device__ __forceinline__ void ld8f(const float* p, float v[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8g(const void* g, int bf16, int64_t i, float v[8]) {
  if (bf16) {
    uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int q = 0; q < 4; ++q) { float2 f = __bfloat1622float2(h[q]); v[2 * q] = f.x; v[2 * q + 1] = f.y; }
  } else {
    ld8f(reinterpret_cast<const float*>(g) + i, v);
  }
}

__global__ void __launch_bounds__(256) lars_norms_kernel(const Chunk* __restrict__ chunks, const float* __restrict__ w32,
                                                         const void* __restrict__ grad, int grad_bf16, float gscale,
                                                         float* __restrict__ sq /* [tensors][2] */) {
  const Chunk c = chunks[blockIdx.x];
  float sw = 0.0f, sg = 0.0f;
  for (int e = threadIdx.x * 8; e < c.len; e += blockDim.x * 8) {
    float w[8], g[8];
    ld8f(w32 + c.start + e, w);
    ld8g(grad, grad_bf16, c.start + e, g);
#pragma unroll
    for (int q = 0; q < 8; ++q) { sw += w[q] * w[q]; const float gq = g[q] * gscale; sg += gq * gq; }
  }
  __shared__ float s_w[8], s_g[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { sw += __shfl_xor_sync(0xffffffffu, sw, o); sg += __shfl_xor_sync(0xffffffffu, sg, o); }
  if ((threadIdx.x & 31) == 0) { s_w[threadIdx.x >> 5] = sw; s_g[threadIdx.x >> 5] = sg; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.0f, b = 0.0f;
    for (int i = 0; i < 8; ++i) { a += s_w[i]; b += s_g[i]; }
    const int t = c.tensor >= 0 ? c.tensor : -1 - c.tensor;
    atomicAdd(sq + 2 * t, a);
    atomicAdd(sq + 2 * t + 1, b);
  }
}

__global__ void __launch_bounds__(256) lars_update_kernel(const Chunk* __restrict__ chunks, const float* __restrict__ sq,
                                                          const void* __restrict__ grad, int grad_bf16, float gscale,
                                                          float* __restrict__ w32, float* __restrict__ mom,
                                                          __nv_bfloat16* __restrict__ w16, float lr, float momentum,
                                                          float wd, float eeta, float eps) {
  const Chunk c = chunks[blockIdx.x];
  float trust = 1.0f, decay = 0.0f;
  if (c.tensor >= 0) {            // adapted tensor: weight decay is part of the scaled gradient
    const float wn = sqrtf(sq[2 * c.tensor]), gn = sqrtf(sq[2 * c.tensor + 1]);
    if (wn > 0.0f && gn > 0.0f) trust = eeta * wn / (gn + wd * wn + eps);
    decay = wd;
  }
  const float step = lr * trust;
  for (int e = threadIdx.x * 8; e < c.len; e += blockDim.x * 8) {
    const int64_t i = c.start + e;
    float w[8], g[8], v[8];
    ld8f(w32 + i, w);
    ld8f(mom + i, v);
    ld8g(grad, grad_bf16, i, g);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      v[q] = momentum * v[q] + step * (g[q] * gscale + decay * w[q]);
      w[q] -= v[q];
    }
    *reinterpret_cast<float4*>(w32 + i) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4*>(w32 + i + 4) = make_float4(w[4], w[5], w[6], w[7]);
    *reinterpret_cast<float4*>(mom + i) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(mom + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    if (w16 != nullptr) {
      uint4 raw;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(w[2 * q], w[2 * q + 1]);
      *reinterpret_cast<uint4*>(w16 + i) = raw;
    }
  }
}

}  // namespace

extern "C" {

int esgd_lars_chunk_elems(void) { return kChunk; }
int esgd_lars_chunk_bytes(void) { return (int)sizeof(Chunk); }

// `chunks`: device array of `num_chunks` Chunk records; `sq`: device fp32 [tensors][2], zeroed by this call.
// All offsets and lengths are multiples of 8 (tensors are padded inside the flat buffers).
int esgd_lars_step(const void* chunks, int num_chunks, int num_tensors, float* sq, const void* grad, int grad_bf16,
                   float grad_scale, float* w32, float* mom, void* w16, float lr, float momentum, float wd, float eeta,
                   float eps, void* stream) {
  if (num_chunks <= 0 || num_tensors <= 0) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(sq, 0, (size_t)num_tensors * 2 * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  lars_norms_kernel<<<num_chunks, 256, 0, s>>>((const Chunk*)chunks, w32, grad, grad_bf16, grad_scale, sq);
  lars_update_kernel<<<num_chunks, 256, 0, s>>>((const Chunk*)chunks, sq, grad, grad_bf16, grad_scale, w32, mom,
                                                (__nv_bfloat16*)w16, lr, momentum, wd, eeta, eps);
  esgd::count_launch(2);
  return (int)cudaGetLastError();
}

}  // extern "C"
