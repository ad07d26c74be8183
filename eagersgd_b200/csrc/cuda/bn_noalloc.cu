// Allocation-free batch-norm forward: see bn_noalloc.h for who needs it and for its rules.
//
// The six per-channel work arrays (sum, sum of squares, mean, inverse std, scale, shift) that
// the regular entry points take from their caller live in one file-scope __device__ array.
// In host code the array's name is only a handle: its device address is fetched once per device
// with cudaGetSymbolAddress and that pointer is what the kernels receive.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <mutex>
#include <stdint.h>
#include "bn_noalloc.h"
#include "launch_count.cuh"

namespace {

constexpr int kMaxC = ESGD_BN_NOALLOC_MAX_CHANNELS;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_bn_scratch[6 * kMaxC];

float* g_scratch_ptr[kMaxDevices];
bool g_scratch_ready[kMaxDevices];
std::mutex g_setup_mutex;

// Device address of the block on the current device (looked up on first use per device).
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return ESGD_BN_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ready[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_bn_scratch);
    if (e != cudaSuccess || p == nullptr) return e != cudaSuccess ? (int)e : ESGD_BN_NOALLOC_SETUP_FAILED;
    g_scratch_ptr[dev] = p;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float v[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 f = __bfloat1622float2(h[q]);
    v[2 * q] = f.x;
    v[2 * q + 1] = f.y;
  }
}

// Threads own a group of 8 channels (16 bytes) and stride over rows; block partials meet in
// shared memory, then one atomic per channel and block.
__global__ void __launch_bounds__(256) na_stats_kernel(const __nv_bfloat16* __restrict__ y, int64_t M, int C,
                                                       float* __restrict__ sum, float* __restrict__ sqsum) {
  const int groups = C / 8;
  const int gpb = groups < 256 ? groups : 256, rows_par = 256 / gpb;
  __shared__ float s_a[256 * 8], s_b[256 * 8];
  for (int g0 = 0; g0 < groups; g0 += gpb) {
    const int gl = threadIdx.x % gpb, rl = threadIdx.x / gpb, g = g0 + gl;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (g < groups && rl < rows_par) {
      for (int64_t r = (int64_t)blockIdx.x * rows_par + rl; r < M; r += (int64_t)gridDim.x * rows_par) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(y + r * C + g * 8), v);
#pragma unroll
        for (int q = 0; q < 8; ++q) { a[q] += v[q]; b[q] += v[q] * v[q]; }
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) { s_a[threadIdx.x * 8 + q] = a[q]; s_b[threadIdx.x * 8 + q] = b[q]; }
    __syncthreads();
    if (rl == 0 && g < groups) {
      for (int rr = 1; rr < rows_par; ++rr)
#pragma unroll
        for (int q = 0; q < 8; ++q) { a[q] += s_a[(rr * gpb + gl) * 8 + q]; b[q] += s_b[(rr * gpb + gl) * 8 + q]; }
#pragma unroll
      for (int q = 0; q < 8; ++q) { atomicAdd(sum + g * 8 + q, a[q]); atomicAdd(sqsum + g * 8 + q, b[q]); }
    }
    __syncthreads();
  }
}

__global__ void na_finalize_kernel(const float* sum, const float* sqsum, const float* gamma, const float* beta,
                                   float* running_mean, float* running_var, float* mean_out, float* invstd_out,
                                   float* scale, float* shift, int C, float inv_count, float unbias, float momentum,
                                   float eps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float mean = sum[c] * inv_count;
  const float var = fmaxf(sqsum[c] * inv_count - mean * mean, 0.0f);
  const float invstd = rsqrtf(var + eps);
  mean_out[c] = mean;
  invstd_out[c] = invstd;
  const float sc = gamma[c] * invstd;
  scale[c] = sc;
  shift[c] = beta[c] - mean * sc;
  if (running_mean != nullptr) running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * mean;
  if (running_var != nullptr) running_var[c] = (1.0f - momentum) * running_var[c] + momentum * var * unbias;
}

__global__ void __launch_bounds__(256) na_apply_kernel(const __nv_bfloat16* __restrict__ y,
                                                       const __nv_bfloat16* __restrict__ res,
                                                       __nv_bfloat16* __restrict__ z, const float* __restrict__ scale,
                                                       const float* __restrict__ shift, int64_t total_groups, int C,
                                                       int relu) {
  const int groups = C / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_groups;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(i % groups);
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(y + i * 8), v);
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = v[q] * scale[g * 8 + q] + shift[g * 8 + q];
    if (res != nullptr) {
      float r[8];
      unpack8(*reinterpret_cast<const uint4*>(res + i * 8), r);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] += r[q];
    }
    if (relu) {
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = fmaxf(v[q], 0.0f);
    }
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
    *reinterpret_cast<uint4*>(z + i * 8) = raw;
  }
}

int clamp_blocks(int64_t want, int64_t cap) { return (int)(want < 1 ? 1 : (want > cap ? cap : want)); }

}  // namespace

extern "C" {

int esgd_bn_forward_noalloc(const void* y, const void* residual, void* z, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, int64_t M, int C, int relu, float momentum,
                            float eps, void* stream) {
  if (y == nullptr || z == nullptr || gamma == nullptr || beta == nullptr || M <= 0 || C <= 0 || (C % 8) != 0)
    return ESGD_BN_NOALLOC_BAD_ARGUMENT;
  // y, residual and z are read and written 16 bytes at a time: a pointer into the middle of a vector
  // would fault on the device, so it is refused here instead
  if ((((uintptr_t)y | (uintptr_t)z | (uintptr_t)residual) & 15u) != 0) return ESGD_BN_NOALLOC_BAD_ARGUMENT;
  if ((((uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)running_mean | (uintptr_t)running_var) & 3u) != 0)
    return ESGD_BN_NOALLOC_BAD_ARGUMENT;
  if (C > kMaxC) return ESGD_BN_NOALLOC_TOO_MANY_CHANNELS;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  float* sum = scratch;
  float* sqsum = scratch + kMaxC;
  float* mean = scratch + 2 * kMaxC;
  float* invstd = scratch + 3 * kMaxC;
  float* scale = scratch + 4 * kMaxC;
  float* shift = scratch + 5 * kMaxC;
  // the accumulators keep the previous call's sums: clear them (contiguous: sum | sqsum)
  cudaError_t e = cudaMemsetAsync(sum, 0, 2 * (size_t)kMaxC * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  const int gpb = C / 8 < 256 ? C / 8 : 256, rows_par = 256 / gpb;
  na_stats_kernel<<<clamp_blocks((M + rows_par * 16 - 1) / (rows_par * 16), 296), 256, 0, s>>>(
      (const __nv_bfloat16*)y, M, C, sum, sqsum);
  const float unbias = M > 1 ? (float)M / (float)(M - 1) : 1.0f;
  na_finalize_kernel<<<(C + 127) / 128, 128, 0, s>>>(sum, sqsum, gamma, beta, running_mean, running_var, mean, invstd,
                                                    scale, shift, C, 1.0f / (float)M, unbias, momentum, eps);
  const int64_t groups = M * (C / 8);
  na_apply_kernel<<<clamp_blocks((groups + 1023) / 1024, 148 * 16), 256, 0, s>>>(
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)residual, (__nv_bfloat16*)z, scale, shift, groups, C, relu);
  esgd::count_launch(3);
  return (int)cudaGetLastError();
}

const char* esgd_bn_forward_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case ESGD_BN_NOALLOC_BAD_ARGUMENT:
      return "bad argument: pointers must be non-null, y / residual / z 16-byte aligned, M and C positive, "
             "C a multiple of 8";
    case ESGD_BN_NOALLOC_TOO_MANY_CHANNELS:
      return "too many channels: the built-in work area holds at most 4096 channels";
    case ESGD_BN_NOALLOC_SETUP_FAILED:
      return "could not obtain the device address of the built-in work area on this device";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

}  // extern "C"
