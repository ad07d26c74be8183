// Fused batch-norm kernels for NHWC bf16 activations viewed as [M = N*H*W, C].
//
//   bn_stats        : per-channel sum / sum of squares (fp32) of a conv output
//   bn_finalize     : mean / inv-std, scale / shift, running-statistics update
//   bn_apply        : z = act(scale*y + shift [+ residual])           (one read, one write)
//   bn_bwd_reduce   : g = dz * [z > 0];  dbeta = sum g, dgamma = sum g*xhat
//   bn_bwd_apply    : dy = gamma*invstd*(g - dbeta/M - xhat*dgamma/M), optional dres = g
//
// Training-mode semantics, momentum and eps follow the reference model
// (official/resnet/resnet_model.py:51-60: decay 0.997, eps 1e-5, fused=True) and its
// CPU restatement (deep500 .../cpp/operators/batchnormalization_op_training.cpp:48-329).
// Threads map to channel groups of 8 (one 16-byte vector), rows are strided over
// blocks, partial sums meet in shared memory and then in fp32 global atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <stdint.h>
#include "launch_count.cuh"

namespace {

__device__ __forceinline__ void st8(__nv_bfloat16* p, const float v[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Block = 256 threads = (C/8 channel groups) x (256/(C/8) row lanes) when C/8 <= 256;
// wider layers loop over channel groups.
struct Map {
  int groups;      // C / 8
  int g_per_blk;   // channel groups handled per pass by a block (<= 256)
  int rows_par;    // rows processed in parallel by a block
};
__device__ __forceinline__ Map make_map(int C) {
  Map m;
  m.groups = C / 8;
  m.g_per_blk = m.groups < 256 ? m.groups : 256;
  m.rows_par = 256 / m.g_per_blk;
  return m;
}

__global__ void __launch_bounds__(256) bn_stats_kernel(const __nv_bfloat16* __restrict__ y, int64_t M, int C,
                                                       float* __restrict__ sum, float* __restrict__ sqsum) {
  const Map mp = make_map(C);
  __shared__ float s_sum[256 * 8], s_sq[256 * 8];
  for (int g0 = 0; g0 < mp.groups; g0 += mp.g_per_blk) {
    const int gl = threadIdx.x % mp.g_per_blk, rl = threadIdx.x / mp.g_per_blk;
    const int g = g0 + gl;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (g < mp.groups && rl < mp.rows_par) {
      const int64_t step = (int64_t)gridDim.x * mp.rows_par;
      for (int64_t r = (int64_t)blockIdx.x * mp.rows_par + rl; r < M; r += 4 * step) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (r + u * step < M) raw[u] = *reinterpret_cast<const uint4*>(y + (r + u * step) * C + g * 8);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (r + u * step < M) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float2 f = __bfloat1622float2(h[q]);
              a[2 * q] += f.x; a[2 * q + 1] += f.y; b[2 * q] += f.x * f.x; b[2 * q + 1] += f.y * f.y;
            }
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) { s_sum[threadIdx.x * 8 + q] = a[q]; s_sq[threadIdx.x * 8 + q] = b[q]; }
    __syncthreads();
    if (rl == 0 && g < mp.groups) {
      for (int rr = 1; rr < mp.rows_par; ++rr) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          a[q] += s_sum[(rr * mp.g_per_blk + gl) * 8 + q];
          b[q] += s_sq[(rr * mp.g_per_blk + gl) * 8 + q];
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) { atomicAdd(sum + g * 8 + q, a[q]); atomicAdd(sqsum + g * 8 + q, b[q]); }
    }
    __syncthreads();
  }
}

// One thread per channel.  Writes mean, invstd, scale = gamma*invstd, shift = beta - mean*scale.
__global__ void bn_finalize_kernel(const float* sum, const float* sqsum, const float* gamma, const float* beta,
                                   float* running_mean, float* running_var, float* mean_out, float* invstd_out,
                                   float* scale, float* shift, int C, float inv_count, float unbias, float momentum,
                                   float eps) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float mean = sum[c] * inv_count;
  float var = fmaxf(sqsum[c] * inv_count - mean * mean, 0.0f);
  float invstd = rsqrtf(var + eps);
  mean_out[c] = mean;
  invstd_out[c] = invstd;
  float sc = gamma[c] * invstd;
  scale[c] = sc;
  shift[c] = beta[c] - mean * sc;
  if (running_mean != nullptr) {
    running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * mean;
    running_var[c] = (1.0f - momentum) * running_var[c] + momentum * var * unbias;
  }
}

// Threads keep a fixed group of 8 channels and walk over rows, so the per-channel
// coefficients live in registers for the whole kernel.
template <int kMinBlocks>
__global__ void __launch_bounds__(256, kMinBlocks) bn_apply_kernel(const __nv_bfloat16* __restrict__ y,
                                                       const __nv_bfloat16* __restrict__ res,
                                                       __nv_bfloat16* __restrict__ z, const float* __restrict__ scale,
                                                       const float* __restrict__ shift, int64_t M, int C, int relu) {
  const Map mp = make_map(C);
  const int gl = threadIdx.x % mp.g_per_blk, rl = threadIdx.x / mp.g_per_blk;
  if (rl >= mp.rows_par) return;
  for (int g = gl; g < mp.groups; g += mp.g_per_blk) {
    float sc[8], sh[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) { sc[q] = scale[g * 8 + q]; sh[q] = shift[g * 8 + q]; }
    const int64_t step = (int64_t)gridDim.x * mp.rows_par;
    for (int64_t r = (int64_t)blockIdx.x * mp.rows_par + rl; r < M; r += 4 * step) {
      uint4 ry[4], rr_[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t rr = r + u * step;
        if (rr < M) {
          ry[u] = *reinterpret_cast<const uint4*>(y + rr * C + g * 8);
          if (res != nullptr) rr_[u] = *reinterpret_cast<const uint4*>(res + rr * C + g * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t rr = r + u * step;
        if (rr < M) {
          const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry[u]);
          const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&rr_[u]);
          float v[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 f = __bfloat1622float2(hy[q]);
            v[2 * q] = f.x * sc[2 * q] + sh[2 * q];
            v[2 * q + 1] = f.y * sc[2 * q + 1] + sh[2 * q + 1];
            if (res != nullptr) {
              float2 rf = __bfloat1622float2(hr[q]);
              v[2 * q] += rf.x; v[2 * q + 1] += rf.y;
            }
            if (relu) { v[2 * q] = fmaxf(v[2 * q], 0.0f); v[2 * q + 1] = fmaxf(v[2 * q + 1], 0.0f); }
          }
          st8(z + rr * C + g * 8, v);
        }
      }
    }
  }
}

template <int kMinBlocks>
__global__ void __launch_bounds__(256, kMinBlocks)
bn_bwd_reduce_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ z,
                     const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean,
                     const float* __restrict__ invstd, const float* __restrict__ fscale,
                     const float* __restrict__ fshift, int64_t M, int C, int relu, float* __restrict__ dbeta,
                     float* __restrict__ dgamma) {
  const Map mp = make_map(C);
  __shared__ float s_a[256 * 8], s_b[256 * 8];
  for (int g0 = 0; g0 < mp.groups; g0 += mp.g_per_blk) {
    const int gl = threadIdx.x % mp.g_per_blk, rl = threadIdx.x / mp.g_per_blk;
    const int g = g0 + gl;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (g < mp.groups && rl < mp.rows_par) {
      float mu[8], fsc[8], fsh[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        mu[q] = mean[g * 8 + q];
        fsc[q] = relu == 2 ? fscale[g * 8 + q] : 0.0f;
        fsh[q] = relu == 2 ? fshift[g * 8 + q] : 0.0f;
      }
      const int64_t step = (int64_t)gridDim.x * mp.rows_par;
      // sum g and g*(y - mean); the 1/std factor is applied once at the end.  Four rows in flight.
      for (int64_t r = (int64_t)blockIdx.x * mp.rows_par + rl; r < M; r += 4 * step) {
        uint4 rd[4], ry[4], rz[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t rr = r + u * step;
          if (rr < M) {
            const int64_t off = rr * C + g * 8;
            rd[u] = *reinterpret_cast<const uint4*>(dz + off);
            ry[u] = *reinterpret_cast<const uint4*>(y + off);
            if (relu == 1) rz[u] = *reinterpret_cast<const uint4*>(z + off);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (r + u * step < M) {
            const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&rd[u]);
            const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry[u]);
            const __nv_bfloat162* hz = reinterpret_cast<const __nv_bfloat162*>(&rz[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float2 d = __bfloat1622float2(hd[q]), yy = __bfloat1622float2(hy[q]);
              if (relu == 1) {
                float2 zz = __bfloat1622float2(hz[q]);
                d.x = zz.x > 0.0f ? d.x : 0.0f;
                d.y = zz.y > 0.0f ? d.y : 0.0f;
              } else if (relu == 2) {   // no residual: the sign of the activation follows from y alone
                d.x = yy.x * fsc[2 * q] + fsh[2 * q] > 0.0f ? d.x : 0.0f;
                d.y = yy.y * fsc[2 * q + 1] + fsh[2 * q + 1] > 0.0f ? d.y : 0.0f;
              }
              a[2 * q] += d.x; a[2 * q + 1] += d.y;
              b[2 * q] += d.x * (yy.x - mu[2 * q]); b[2 * q + 1] += d.y * (yy.y - mu[2 * q + 1]);
            }
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) b[q] *= invstd[g * 8 + q];
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) { s_a[threadIdx.x * 8 + q] = a[q]; s_b[threadIdx.x * 8 + q] = b[q]; }
    __syncthreads();
    if (rl == 0 && g < mp.groups) {
      for (int rr = 1; rr < mp.rows_par; ++rr) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          a[q] += s_a[(rr * mp.g_per_blk + gl) * 8 + q];
          b[q] += s_b[(rr * mp.g_per_blk + gl) * 8 + q];
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) { atomicAdd(dbeta + g * 8 + q, a[q]); atomicAdd(dgamma + g * 8 + q, b[q]); }
    }
    __syncthreads();
  }
}

// dy = a*g + b*y + c per channel, with a = gamma*invstd, b = -gamma*invstd^2*dgamma/M,
// c = gamma*invstd*(mean*invstd*dgamma - dbeta)/M held in registers.
template <int kMinBlocks>
__global__ void __launch_bounds__(256, kMinBlocks)
bn_bwd_apply_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ z,
                    const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean,
                    const float* __restrict__ invstd, const float* __restrict__ gamma,
                    const float* __restrict__ dbeta, const float* __restrict__ dgamma,
                    const float* __restrict__ fscale, const float* __restrict__ fshift,
                    __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dres, int64_t M, int C, int relu,
                    float inv_count) {
  const Map mp = make_map(C);
  const int gl = threadIdx.x % mp.g_per_blk, rl = threadIdx.x / mp.g_per_blk;
  if (rl >= mp.rows_par) return;
  for (int g = gl; g < mp.groups; g += mp.g_per_blk) {
    float ca[8], cb[8], cc[8], fsc[8], fsh[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int c = g * 8 + q;
      fsc[q] = relu == 2 ? fscale[c] : 0.0f;
      fsh[q] = relu == 2 ? fshift[c] : 0.0f;
      const float is = invstd[c], gm = gamma[c], dg = dgamma[c] * inv_count, db = dbeta[c] * inv_count;
      ca[q] = gm * is;
      cb[q] = -gm * is * is * dg;
      cc[q] = gm * is * (mean[c] * is * dg - db);
    }
    const int64_t step = (int64_t)gridDim.x * mp.rows_par;
    for (int64_t r = (int64_t)blockIdx.x * mp.rows_par + rl; r < M; r += 4 * step) {
      uint4 rd[4], ry[4], rz[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t rr = r + u * step;
        if (rr < M) {
          const int64_t off = rr * C + g * 8;
          rd[u] = *reinterpret_cast<const uint4*>(dz + off);
          ry[u] = *reinterpret_cast<const uint4*>(y + off);
          if (relu == 1) rz[u] = *reinterpret_cast<const uint4*>(z + off);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t rr = r + u * step;
        if (rr < M) {
          const int64_t off = rr * C + g * 8;
          const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&rd[u]);
          const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry[u]);
          const __nv_bfloat162* hz = reinterpret_cast<const __nv_bfloat162*>(&rz[u]);
          float d[8], o[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 dd = __bfloat1622float2(hd[q]), yy = __bfloat1622float2(hy[q]);
            if (relu == 1) {
              float2 zz = __bfloat1622float2(hz[q]);
              dd.x = zz.x > 0.0f ? dd.x : 0.0f;
              dd.y = zz.y > 0.0f ? dd.y : 0.0f;
            } else if (relu == 2) {
              dd.x = yy.x * fsc[2 * q] + fsh[2 * q] > 0.0f ? dd.x : 0.0f;
              dd.y = yy.y * fsc[2 * q + 1] + fsh[2 * q + 1] > 0.0f ? dd.y : 0.0f;
            }
            d[2 * q] = dd.x; d[2 * q + 1] = dd.y;
            o[2 * q] = ca[2 * q] * dd.x + cb[2 * q] * yy.x + cc[2 * q];
            o[2 * q + 1] = ca[2 * q + 1] * dd.y + cb[2 * q + 1] * yy.y + cc[2 * q + 1];
          }
          if (dres != nullptr) st8(dres + off, d);
          st8(dy + off, o);
        }
      }
    }
  }
}

int blocks_for(int64_t work_items, int per_block, int64_t cap = 148 * 16) {
  int64_t b = (work_items + per_block - 1) / per_block;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
// Reductions end with a shared-memory pass and atomics per block: few, long-running blocks.
constexpr int64_t kReduceGridCap = 148 * 2;

}  // namespace

// Resident blocks per SM the three bandwidth-bound kernels are compiled for (a register budget): chosen by
// measurement, overridable for experiments with ESGD_BN_OCC="apply,reduce,bwd_apply" (each 2, 3 or 4).
static int occupancy_choice(int which) {
  static int choice[3] = {0, 0, 0};
  if (choice[0] == 0) {
    int c[3] = {2, 2, 2};
    if (const char* e = getenv("ESGD_BN_OCC")) sscanf(e, "%d,%d,%d", &c[0], &c[1], &c[2]);
    for (int i = 2; i >= 0; --i) choice[i] = c[i] >= 2 && c[i] <= 4 ? c[i] : 2;
  }
  return choice[which];
}

extern "C" {

// sum / sqsum must be zeroed by the caller (they accumulate).
int esgd_bn_stats(const void* y, int64_t M, int C, float* sum, float* sqsum, void* stream) {
  if (C % 8) return -1;
  int g = C / 8 < 256 ? C / 8 : 256;
  int rows_par = 256 / g;
  bn_stats_kernel<<<blocks_for(M, rows_par * 16, kReduceGridCap), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, M, C, sum, sqsum);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_bn_finalize(const float* sum, const float* sqsum, const float* gamma, const float* beta,
                     float* running_mean, float* running_var, float* mean, float* invstd, float* scale,
                     float* shift, int C, int64_t count, float momentum, float eps, void* stream) {
  float unbias = count > 1 ? (float)count / (float)(count - 1) : 1.0f;
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      sum, sqsum, gamma, beta, running_mean, running_var, mean, invstd, scale, shift, C, 1.0f / (float)count,
      unbias, momentum, eps);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_bn_apply(const void* y, const void* residual, void* z, const float* scale, const float* shift, int64_t M,
                  int C, int relu, void* stream) {
  if (C % 8) return -1;
  int g = C / 8 < 256 ? C / 8 : 256;
  int rows_par = 256 / g;
#define ESGD_BN_APPLY(MB)                                                                          \
  bn_apply_kernel<MB><<<blocks_for(M, rows_par * 8), 256, 0, (cudaStream_t)stream>>>(             \
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)residual, (__nv_bfloat16*)z, scale, shift, M, C, relu)
  switch (occupancy_choice(0)) {
    case 3: ESGD_BN_APPLY(3); break;
    case 4: ESGD_BN_APPLY(4); break;
    default: ESGD_BN_APPLY(2); break;
  }
  esgd::count_launch();
  return (int)cudaGetLastError();
}

// dbeta / dgamma must be zeroed by the caller.
// relu: 0 none, 1 mask from the saved output z (needed with a residual), 2 mask recomputed from y with
// the forward scale / shift (no read of z).
int esgd_bn_bwd_reduce(const void* dz, const void* z, const void* y, const float* mean, const float* invstd,
                       const float* fscale, const float* fshift, int64_t M, int C, int relu, float* dbeta,
                       float* dgamma, void* stream) {
  if (C % 8) return -1;
  int g = C / 8 < 256 ? C / 8 : 256;
  int rows_par = 256 / g;
#define ESGD_BN_REDUCE(MB)                                                                                     \
  bn_bwd_reduce_kernel<MB><<<blocks_for(M, rows_par * 16, kReduceGridCap), 256, 0, (cudaStream_t)stream>>>(   \
      (const __nv_bfloat16*)dz, (const __nv_bfloat16*)z, (const __nv_bfloat16*)y, mean, invstd, fscale, fshift, M, C, \
      relu, dbeta, dgamma)
  switch (occupancy_choice(1)) {
    case 3: ESGD_BN_REDUCE(3); break;
    default: ESGD_BN_REDUCE(2); break;
  }
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_bn_bwd_apply(const void* dz, const void* z, const void* y, const float* mean, const float* invstd,
                      const float* gamma, const float* dbeta, const float* dgamma, const float* fscale,
                      const float* fshift, void* dy, void* dres, int64_t M, int C, int relu, void* stream) {
  if (C % 8) return -1;
  int g = C / 8 < 256 ? C / 8 : 256;
  int rows_par = 256 / g;
#define ESGD_BN_BWD_APPLY(MB)                                                                              \
  bn_bwd_apply_kernel<MB><<<blocks_for(M, rows_par * 8), 256, 0, (cudaStream_t)stream>>>(                   \
      (const __nv_bfloat16*)dz, (const __nv_bfloat16*)z, (const __nv_bfloat16*)y, mean, invstd, gamma, dbeta, \
      dgamma, fscale, fshift, (__nv_bfloat16*)dy, (__nv_bfloat16*)dres, M, C, relu, 1.0f / (float)M)
  switch (occupancy_choice(2)) {
    case 3: ESGD_BN_BWD_APPLY(3); break;
    case 4: ESGD_BN_BWD_APPLY(4); break;
    default: ESGD_BN_BWD_APPLY(2); break;
  }
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // extern "C"
