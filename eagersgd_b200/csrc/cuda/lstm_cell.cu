// Fused LSTM cell kernels (gate non-linearities + state update, forward and backward).
//
// The projections run on the tensor cores: x.W_ih^T for all time steps as one GEMM, and per
// time step the recurrent product in swapped form  G^T[4H, B] = W_hh[4H, H] . h_{t-1}^T  so
// that the large dimension (4H) fills the 128-row MMA tile and the small batch is the N
// dimension.  These kernels consume that fp32 [4H, B] product directly.
//
//   forward : pre = xproj[b, :] + hprojT[:, b] + bias ; i,f,o = sigmoid, g = tanh
//             c_t = f*c_{t-1} + i*g ; h_t = o*tanh(c_t) ; gate activations are kept for backward
//   backward: given dh_t (from the layer above plus the recurrence) and dc_t, produce the
//             pre-activation gradients dG[b, 4H] (bf16) and dc_{t-1}
//
// Gate order i, f, g, o as in torch.nn.LSTM, which the reference model uses through cuDNN
// (deep500 samples/ucf101_resnetlstm.py:41-59).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_count.cuh"

extern "C" void esgd_gemm_set_chained(int on);

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// One thread per (b, j): B*H threads.
__global__ void __launch_bounds__(256)
lstm_cell_fwd_kernel(const __nv_bfloat16* __restrict__ xproj,   // [B, 4H]
                     float* __restrict__ hprojT,                // [4H, ldh] (ldh >= B), may be null at t = 0
                     const float* __restrict__ bias,            // [4H] (b_ih + b_hh)
                     const float* __restrict__ c_prev,          // [B, H] or null
                     float* __restrict__ c_out,                 // [B, H]
                     __nv_bfloat16* __restrict__ h_out,         // [B, H]
                     __nv_bfloat16* __restrict__ gates,         // [B, 4H] activations i, f, g, o
                     int B, int H, int ldh, int clear) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  float pre[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int row = k * H + j;
    float v = __bfloat162float(xproj[(size_t)b * 4 * H + row]) + bias[row];
    if (hprojT != nullptr) {
      v += hprojT[(size_t)row * ldh + b];
      if (clear) hprojT[(size_t)row * ldh + b] = 0.0f;   // each element has one reader: ready for the next step's split-K sums
    }
    pre[k] = v;
  }
  const float ig = sigmoidf_(pre[0]), fg = sigmoidf_(pre[1]), gg = tanhf(pre[2]), og = sigmoidf_(pre[3]);
  const float cp = c_prev != nullptr ? c_prev[idx] : 0.0f;
  const float c = fg * cp + ig * gg;
  c_out[idx] = c;
  h_out[idx] = __float2bfloat16(og * tanhf(c));
  __nv_bfloat16* gp = gates + (size_t)b * 4 * H + j;
  gp[0] = __float2bfloat16(ig);
  gp[H] = __float2bfloat16(fg);
  gp[2 * H] = __float2bfloat16(gg);
  gp[3 * H] = __float2bfloat16(og);
}

__global__ void __launch_bounds__(256)
lstm_cell_bwd_kernel(const __nv_bfloat16* __restrict__ gates,   // [B, 4H] saved activations
                     const float* __restrict__ c_prev,          // [B, H] or null
                     const float* __restrict__ c_cur,           // [B, H]
                     const __nv_bfloat16* __restrict__ dh_ext,  // [B, H] gradient from above (may be null)
                     float* __restrict__ dh_recT,               // [H, ldr] recurrent gradient, transposed (may be null)
                     float* __restrict__ dc,                    // [B, H] in: dc_t, out: dc_{t-1}
                     __nv_bfloat16* __restrict__ dgates,        // [B, 4H] pre-activation gradients
                     int B, int H, int ldr, int clear) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  const __nv_bfloat16* gp = gates + (size_t)b * 4 * H + j;
  const float ig = __bfloat162float(gp[0]), fg = __bfloat162float(gp[H]), gg = __bfloat162float(gp[2 * H]),
              og = __bfloat162float(gp[3 * H]);
  float dh = dh_ext != nullptr ? __bfloat162float(dh_ext[idx]) : 0.0f;
  if (dh_recT != nullptr) {
    dh += dh_recT[(size_t)j * ldr + b];
    if (clear) dh_recT[(size_t)j * ldr + b] = 0.0f;
  }
  const float tc = tanhf(c_cur[idx]);
  const float dct = dc[idx] + dh * og * (1.0f - tc * tc);
  const float cp = c_prev != nullptr ? c_prev[idx] : 0.0f;
  const float d_i = dct * gg * ig * (1.0f - ig);
  const float d_f = dct * cp * fg * (1.0f - fg);
  const float d_g = dct * ig * (1.0f - gg * gg);
  const float d_o = dh * tc * og * (1.0f - og);
  dc[idx] = dct * fg;
  __nv_bfloat16* dp = dgates + (size_t)b * 4 * H + j;
  dp[0] = __float2bfloat16(d_i);
  dp[H] = __float2bfloat16(d_f);
  dp[2 * H] = __float2bfloat16(d_g);
  dp[3 * H] = __float2bfloat16(d_o);
}

// Tiled forms for the sequence loop.  The recurrent products arrive transposed ([4H, B] and [H, B], batch fastest)
// while everything else is [B, H] (unit fastest): a block takes kJT hidden units x all B batch rows, moves its part
// of the transposed product through shared memory with contiguous accesses (and zeroes it behind itself for the next
// step's split-K sums), then works unit-fastest.  B <= kMaxTileB.
constexpr int kJT = 16;
constexpr int kMaxTileB = 32;

__global__ void __launch_bounds__(256)
lstm_cell_fwd_tiled_kernel(const __nv_bfloat16* __restrict__ xproj, float* __restrict__ hprojT,
                           const float* __restrict__ bias, const float* __restrict__ c_prev, float* __restrict__ c_out,
                           __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ gates, int B, int H,
                           int chained) {
  __shared__ float hp[4][kJT][kMaxTileB + 1];
  if (chained) {   // started early, behind a kernel that may still run: wait for it, then let the next one be scheduled
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  const int j0 = blockIdx.x * kJT;
  const int n = kJT * B;                        // elements per gate in this block; contiguous in hprojT
  if (hprojT != nullptr) {
    constexpr int kPer = kJT * kMaxTileB / 256;   // elements per thread and gate, at most
    float v[4][kPer];
#pragma unroll
    for (int k = 0; k < 4; ++k)                   // every load is issued before the first store
#pragma unroll
      for (int r = 0; r < kPer; ++r) {
        const int i = threadIdx.x + r * 256;
        v[k][r] = i < n ? hprojT[((size_t)k * H + j0) * B + i] : 0.0f;
      }
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int r = 0; r < kPer; ++r) {
        const int i = threadIdx.x + r * 256;
        if (i < n) {
          hp[k][i / B][i % B] = v[k][r];
          hprojT[((size_t)k * H + j0) * B + i] = 0.0f;
        }
      }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int b = i / kJT, jj = i % kJT, j = j0 + jj;
    const size_t idx = (size_t)b * H + j;
    float pre[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v = __bfloat162float(xproj[(size_t)b * 4 * H + k * H + j]) + bias[k * H + j];
      if (hprojT != nullptr) v += hp[k][jj][b];
      pre[k] = v;
    }
    const float ig = sigmoidf_(pre[0]), fg = sigmoidf_(pre[1]), gg = tanhf(pre[2]), og = sigmoidf_(pre[3]);
    const float cp = c_prev != nullptr ? c_prev[idx] : 0.0f;
    const float c = fg * cp + ig * gg;
    c_out[idx] = c;
    h_out[idx] = __float2bfloat16(og * tanhf(c));
    __nv_bfloat16* gp = gates + (size_t)b * 4 * H + j;
    gp[0] = __float2bfloat16(ig);
    gp[H] = __float2bfloat16(fg);
    gp[2 * H] = __float2bfloat16(gg);
    gp[3 * H] = __float2bfloat16(og);
  }
}

__global__ void __launch_bounds__(256)
lstm_cell_bwd_tiled_kernel(const __nv_bfloat16* __restrict__ gates, const float* __restrict__ c_prev,
                           const float* __restrict__ c_cur, const __nv_bfloat16* __restrict__ dh_ext,
                           float* __restrict__ dh_recT, float* __restrict__ dc, __nv_bfloat16* __restrict__ dgates,
                           int B, int H, int chained) {
  __shared__ float dr[kJT][kMaxTileB + 1];
  if (chained) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  const int j0 = blockIdx.x * kJT;
  const int n = kJT * B;
  if (dh_recT != nullptr) {
    float* src = dh_recT + (size_t)j0 * B;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      dr[i / B][i % B] = src[i];
      src[i] = 0.0f;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int b = i / kJT, jj = i % kJT, j = j0 + jj;
    const size_t idx = (size_t)b * H + j;
    const __nv_bfloat16* gp = gates + (size_t)b * 4 * H + j;
    const float ig = __bfloat162float(gp[0]), fg = __bfloat162float(gp[H]), gg = __bfloat162float(gp[2 * H]),
                og = __bfloat162float(gp[3 * H]);
    float dh = dh_ext != nullptr ? __bfloat162float(dh_ext[idx]) : 0.0f;
    if (dh_recT != nullptr) dh += dr[jj][b];
    const float tc = tanhf(c_cur[idx]);
    const float dct = dc[idx] + dh * og * (1.0f - tc * tc);
    const float cp = c_prev != nullptr ? c_prev[idx] : 0.0f;
    dc[idx] = dct * fg;
    __nv_bfloat16* dp = dgates + (size_t)b * 4 * H + j;
    dp[0] = __float2bfloat16(dct * gg * ig * (1.0f - ig));
    dp[H] = __float2bfloat16(dct * cp * fg * (1.0f - fg));
    dp[2 * H] = __float2bfloat16(dct * ig * (1.0f - gg * gg));
    dp[3 * H] = __float2bfloat16(dh * tc * og * (1.0f - og));
  }
}

// A link of a chain of dependent launches: the kernel may be scheduled before the one ahead of it in the stream has
// finished (it waits for it inside, with griddepcontrol.wait), which hides the launch latency between the steps.
template <class... KArgs, class... Args>
int launch_chained(void (*kernel)(KArgs...), int grid, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

int cell_fwd(const void* xproj, float* hprojT, const float* bias, const float* c_prev, float* c_out, void* h_out,
             void* gates, int B, int H, int ldh, int clear, void* stream) {
  if (clear && ldh == B && B <= kMaxTileB && H % kJT == 0) {
    esgd::count_launch();
    return launch_chained(lstm_cell_fwd_tiled_kernel, H / kJT, (cudaStream_t)stream, (const __nv_bfloat16*)xproj, hprojT,
                          bias, c_prev, c_out, (__nv_bfloat16*)h_out, (__nv_bfloat16*)gates, B, H, 1);
  }
  lstm_cell_fwd_kernel<<<(B * H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)xproj, hprojT, bias, c_prev, c_out, (__nv_bfloat16*)h_out, (__nv_bfloat16*)gates, B, H,
      ldh, clear);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int cell_bwd(const void* gates, const float* c_prev, const float* c_cur, const void* dh_ext, float* dh_recT, float* dc,
             void* dgates, int B, int H, int ldr, int clear, void* stream) {
  if (clear && ldr == B && B <= kMaxTileB && H % kJT == 0) {
    esgd::count_launch();
    return launch_chained(lstm_cell_bwd_tiled_kernel, H / kJT, (cudaStream_t)stream, (const __nv_bfloat16*)gates, c_prev,
                          c_cur, (const __nv_bfloat16*)dh_ext, dh_recT, dc, (__nv_bfloat16*)dgates, B, H, 1);
  }
  lstm_cell_bwd_kernel<<<(B * H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gates, c_prev, c_cur, (const __nv_bfloat16*)dh_ext, dh_recT, dc, (__nv_bfloat16*)dgates,
      B, H, ldr, clear);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

struct ChainScope {   // the GEMM launches of this thread are chain links while one of these is alive
  ChainScope() { esgd_gemm_set_chained(1); }
  ~ChainScope() { esgd_gemm_set_chained(0); }
};

// Split-K factor that brings a recurrent GEMM of `m` output rows to about one CTA per SM.
int splits_for(int m, int k) {
  const int tiles = (m + 127) / 128;
  int s = 128 / (tiles < 1 ? 1 : tiles);
  const int kb = (k + 63) / 64;
  if (s > kb / 4) s = kb / 4;       // at least four k-blocks per split
  return s < 1 ? 1 : s;
}

}  // namespace

extern "C" {

int esgd_lstm_cell_fwd(const void* xproj, const float* hprojT, const float* bias, const float* c_prev, float* c_out,
                       void* h_out, void* gates, int B, int H, int ldh, void* stream) {
  return cell_fwd(xproj, const_cast<float*>(hprojT), bias, c_prev, c_out, h_out, gates, B, H, ldh, 0, stream);
}

int esgd_lstm_cell_bwd(const void* gates, const float* c_prev, const float* c_cur, const void* dh_ext,
                       const float* dh_recT, float* dc, void* dgates, int B, int H, int ldr, void* stream) {
  return cell_bwd(gates, c_prev, c_cur, dh_ext, const_cast<float*>(dh_recT), dc, dgates, B, H, ldr, 0, stream);
}

// ---- whole sequences: the time loop runs here, not in Python ----------------------------------------------------
// One call per layer and direction issues every launch of the recurrence (per step: the swapped recurrent GEMM
// on the tensor cores and the fused cell kernel), so the GPU never waits for an interpreter between steps.

int esgd_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                   int b_mn, int out_mode, const float* bias, int relu, int splits, float* col_sum, float* col_sqsum,
                   const void* residual, int ldr, int* error_flag, void* stream);
void esgd_gemm_set_chained(int on);

// xproj [T*B, 4H] bf16 (input projection of every step), w_hh [4H, H] bf16, bias [4H] fp32;
// out: c [T, B, H] fp32, y [T, B, H] bf16, gates [T, B, 4H] bf16; scratch hprojT [4H, B] fp32.
int esgd_lstm_seq_fwd(const void* xproj, const void* w_hh, const float* bias, float* c, void* y, void* gates,
                      float* hprojT, int T, int B, int H, int* error_flag, void* stream) {
  if (T <= 0 || B <= 0 || H <= 0 || (B % 8) || (H % 8)) return -1;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)xproj;
  __nv_bfloat16* yp = (__nv_bfloat16*)y;
  __nv_bfloat16* gp = (__nv_bfloat16*)gates;
  const size_t bh = (size_t)B * H;
  // The product is split over K so that about every SM has a tile (4H / 128 row tiles alone leave most idle); the
  // partial sums meet in hprojT by fp32 atomics, and the cell kernel that reads an element zeroes it again.
  const int splits = splits_for(4 * H, H);
  cudaError_t e = cudaMemsetAsync(hprojT, 0, (size_t)4 * bh * sizeof(float), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  ChainScope chain;
  for (int t = 0; t < T; ++t) {
    if (t > 0) {   // hprojT[4H, B] += W_hh[4H, H] . h_{t-1}[B, H]^T
      int rc = esgd_gemm_bf16(w_hh, yp + (t - 1) * bh, hprojT, 4 * H, B, H, H, H, B, 0, 0, 2, nullptr, 0, splits,
                              nullptr, nullptr, nullptr, 0, error_flag, stream);
      if (rc != 0) return rc;
    }
    int rc = cell_fwd(xp + (size_t)t * 4 * bh, t > 0 ? hprojT : nullptr, bias, t > 0 ? c + (t - 1) * bh : nullptr,
                      c + t * bh, yp + t * bh, gp + (size_t)t * 4 * bh, B, H, B, 1, stream);
    if (rc != 0) return rc;
  }
  return 0;
}

// Recurrent half of the backward pass: dG [T, B, 4H] bf16 (pre-activation gradients of every step) from
// dy [T, B, H] bf16, the saved gates and cell states.  Scratch: dc [B, H] fp32 (zeroed here), dh_recT [H, B] fp32.
int esgd_lstm_seq_bwd(const void* gates, const float* c, const void* dy, const void* w_hh, void* dG, float* dc,
                      float* dh_recT, int T, int B, int H, int* error_flag, void* stream) {
  if (T <= 0 || B <= 0 || H <= 0 || (B % 8) || (H % 8)) return -1;
  const __nv_bfloat16* gp = (const __nv_bfloat16*)gates;
  const __nv_bfloat16* dyp = (const __nv_bfloat16*)dy;
  __nv_bfloat16* dgp = (__nv_bfloat16*)dG;
  const size_t bh = (size_t)B * H;
  cudaError_t e = cudaMemsetAsync(dc, 0, bh * sizeof(float), (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(dh_recT, 0, bh * sizeof(float), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  const int splits = splits_for(H, 4 * H);   // H / 128 row tiles only: the split over K = 4H is what fills the GPU
  ChainScope chain;
  for (int t = T - 1; t >= 0; --t) {
    int rc = cell_bwd(gp + (size_t)t * 4 * bh, t > 0 ? c + (t - 1) * bh : nullptr, c + t * bh, dyp + t * bh,
                      t < T - 1 ? dh_recT : nullptr, dc, dgp + (size_t)t * 4 * bh, B, H, B, 1, stream);
    if (rc != 0) return rc;
    if (t > 0) {   // dh_recT[H, B] += W_hh^T . dG_t^T: A stored [K = 4H][M = H]
      rc = esgd_gemm_bf16(w_hh, dgp + (size_t)t * 4 * bh, dh_recT, H, B, 4 * H, H, 4 * H, B, 1, 0, 2, nullptr, 0, splits,
                          nullptr, nullptr, nullptr, 0, error_flag, stream);
      if (rc != 0) return rc;
    }
  }
  return 0;
}

}  // extern "C"
