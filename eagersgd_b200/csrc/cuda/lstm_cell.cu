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

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// One thread per (b, j): B*H threads.
__global__ void __launch_bounds__(256)
lstm_cell_fwd_kernel(const __nv_bfloat16* __restrict__ xproj,   // [B, 4H]
                     const float* __restrict__ hprojT,          // [4H, ldh] (ldh >= B), may be null at t = 0
                     const float* __restrict__ bias,            // [4H] (b_ih + b_hh)
                     const float* __restrict__ c_prev,          // [B, H] or null
                     float* __restrict__ c_out,                 // [B, H]
                     __nv_bfloat16* __restrict__ h_out,         // [B, H]
                     __nv_bfloat16* __restrict__ gates,         // [B, 4H] activations i, f, g, o
                     int B, int H, int ldh) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  float pre[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int row = k * H + j;
    float v = __bfloat162float(xproj[(size_t)b * 4 * H + row]) + bias[row];
    if (hprojT != nullptr) v += hprojT[(size_t)row * ldh + b];
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
                     const float* __restrict__ dh_recT,         // [H, ldr] recurrent gradient, transposed (may be null)
                     float* __restrict__ dc,                    // [B, H] in: dc_t, out: dc_{t-1}
                     __nv_bfloat16* __restrict__ dgates,        // [B, 4H] pre-activation gradients
                     int B, int H, int ldr) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  const __nv_bfloat16* gp = gates + (size_t)b * 4 * H + j;
  const float ig = __bfloat162float(gp[0]), fg = __bfloat162float(gp[H]), gg = __bfloat162float(gp[2 * H]),
              og = __bfloat162float(gp[3 * H]);
  float dh = dh_ext != nullptr ? __bfloat162float(dh_ext[idx]) : 0.0f;
  if (dh_recT != nullptr) dh += dh_recT[(size_t)j * ldr + b];
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

}  // namespace

extern "C" {

int esgd_lstm_cell_fwd(const void* xproj, const float* hprojT, const float* bias, const float* c_prev, float* c_out,
                       void* h_out, void* gates, int B, int H, int ldh, void* stream) {
  lstm_cell_fwd_kernel<<<(B * H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)xproj, hprojT, bias, c_prev, c_out, (__nv_bfloat16*)h_out, (__nv_bfloat16*)gates, B, H,
      ldh);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

int esgd_lstm_cell_bwd(const void* gates, const float* c_prev, const float* c_cur, const void* dh_ext,
                       const float* dh_recT, float* dc, void* dgates, int B, int H, int ldr, void* stream) {
  lstm_cell_bwd_kernel<<<(B * H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gates, c_prev, c_cur, (const __nv_bfloat16*)dh_ext, dh_recT, dc, (__nv_bfloat16*)dgates,
      B, H, ldr);
  esgd::count_launch();
  return (int)cudaGetLastError();
}

}  // extern "C"
