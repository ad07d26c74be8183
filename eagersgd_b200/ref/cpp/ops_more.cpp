// CPU oracles, second part: the operators of the reference's C++ operator set that ops.cpp does not have,
// each with its backward pass, and the backward passes of max pool / global average pool / softmax / GEMM /
// ReLU (deep500/frameworks/reference/custom_operators/cpp/operators/: add_op.cpp, sum_op.cpp,
// averagepool_op.cpp, batchnormalization_op_inference.cpp, matmul_op.cpp, reshape_op.cpp, maxpool_op.cpp,
// globalaveragepool_op.cpp, softmax_op.cpp, gemm_op.cpp, relu_op.cpp).  Plain loops, fp32 data, double
// accumulation: written to be obviously right, not fast.  NCHW.
#include <stdint.h>
#include <string.h>
#include <cmath>
#include <limits>

#define IDX4(n, c, h, w, C, H, W) ((((int64_t)(n) * (C) + (c)) * (H) + (h)) * (W) + (w))

extern "C" {

// ---- Add / Sum (element-wise; the gradient of each input is the output gradient) -----------------------------
void ref_add_fwd(const float* a, const float* b, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = a[i] + b[i];
}
void ref_add_bwd(const float* dy, float* da, float* db, int64_t n) {
  memcpy(da, dy, (size_t)n * sizeof(float));
  memcpy(db, dy, (size_t)n * sizeof(float));
}
void ref_sum_fwd(const float* const* inputs, int num_inputs, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    double s = 0;
    for (int k = 0; k < num_inputs; ++k) s += inputs[k][i];
    y[i] = (float)s;
  }
}
void ref_sum_bwd(const float* dy, float* const* dinputs, int num_inputs, int64_t n) {
  for (int k = 0; k < num_inputs; ++k) memcpy(dinputs[k], dy, (size_t)n * sizeof(float));
}

// ---- Reshape: data is untouched, only the gradient's view changes ------------------------------------------------
void ref_reshape_fwd(const float* x, float* y, int64_t n) { memcpy(y, x, (size_t)n * sizeof(float)); }
void ref_reshape_bwd(const float* dy, float* dx, int64_t n) { memcpy(dx, dy, (size_t)n * sizeof(float)); }

// ---- ReLU backward --------------------------------------------------------------------------------------------------
void ref_relu_bwd(const float* x, const float* dy, float* dx, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dx[i] = x[i] > 0 ? dy[i] : 0.0f;
}

// ---- MatMul [M,K] x [K,N] and its two gradients ---------------------------------------------------------------------
void ref_matmul_fwd(const float* A, const float* B, float* Y, int M, int N, int K) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double s = 0;
      for (int k = 0; k < K; ++k) s += (double)A[(int64_t)i * K + k] * B[(int64_t)k * N + j];
      Y[(int64_t)i * N + j] = (float)s;
    }
}
void ref_matmul_bwd(const float* A, const float* B, const float* dY, float* dA, float* dB, int M, int N, int K) {
  for (int i = 0; i < M; ++i)          // dA = dY B^T
    for (int k = 0; k < K; ++k) {
      double s = 0;
      for (int j = 0; j < N; ++j) s += (double)dY[(int64_t)i * N + j] * B[(int64_t)k * N + j];
      dA[(int64_t)i * K + k] = (float)s;
    }
  for (int k = 0; k < K; ++k)          // dB = A^T dY
    for (int j = 0; j < N; ++j) {
      double s = 0;
      for (int i = 0; i < M; ++i) s += (double)A[(int64_t)i * K + k] * dY[(int64_t)i * N + j];
      dB[(int64_t)k * N + j] = (float)s;
    }
}

// ---- GEMM backward: Y = alpha op(A) op(B) + beta C -------------------------------------------------------------------
void ref_gemm_bwd(const float* A, const float* B, const float* dY, float* dA, float* dB, float* dC, int M, int N, int K,
                  int trans_a, int trans_b, float alpha, float beta) {
  // gradients with respect to op(A) [M,K] and op(B) [K,N], stored back in the layout A and B have
  for (int i = 0; i < M; ++i)
    for (int k = 0; k < K; ++k) {
      double s = 0;
      for (int j = 0; j < N; ++j) {
        const float b = trans_b ? B[(int64_t)j * K + k] : B[(int64_t)k * N + j];
        s += (double)dY[(int64_t)i * N + j] * b;
      }
      if (trans_a) dA[(int64_t)k * M + i] = (float)(alpha * s);
      else dA[(int64_t)i * K + k] = (float)(alpha * s);
    }
  for (int k = 0; k < K; ++k)
    for (int j = 0; j < N; ++j) {
      double s = 0;
      for (int i = 0; i < M; ++i) {
        const float a = trans_a ? A[(int64_t)k * M + i] : A[(int64_t)i * K + k];
        s += (double)a * dY[(int64_t)i * N + j];
      }
      if (trans_b) dB[(int64_t)j * K + k] = (float)(alpha * s);
      else dB[(int64_t)k * N + j] = (float)(alpha * s);
    }
  if (dC != nullptr)
    for (int64_t i = 0; i < (int64_t)M * N; ++i) dC[i] = beta * dY[i];
}

// ---- Softmax backward (rows): dx = y * (dy - sum(dy * y)) -------------------------------------------------------------
void ref_softmax_bwd(const float* y, const float* dy, float* dx, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    double dot = 0;
    for (int c = 0; c < cols; ++c) dot += (double)dy[(int64_t)r * cols + c] * y[(int64_t)r * cols + c];
    for (int c = 0; c < cols; ++c)
      dx[(int64_t)r * cols + c] = (float)(y[(int64_t)r * cols + c] * (dy[(int64_t)r * cols + c] - dot));
  }
}

// ---- Max pool backward: the gradient goes to the first maximum of every window -------------------------------------------
void ref_maxpool_bwd(const float* x, const float* dy, float* dx, int N, int C, int H, int W, int k, int stride, int pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  memset(dx, 0, (size_t)N * C * H * W * sizeof(float));
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int p = 0; p < Ho; ++p)
        for (int q = 0; q < Wo; ++q) {
          float m = -std::numeric_limits<float>::infinity();
          int bh = -1, bw = -1;
          for (int r = 0; r < k; ++r)
            for (int s = 0; s < k; ++s) {
              const int h = p * stride + r - pad, w = q * stride + s - pad;
              if (h >= 0 && h < H && w >= 0 && w < W && x[IDX4(n, c, h, w, C, H, W)] > m) {
                m = x[IDX4(n, c, h, w, C, H, W)];
                bh = h; bw = w;
              }
            }
          if (bh >= 0) dx[IDX4(n, c, bh, bw, C, H, W)] += dy[IDX4(n, c, p, q, C, Ho, Wo)];
        }
}

// ---- Average pool (count_include_pad selectable) and its backward ----------------------------------------------------------
void ref_avgpool_fwd(const float* x, float* y, int N, int C, int H, int W, int k, int stride, int pad, int include_pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int p = 0; p < Ho; ++p)
        for (int q = 0; q < Wo; ++q) {
          double s = 0;
          int cnt = 0;
          for (int r = 0; r < k; ++r)
            for (int t = 0; t < k; ++t) {
              const int h = p * stride + r - pad, w = q * stride + t - pad;
              if (h >= 0 && h < H && w >= 0 && w < W) { s += x[IDX4(n, c, h, w, C, H, W)]; ++cnt; }
            }
          y[IDX4(n, c, p, q, C, Ho, Wo)] = (float)(s / (include_pad ? k * k : (cnt > 0 ? cnt : 1)));
        }
}
void ref_avgpool_bwd(const float* dy, float* dx, int N, int C, int H, int W, int k, int stride, int pad, int include_pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  memset(dx, 0, (size_t)N * C * H * W * sizeof(float));
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int p = 0; p < Ho; ++p)
        for (int q = 0; q < Wo; ++q) {
          int cnt = 0;
          for (int r = 0; r < k; ++r)
            for (int t = 0; t < k; ++t) {
              const int h = p * stride + r - pad, w = q * stride + t - pad;
              if (h >= 0 && h < H && w >= 0 && w < W) ++cnt;
            }
          const float g = dy[IDX4(n, c, p, q, C, Ho, Wo)] / (float)(include_pad ? k * k : (cnt > 0 ? cnt : 1));
          for (int r = 0; r < k; ++r)
            for (int t = 0; t < k; ++t) {
              const int h = p * stride + r - pad, w = q * stride + t - pad;
              if (h >= 0 && h < H && w >= 0 && w < W) dx[IDX4(n, c, h, w, C, H, W)] += g;
            }
        }
}

// ---- Global average pool backward ----------------------------------------------------------------------------------------------
void ref_global_avgpool_bwd(const float* dy, float* dx, int N, int C, int HW) {
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int i = 0; i < HW; ++i) dx[((int64_t)n * C + c) * HW + i] = dy[(int64_t)n * C + c] / (float)HW;
}

// ---- Batch norm, inference mode: y = gamma (x - mean) / sqrt(var + eps) + beta, and its gradients -------------------------------
void ref_batchnorm_infer_fwd(const float* x, const float* gamma, const float* beta, const float* mean, const float* var,
                             float* y, int N, int C, int HW, float eps) {
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      const double inv = 1.0 / std::sqrt((double)var[c] + eps);
      for (int i = 0; i < HW; ++i) {
        const int64_t o = ((int64_t)n * C + c) * HW + i;
        y[o] = (float)(gamma[c] * (x[o] - mean[c]) * inv + beta[c]);
      }
    }
}
void ref_batchnorm_infer_bwd(const float* x, const float* gamma, const float* mean, const float* var, const float* dy,
                             float* dx, float* dgamma, float* dbeta, int N, int C, int HW, float eps) {
  for (int c = 0; c < C; ++c) {
    const double inv = 1.0 / std::sqrt((double)var[c] + eps);
    double dg = 0, db = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) {
        const int64_t o = ((int64_t)n * C + c) * HW + i;
        dx[o] = (float)(dy[o] * gamma[c] * inv);
        dg += (double)dy[o] * (x[o] - mean[c]) * inv;
        db += dy[o];
      }
    dgamma[c] = (float)dg;
    dbeta[c] = (float)db;
  }
}

}  // extern "C"
