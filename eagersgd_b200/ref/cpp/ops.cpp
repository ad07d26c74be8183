// Naive C++ restatements of the hot operators, the CPU oracles of the CUDA kernels
// (same role as the reference's deep500/frameworks/reference/custom_operators/cpp/operators/*.cpp
// and cpp/utility/*.hpp: cross-correlation loop nests for convolution and its two gradients,
// per-channel batch-norm training forward / backward, triple-loop GEMM, softmax, pooling, ReLU).
// Plain loops, fp32 storage with double accumulation, NCHW, OpenMP over the batch.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>

#define IDX4(n, c, h, w, C, H, W) ((((int64_t)(n) * (C) + (c)) * (H) + (h)) * (W) + (w))

extern "C" {

void ref_conv2d_fwd(const float* x, const float* w, float* y, int N, int C, int H, int W, int K, int R, int S,
                    int stride, int pad) {
  const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
#pragma omp parallel for collapse(2)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k)
      for (int p = 0; p < Ho; ++p)
        for (int q = 0; q < Wo; ++q) {
          double acc = 0;
          for (int c = 0; c < C; ++c)
            for (int r = 0; r < R; ++r)
              for (int s = 0; s < S; ++s) {
                const int h = p * stride + r - pad, ww = q * stride + s - pad;
                if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
                acc += (double)x[IDX4(n, c, h, ww, C, H, W)] * w[IDX4(k, c, r, s, C, R, S)];
              }
          y[IDX4(n, k, p, q, K, Ho, Wo)] = (float)acc;
        }
}

// dx: cross-correlation of the (dilated) dy with the flipped filter, written as a scatter.
void ref_conv2d_dgrad(const float* dy, const float* w, float* dx, int N, int C, int H, int W, int K, int R, int S,
                      int stride, int pad) {
  const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
#pragma omp parallel for collapse(2)
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int h = 0; h < H; ++h)
        for (int ww = 0; ww < W; ++ww) {
          double acc = 0;
          for (int k = 0; k < K; ++k)
            for (int r = 0; r < R; ++r)
              for (int s = 0; s < S; ++s) {
                const int ph = h + pad - r, pw = ww + pad - s;
                if (ph < 0 || pw < 0 || ph % stride || pw % stride) continue;
                const int p = ph / stride, q = pw / stride;
                if (p >= Ho || q >= Wo) continue;
                acc += (double)dy[IDX4(n, k, p, q, K, Ho, Wo)] * w[IDX4(k, c, r, s, C, R, S)];
              }
          dx[IDX4(n, c, h, ww, C, H, W)] = (float)acc;
        }
}

// dw: cross-correlation of x with dy over the batch ("swap axes").
void ref_conv2d_wgrad(const float* x, const float* dy, float* dw, int N, int C, int H, int W, int K, int R, int S,
                      int stride, int pad) {
  const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
#pragma omp parallel for collapse(2)
  for (int k = 0; k < K; ++k)
    for (int c = 0; c < C; ++c)
      for (int r = 0; r < R; ++r)
        for (int s = 0; s < S; ++s) {
          double acc = 0;
          for (int n = 0; n < N; ++n)
            for (int p = 0; p < Ho; ++p)
              for (int q = 0; q < Wo; ++q) {
                const int h = p * stride + r - pad, ww = q * stride + s - pad;
                if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
                acc += (double)x[IDX4(n, c, h, ww, C, H, W)] * dy[IDX4(n, k, p, q, K, Ho, Wo)];
              }
          dw[IDX4(k, c, r, s, C, R, S)] = (float)acc;
        }
}

void ref_batchnorm_train_fwd(const float* x, const float* gamma, const float* beta, float* y, float* running_mean,
                             float* running_var, float* save_mean, float* save_invstd, int N, int C, int HW,
                             float momentum, float eps) {
  const double m = (double)N * HW;
#pragma omp parallel for
  for (int c = 0; c < C; ++c) {
    double s = 0, s2 = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) { double v = x[((int64_t)n * C + c) * HW + i]; s += v; s2 += v * v; }
    const double mean = s / m, var = std::max(s2 / m - mean * mean, 0.0), invstd = 1.0 / std::sqrt(var + eps);
    save_mean[c] = (float)mean;
    save_invstd[c] = (float)invstd;
    running_mean[c] = (float)((1 - momentum) * running_mean[c] + momentum * mean);
    running_var[c] = (float)((1 - momentum) * running_var[c] + momentum * var * m / std::max(m - 1, 1.0));
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) {
        const int64_t o = ((int64_t)n * C + c) * HW + i;
        y[o] = (float)((x[o] - mean) * invstd * gamma[c] + beta[c]);
      }
  }
}

void ref_batchnorm_train_bwd(const float* x, const float* gamma, const float* save_mean, const float* save_invstd,
                             const float* dy, float* dx, float* dgamma, float* dbeta, int N, int C, int HW) {
  const double m = (double)N * HW;
#pragma omp parallel for
  for (int c = 0; c < C; ++c) {
    double db = 0, dg = 0;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) {
        const int64_t o = ((int64_t)n * C + c) * HW + i;
        db += dy[o];
        dg += dy[o] * (x[o] - save_mean[c]) * save_invstd[c];
      }
    dbeta[c] = (float)db;
    dgamma[c] = (float)dg;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) {
        const int64_t o = ((int64_t)n * C + c) * HW + i;
        const double xhat = (x[o] - save_mean[c]) * save_invstd[c];
        dx[o] = (float)(gamma[c] * save_invstd[c] * (dy[o] - db / m - xhat * dg / m));
      }
  }
}

// C = alpha * op(A) op(B) + beta * C, four transpose cases (gemm.hpp).
void ref_gemm(const float* A, const float* B, float* C, int M, int N, int K, int trans_a, int trans_b, float alpha,
              float beta) {
#pragma omp parallel for
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double acc = 0;
      for (int k = 0; k < K; ++k) {
        const float a = trans_a ? A[(int64_t)k * M + i] : A[(int64_t)i * K + k];
        const float b = trans_b ? B[(int64_t)j * K + k] : B[(int64_t)k * N + j];
        acc += (double)a * b;
      }
      C[(int64_t)i * N + j] = (float)(alpha * acc + beta * C[(int64_t)i * N + j]);
    }
}

void ref_softmax(const float* x, float* y, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    float mx = -std::numeric_limits<float>::infinity();
    for (int c = 0; c < cols; ++c) mx = std::max(mx, x[(int64_t)r * cols + c]);
    double s = 0;
    for (int c = 0; c < cols; ++c) s += std::exp((double)x[(int64_t)r * cols + c] - mx);
    for (int c = 0; c < cols; ++c) y[(int64_t)r * cols + c] = (float)(std::exp((double)x[(int64_t)r * cols + c] - mx) / s);
  }
}

void ref_maxpool(const float* x, float* y, int N, int C, int H, int W, int k, int stride, int pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int p = 0; p < Ho; ++p)
        for (int q = 0; q < Wo; ++q) {
          float m = -std::numeric_limits<float>::infinity();
          for (int r = 0; r < k; ++r)
            for (int s = 0; s < k; ++s) {
              const int h = p * stride + r - pad, w = q * stride + s - pad;
              if (h >= 0 && h < H && w >= 0 && w < W) m = std::max(m, x[IDX4(n, c, h, w, C, H, W)]);
            }
          y[IDX4(n, c, p, q, C, Ho, Wo)] = m;
        }
}

void ref_global_avgpool(const float* x, float* y, int N, int C, int HW) {
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      double s = 0;
      for (int i = 0; i < HW; ++i) s += x[((int64_t)n * C + c) * HW + i];
      y[(int64_t)n * C + c] = (float)(s / HW);
    }
}

void ref_relu(const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = x[i] > 0 ? x[i] : 0;
}

}  // extern "C"
