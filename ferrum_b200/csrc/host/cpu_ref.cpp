// Plain single-threaded C++ restatements of the reference's CPU arithmetic.  They are
// the oracles of the CPU test-suite and the "reference CPU" arm of the small-size
// comparisons: same loop structure and operation order as the Rust code they cite, no
// vectorisation tricks, fp32 storage.
//
//   matmul      ferrum-core/src/tensor.rs:2487-2558   (i-j-p triple loop)
//   train_xor   ferrum-examples/src/train_xor.rs:9-153 (2 -> H tanh -> 1 sigmoid, MSE,
//               hand-written backward, full-batch gradient descent)
//   adam / sgd  ferrum-optim/src/adam.rs:91-146, sgd.rs:81-120
//   layer_norm  row-wise form (ferrum-nn/src/transformer.rs:316-342)
//   softmax     ferrum-cuda/src/kernels.rs:523-621 (per row, max-subtracted)
#include <cmath>
#include <cstdint>
#include <vector>

#define FB_API extern "C" __attribute__((visibility("default")))

FB_API void fb_ref_matmul(const float* a, const float* b, float* c, int M, int K, int N) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float s = 0.f;
      for (int p = 0; p < K; ++p) s += a[i * K + p] * b[p * N + j];
      c[i * N + j] = s;
    }
}

// y = x W^T + b, W [out, in]
FB_API void fb_ref_linear(const float* x, const float* w, const float* b, float* y, int B, int in, int out) {
  for (int i = 0; i < B; ++i)
    for (int o = 0; o < out; ++o) {
      float s = b ? b[o] : 0.f;
      for (int p = 0; p < in; ++p) s += x[i * in + p] * w[o * in + p];
      y[i * out + o] = s;
    }
}

FB_API void fb_ref_softmax_rows(const float* x, float* y, int rows, int cols, int log_mode) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float m = xr[0];
    for (int c = 1; c < cols; ++c) m = std::fmax(m, xr[c]);
    double s = 0.0;
    for (int c = 0; c < cols; ++c) s += std::exp(static_cast<double>(xr[c] - m));
    for (int c = 0; c < cols; ++c)
      y[r * cols + c] = log_mode ? static_cast<float>(xr[c] - m - std::log(s))
                                 : static_cast<float>(std::exp(static_cast<double>(xr[c] - m)) / s);
  }
}

FB_API void fb_ref_layernorm_rows(const float* x, const float* gamma, const float* beta, float* y, int rows,
                                  int cols, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double mu = 0.0;
    for (int c = 0; c < cols; ++c) mu += xr[c];
    mu /= cols;
    double var = 0.0;
    for (int c = 0; c < cols; ++c) var += (xr[c] - mu) * (xr[c] - mu);
    var /= cols;
    const double rs = 1.0 / std::sqrt(var + eps);
    for (int c = 0; c < cols; ++c)
      y[r * cols + c] = static_cast<float>((xr[c] - mu) * rs * (gamma ? gamma[c] : 1.f) + (beta ? beta[c] : 0.f));
  }
}

FB_API void fb_ref_adam_step(float* p, const float* g, float* m, float* v, long long n, float lr, float b1,
                             float b2, float eps, float wd, int t) {
  const float bc1 = 1.f - std::pow(b1, static_cast<float>(t));
  const float bc2 = 1.f - std::pow(b2, static_cast<float>(t));
  for (long long i = 0; i < n; ++i) {
    if (wd != 0.f) p[i] -= lr * wd * p[i];
    m[i] = b1 * m[i] + (1.f - b1) * g[i];
    v[i] = b2 * v[i] + (1.f - b2) * g[i] * g[i];
    p[i] -= lr * (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps);
  }
}

FB_API void fb_ref_sgd_step(float* p, const float* g, float* vel, long long n, float lr, float mu, float wd,
                            int nesterov, int first) {
  for (long long i = 0; i < n; ++i) {
    float gi = g[i] + wd * p[i];
    if (mu != 0.f) {
      const float vi = first ? gi : mu * vel[i] + gi;
      vel[i] = vi;
      gi = nesterov ? gi + mu * vi : vi;
    }
    p[i] -= lr * gi;
  }
}

// Full-batch training of  x[4,2] -> (W1 [2,H], b1 [H]) tanh -> (W2 [H,1], b2 [1]) sigmoid  with MSE
// (loss_kind 0) or the reference's BCE (loss_kind 1), hand-written backward, plain gradient descent.
// Weights are updated in place; losses[e] is the loss before the update of epoch e.
FB_API void fb_ref_train_xor(float* w1, float* b1, float* w2, float* b2, int H, float lr, int epochs,
                             int loss_kind, float* losses) {
  const float X[4][2] = {{0, 0}, {0, 1}, {1, 0}, {1, 1}};
  const float Y[4] = {0, 1, 1, 0};
  std::vector<float> h(4 * H), gw1(2 * H), gb1(H), gw2(H);
  for (int e = 0; e < epochs; ++e) {
    float out[4], dz2[4];
    double loss = 0.0;
    for (int i = 0; i < 4; ++i) {
      for (int j = 0; j < H; ++j) h[i * H + j] = std::tanh(X[i][0] * w1[j] + X[i][1] * w1[H + j] + b1[j]);
      float z = b2[0];
      for (int j = 0; j < H; ++j) z += h[i * H + j] * w2[j];
      out[i] = 1.f / (1.f + std::exp(-z));
      float dout;
      if (loss_kind == 0) {
        loss += (out[i] - Y[i]) * (out[i] - Y[i]);
        dout = 2.f * (out[i] - Y[i]) / 4.f;
      } else {
        const float eps = 1e-7f, pc = out[i] + eps, q = (1.f + eps) - pc;
        loss += -(Y[i] * std::log(pc) + (1.f - Y[i]) * std::log(q));
        dout = -(Y[i] / pc - (1.f - Y[i]) / q) / 4.f;
      }
      dz2[i] = dout * out[i] * (1.f - out[i]);
    }
    losses[e] = static_cast<float>(loss / 4.0);
    for (int j = 0; j < H; ++j) gw2[j] = gb1[j] = gw1[j] = gw1[H + j] = 0.f;
    float gb2 = 0.f;
    for (int i = 0; i < 4; ++i) {
      gb2 += dz2[i];
      for (int j = 0; j < H; ++j) {
        gw2[j] += h[i * H + j] * dz2[i];
        const float dz1 = dz2[i] * w2[j] * (1.f - h[i * H + j] * h[i * H + j]);
        gw1[j] += X[i][0] * dz1;
        gw1[H + j] += X[i][1] * dz1;
        gb1[j] += dz1;
      }
    }
    for (int j = 0; j < H; ++j) {
      w1[j] -= lr * gw1[j];
      w1[H + j] -= lr * gw1[H + j];
      b1[j] -= lr * gb1[j];
      w2[j] -= lr * gw2[j];
    }
    b2[0] -= lr * gb2;
  }
}
