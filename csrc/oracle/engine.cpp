#include "engine.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <stdexcept>

#include "../core/adapter.hpp"
#include "../core/philox.h"

namespace ono::oracle {

// ---- small dense kernels (row-major) ----------------------------------------------------------
// The hot loops are plain C++ written so that the compiler vectorises them (unit-stride updates and `omp simd` reductions),
// compiled once per instruction-set level and picked at load time by the CPU that runs them: a node binary built on one
// machine runs on another. Summation order inside a dot product therefore depends on the vector width; every comparison
// against this engine allows for rounding.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__) && !defined(ONO_NO_CLONES)
#define ONO_HOT __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))
#else
#define ONO_HOT
#endif

// c[0..n) += a * b[0..n)
#define ONO_AXPY(c, a, b, n)                             \
  _Pragma("omp simd") for (size_t j_ = 0; j_ < (n); ++j_) (c)[j_] += (a) * (b)[j_]

// C[M,N] (+)= A[M,K] * B[K,N]
ONO_HOT static void gemm_nn(const float* A, const float* B, float* C, size_t M, size_t N, size_t K, bool accumulate) {
  if (!accumulate) std::fill(C, C + M * N, 0.f);
  for (size_t i = 0; i < M; ++i) {
    float* c = C + i * N;
    size_t k = 0;
    for (; k + 4 <= K; k += 4) {       // four rows of B per pass over c: a quarter of the loads and stores of c
      const float a0 = A[i * K + k], a1 = A[i * K + k + 1], a2 = A[i * K + k + 2], a3 = A[i * K + k + 3];
      if (a0 == 0.f && a1 == 0.f && a2 == 0.f && a3 == 0.f) continue;
      const float *b0 = B + k * N, *b1 = b0 + N, *b2 = b1 + N, *b3 = b2 + N;
#pragma omp simd
      for (size_t j = 0; j < N; ++j) c[j] += a0 * b0[j] + a1 * b1[j] + a2 * b2[j] + a3 * b3[j];
    }
    for (; k < K; ++k) {
      const float a = A[i * K + k];
      if (a == 0.f) continue;
      const float* b = B + k * N;
      ONO_AXPY(c, a, b, N);
    }
  }
}
// C[K,N] += A[M,K]^T * D[M,N]
ONO_HOT static void gemm_tn_acc(const float* A, const float* D, float* C, size_t M, size_t N, size_t K) {
  size_t i = 0;
  for (; i + 4 <= M; i += 4) {         // four samples per pass over a row of C
    const float *d0 = D + i * N, *d1 = d0 + N, *d2 = d1 + N, *d3 = d2 + N;
    for (size_t k = 0; k < K; ++k) {
      const float a0 = A[i * K + k], a1 = A[(i + 1) * K + k], a2 = A[(i + 2) * K + k], a3 = A[(i + 3) * K + k];
      if (a0 == 0.f && a1 == 0.f && a2 == 0.f && a3 == 0.f) continue;
      float* c = C + k * N;
#pragma omp simd
      for (size_t j = 0; j < N; ++j) c[j] += a0 * d0[j] + a1 * d1[j] + a2 * d2[j] + a3 * d3[j];
    }
  }
  for (; i < M; ++i) {
    const float* d = D + i * N;
    for (size_t k = 0; k < K; ++k) {
      const float a = A[i * K + k];
      if (a == 0.f) continue;
      float* c = C + k * N;
      ONO_AXPY(c, a, d, N);
    }
  }
}
ONO_HOT static float dot(const float* a, const float* b, size_t n) {
  float s = 0.f;
#pragma omp simd reduction(+ : s)
  for (size_t j = 0; j < n; ++j) s += a[j] * b[j];
  return s;
}
// C[M,K] = D[M,N] * W[K,N]^T
ONO_HOT static void gemm_nt(const float* D, const float* W, float* C, size_t M, size_t N, size_t K) {
  for (size_t i = 0; i < M; ++i) {
    const float* d = D + i * N;
    for (size_t k = 0; k < K; ++k) {
      const float* w = W + k * N;
      float s = 0.f;
#pragma omp simd reduction(+ : s)
      for (size_t j = 0; j < N; ++j) s += d[j] * w[j];
      C[i * K + k] = s;
    }
  }
}
// Convolution backward for one sample. dcol[ckk, npix] = K[F, ckk]^T delta[F, npix]
ONO_HOT static void conv_dcol(const float* kernels, const float* delta, float* dcol, size_t F, size_t ckk, size_t npix) {
  std::fill(dcol, dcol + ckk * npix, 0.f);
  for (size_t f = 0; f < F; ++f) {
    const float* dd = delta + f * npix;
    for (size_t q = 0; q < ckk; ++q) {
      const float kv = kernels[f * ckk + q];
      if (kv == 0.f) continue;
      float* dc = dcol + q * npix;
      ONO_AXPY(dc, kv, dd, npix);
    }
  }
}
// dK[F, ckk] += delta[F, npix] col[ckk, npix]^T ; db[F] += row sums of delta
ONO_HOT static void conv_dk(const float* delta, const float* col, float* dk, float* db, size_t F, size_t ckk, size_t npix) {
  for (size_t f = 0; f < F; ++f) {
    const float* dd = delta + f * npix;
    for (size_t q = 0; q < ckk; ++q) {
      const float* cc = col + q * npix;
      float s = 0.f;
#pragma omp simd reduction(+ : s)
      for (size_t i = 0; i < npix; ++i) s += dd[i] * cc[i];
      dk[f * ckk + q] += s;
    }
    float sb = 0.f;
#pragma omp simd reduction(+ : sb)
    for (size_t i = 0; i < npix; ++i) sb += dd[i];
    db[f] += sb;
  }
}

// ---- activations ------------------------------------------------------------------------------
// exp and tanh as branch-free float code the compiler vectorises (Cephes-style range reduction and polynomials, a few ulp
// from libm): a LeNet-5 sample runs ~6 500 of them, which cost as much as its convolutions when taken one libm call at a time.
static inline float exp_poly(float x) {
  x = std::min(88.f, std::max(-87.f, x));
  const float n = std::nearbyint(x * 1.44269504088896341f);
  const float r = (x - n * 0.693359375f) - n * -2.12194440e-4f;
  float p = 1.9875691500e-4f;
  p = p * r + 1.3981999507e-3f;
  p = p * r + 8.3334519073e-3f;
  p = p * r + 4.1665795894e-2f;
  p = p * r + 1.6666665459e-1f;
  p = p * r + 5.0000001201e-1f;
  const float e = p * r * r + r + 1.f;
  int32_t bits = ((int32_t)n + 127) << 23;
  float scale;
  std::memcpy(&scale, &bits, 4);
  return e * scale;
}
ONO_HOT static void act_sigmoid(float* y, size_t n, float amp) {
#pragma omp simd
  for (size_t i = 0; i < n; ++i) y[i] = amp / (1.f + exp_poly(-y[i]));
}
ONO_HOT static void act_tanh(float* y, size_t n, float amp) {
#pragma omp simd
  for (size_t i = 0; i < n; ++i) {
    const float x = y[i], ax = std::fabs(x), z = x * x;
    float small = -5.70498872745e-3f;
    small = small * z + 2.06390887954e-2f;
    small = small * z - 5.37397155531e-2f;
    small = small * z + 1.33314422036e-1f;
    small = small * z - 3.33332819422e-1f;
    small = small * z * x + x;
    const float big = std::copysign(1.f - 2.f / (exp_poly(2.f * ax) + 1.f), x);
    y[i] = amp * (ax < 0.625f ? small : big);
  }
}

ActFn ActFn::from_spec(const Json& j) {
  ActFn a;
  if (j.is_null()) return a;
  if (j.is_string()) {
    if (j.as_string() == "softmax") a.kind = Act::Softmax;
    else if (j.as_string() == "gelu") a.kind = Act::Gelu;
    else throw std::runtime_error("unknown activation " + j.as_string());
    return a;
  }
  const auto& m = j.members().at(0);
  if (m.first == "sigmoid") { a.kind = Act::Sigmoid; a.param = (float)m.second.at("amp").as_double(); }
  else if (m.first == "tanh") { a.kind = Act::Tanh; a.param = (float)m.second.at("amp").as_double(); }
  else if (m.first == "relu" || m.first == "re_l_u") { a.kind = Act::ReLU; a.param = (float)m.second.at("slope").as_double(); }
  else throw std::runtime_error("unknown activation " + m.first);
  return a;
}

void Layer::apply_act(std::vector<float>& y, size_t B, size_t width) {
  switch (act.kind) {
    case Act::None: break;
    case Act::Sigmoid: act_sigmoid(y.data(), y.size(), act.param); break;
    case Act::Tanh: act_tanh(y.data(), y.size(), act.param); break;
    case Act::ReLU: for (auto& v : y) v = std::max(v, act.param * v); break;
    case Act::Gelu:
      pre_ = y;
      for (auto& v : y) v = 0.5f * v * (1.f + std::erf(v * 0.70710678118654752f));
      break;
    case Act::Softmax:
      for (size_t b = 0; b < B; ++b) {
        float* r = y.data() + b * width;
        const float mx = *std::max_element(r, r + width);
        float z = 0.f;
        for (size_t j = 0; j < width; ++j) { r[j] = std::exp(r[j] - mx); z += r[j]; }
        const float inv = 1.f / z;
        for (size_t j = 0; j < width; ++j) r[j] *= inv;
      }
      break;
  }
  if (act.kind != Act::None) acts_ = y;
}

void Layer::act_backward(std::vector<float>& d, size_t B, size_t width) {
  const float p = act.param;
  switch (act.kind) {
    case Act::None: break;
    case Act::Sigmoid: for (size_t i = 0; i < d.size(); ++i) d[i] *= acts_[i] * (1.f - acts_[i] / p); break;
    case Act::Tanh: for (size_t i = 0; i < d.size(); ++i) d[i] *= p - acts_[i] * acts_[i] / p; break;
    case Act::ReLU:
      for (size_t i = 0; i < d.size(); ++i)
        if (acts_[i] <= 0.f) d[i] = leaky_relu_exact ? p * d[i] : p * acts_[i];
      break;
    case Act::Gelu:
      for (size_t i = 0; i < d.size(); ++i) {
        const float z = pre_[i];
        const float cdf = 0.5f * (1.f + std::erf(z * 0.70710678118654752f));
        const float pdf = 0.3989422804014327f * std::exp(-0.5f * z * z);
        d[i] *= cdf + z * pdf;
      }
      break;
    case Act::Softmax:
      for (size_t b = 0; b < B; ++b) {
        const float* a = acts_.data() + b * width;
        float* db = d.data() + b * width;
        float dot = 0.f;
        for (size_t j = 0; j < width; ++j) dot += a[j] * db[j];
        for (size_t j = 0; j < width; ++j) db[j] = a[j] * (db[j] - dot);
      }
      break;
  }
}

// ---- layers -----------------------------------------------------------------------------------
namespace {

class Dense final : public Layer {
 public:
  Dense(size_t in, size_t out) : in_(in), out_(out) {}
  size_t n_params() const override { return (in_ + 1) * out_; }
  size_t in_size() const override { return in_; }
  size_t out_size() const override { return out_; }
  void forward(const float* params, const float* x, size_t B, std::vector<float>& y) override {
    x_.assign(x, x + B * in_);
    y.resize(B * out_);
    gemm_nn(x, params, y.data(), B, out_, in_, false);
    const float* b = params + in_ * out_;
    for (size_t i = 0; i < B; ++i)
      for (size_t j = 0; j < out_; ++j) y[i * out_ + j] += b[j];
    apply_act(y, B, out_);
  }
  void backward(const float* params, float* grad, std::vector<float>& d, size_t B, std::vector<float>& dx) override {
    act_backward(d, B, out_);
    gemm_tn_acc(x_.data(), d.data(), grad, B, out_, in_);  // dW = X^T d
    float* gb = grad + in_ * out_;
    for (size_t i = 0; i < B; ++i)
      for (size_t j = 0; j < out_; ++j) gb[j] += d[i * out_ + j];
    if (!need_dx) { dx.clear(); return; }
    dx.resize(B * in_);
    gemm_nt(d.data(), params, dx.data(), B, out_, in_);  // dX = d W^T
  }

 private:
  size_t in_, out_;
  std::vector<float> x_;
};

class Conv2d final : public Layer {
 public:
  Conv2d(size_t c, size_t h, size_t w, size_t f, size_t k, size_t s, size_t p)
      : C_(c), H_(h), W_(w), F_(f), K_(k), S_(s), P_(p) {
    OH_ = (H_ + 2 * P_ - K_) / S_ + 1;
    OW_ = (W_ + 2 * P_ - K_) / S_ + 1;
  }
  size_t n_params() const override { return F_ * C_ * K_ * K_ + F_; }
  size_t in_size() const override { return C_ * H_ * W_; }
  size_t out_size() const override { return F_ * OH_ * OW_; }
  void forward(const float* params, const float* x, size_t B, std::vector<float>& y) override {
    x_.assign(x, x + B * in_size());
    y.assign(B * out_size(), 0.f);
    const size_t ckk = C_ * K_ * K_, npix = OH_ * OW_;
    col_.resize(ckk * npix);
    const float* bias = params + F_ * ckk;
    for (size_t b = 0; b < B; ++b) {
      im2col(x + b * in_size());
      float* yb = y.data() + b * out_size();
      gemm_nn(params, col_.data(), yb, F_, npix, ckk, false);  // [F,Ckk] x [Ckk, oh*ow]
      for (size_t f = 0; f < F_; ++f)
        for (size_t i = 0; i < npix; ++i) yb[f * npix + i] += bias[f];
    }
    apply_act(y, B, out_size());
  }
  void backward(const float* params, float* grad, std::vector<float>& d, size_t B, std::vector<float>& dx) override {
    act_backward(d, B, out_size());
    const size_t ckk = C_ * K_ * K_, npix = OH_ * OW_;
    if (need_dx) dx.assign(B * in_size(), 0.f);
    else dx.clear();
    dcol_.resize(ckk * npix);
    float* gb = grad + F_ * ckk;
    for (size_t b = 0; b < B; ++b) {
      const float* db = d.data() + b * out_size();
      // col_delta = K^T delta  -> col2im scatter-add (conv2d.rs:161-172, 240-266)
      if (need_dx) {
        conv_dcol(params, db, dcol_.data(), F_, ckk, npix);
        col2im(dx.data() + b * in_size());
      }
      // dK += delta col^T (conv2d.rs:174-180)
      im2col(x_.data() + b * in_size());
      conv_dk(db, col_.data(), grad, gb, F_, ckk, npix);
    }
  }

 private:
  // Output columns [lo, hi) of a row whose input column ox * S + kx - P falls inside the image.
  void valid_span(size_t kx, size_t& lo, size_t& hi) const {
    lo = kx >= P_ ? 0 : (P_ - kx + S_ - 1) / S_;
    const long last = (long)W_ - 1 + (long)P_ - (long)kx;          // largest ox * S allowed
    hi = last < 0 ? 0 : std::min(OW_, (size_t)last / S_ + 1);
    if (lo > hi) lo = hi;
  }
  void im2col(const float* x) {
    const size_t npix = OH_ * OW_;
    for (size_t c = 0; c < C_; ++c)
      for (size_t ky = 0; ky < K_; ++ky)
        for (size_t kx = 0; kx < K_; ++kx) {
          float* row = col_.data() + ((c * K_ + ky) * K_ + kx) * npix;
          size_t lo, hi;
          valid_span(kx, lo, hi);
          for (size_t oy = 0; oy < OH_; ++oy) {
            const long iy = (long)(oy * S_ + ky) - (long)P_;
            float* r = row + oy * OW_;
            if (iy < 0 || iy >= (long)H_) { std::fill(r, r + OW_, 0.f); continue; }
            std::fill(r, r + lo, 0.f);
            if (hi > lo) {
              const float* src = x + (c * H_ + iy) * W_ + (lo * S_ + kx - P_);   // lo * S + kx >= P inside the span
              if (S_ == 1) std::copy(src, src + (hi - lo), r + lo);
              else for (size_t ox = lo; ox < hi; ++ox) r[ox] = src[(ox - lo) * S_];
            }
            std::fill(r + hi, r + OW_, 0.f);
          }
        }
  }
  void col2im(float* dx) {
    const size_t npix = OH_ * OW_;
    for (size_t c = 0; c < C_; ++c)
      for (size_t ky = 0; ky < K_; ++ky)
        for (size_t kx = 0; kx < K_; ++kx) {
          const float* row = dcol_.data() + ((c * K_ + ky) * K_ + kx) * npix;
          size_t lo, hi;
          valid_span(kx, lo, hi);
          for (size_t oy = 0; oy < OH_; ++oy) {
            const long iy = (long)(oy * S_ + ky) - (long)P_;
            if (iy < 0 || iy >= (long)H_ || hi <= lo) continue;
            float* dst = dx + (c * H_ + iy) * W_ + (lo * S_ + kx - P_);
            const float* r = row + oy * OW_ + lo;
            if (S_ == 1) { for (size_t t = 0; t < hi - lo; ++t) dst[t] += r[t]; }
            else for (size_t t = 0; t < hi - lo; ++t) dst[t * S_] += r[t];
          }
        }
  }
  size_t C_, H_, W_, F_, K_, S_, P_, OH_, OW_;
  std::vector<float> x_, col_, dcol_;
};

class MaxPool final : public Layer {
 public:
  MaxPool(size_t c, size_t h, size_t w, size_t k, size_t s, size_t p) : C_(c), H_(h), W_(w), K_(k), S_(s), P_(p) {
    OH_ = (H_ + 2 * P_ - K_) / S_ + 1;
    OW_ = (W_ + 2 * P_ - K_) / S_ + 1;
  }
  size_t n_params() const override { return 0; }
  size_t in_size() const override { return C_ * H_ * W_; }
  size_t out_size() const override { return C_ * OH_ * OW_; }
  void forward(const float*, const float* x, size_t B, std::vector<float>& y) override {
    y.resize(B * out_size());
    arg_.resize(B * out_size());
    for (size_t b = 0; b < B; ++b)
      for (size_t c = 0; c < C_; ++c) {
        const float* xc = x + b * in_size() + c * H_ * W_;
        for (size_t oy = 0; oy < OH_; ++oy)
          for (size_t ox = 0; ox < OW_; ++ox) {
            // Zero padding takes part in the max; on ties the last element in scan order wins
            // (Iterator::max_by), max_pooling.rs:97-118.
            float best = -INFINITY;
            long by = 0, bx = 0;
            for (size_t ky = 0; ky < K_; ++ky)
              for (size_t kx = 0; kx < K_; ++kx) {
                const long py = (long)(oy * S_ + ky), px = (long)(ox * S_ + kx);  // padded coords
                const long iy = py - (long)P_, ix = px - (long)P_;
                const float v = (iy >= 0 && iy < (long)H_ && ix >= 0 && ix < (long)W_) ? xc[iy * W_ + ix] : 0.f;
                if (v >= best) { best = v; by = py; bx = px; }
              }
            const size_t o = b * out_size() + (c * OH_ + oy) * OW_ + ox;
            y[o] = best;
            arg_[o] = {by, bx};
          }
      }
    apply_act(y, B, out_size());
  }
  void backward(const float*, float*, std::vector<float>& d, size_t B, std::vector<float>& dx) override {
    act_backward(d, B, out_size());
    dx.assign(B * in_size(), 0.f);
    for (size_t b = 0; b < B; ++b)
      for (size_t c = 0; c < C_; ++c)
        for (size_t i = 0; i < OH_ * OW_; ++i) {
          const size_t o = b * out_size() + c * OH_ * OW_ + i;
          const long iy = arg_[o].first - (long)P_, ix = arg_[o].second - (long)P_;
          if (iy >= 0 && iy < (long)H_ && ix >= 0 && ix < (long)W_) dx[b * in_size() + (c * H_ + iy) * W_ + ix] += d[o];
        }
  }

 private:
  size_t C_, H_, W_, K_, S_, P_, OH_, OW_;
  std::vector<std::pair<long, long>> arg_;
};

}  // namespace

std::unique_ptr<Layer> make_layer(const Json& spec, size_t input_size) {
  const auto& m = spec.members().at(0);
  const Json& b = m.second;
  std::unique_ptr<Layer> l;
  auto u = [](const Json& v) { return (size_t)v.as_u64(); };
  if (m.first == "dense") {
    l = std::make_unique<Dense>(u(b.at("dim")[0]), u(b.at("dim")[1]));
  } else if (m.first == "conv") {
    const Json& i = b.at("input_dim");
    const Json& k = b.at("kernel_dim");
    l = std::make_unique<Conv2d>(u(i[0]), u(i[1]), u(i[2]), u(k[0]), u(k[2]), u(b.at("stride")), u(b.at("padding")));
  } else if (m.first == "max_pooling") {
    const Json& i = b.at("input_dim");
    l = std::make_unique<MaxPool>(u(i[0]), u(i[1]), u(i[2]), u(b.at("filter_size")), u(b.at("stride")), u(b.at("padding")));
  } else {
    throw std::runtime_error("unknown layer spec " + m.first);
  }
  if (l->in_size() != input_size)
    throw std::runtime_error("layer expects an input of " + std::to_string(l->in_size()) + " but the incoming size is " + std::to_string(input_size));
  if (const Json* a = b.find("act_fn")) l->act = ActFn::from_spec(*a);
  return l;
}

Sequential::Sequential(const Json& layer_specs, size_t x_size, bool leaky_relu_exact) {
  size_t in = x_size;
  for (auto& ls : layer_specs.items()) {
    auto l = make_layer(ls, in);
    l->leaky_relu_exact = leaky_relu_exact;
    offsets_.push_back(n_params_);
    n_params_ += l->n_params();
    in = l->out_size();
    layers_.push_back(std::move(l));
  }
  if (layers_.empty()) throw std::runtime_error("model must have at least one layer");
  layers_.front()->need_dx = false;
  outs_.resize(layers_.size());
}

const std::vector<float>& Sequential::forward(const float* params, const float* x, size_t B) {
  const float* cur = x;
  for (size_t i = 0; i < layers_.size(); ++i) {
    layers_[i]->forward(params + offsets_[i], cur, B, outs_[i]);
    cur = outs_[i].data();
  }
  return outs_.back();
}

void Sequential::backward(const float* params, float* grad, std::vector<float>& d, size_t B) {
  std::vector<float>* cur = &d;
  std::vector<float>* bufs[2] = {&dx_a_, &dx_b_};
  int flip = 0;
  for (size_t i = layers_.size(); i-- > 0;) {
    std::vector<float>* nxt = bufs[flip];
    layers_[i]->backward(params + offsets_[i], grad + offsets_[i], *cur, B, *nxt);
    cur = nxt;
    flip ^= 1;
  }
}

// ---- loss -------------------------------------------------------------------------------------
double loss_prime(Loss kind, const float* yp, const float* y, size_t n, std::vector<float>& delta) {
  delta.resize(n);
  const float fn = (float)n;
  double total = 0.0;
  if (kind == Loss::Mse) {
    const float two_over_n = 2.0f / fn;
    for (size_t i = 0; i < n; ++i) {
      const float diff = yp[i] - y[i];
      total += (double)(diff * diff);
      delta[i] = diff * two_over_n;
    }
  } else {
    const float one_over_n = 1.0f / fn;
    for (size_t i = 0; i < n; ++i) {
      const float safe = std::max(yp[i], 1.1920929e-07f);
      total -= (double)(y[i] * std::log(safe));
      delta[i] = -(y[i] / safe) * one_over_n;
    }
  }
  return total / (double)fn;
}

// ---- optimizers -------------------------------------------------------------------------------
OptimizerSpec OptimizerSpec::from_spec(const Json& j) {
  OptimizerSpec o;
  const auto& m = j.members().at(0);
  const Json& b = m.second;
  auto lr_of = [&]() { return (float)(b.has("learning_rate") ? b.at("learning_rate") : b.at("lr")).as_double(); };
  o.lr = lr_of();
  if (m.first == "gradient_descent") o.kind = GradientDescent;
  else if (m.first == "gradient_descent_with_momentum") { o.kind = Momentum; o.mu = (float)(b.has("momentum") ? b.at("momentum") : b.at("mu")).as_double(); }
  else if (m.first == "adam") {
    o.kind = Adam;
    o.b1 = (float)(b.has("beta1") ? b.at("beta1") : b.at("b1")).as_double();
    o.b2 = (float)(b.has("beta2") ? b.at("beta2") : b.at("b2")).as_double();
    o.eps = (float)(b.has("epsilon") ? b.at("epsilon") : b.at("eps")).as_double();
  } else throw std::runtime_error("unknown optimizer " + m.first);
  return o;
}

Optimizer::Optimizer(const OptimizerSpec& spec, size_t n) : spec_(spec) {
  if (spec.kind != OptimizerSpec::GradientDescent) m_.assign(n, 0.f);
  if (spec.kind == OptimizerSpec::Adam) v_.assign(n, 0.f);
}

void Optimizer::reset() {
  std::fill(m_.begin(), m_.end(), 0.f);
  std::fill(v_.begin(), v_.end(), 0.f);
  b1t_ = b2t_ = 1.f;
}

void Optimizer::load_state(const float* m, const float* v, float b1t, float b2t) {
  if (m && !m_.empty()) std::copy(m, m + m_.size(), m_.begin());
  if (v && !v_.empty()) std::copy(v, v + v_.size(), v_.begin());
  if (spec_.kind == OptimizerSpec::Adam) { b1t_ = b1t; b2t_ = b2t; }
}

void Optimizer::step(float* p, const float* g, size_t n) {
  const auto& s = spec_;
  if (s.kind == OptimizerSpec::GradientDescent) {
    for (size_t i = 0; i < n; ++i) p[i] -= s.lr * g[i];
  } else if (s.kind == OptimizerSpec::Momentum) {
    for (size_t i = 0; i < n; ++i) {
      m_[i] = s.mu * m_[i] + g[i];
      p[i] -= s.lr * m_[i];
    }
  } else {
    b1t_ *= s.b1;
    b2t_ *= s.b2;
    const float step = s.lr * std::sqrt(1.f - b2t_) / (1.f - b1t_);
    for (size_t i = 0; i < n; ++i) {
      m_[i] = s.b1 * m_[i] + (1.f - s.b1) * g[i];
      v_[i] = s.b2 * v_[i] + (1.f - s.b2) * g[i] * g[i];
      p[i] -= step * m_[i] / (std::sqrt(v_[i]) + s.eps);
    }
  }
}

// ---- parameter generators ---------------------------------------------------------------------
size_t param_gen_size(const Json& spec) {
  const auto& m = spec.members().at(0);
  if (m.first == "const" || m.first == "rand") return (size_t)m.second.at("limit").as_u64();
  if (m.first == "inline") return m.second.at("params").size();
  if (m.first == "chained") {
    size_t n = 0;
    for (auto& s : m.second.at("specs").items()) n += param_gen_size(s);
    return n;
  }
  throw std::runtime_error("unknown param_gen " + m.first);
}

void param_gen_fill(const Json& spec, uint64_t seed, std::vector<float>& out) {
  const auto& m = spec.members().at(0);
  const Json& b = m.second;
  if (m.first == "const") {
    out.insert(out.end(), (size_t)b.at("limit").as_u64(), (float)b.at("value").as_double());
  } else if (m.first == "inline") {
    for (auto& v : b.at("params").items()) out.push_back((float)v.as_double());
  } else if (m.first == "rand") {
    int kind;
    float lo, hi;
    resolve_distribution(b.at("distribution"), kind, lo, hi);
    const uint64_t off = b.has("index_offset") ? b.at("index_offset").as_u64() : 0;
    const size_t n = (size_t)b.at("limit").as_u64();
    for (size_t i = 0; i < n; ++i) out.push_back(philox_sample(off + i, seed, kind, lo, hi));
  } else if (m.first == "chained") {
    for (auto& s : b.at("specs").items()) param_gen_fill(s, seed, out);
  } else {
    throw std::runtime_error("unknown param_gen " + m.first);
  }
}

// ---- dataset ----------------------------------------------------------------------------------
void Dataset::shuffle(uint64_t seed, uint64_t epoch) {
  const size_t n = rows();
  if (n < 2) return;
  std::vector<float> tx(x_size), ty(y_size);
  const uint64_t key = seed ^ (0x9E3779B97F4A7C15ull * (epoch + 1));
  for (size_t i = n - 1; i > 0; --i) {
    const Philox4 r = philox4x32_10(i, key);
    const uint64_t rnd = ((uint64_t)r.v[0] << 32) | r.v[1];
    const size_t j = (size_t)(rnd % (i + 1));
    if (i == j) continue;
    std::swap_ranges(samples.begin() + i * x_size, samples.begin() + (i + 1) * x_size, samples.begin() + j * x_size);
    std::swap_ranges(labels.begin() + i * y_size, labels.begin() + (i + 1) * y_size, labels.begin() + j * y_size);
  }
}

void Dataset::append(const Dataset& o) {
  samples.insert(samples.end(), o.samples.begin(), o.samples.end());
  labels.insert(labels.end(), o.labels.begin(), o.labels.end());
}

Dataset Dataset::slice(size_t b, size_t e) const {
  Dataset d;
  d.x_size = x_size;
  d.y_size = y_size;
  d.samples.assign(samples.begin() + b * x_size, samples.begin() + e * x_size);
  d.labels.assign(labels.begin() + b * y_size, labels.begin() + e * y_size);
  return d;
}

std::vector<Dataset> Dataset::partition(size_t n) const {
  std::vector<Dataset> out;
  for (auto& [b, e] : dataset_partitions(rows(), n)) out.push_back(slice(b, e));
  return out;
}

// ---- round trainer ----------------------------------------------------------------------------
RoundTrainer::RoundTrainer(const Json& ts, Dataset dataset, bool leaky_relu_exact)
    : model_(ts.at("layers"), (size_t)ts.at("dataset").at("x_size").as_u64(), leaky_relu_exact), data_(std::move(dataset)) {
  loss_ = ts.at("loss_fn").as_string() == "mse" ? Loss::Mse : Loss::CrossEntropy;
  opt_ = OptimizerSpec::from_spec(ts.at("optimizer"));
  batch_size_ = (size_t)ts.at("batch_size").as_u64();
  max_epochs_ = (size_t)ts.at("max_epochs").as_u64();
  offline_epochs_ = (size_t)ts.at("offline_epochs").as_u64();
  if (const Json* s = ts.find("seed"); s && !s->is_null()) seed_ = s->as_u64();
  else seed_ = (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
  data_.x_size = (size_t)ts.at("dataset").at("x_size").as_u64();
  data_.y_size = (size_t)ts.at("dataset").at("y_size").as_u64();
  grad_.assign(model_.n_params(), 0.f);
}

TrainResult RoundTrainer::train(float* params, float* residual) {
  TrainResult res;
  const size_t remaining = max_epochs_ > epoch_ ? max_epochs_ - epoch_ : 0;
  const size_t todo = std::min(remaining, offline_epochs_ + 1);
  const size_t n = data_.rows(), P = model_.n_params();
  if (n == 0) throw std::runtime_error("empty epoch: the worker has no samples");
  for (size_t e = 0; e < todo; ++e) {
    data_.shuffle(seed_, epoch_base_ + epoch_);
    double total = 0.0;
    size_t batches = 0;
    for (size_t lo = 0; lo < n; lo += batch_size_) {
      const size_t B = std::min(batch_size_, n - lo);  // the ragged tail is used (dataset.rs:85-95)
      const auto& out = model_.forward(params, data_.samples.data() + lo * data_.x_size, B);
      total += loss_prime(loss_, out.data(), data_.labels.data() + lo * data_.y_size, out.size(), delta_);
      model_.backward(params, grad_.data(), delta_, B);
      // stateless SGD at the optimizer's learning rate + residual accumulation + zero_grad
      // (sequential.rs:129-141, backprop_trainer.rs:67-70)
      for (size_t i = 0; i < P; ++i) {
        params[i] -= opt_.lr * grad_[i];
        residual[i] += grad_[i];
        grad_[i] = 0.f;
      }
      ++batches;
    }
    res.losses.push_back(total / (double)batches);
    ++epoch_;
  }
  res.is_last = epoch_ >= max_epochs_;
  return res;
}

std::pair<double, double> RoundTrainer::evaluate(const float* params, const Dataset& d, size_t batch) {
  const size_t n = d.rows();
  double loss = 0.0;
  size_t correct = 0, batches = 0;
  std::vector<float> tmp;
  for (size_t lo = 0; lo < n; lo += batch) {
    const size_t B = std::min(batch, n - lo);
    const auto& out = model_.forward(params, d.samples.data() + lo * d.x_size, B);
    loss += loss_prime(loss_, out.data(), d.labels.data() + lo * d.y_size, out.size(), tmp);
    const size_t C = d.y_size;
    for (size_t b = 0; b < B; ++b) {
      const float* o = out.data() + b * C;
      const float* y = d.labels.data() + (lo + b) * C;
      if (std::max_element(o, o + C) - o == std::max_element(y, y + C) - y) ++correct;
    }
    ++batches;
  }
  return {batches ? loss / (double)batches : 0.0, n ? (double)correct / (double)n : 0.0};
}

}  // namespace ono::oracle
