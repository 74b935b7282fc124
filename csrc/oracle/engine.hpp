// CPU restatement of the reference's neural-network engine (machine_learning/src): same maths,
// same round semantics, f32 compute with f64 loss accumulation. It is the numerical authority for
// the CUDA kernels' tests, the engine behind CPU ranks, and the timed CPU baseline.
//
//   Layer / Sequential   arch/layers/{dense,conv/conv2d,max_pooling,relu,sigmoid,tanh,softmax}.rs,
//                        arch/sequential.rs:43-148
//   losses               arch/loss/{mse,cross_entropy}.rs
//   optimizers           optimization/{gradient_descent,gradient_descent_with_momentum,adam}.rs
//   param generators     initialization/* (streams replaced by Philox counters keyed by global index)
//   dataset              datasets/{dataset,inmem_src}.rs
//   round trainer        training/backprop_trainer.rs:101-141
//
// Tensors are flat row-major float arrays; images are NCHW like the reference's Array4.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../core/json.hpp"

namespace ono::oracle {

enum class Act { None, Sigmoid, Softmax, Tanh, ReLU, Gelu };

struct ActFn {
  Act kind = Act::None;
  float param = 0.f;
  static ActFn from_spec(const Json& j);  // ActFnSpec or null
};

class Layer {
 public:
  virtual ~Layer() = default;
  virtual size_t n_params() const = 0;
  virtual size_t in_size() const = 0;
  virtual size_t out_size() const = 0;
  // y[B, out] = f(x[B, in]; params). Keeps whatever backward needs.
  virtual void forward(const float* params, const float* x, size_t B, std::vector<float>& y) = 0;
  // d[B, out] is the gradient w.r.t. this layer's output (after activation). Writes the parameter
  // gradient into grad (+=) and the gradient w.r.t. the input into dx[B, in].
  virtual void backward(const float* params, float* grad, std::vector<float>& d, size_t B, std::vector<float>& dx) = 0;
  ActFn act;
  bool leaky_relu_exact = true;  // false reproduces relu.rs:41-45 (d := slope * a where a <= 0)
  bool need_dx = true;           // false for a model's first layer: nobody consumes the gradient w.r.t. the input

 protected:
  void apply_act(std::vector<float>& y, size_t B, size_t width);
  void act_backward(std::vector<float>& d, size_t B, size_t width);  // uses acts_
  std::vector<float> acts_;  // stored activations (post-activation output)
  std::vector<float> pre_;   // stored pre-activations (GELU only)
};

std::unique_ptr<Layer> make_layer(const Json& layer_spec, size_t input_size);

class Sequential {
 public:
  Sequential() = default;
  Sequential(const Json& layer_specs, size_t x_size, bool leaky_relu_exact = true);
  size_t n_params() const { return n_params_; }
  size_t out_size() const { return layers_.back()->out_size(); }
  const std::vector<float>& forward(const float* params, const float* x, size_t B);
  // d = dLoss/dOutput [B, out]; accumulates into grad[n_params].
  void backward(const float* params, float* grad, std::vector<float>& d, size_t B);
  std::vector<size_t> layer_offsets() const { return offsets_; }
  size_t n_layers() const { return layers_.size(); }

 private:
  std::vector<std::unique_ptr<Layer>> layers_;
  std::vector<size_t> offsets_;
  std::vector<std::vector<float>> outs_;
  std::vector<float> dx_a_, dx_b_;
  size_t n_params_ = 0;
};

enum class Loss { Mse, CrossEntropy };
// Returns the loss; fills delta[B*C] (mse.rs:25-48, cross_entropy.rs:25-48; n = B*C).
double loss_prime(Loss kind, const float* y_pred, const float* y, size_t n, std::vector<float>& delta);

struct OptimizerSpec {
  enum Kind { GradientDescent, Momentum, Adam } kind = GradientDescent;
  float lr = 0.01f, mu = 0.f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f;
  static OptimizerSpec from_spec(const Json& j);
};

class Optimizer {
 public:
  Optimizer() = default;
  Optimizer(const OptimizerSpec& spec, size_t n);
  void step(float* params, const float* grad, size_t n);  // n must equal the constructed size
  const OptimizerSpec& spec() const { return spec_; }
  void reset();
  // The state a later run needs to continue exactly here (empty vectors where the optimizer keeps none).
  const std::vector<float>& m() const { return m_; }
  const std::vector<float>& v() const { return v_; }
  float b1t() const { return b1t_; }
  float b2t() const { return b2t_; }
  // m / v: n floats each, or null to leave the moment as it is; ignored where the optimizer keeps none.
  void load_state(const float* m, const float* v, float b1t, float b2t);

 private:
  OptimizerSpec spec_;
  std::vector<float> m_, v_;
  float b1t_ = 1.f, b2t_ = 1.f;
};

// Fills out[0..n) from a ParamGenSpec (const / inline / rand / chained). Random values come from
// Philox keyed by (seed, index_offset + i), so the same element gets the same value however the
// model is sharded. Returns the number of elements produced (the spec's total size).
size_t param_gen_size(const Json& spec);
void param_gen_fill(const Json& spec, uint64_t seed, std::vector<float>& out);

struct Dataset {
  std::vector<float> samples, labels;
  size_t x_size = 0, y_size = 0;
  size_t rows() const { return x_size ? samples.size() / x_size : 0; }
  // Fisher-Yates row shuffle (inmem_src.rs:31-43) driven by Philox(seed, epoch).
  void shuffle(uint64_t seed, uint64_t epoch);
  void append(const Dataset& other);
  Dataset slice(size_t row_begin, size_t row_end) const;
  std::vector<Dataset> partition(size_t n) const;  // dataset.rs:104-119
};

struct TrainResult {
  std::vector<double> losses;  // mean batch loss of each epoch run in this round
  bool is_last = false;
};

// One worker's trainer (backprop_trainer.rs). `train` runs min(remaining, offline_epochs+1) local
// epochs of stateless SGD at the optimizer's learning rate on `params` (mutated in place) and sums
// the per-batch gradients into `residual`.
class RoundTrainer {
 public:
  RoundTrainer(const Json& trainer_spec, Dataset dataset, bool leaky_relu_exact = true);
  TrainResult train(float* params, float* residual);
  size_t n_params() const { return model_.n_params(); }
  size_t epochs_done() const { return epoch_; }
  size_t max_epochs() const { return max_epochs_; }
  const OptimizerSpec& optimizer_spec() const { return opt_; }
  Dataset& dataset() { return data_; }
  Sequential& model() { return model_; }
  void set_epochs_done(size_t e) { epoch_ = e; }
  // A resumed run continues the shuffle sequence of the saved one. Every epoch permutes the order the previous epoch
  // left, so the permutations of the epochs already done are replayed on the fresh partition first.
  void set_epoch_base(size_t e) {
    for (size_t k = 0; k < e; ++k) data_.shuffle(seed_, k);
    epoch_base_ = e;
  }
  // Mean loss and accuracy (arg-max match) of `params` over a dataset; used for evaluation.
  std::pair<double, double> evaluate(const float* params, const Dataset& d, size_t batch = 256);

 private:
  Sequential model_;
  Dataset data_;
  Loss loss_ = Loss::Mse;
  OptimizerSpec opt_;
  size_t batch_size_ = 1, max_epochs_ = 1, offline_epochs_ = 0, epoch_ = 0, epoch_base_ = 0;
  uint64_t seed_ = 0;
  std::vector<float> grad_, delta_;
};

}  // namespace ono::oracle
