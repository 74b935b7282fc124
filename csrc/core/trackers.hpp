// Run-level policies of the orchestrator's event loop (orchestrator/src/sessions/
// {convergence_tracker,switch_tracker,loss_recorder}.rs), plus the gradient-norm variant of the
// switch test that BASELINE-style runs use on this runtime.
#pragma once
#include <cmath>
#include <deque>
#include <map>
#include <optional>
#include <stdexcept>

namespace ono {

// Early stopping: `winsize` consecutive records whose |delta| <= tolerance (convergence_tracker.rs:36-55).
class ConvergenceTracker {
 public:
  ConvergenceTracker(size_t winsize, double tolerance) : win_(winsize), tol_(tolerance) {
    if (winsize < 2) throw std::invalid_argument("window must be greater than one");
    if (!(tolerance >= 0.0)) throw std::invalid_argument("tolerance must be non-negative");
  }
  void record(double loss) {
    if (last_ && std::fabs(*last_ - loss) > tol_) count_ = 0;
    ++count_;
    last_ = loss;
  }
  bool converged() const { return count_ == win_; }
  size_t count() const { return count_; }

 private:
  size_t win_;
  double tol_;
  std::optional<double> last_;
  size_t count_ = 0;
};

// Strategy switch: mean over the window of |x_i - x_{i-1}| / x_{i-1} <= threshold
// (switch_tracker.rs:48-62). The tracked series is the max worker loss per round in the reference;
// with switch_metric = "grad_norm" it is the global gradient L2 norm per step.
class SwitchTracker {
 public:
  SwitchTracker(size_t winsize, double threshold) : win_(winsize), thr_(threshold) {
    if (winsize < 2) throw std::invalid_argument("window must be greater than one");
  }
  void record(double v) {
    if (vals_.size() == win_) vals_.pop_front();
    vals_.push_back(v);
  }
  bool should_switch() const {
    if (vals_.size() < win_) return false;
    double sum = 0.0;
    for (size_t i = 1; i < win_; ++i) sum += std::fabs(vals_[i] - vals_[i - 1]) / vals_[i - 1];
    return sum / double(win_ - 1) <= thr_;
  }
  size_t filled() const { return vals_.size(); }

 private:
  size_t win_;
  double thr_;
  std::deque<double> vals_;
};

// Last loss per worker; aggregates only once every live worker has reported (loss_recorder.rs:23-68).
class LossRecorder {
 public:
  void record(size_t worker, double loss) {
    if (std::isnormal(loss) || loss == 0.0) losses_[worker] = loss;
  }
  std::optional<double> max(size_t workers) const {
    if (workers == 0 || losses_.size() != workers) return std::nullopt;
    double m = losses_.begin()->second;
    for (auto& kv : losses_) m = std::fmax(m, kv.second);
    return m;
  }
  std::optional<double> mean(size_t workers) const {
    if (workers == 0 || losses_.size() != workers) return std::nullopt;
    double s = 0.0;
    for (auto& kv : losses_) s += kv.second;
    return s / double(workers);
  }
  void clear() { losses_.clear(); }
  void forget(size_t worker) { losses_.erase(worker); }
  size_t size() const { return losses_.size(); }

 private:
  std::map<size_t, double> losses_;
};

// The orchestrator's reaction to loss reports (orchestrator/src/sessions/event_listener.rs:108-186):
// record each worker's last loss; once every live worker has reported take the max, clear, feed the
// early-stopping tracker (-> Stop) and then the switch tracker (-> Switch, armed once).
class SessionPolicy {
 public:
  enum Decision { Nothing = 0, Stop = 1, Switch = 2 };
  explicit SessionPolicy(size_t nworkers) : workers_left_(nworkers) {}
  void enable_early_stopping(size_t window, double tolerance) { conv_.emplace(window, tolerance); }
  void enable_switch(size_t window, double threshold) { switch_.emplace(window, threshold); }
  Decision on_losses(size_t worker, const double* losses, size_t n) {
    if (stopped_) return Nothing;
    if (n) recorder_.record(worker, losses[n - 1]);
    if (workers_left_ == 0) return Nothing;
    const auto loss = recorder_.max(workers_left_);
    if (!loss) return Nothing;
    recorder_.clear();
    last_max_ = *loss;
    return feed(*loss, true);
  }
  // Gradient-norm variant of the switch test: one value per synchronised step.
  Decision on_metric(double value) {
    if (stopped_) return Nothing;
    return feed(value, false);
  }
  void worker_left(size_t worker) {
    if (workers_left_) --workers_left_;
    recorder_.forget(worker);
  }
  size_t workers_left() const { return workers_left_; }
  bool stopped() const { return stopped_; }
  std::optional<double> last_max() const { return last_max_; }

 private:
  Decision feed(double v, bool from_loss) {
    if (from_loss && conv_) {
      conv_->record(v);
      if (conv_->converged()) { stopped_ = true; return Stop; }
    }
    if (switch_ && (from_loss != metric_is_external_)) {
      switch_->record(v);
      if (switch_->should_switch()) { switch_.reset(); return Switch; }
    }
    return Nothing;
  }

 public:
  // When true the switch tracker listens to on_metric() values instead of losses.
  void set_switch_on_metric(bool v) { metric_is_external_ = v; }

 private:
  size_t workers_left_;
  LossRecorder recorder_;
  std::optional<ConvergenceTracker> conv_;
  std::optional<SwitchTracker> switch_;
  bool stopped_ = false, metric_is_external_ = false;
  std::optional<double> last_max_;
};

}  // namespace ono
