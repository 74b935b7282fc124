// N CPU ranks in one process (one thread per rank) running the reference's three strategies over
// shared host memory: the oracle for the distributed semantics and the engine behind `cpu:` nodes.
//
//   all-reduce worker      worker/src/workers/all_reduce.rs:57-153 + middlewares/worker_ring.rs:82-204
//   parameter-server worker worker/src/workers/parameter_server.rs:56-96 + middlewares/server_cluster.rs
//   stores                 parameter_server/src/storage/{blocking,wild}
//   synchronizers          parameter_server/src/synchronization/{barrier,non_blocking}.rs
//   strategy switch        node/src/router.rs:188-341, worker/src/builder.rs:165-200
//   orchestrator policy    orchestrator/src/sessions/event_listener.rs:108-219
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../core/dyn_barrier.hpp"
#include "../core/json.hpp"
#include "../core/trackers.hpp"
#include "engine.hpp"

namespace ono::oracle {

// ---- parameter-server storage -----------------------------------------------------------------
class Store {
 public:
  virtual ~Store() = default;
  virtual size_t len() const = 0;
  virtual void accumulate(const float* grad, size_t n) = 0;
  virtual void update_params() = 0;
  virtual void pull_params(float* out) = 0;
  virtual Optimizer& optimizer() = 0;
  // Parameters and optimizer state of the shard as one consistent copy (taken under the store's lock).
  virtual void snapshot(std::vector<float>& params, std::vector<float>& m, std::vector<float>& v, float& b1t, float& b2t) = 0;
};

// Two gradient accumulators flipped by the single updater; update = mean over workers, optimizer,
// zero the frozen buffer (storage/blocking/store.rs:84-108, shard.rs:56-92).
class BlockingStore final : public Store {
 public:
  BlockingStore(std::vector<float> params, const OptimizerSpec& opt, size_t nworkers);
  size_t len() const override { return params_.size(); }
  void accumulate(const float* grad, size_t n) override;
  void update_params() override;
  void pull_params(float* out) override;
  Optimizer& optimizer() override { return opt_; }
  void snapshot(std::vector<float>& params, std::vector<float>& m, std::vector<float>& v, float& b1t, float& b2t) override;

 private:
  std::vector<float> params_, acc_[2];
  int active_ = 0;
  size_t nworkers_;
  Optimizer opt_;
  std::mutex mu_;
};

// Hogwild: the optimizer is applied at once, without averaging; update_params is a no-op
// (storage/wild/shard.rs:43-58). A mutex keeps the C++ memory model honest; the semantics
// (per-push application, no division) are the reference's.
class WildStore final : public Store {
 public:
  WildStore(std::vector<float> params, const OptimizerSpec& opt);
  size_t len() const override { return params_.size(); }
  void accumulate(const float* grad, size_t n) override;
  void update_params() override {}
  void pull_params(float* out) override;
  Optimizer& optimizer() override { return opt_; }
  void snapshot(std::vector<float>& params, std::vector<float>& m, std::vector<float>& v, float& b1t, float& b2t) override;

 private:
  std::vector<float> params_;
  Optimizer opt_;
  std::mutex mu_;
};

class Synchronizer {
 public:
  virtual ~Synchronizer() = default;
  // accumulate grad, (wait,) update, copy the fresh parameters into params_out
  virtual void step(Store& store, const float* grad, size_t n, float* params_out) = 0;
  virtual void leave(Store& store) = 0;  // the calling worker will not come back
};

class BarrierSync final : public Synchronizer {
 public:
  explicit BarrierSync(size_t nworkers) : barrier_(nworkers) {}
  void step(Store& store, const float* grad, size_t n, float* params_out) override;
  void leave(Store& store) override;

 private:
  DynBarrier barrier_;
};

class NonBlockingSync final : public Synchronizer {
 public:
  void step(Store& store, const float* grad, size_t n, float* params_out) override;
  void leave(Store&) override {}
};

// ---- events -----------------------------------------------------------------------------------
struct ClusterEvent {
  std::string kind;            // losses | upgrading | upgraded | switch | worker_done | error | complete
  size_t worker = 0;
  std::vector<double> losses;
  std::string text;            // stop reason / error message
};

struct ClusterOptions {
  std::string wire = "f32";        // "f32" | "f16" (the reference always uses f16 for gradients)
  bool sparse = false;             // SparseCapable serializer
  double sparse_r = 0.0;
  bool leaky_relu_exact = true;
  bool switch_resets_progress = false;
  // Optimizer state to start from (global parameter order; empty = fresh state) and the number of epochs the saved
  // run had done (offsets the shuffle sequence). The reference has no such thing: it exports weights only.
  std::vector<float> init_m, init_v;
  float init_b1t = 1.f, init_b2t = 1.f;
  size_t start_epoch = 0;
  // Every `checkpoint_every` epochs (counted from the saved run's first epoch) the leading worker takes a copy of the
  // parameters and the optimizer state and announces it with a "checkpoint" event; the host fetches it with
  // pop_checkpoint() and writes the files. 0 = never.
  size_t checkpoint_every = 0;
};

struct ClusterState {              // optimizer state at the end of a run, global parameter order
  std::vector<float> m, v;
  float b1t = 1.f, b2t = 1.f;
  size_t epochs = 0;
};

class LocalCluster {
 public:
  // `plan` is the document produced by adapt_configs(); `data` the whole dataset (partitioned by
  // the plan's row ranges).
  LocalCluster(Json plan, Dataset data, ClusterOptions opts);
  ~LocalCluster();
  void start();
  void request_stop();                                  // StopAfterEpoch to every worker
  bool next_event(ClusterEvent& ev, int timeout_ms);    // false on timeout
  void join();
  bool finished() const { return finished_.load(); }
  const std::vector<float>& final_params() const { return final_params_; }
  const ClusterState& final_state() const { return final_state_; }
  // The oldest checkpoint not fetched yet (see ClusterOptions::checkpoint_every); false if there is none.
  bool pop_checkpoint(std::vector<float>& params, ClusterState& state);
  const std::string& stop_reason() const { return stop_reason_; }
  bool switched() const { return switched_.load(); }

 private:
  struct Server {
    std::unique_ptr<Store> store;
    std::unique_ptr<Synchronizer> sync;
    std::vector<std::pair<size_t, size_t>> ranges;  // global ranges concatenated into the shard
  };
  void emit(ClusterEvent ev);
  void run_all();
  void all_reduce_worker(size_t w);
  void ps_worker(size_t w, RoundTrainer& trainer, std::vector<float>& params);
  void ring_all_reduce(size_t w, std::vector<float>& residual, std::vector<float>& grad);
  SessionPolicy::Decision report_losses(size_t w, const std::vector<double>& losses);
  void build_servers(const Json& server_list, const std::vector<std::vector<float>>* inline_params);
  void gather_final_from_servers();
  void note_epochs(size_t done);
  // Called by the leading worker between rounds, when no update is in flight on its side.
  void maybe_checkpoint(size_t epochs_done, const std::vector<float>* replica, const Optimizer* replica_opt);

  Json plan_;
  Dataset data_;
  ClusterOptions opts_;
  uint64_t seed_ = 0;
  size_t n_params_ = 0, nworkers_ = 0;
  std::vector<std::thread> threads_;
  std::thread main_;
  std::mutex ev_mu_;
  std::condition_variable ev_cv_;
  std::deque<ClusterEvent> events_;
  std::mutex policy_mu_;
  std::unique_ptr<SessionPolicy> policy_;
  std::atomic<bool> stop_{false}, finished_{false}, switched_{false};
  std::string stop_reason_ = "max_epochs";
  std::vector<float> final_params_;
  ClusterState final_state_;
  struct Checkpoint { std::vector<float> params; ClusterState state; };
  std::mutex ckpt_mu_;
  std::deque<Checkpoint> ckpts_;
  size_t ckpt_mark_ = 0, ps_leader_ = 0;
  std::vector<Server> servers_;
  // all-reduce shared state
  std::vector<std::vector<float>*> ring_bufs_;          // each worker's residual (scatter) buffer
  std::vector<std::vector<float>*> ring_grads_;         // each worker's gathered gradient buffer
  std::vector<std::vector<float>> ring_msgs_;          // what each worker put on the wire this hop
  std::unique_ptr<DynBarrier> ring_barrier_;
  std::atomic<int> round_decision_{0};                  // decision published by the round leader
  std::vector<std::vector<float>> ar_params_;           // canonical params per worker (replicas)
  std::vector<std::unique_ptr<RoundTrainer>> trainers_;
  std::vector<int> pending_decision_;
};

}  // namespace ono::oracle
