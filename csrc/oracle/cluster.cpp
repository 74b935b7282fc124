#include "cluster.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <stdexcept>

#include "../core/adapter.hpp"
#include "../core/codec.hpp"

namespace ono::oracle {

// ---- stores -----------------------------------------------------------------------------------
BlockingStore::BlockingStore(std::vector<float> params, const OptimizerSpec& opt, size_t nworkers)
    : params_(std::move(params)), nworkers_(nworkers), opt_(opt, params_.size()) {
  acc_[0].assign(params_.size(), 0.f);
  acc_[1].assign(params_.size(), 0.f);
}

void BlockingStore::accumulate(const float* grad, size_t n) {
  if (n != params_.size()) return;  // pserver.rs:145-151: wrong-sized gradients are ignored
  std::lock_guard<std::mutex> lk(mu_);
  float* a = acc_[active_].data();
  for (size_t i = 0; i < n; ++i) a[i] += grad[i];
}

void BlockingStore::update_params() {
  std::lock_guard<std::mutex> lk(mu_);
  const int frozen = active_;
  active_ ^= 1;  // new pushes land in the other accumulator while this one is applied
  float* g = acc_[frozen].data();
  const float inv = 1.0f / (float)nworkers_;
  for (size_t i = 0; i < params_.size(); ++i) g[i] *= inv;  // shard.rs:78-83
  opt_.step(params_.data(), g, params_.size());
  std::fill(acc_[frozen].begin(), acc_[frozen].end(), 0.f);
}

void BlockingStore::pull_params(float* out) {
  std::lock_guard<std::mutex> lk(mu_);
  std::copy(params_.begin(), params_.end(), out);
}

void BlockingStore::snapshot(std::vector<float>& params, std::vector<float>& m, std::vector<float>& v, float& b1t, float& b2t) {
  std::lock_guard<std::mutex> lk(mu_);
  params = params_;
  m = opt_.m();
  v = opt_.v();
  b1t = opt_.b1t();
  b2t = opt_.b2t();
}

WildStore::WildStore(std::vector<float> params, const OptimizerSpec& opt) : params_(std::move(params)), opt_(opt, params_.size()) {}

void WildStore::accumulate(const float* grad, size_t n) {
  if (n != params_.size()) return;
  std::lock_guard<std::mutex> lk(mu_);
  opt_.step(params_.data(), grad, n);
}

void WildStore::pull_params(float* out) {
  std::lock_guard<std::mutex> lk(mu_);
  std::copy(params_.begin(), params_.end(), out);
}

void WildStore::snapshot(std::vector<float>& params, std::vector<float>& m, std::vector<float>& v, float& b1t, float& b2t) {
  std::lock_guard<std::mutex> lk(mu_);
  params = params_;
  m = opt_.m();
  v = opt_.v();
  b1t = opt_.b1t();
  b2t = opt_.b2t();
}

// ---- synchronizers ----------------------------------------------------------------------------
void BarrierSync::step(Store& store, const float* grad, size_t n, float* params_out) {
  store.accumulate(grad, n);
  barrier_.wait_with([&] { store.update_params(); });
  store.pull_params(params_out);
}

void BarrierSync::leave(Store& store) {
  barrier_.leave([&] { store.update_params(); });
}

void NonBlockingSync::step(Store& store, const float* grad, size_t n, float* params_out) {
  store.accumulate(grad, n);
  store.update_params();
  store.pull_params(params_out);
}

// ---- cluster plumbing -------------------------------------------------------------------------
LocalCluster::LocalCluster(Json plan, Dataset data, ClusterOptions opts)
    : plan_(std::move(plan)), data_(std::move(data)), opts_(std::move(opts)) {
  ckpt_mark_ = opts_.checkpoint_every ? opts_.start_epoch / opts_.checkpoint_every : 0;
  n_params_ = (size_t)plan_.at("n_params").as_u64();
  nworkers_ = plan_.at("workers").size();
  if (const Json* s = plan_.find("seed"); s && !s->is_null()) seed_ = s->as_u64();
  else seed_ = (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
  policy_ = std::make_unique<SessionPolicy>(nworkers_);
  if (const Json* e = plan_.find("early_stopping"); e && !e->is_null())
    policy_->enable_early_stopping((size_t)e->at("window").as_u64(), e->at("tolerance").as_double());
  if (const Json* s = plan_.find("switch"); s && !s->is_null())
    policy_->enable_switch((size_t)s->at("window").as_u64(), s->at("threshold").as_double());
}

LocalCluster::~LocalCluster() {
  request_stop();
  join();
}

void LocalCluster::emit(ClusterEvent ev) {
  {
    std::lock_guard<std::mutex> lk(ev_mu_);
    events_.push_back(std::move(ev));
  }
  ev_cv_.notify_all();
}

bool LocalCluster::next_event(ClusterEvent& ev, int timeout_ms) {
  std::unique_lock<std::mutex> lk(ev_mu_);
  if (!ev_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !events_.empty(); })) return false;
  ev = std::move(events_.front());
  events_.pop_front();
  return true;
}

void LocalCluster::request_stop() {
  bool expected = false;
  if (stop_.compare_exchange_strong(expected, true)) {
    std::lock_guard<std::mutex> lk(policy_mu_);
    if (stop_reason_ == "max_epochs") stop_reason_ = "stopped";
  }
}

void LocalCluster::start() { main_ = std::thread([this] { run_all(); }); }

void LocalCluster::join() {
  if (main_.joinable()) main_.join();
}

SessionPolicy::Decision LocalCluster::report_losses(size_t w, const std::vector<double>& losses) {
  for (double l : losses)
    if (!std::isfinite(l)) {  // comms/src/handles/worker.rs:110-120: a non-finite loss aborts the run
      ClusterEvent ev;
      ev.kind = "error";
      ev.worker = w;
      ev.text = "worker reported a non-finite loss";
      emit(std::move(ev));
      request_stop();
      std::lock_guard<std::mutex> lk(policy_mu_);
      stop_reason_ = "error";
      return SessionPolicy::Stop;
    }
  ClusterEvent ev;
  ev.kind = "losses";
  ev.worker = w;
  ev.losses = losses;
  emit(std::move(ev));
  std::lock_guard<std::mutex> lk(policy_mu_);
  const auto d = policy_->on_losses(w, losses.data(), losses.size());
  if (d == SessionPolicy::Stop) {
    stop_reason_ = "early_stopping";
    stop_.store(true);
  }
  return d;
}

// ---- ring all-reduce --------------------------------------------------------------------------
namespace {

// near-equal split, the first `rem` chunks one element longer (worker/src/middlewares/mod.rs:15-59)
void chunk_bounds(size_t n, size_t parts, size_t c, size_t& lo, size_t& hi) {
  const size_t base = n / parts, rem = n % parts;
  lo = base * c + std::min(c, rem);
  hi = lo + base + (c < rem ? 1 : 0);
}

// What the receiver of `src[0..n)` decodes, given the wire format. Returns the sparse threshold
// (negative when the message went out dense).
float encode_decode(const float* src, size_t n, const ClusterOptions& o, uint64_t seed, std::vector<float>& out) {
  out.resize(n);
  if (o.sparse) {
    Compressed c = compress_gradient(src, n, true, o.sparse_r, seed);
    if (c.sparse) {
      sparse_lift(out, c.bytes.data(), c.bytes.size());
      out.resize(n, 0.f);
      return c.threshold;
    }
  }
  if (o.wire == "f16" || o.sparse) {
    for (size_t i = 0; i < n; ++i) out[i] = f16_round_trip(src[i]);
  } else {
    std::copy(src, src + n, out.begin());
  }
  return -1.f;
}

}  // namespace

void LocalCluster::ring_all_reduce(size_t w, std::vector<float>& residual, std::vector<float>& grad) {
  const size_t n = nworkers_, P = n_params_;
  grad.assign(P, 0.f);
  ring_bufs_[w] = &residual;
  ring_grads_[w] = &grad;
  const size_t prev = (w + n - 1) % n;
  size_t i = w;
  size_t lo, hi;
  // scatter-reduce (worker_ring.rs:112-147)
  for (size_t s = 0; s + 1 < n; ++s) {
    chunk_bounds(P, n, i, lo, hi);
    const float thr = encode_decode(residual.data() + lo, hi - lo, opts_, seed_ + s * 131 + w, ring_msgs_[w]);
    if (thr >= 0.f) {
      for (size_t k = lo; k < hi; ++k)
        if (std::fabs(residual[k]) >= thr) residual[k] = 0.f;  // sent entries leave the residual
    } else {
      std::fill(residual.begin() + lo, residual.begin() + hi, 0.f);
    }
    ring_barrier_->wait_with(nullptr);
    i = (i + n - 1) % n;
    chunk_bounds(P, n, i, lo, hi);
    const std::vector<float>& msg = ring_msgs_[prev];
    for (size_t k = lo; k < hi; ++k) residual[k] += msg[k - lo];
    ring_barrier_->wait_with(nullptr);
  }
  // all-gather (worker_ring.rs:155-204)
  i = (w + 1) % n;
  chunk_bounds(P, n, i, lo, hi);
  std::copy(residual.begin() + lo, residual.begin() + hi, grad.begin() + lo);
  if (n == 1) {
    std::fill(residual.begin() + lo, residual.begin() + hi, 0.f);
    return;
  }
  for (size_t j = 0; j + 1 < n; ++j) {
    chunk_bounds(P, n, i, lo, hi);
    const float thr = encode_decode(grad.data() + lo, hi - lo, opts_, seed_ + 7919 + j * 131 + w, ring_msgs_[w]);
    if (thr >= 0.f) {
      for (size_t k = lo; k < hi; ++k)
        if (std::fabs(grad[k]) < thr) grad[k] = 0.f;
    } else if (j == 0) {
      std::fill(residual.begin() + lo, residual.begin() + hi, 0.f);
    }
    ring_barrier_->wait_with(nullptr);
    i = (i + n - 1) % n;
    chunk_bounds(P, n, i, lo, hi);
    const std::vector<float>& msg = ring_msgs_[prev];
    std::copy(msg.begin(), msg.begin() + (hi - lo), grad.begin() + lo);
    ring_barrier_->wait_with(nullptr);
  }
  const float inv = 1.0f / (float)n;  // worker_ring.rs:101-105
  for (auto& g : grad) g *= inv;
}

// ---- helpers ----------------------------------------------------------------------------------
namespace {

std::vector<std::pair<size_t, size_t>> ranges_of(const Json& j) {
  std::vector<std::pair<size_t, size_t>> r;
  for (auto& p : j.items()) r.emplace_back((size_t)p[0].as_u64(), (size_t)p[1].as_u64());
  return r;
}

std::vector<float> model_init(const Json& plan, uint64_t seed) {
  std::vector<float> v;
  for (auto& l : plan.at("layers").items())
    if (!l.at("param_gen").is_null()) param_gen_fill(l.at("param_gen"), seed, v);
  return v;
}

void gather_ranges(const std::vector<float>& full, const std::vector<std::pair<size_t, size_t>>& ranges, std::vector<float>& out) {
  out.clear();
  for (auto& [b, e] : ranges) out.insert(out.end(), full.begin() + b, full.begin() + e);
}

void scatter_ranges(const std::vector<float>& shard, const std::vector<std::pair<size_t, size_t>>& ranges, std::vector<float>& full) {
  size_t cur = 0;
  for (auto& [b, e] : ranges) {
    std::copy(shard.begin() + cur, shard.begin() + cur + (e - b), full.begin() + b);
    cur += e - b;
  }
}

}  // namespace

void LocalCluster::build_servers(const Json& server_list, const std::vector<std::vector<float>>* inline_params) {
  servers_.clear();
  std::vector<float> init;
  if (!inline_params) init = model_init(plan_, seed_);
  size_t idx = 0;
  for (auto& sj : server_list.items()) {
    Server s;
    s.ranges = ranges_of(sj.at("ranges"));
    std::vector<float> shard;
    if (inline_params) shard = (*inline_params)[idx];
    else gather_ranges(init, s.ranges, shard);
    const Json& spec = sj.at("spec");
    const OptimizerSpec opt = OptimizerSpec::from_spec(spec.at("optimizer"));
    const size_t nw = (size_t)spec.at("nworkers").as_u64();
    if (spec.at("store").as_string() == "wild") s.store = std::make_unique<WildStore>(std::move(shard), opt);
    else s.store = std::make_unique<BlockingStore>(std::move(shard), opt, nw);
    if (!inline_params && (opts_.init_m.size() == n_params_ || opts_.init_v.size() == n_params_)) {
      std::vector<float> m, v;       // this shard's slice of the saved moments
      if (opts_.init_m.size() == n_params_) gather_ranges(opts_.init_m, s.ranges, m);
      if (opts_.init_v.size() == n_params_) gather_ranges(opts_.init_v, s.ranges, v);
      s.store->optimizer().load_state(m.empty() ? nullptr : m.data(), v.empty() ? nullptr : v.data(), opts_.init_b1t, opts_.init_b2t);
    }
    if (spec.at("synchronizer").is_string()) s.sync = std::make_unique<NonBlockingSync>();
    else s.sync = std::make_unique<BarrierSync>(nw);
    servers_.push_back(std::move(s));
    ++idx;
  }
}

void LocalCluster::note_epochs(size_t done) {
  std::lock_guard<std::mutex> lk(policy_mu_);
  final_state_.epochs = std::max(final_state_.epochs, opts_.start_epoch + done);
}

void LocalCluster::maybe_checkpoint(size_t epochs_done, const std::vector<float>* replica, const Optimizer* replica_opt) {
  const size_t every = opts_.checkpoint_every;
  if (every == 0) return;
  const size_t at = opts_.start_epoch + epochs_done, mark = at / every;
  if (mark <= ckpt_mark_) return;
  ckpt_mark_ = mark;
  Checkpoint c;
  c.state.epochs = at;
  if (replica) {                 // all-reduce: every replica holds the whole model and its own (identical) optimizer
    c.params = *replica;
    c.state.m = replica_opt->m().empty() ? std::vector<float>(n_params_, 0.f) : replica_opt->m();
    c.state.v = replica_opt->v().empty() ? std::vector<float>(n_params_, 0.f) : replica_opt->v();
    c.state.b1t = replica_opt->b1t();
    c.state.b2t = replica_opt->b2t();
  } else {                       // parameter server: the shards are authoritative
    c.params.assign(n_params_, 0.f);
    c.state.m.assign(n_params_, 0.f);
    c.state.v.assign(n_params_, 0.f);
    std::vector<float> p, m, v;
    for (auto& s : servers_) {
      s.store->snapshot(p, m, v, c.state.b1t, c.state.b2t);
      scatter_ranges(p, s.ranges, c.params);
      if (!m.empty()) scatter_ranges(m, s.ranges, c.state.m);
      if (!v.empty()) scatter_ranges(v, s.ranges, c.state.v);
    }
  }
  {
    std::lock_guard<std::mutex> lk(ckpt_mu_);
    ckpts_.push_back(std::move(c));
  }
  ClusterEvent ev;
  ev.kind = "checkpoint";
  ev.text = std::to_string(at);
  emit(std::move(ev));
}

bool LocalCluster::pop_checkpoint(std::vector<float>& params, ClusterState& state) {
  std::lock_guard<std::mutex> lk(ckpt_mu_);
  if (ckpts_.empty()) return false;
  params = std::move(ckpts_.front().params);
  state = std::move(ckpts_.front().state);
  ckpts_.pop_front();
  return true;
}

void LocalCluster::gather_final_from_servers() {
  final_params_.assign(n_params_, 0.f);
  final_state_.m.assign(n_params_, 0.f);
  final_state_.v.assign(n_params_, 0.f);
  for (auto& s : servers_) {
    std::vector<float> shard(s.store->len());
    s.store->pull_params(shard.data());
    scatter_ranges(shard, s.ranges, final_params_);
    const Optimizer& o = s.store->optimizer();
    if (!o.m().empty()) scatter_ranges(o.m(), s.ranges, final_state_.m);
    if (!o.v().empty()) scatter_ranges(o.v(), s.ranges, final_state_.v);
    final_state_.b1t = o.b1t();
    final_state_.b2t = o.b2t();
  }
}

// ---- workers ----------------------------------------------------------------------------------
void LocalCluster::all_reduce_worker(size_t w) {
  RoundTrainer& trainer = *trainers_[w];
  std::vector<float>& params = ar_params_[w];
  std::vector<float> scratch = params, residual(n_params_, 0.f), grad;
  Optimizer opt(trainer.optimizer_spec(), n_params_);
  if (opts_.init_m.size() == n_params_ || opts_.init_v.size() == n_params_)
    opt.load_state(opts_.init_m.size() == n_params_ ? opts_.init_m.data() : nullptr,
                   opts_.init_v.size() == n_params_ ? opts_.init_v.data() : nullptr, opts_.init_b1t, opts_.init_b2t);
  struct Keep {      // worker 0's replica is the run's result (session.rs:371-412); so is its optimizer state
    LocalCluster& c; Optimizer& o; size_t w, n;
    ~Keep() {
      if (w != 0) return;
      c.final_state_.m = o.m().empty() ? std::vector<float>(n, 0.f) : o.m();
      c.final_state_.v = o.v().empty() ? std::vector<float>(n, 0.f) : o.v();
      c.final_state_.b1t = o.b1t();
      c.final_state_.b2t = o.b2t();
    }
  } keep{*this, opt, w, n_params_};
  while (true) {
    TrainResult res = trainer.train(scratch.data(), residual.data());
    const auto d = report_losses(w, res.losses);
    if (d == SessionPolicy::Switch) round_decision_.store((int)SessionPolicy::Switch);
    // Every worker sees the same verdict for this round: the last arriver snapshots it.
    ring_barrier_->wait_with([this] {
      const int sw = round_decision_.load();
      pending_decision_[0] = stop_.load() ? (int)SessionPolicy::Stop : sw;
    });
    const int verdict = pending_decision_[0];
    if (verdict == (int)SessionPolicy::Stop) break;
    if (verdict == (int)SessionPolicy::Switch) break;
    ring_all_reduce(w, residual, grad);
    opt.step(params.data(), grad.data(), n_params_);  // all_reduce.rs:126
    scratch = params;                                   // all_reduce.rs:131-132
    if (w == 0) maybe_checkpoint(trainer.epochs_done(), &params, &opt);
    if (res.is_last) break;
  }
  note_epochs(trainer.epochs_done());
}

void LocalCluster::ps_worker(size_t w, RoundTrainer& trainer, std::vector<float>& params) {
  std::vector<float> residual(n_params_, 0.f), g, wire, shard;
  for (auto& s : servers_) {  // initial pull (pserver.rs:119)
    shard.resize(s.store->len());
    s.store->pull_params(shard.data());
    scatter_ranges(shard, s.ranges, params);
  }
  while (true) {
    if (stop_.load()) break;
    TrainResult res = trainer.train(params.data(), residual.data());
    size_t si = 0;
    for (auto& s : servers_) {
      gather_ranges(residual, s.ranges, g);
      const float thr = encode_decode(g.data(), g.size(), opts_, seed_ + 31 * w + si, wire);
      shard.resize(g.size());
      s.sync->step(*s.store, wire.data(), wire.size(), shard.data());
      scatter_ranges(shard, s.ranges, params);
      // server_cluster.rs:85-104: dense -> clear the residual, sparse -> keep what was not sent
      for (auto& [b, e] : s.ranges)
        for (size_t k = b; k < e; ++k)
          if (thr < 0.f || std::fabs(residual[k]) >= thr) residual[k] = 0.f;
      ++si;
    }
    report_losses(w, res.losses);
    // (with the barrier synchroniser every server has taken this round's update from every worker by now and cannot
    // take the next before this worker pushes again: the copy is one consistent round)
    if (w == ps_leader_) maybe_checkpoint(trainer.epochs_done(), nullptr, nullptr);
    if (res.is_last) break;
  }
  for (auto& s : servers_) s.sync->leave(*s.store);
  note_epochs(trainer.epochs_done());
  ClusterEvent ev;
  ev.kind = "worker_done";
  ev.worker = w;
  emit(std::move(ev));
}

// ---- orchestration of one run -----------------------------------------------------------------
void LocalCluster::run_all() {
  try {
    const std::string algo = plan_.at("algorithm").as_string();
    const Json& workers = plan_.at("workers");
    // every worker's dataset partition (session.rs:465-504)
    std::vector<Dataset> parts;
    for (auto& wj : workers.items())
      parts.push_back(data_.slice((size_t)wj.at("partition")[0].as_u64(), (size_t)wj.at("partition")[1].as_u64()));

    if (algo == "parameter_server") {
      build_servers(plan_.at("servers"), nullptr);
      std::vector<std::unique_ptr<RoundTrainer>> trainers;
      std::vector<std::vector<float>> params(nworkers_, std::vector<float>(n_params_, 0.f));
      for (size_t w = 0; w < nworkers_; ++w)
        trainers.push_back(std::make_unique<RoundTrainer>(workers[w].at("spec").at("trainer"), std::move(parts[w]), opts_.leaky_relu_exact));
      for (auto& t : trainers) t->set_epoch_base(opts_.start_epoch);
      for (size_t w = 0; w < nworkers_; ++w)
        threads_.emplace_back([this, w, &trainers, &params] {
          try { ps_worker(w, *trainers[w], params[w]); }
          catch (const std::exception& e) { ClusterEvent ev; ev.kind = "error"; ev.worker = w; ev.text = e.what(); emit(std::move(ev)); request_stop(); for (auto& s : servers_) s.sync->leave(*s.store); }
        });
      for (auto& t : threads_) t.join();
      threads_.clear();
      gather_final_from_servers();
    } else {
      // all-reduce phase (also the first phase of a strategy switch)
      const std::vector<float> init = model_init(plan_, seed_);
      ar_params_.assign(nworkers_, init);
      trainers_.clear();
      for (size_t w = 0; w < nworkers_; ++w)
        trainers_.push_back(std::make_unique<RoundTrainer>(workers[w].at("spec").at("trainer"), parts[w], opts_.leaky_relu_exact));
      for (auto& t : trainers_) t->set_epoch_base(opts_.start_epoch);
      ring_bufs_.assign(nworkers_, nullptr);
      ring_grads_.assign(nworkers_, nullptr);
      ring_msgs_.assign(nworkers_, {});
      ring_barrier_ = std::make_unique<DynBarrier>(nworkers_);
      pending_decision_.assign(1, 0);
      std::atomic<bool> failed{false};
      for (size_t w = 0; w < nworkers_; ++w)
        threads_.emplace_back([this, w, &failed] {
          try { all_reduce_worker(w); }
          catch (const std::exception& e) {
            failed.store(true);
            ClusterEvent ev; ev.kind = "error"; ev.worker = w; ev.text = e.what(); emit(std::move(ev));
            request_stop();
            ring_barrier_->leave(nullptr);
          }
        });
      for (auto& t : threads_) t.join();
      threads_.clear();
      final_params_ = ar_params_[0];  // session.rs:371-412: worker 0's replica
      const bool do_switch = !failed.load() && algo == "strategy_switch" && pending_decision_[0] == (int)SessionPolicy::Switch;
      if (do_switch) {
        switched_.store(true);
        { ClusterEvent ev; ev.kind = "switch"; emit(std::move(ev)); }
        const Json& actions = plan_.at("switch").at("post_actions");
        // promoted workers keep their slice of the replica as the server's parameters
        Json server_list = Json::array();
        std::vector<std::vector<float>> shards;
        std::vector<size_t> promoted, remaining;
        for (size_t w = 0; w < nworkers_; ++w) {
          const Json& a = actions[w];
          if (a.at("action").as_string() == "upgrade") {
            { ClusterEvent ev; ev.kind = "upgrading"; ev.worker = w; emit(std::move(ev)); }
            Json s = Json::object();
            s.set("ranges", a.at("ranges"));
            s.set("spec", a.at("spec"));
            // keep server order = server_index
            while (server_list.size() <= (size_t)a.at("server_index").as_u64()) { server_list.push(Json()); shards.emplace_back(); }
            const size_t si = (size_t)a.at("server_index").as_u64();
            server_list.items()[si] = s;
            gather_ranges(ar_params_[w], ranges_of(a.at("ranges")), shards[si]);
            promoted.push_back(w);
          } else remaining.push_back(w);
        }
        build_servers(server_list, &shards);
        // router.rs:305-341 + builder.rs:183-196: a promoted node splits its data over the
        // remaining workers, which append it to their own
        std::vector<Dataset> new_data;
        for (size_t w : remaining) new_data.push_back(trainers_[w]->dataset());
        for (size_t w : promoted) {
          auto pieces = trainers_[w]->dataset().partition(remaining.size());
          for (size_t k = 0; k < remaining.size(); ++k) new_data[k].append(pieces[k]);
          { std::lock_guard<std::mutex> lk(policy_mu_); policy_->worker_left(w); }
          ClusterEvent ev; ev.kind = "upgraded"; ev.worker = w; emit(std::move(ev));
        }
        std::vector<std::unique_ptr<RoundTrainer>> trainers;
        std::vector<std::vector<float>> params(remaining.size(), std::vector<float>(n_params_, 0.f));
        for (size_t k = 0; k < remaining.size(); ++k) {
          const size_t w = remaining[k];
          trainers.push_back(std::make_unique<RoundTrainer>(actions[w].at("trainer_spec"), std::move(new_data[k]), opts_.leaky_relu_exact));
          // builder.rs:179-181 rebuilds the trainer, restarting the epoch counter; carrying it over
          // is this runtime's default
          if (!opts_.switch_resets_progress) trainers.back()->set_epochs_done(trainers_[w]->epochs_done());
          trainers.back()->set_epoch_base(opts_.start_epoch);
        }
        bool work_left = false;
        for (auto& t : trainers) work_left = work_left || t->epochs_done() < t->max_epochs();
        if (work_left && !stop_.load()) {
          ps_leader_ = remaining.front();
          for (size_t k = 0; k < remaining.size(); ++k)
            threads_.emplace_back([this, k, &remaining, &trainers, &params] {
              try { ps_worker(remaining[k], *trainers[k], params[k]); }
              catch (const std::exception& e) { ClusterEvent ev; ev.kind = "error"; ev.worker = remaining[k]; ev.text = e.what(); emit(std::move(ev)); request_stop(); for (auto& s : servers_) s.sync->leave(*s.store); }
            });
          for (auto& t : threads_) t.join();
          threads_.clear();
        }
        gather_final_from_servers();
      } else {
        for (size_t w = 0; w < nworkers_; ++w) { ClusterEvent ev; ev.kind = "worker_done"; ev.worker = w; emit(std::move(ev)); }
      }
    }
  } catch (const std::exception& e) {
    ClusterEvent ev;
    ev.kind = "error";
    ev.text = e.what();
    emit(std::move(ev));
    std::lock_guard<std::mutex> lk(policy_mu_);
    stop_reason_ = "error";
  }
  finished_.store(true);
  ClusterEvent done;
  done.kind = "complete";
  {
    std::lock_guard<std::mutex> lk(policy_mu_);
    done.text = stop_reason_;
  }
  emit(std::move(done));
}

}  // namespace ono::oracle
