// Orchestrator-side training session for the native executables (header-only).
//
// Counterpart of orchestrator/src/lib.rs:52-89 (`train`) and orchestrator/src/sessions/session.rs:36-627:
// validate, plan, start the ranks, relay their events, collect the final parameters. Two backends:
//
//   * addresses `cpu:<i>`   - in-process CPU ranks (threads) running the C++ engine and strategies
//                             (oracle/cluster.hpp);
//   * addresses `host:port` - node processes already listening there (one per GPU or CPU rank); the
//                             orchestrator hands each its role spec and dataset partition over the framed
//                             control channel (core/wire.hpp) exactly as session.rs:57-91,465-504 does, then
//                             relays `event` messages until every node said `done`.
//
// The event kinds are the reference's TrainingEvent stream (orchestrator/src/sessions/mod.rs:47-70) in
// flattened form: losses | upgrading | upgraded | switch | worker_done | error | complete.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "core/adapter.hpp"
#include "core/codec.hpp"
#include "core/configs.hpp"
#include "core/json.hpp"
#include "core/wire.hpp"
#include "oracle/cluster.hpp"

namespace ono {

struct TrainingEvent {
  std::string kind;
  size_t worker = 0;
  std::vector<double> losses;
  std::string text;
};

// Samples and labels of a dataset config as flat arrays (csv/tsv converted to packed f32 first:
// orchestrator/src/dataset_format.rs:58-86).
inline oracle::Dataset load_dataset(const DatasetConfig& d) {
  oracle::Dataset out;
  out.x_size = d.x_size;
  out.y_size = d.y_size;
  if (d.is_inline) {
    out.samples = d.samples;
    out.labels = d.labels;
  } else {
    out.samples = read_f32_file(ensure_binary_dataset(d.samples_path));
    out.labels = read_f32_file(ensure_binary_dataset(d.labels_path));
  }
  return out;
}

// Per-epoch mean loss over the workers that are still training (orchestra-py/src/session.rs:115-153;
// promoted workers stop counting, as the TUI does: orchestui/src/ui/screens/training.rs:527-562).
class ProgressAggregator {
 public:
  explicit ProgressAggregator(size_t workers) : live_(workers) {}
  // returns the epochs completed by this call
  std::vector<double> add(size_t worker, const std::vector<double>& losses) {
    for (double l : losses) per_epoch_[next_[worker]++].push_back(l);
    return flush(false);
  }
  std::vector<double> worker_left() {
    if (live_ > 1) --live_;
    return flush(false);
  }
  std::vector<double> finish() { return flush(true); }
  const std::vector<double>& history() const { return history_; }

 private:
  std::vector<double> flush(bool final) {
    std::vector<double> fresh;
    while (true) {
      auto it = per_epoch_.find(history_.size());
      if (it == per_epoch_.end() || it->second.empty() || (it->second.size() < live_ && !final)) break;
      double s = 0;
      for (double v : it->second) s += v;
      history_.push_back(s / (double)it->second.size());
      fresh.push_back(history_.back());
    }
    return fresh;
  }
  size_t live_;
  std::map<size_t, std::vector<double>> per_epoch_;
  std::map<size_t, size_t> next_;
  std::vector<double> history_;
};

class Session {
 public:
  virtual ~Session() = default;
  virtual size_t n_workers() const = 0;
  virtual bool next_event(TrainingEvent& ev, int timeout_ms) = 0;  // false on timeout
  virtual void stop() = 0;                                         // StopAfterEpoch to every worker
  virtual std::vector<float> final_params() = 0;                   // after the `complete` event
  virtual bool switched() const { return false; }
  virtual Json run_metrics() const { return Json::object(); }      // what the ranks reported about the run, if anything
};

class LocalSession final : public Session {
 public:
  LocalSession(const Json& plan, const TrainingConfig& t, oracle::Dataset data) {
    oracle::ClusterOptions o;
    o.wire = t.b200.wire_dtype == "f16" ? "f16" : "f32";
    o.sparse = t.serializer.sparse;
    o.sparse_r = t.serializer.r;
    o.leaky_relu_exact = t.b200.leaky_relu_exact;
    o.switch_resets_progress = t.b200.switch_resets_progress;
    workers_ = plan.at("workers").size();
    // resume (additive): the weights come through the plan (`b200.init_from`), the optimizer state and the position in
    // the shuffle sequence from the sidecar a previous run wrote
    n_params_ = (size_t)plan.at("n_params").as_u64();
    state_path_ = t.b200.state_path;
    long long start = t.b200.start_epoch;
    if (!t.b200.init_state_from.empty()) {
      StateSidecar st = load_state_sidecar(t.b200.init_state_from, n_params_);
      o.init_m = std::move(st.m);
      o.init_v = std::move(st.v);
      o.init_b1t = st.b1t;
      o.init_b2t = st.b2t;
      if (start < 0) start = (long long)st.epochs;
    }
    o.start_epoch = start > 0 ? (size_t)start : 0;
    if (const Json* op = plan.at("workers")[0].at("spec").at("trainer").find("optimizer"); op && op->is_object() && !op->members().empty())
      opt_kind_ = op->members().at(0).first;
    cluster_ = std::make_unique<oracle::LocalCluster>(plan, std::move(data), o);
    cluster_->start();
  }
  size_t n_workers() const override { return workers_; }
  bool next_event(TrainingEvent& ev, int timeout_ms) override {
    oracle::ClusterEvent ce;
    if (!cluster_->next_event(ce, timeout_ms)) return false;
    ev = TrainingEvent{ce.kind, ce.worker, ce.losses, ce.text};
    return true;
  }
  void stop() override { cluster_->request_stop(); }
  std::vector<float> final_params() override {
    cluster_->join();
    if (!state_path_.empty() && !state_written_) {
      const oracle::ClusterState& cs = cluster_->final_state();
      StateSidecar st;
      st.m = cs.m.empty() ? std::vector<float>(n_params_, 0.f) : cs.m;
      st.v = cs.v.empty() ? std::vector<float>(n_params_, 0.f) : cs.v;
      st.b1t = cs.b1t;
      st.b2t = cs.b2t;
      st.epochs = cs.epochs;
      st.optimizer = opt_kind_;
      save_state_sidecar(state_path_, st);
      state_written_ = true;
    }
    return cluster_->final_params();
  }
  bool switched() const override { return cluster_->switched(); }

 private:
  size_t workers_ = 0, n_params_ = 0;
  std::string state_path_, opt_kind_;
  bool state_written_ = false;
  std::unique_ptr<oracle::LocalCluster> cluster_;
};

class RemoteSession final : public Session {
 public:
  RemoteSession(const Json& plan, const ModelConfig& model, const TrainingConfig& training, const oracle::Dataset& data) {
    workers_ = plan.at("workers").size();
    const auto& addrs = training.addrs;
    std::map<size_t, std::pair<size_t, size_t>> part;
    for (auto& w : plan.at("workers").items()) {
      const auto& p = w.at("partition");
      part[(size_t)w.at("rank").as_u64()] = {(size_t)p[0].as_u64(), (size_t)p[1].as_u64()};
    }
    int master_port = 0;
    {
      int fd = wire::listen_on("127.0.0.1", 0, &master_port);
      ::close(fd);
    }
    std::string master_addr = addrs[0].substr(0, addrs[0].rfind(':'));
    if (master_addr == "localhost") master_addr = "127.0.0.1";
    const std::string my_id = wire::uuid4();
    for (auto& a : addrs) {
      const size_t c = a.rfind(':');
      if (c == std::string::npos) throw InvalidConfig("address `" + a + "` is not host:port");
      chs_.push_back(std::make_unique<wire::Channel>(wire::connect(a.substr(0, c), std::stoi(a.substr(c + 1)))));
      chs_.back()->connect_as("Orchestrator", my_id);
      if (chs_.back()->peer_entity != "Node") throw wire::WireError(a + " answered as " + chs_.back()->peer_entity + ", expected a node");
    }
    // the job carries the configs without the dataset: every node gets only its partition
    TrainingConfig lean = training;
    lean.dataset.is_inline = true;
    lean.dataset.samples.clear();
    lean.dataset.labels.clear();
    lean.dataset.rows_hint = data.rows();
    for (size_t r = 0; r < chs_.size(); ++r) {
      Json job = Json::object();
      job.set("model", model.to_json());
      job.set("training", lean.to_json(false));
      job.set("rank", Json((unsigned long long)r));
      job.set("world", Json((unsigned long long)addrs.size()));
      job.set("master_addr", master_addr);
      job.set("master_port", master_port);
      job.set("plan", plan);          // every node works from the orchestrator's plan (roles, ranges, partitions), not from its own
      Json spec = Json::object();
      spec.set("spec", job);
      chs_[r]->send_command(Json::tagged("create_node", spec));
      auto it = part.find(r);
      const size_t b = it == part.end() ? 0 : it->second.first, e = it == part.end() ? 0 : it->second.second;
      chs_[r]->send_dataset(data.samples.data() + b * data.x_size, (e - b) * data.x_size,
                            data.labels.data() + b * data.y_size, (e - b) * data.y_size);
    }
    remaining_ = chs_.size();
    for (size_t r = 0; r < chs_.size(); ++r) readers_.emplace_back([this, r] { reader(r); });
  }
  ~RemoteSession() override {
    close_all();
    for (auto& t : readers_)
      if (t.joinable()) t.join();
  }
  size_t n_workers() const override { return workers_; }
  void stop() override {
    for (auto& c : chs_) try { c->send_command(Json("stop_after_epoch")); } catch (const wire::WireError&) {}
  }
  bool next_event(TrainingEvent& ev, int timeout_ms) override {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !q_.empty(); })) return false;
    ev = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  std::vector<float> final_params() override {
    if (!failed_) {
      try {
        chs_[0]->send_command(Json("request_params"));
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait_for(lk, std::chrono::seconds(600), [&] { return got_metrics_ || failed_; });
      } catch (const wire::WireError&) {}
    }
    close_all();
    return params_;
  }
  bool switched() const override {
    if (const Json* s = metrics_.find("switched")) return s->is_bool() && s->as_bool();
    return false;
  }
  const Json& metrics() const { return metrics_; }
  Json run_metrics() const override { return metrics_.is_object() ? metrics_ : Json::object(); }

 private:
  void push(TrainingEvent ev) {
    { std::lock_guard<std::mutex> lk(mu_); q_.push_back(std::move(ev)); }
    cv_.notify_all();
  }
  void node_done(size_t rank, bool lost) {
    bool last;
    {
      std::lock_guard<std::mutex> lk(mu_);
      last = --remaining_ == 0;
      if (lost) failed_ = true;
    }
    if (lost)  // the reference ends the whole session on a worker io error (event_listener.rs:128-132)
      for (size_t r = 0; r < chs_.size(); ++r)
        if (r != rank) try { chs_[r]->send_command(Json("abort")); } catch (const wire::WireError&) {}
    if (last) {
      TrainingEvent c = complete_;
      if (failed_ || c.kind.empty()) c = TrainingEvent{"complete", 0, {}, failed_ ? "error" : (c.text.empty() ? "error" : c.text)};
      push(c);
    }
    cv_.notify_all();
  }
  void reader(size_t rank) {
    bool done_sent = false;
    try {
      while (true) {
        wire::Message m = chs_[rank]->recv(-1);
        if (m.kind == wire::KIND_PARAMS) {
          if (rank == 0) { std::lock_guard<std::mutex> lk(mu_); params_ = std::move(m.floats); }
          continue;
        }
        if (m.is_command("done")) {
          done_sent = true;
          node_done(rank, false);
          if (rank != 0) return;
          continue;
        }
        const Json* evj = m.variant("event");
        if (!evj) continue;
        TrainingEvent ev;
        ev.kind = evj->at("kind").as_string();
        ev.worker = (size_t)evj->at("worker").as_u64();
        if (const Json* l = evj->find("losses"))
          for (auto& v : l->items()) ev.losses.push_back(v.is_null() ? std::nan("") : v.as_double());
        if (const Json* t = evj->find("text"); t && t->is_string()) ev.text = t->as_string();
        if (ev.kind == "heartbeat") continue;   // liveness only
        if (ev.kind == "metrics") {
          { std::lock_guard<std::mutex> lk(mu_); metrics_ = Json::parse(ev.text); got_metrics_ = true; }
          cv_.notify_all();
          return;
        }
        if (ev.kind == "complete") {
          if (rank == 0) { std::lock_guard<std::mutex> lk(mu_); complete_ = ev; }
          continue;
        }
        if (ev.kind == "error") { std::lock_guard<std::mutex> lk(mu_); failed_ = true; }
        push(std::move(ev));
      }
    } catch (const std::exception& e) {
      if (closing_) return;
      push(TrainingEvent{"error", rank, {}, "node " + std::to_string(rank) + " lost: " + e.what()});
      if (!done_sent) node_done(rank, true);
      else { std::lock_guard<std::mutex> lk(mu_); failed_ = true; cv_.notify_all(); }
    }
  }
  void close_all() {
    closing_ = true;
    for (auto& c : chs_) {
      if (!c->open()) continue;
      try { c->send_command(Json("disconnect")); } catch (const wire::WireError&) {}
      c->close();
    }
  }

  size_t workers_ = 0, remaining_ = 0;
  std::vector<std::unique_ptr<wire::Channel>> chs_;
  std::vector<std::thread> readers_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<TrainingEvent> q_;
  TrainingEvent complete_;
  std::vector<float> params_;
  Json metrics_ = Json::object();
  bool got_metrics_ = false;
  std::atomic<bool> failed_{false}, closing_{false};
};

// All-pairs latency probe (orchestrator/src/configs/stat_requester.rs:32-72): node i pings nodes 0..i-1 and accepts the
// n-i-1 later ones; the maximum round-trip time per pair feeds the role assignment.
inline std::map<std::string, std::map<std::string, uint64_t>> obtain_stats(const std::vector<std::string>& addrs, int rounds = 10) {
  std::vector<wire::Channel> chs;
  for (auto& a : addrs) {
    const size_t c = a.rfind(':');
    if (c == std::string::npos) throw InvalidConfig("address `" + a + "` is not host:port");
    chs.push_back(wire::connect(a.substr(0, c), std::stoi(a.substr(c + 1))));
    chs.back().connect_as("Orchestrator");
  }
  const size_t n = addrs.size();
  for (size_t i = 0; i < n; ++i) {
    Json peers = Json::array();
    for (size_t j = 0; j < i; ++j) peers.push(addrs[j]);
    Json body = Json::object();
    body.set("addrs", peers);
    body.set("rounds", rounds);
    body.set("incoming", Json((unsigned long long)(n - i - 1)));
    chs[i].send_command(Json::tagged("stats_request", Json::tagged("ping", body)));
  }
  std::map<std::string, std::map<std::string, uint64_t>> stats;
  for (auto& a : addrs) stats[a];
  for (size_t i = 0; i < n; ++i) {
    wire::Message m = chs[i].recv(120000);
    if (const Json* resp = m.variant("stats_response"))
      if (const Json* st = resp->find("stats"); st && st->is_object())
        if (const Json* ping = st->find("ping"))
          if (const Json* rtts = ping->find("rtts"))
            for (auto& [peer, v] : rtts->members()) {
              const uint64_t mx = (uint64_t)v.at("max").as_double();
              stats[addrs[i]][peer] = mx;
              stats[peer][addrs[i]] = mx;
            }
    chs[i].send_command(Json("disconnect"));
    chs[i].close();
  }
  return stats;
}

// Validate + plan + start. With `b200.probe` the nodes' pairwise latency is measured first and used for the plan.
inline std::unique_ptr<Session> start_session(const ModelConfig& model, const TrainingConfig& training,
                                              oracle::Dataset data, Json* plan_out = nullptr) {
  validate_configs(model, training);
  bool all_cpu = true, any_cpu = false;
  for (auto& a : training.addrs) {
    const bool cpu = a.rfind("cpu:", 0) == 0;
    all_cpu = all_cpu && cpu;
    any_cpu = any_cpu || cpu;
  }
  if (any_cpu && !all_cpu) throw InvalidConfig("addrs must all be cpu:<i> or all host:port");
  Json plan = (!all_cpu && training.b200.probe)
                  ? adapt_configs(model, training, Calculator(obtain_stats(training.addrs)))
                  : adapt_configs(model, training, Calculator::uniform(training.addrs));
  if (plan_out) *plan_out = plan;
  if (all_cpu) return std::make_unique<LocalSession>(plan, training, std::move(data));
  return std::make_unique<RemoteSession>(plan, model, training, data);
}

}  // namespace ono
