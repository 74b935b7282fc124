// One rank of a multi-process CPU session, natively: the C++ trainer on this node's partition and a TCP mesh to the
// other nodes for the gradient exchange. This is the reference's data plane between node processes
// (node/src/router.rs:166-220, worker/src/middlewares/{worker_ring,server_cluster}.rs, comms/src/connection) rebuilt on
// this runtime's ownership model: every parameter range has one owner; each worker sends the owner its residual for that
// range (f32, or packed f16 with `wire_dtype: "f16"`, the reference's wire), the owner averages, applies the optimizer
// and sends the fresh range to every rank. All-reduce = every rank owns 1/N; parameter server = the server ranks own
// their shards. Decisions (early stop, stop request) are taken by every rank from the same gathered losses, as on the
// GPU ranks, so no extra messaging is needed.
//
// Covered here (the caller checks `NetRank::supports`):
//   * all_reduce: the owner-based exchange above; with the sparse serializer the reference's ring itself, every hop's
//     chunk thresholded and encoded anew (exchange_ring_sparse);
//   * parameter_server with the barrier synchroniser and the blocking store (exchange), also with the sparse serializer:
//     one thresholded message per worker and server shard, unsent entries kept by the worker (exchange_sparse);
//   * parameter_server with the non-blocking synchroniser on either store: every push applied on arrival, alone, and
//     answered with the shard as it stands (exchange_async);
//   * strategy_switch: all-reduce first; at the switch the promoted ranks keep their ranges, hand their samples to the
//     remaining workers and serve (do_switch).
// A wild store behind a barrier runs in a rank process instead.
#pragma once
#include <atomic>
#include <cmath>
#include <mutex>
#include <deque>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <random>
#include <thread>

#include "core/codec.hpp"
#include "core/session.hpp"

namespace ono {

class NetRank {
 public:
  using Emit = std::function<void(const TrainingEvent&)>;

  static bool supports(const Json& plan, const TrainingConfig& training) {
    const std::string algo = plan.at("algorithm").as_string();
    if (algo == "strategy_switch") {
      // all-reduce first, then the promoted ranks become servers in place (see do_switch)
      for (auto& a : plan.at("switch").at("post_actions").items()) {
        if (a.at("action").as_string() != "upgrade") continue;
        const Json& sp = a.at("spec");
        const bool barrier = sp.at("synchronizer").is_string() ? sp.at("synchronizer").as_string() == "barrier"
                                                                : sp.at("synchronizer").find("barrier") != nullptr;
        if (barrier && sp.at("store").as_string() != "blocking") return false;
      }
      return true;
    }
    // the sparse serializer: one thresholded message per worker and server shard under the parameter server
    // (exchange_sparse), re-encoded at every hop of the ring under all-reduce (exchange_ring_sparse)
    if (training.serializer.sparse && algo == "all_reduce" && plan.at("workers").size() < 2) return false;
    if (algo == "parameter_server")
      for (auto& s : plan.at("servers").items()) {
        const Json& sp = s.at("spec");
        const bool barrier = sp.at("synchronizer").is_string() ? sp.at("synchronizer").as_string() == "barrier"
                                                                : sp.at("synchronizer").find("barrier") != nullptr;
        // barrier + blocking store: one averaged update per round; non-blocking synchroniser (either store): every push is
        // applied on arrival. A wild store behind a barrier stays with the rank processes.
        if (barrier && sp.at("store").as_string() != "blocking") return false;
      }
    return true;
  }

  NetRank(Json plan, const TrainingConfig& training, size_t rank, int listen_fd, std::string node_id, std::vector<float> xs,
          std::vector<float> ys, Emit emit, std::atomic<bool>& stop)
      : plan_(std::move(plan)), rank_(rank), world_(training.addrs.size()), listen_fd_(listen_fd), node_id_(std::move(node_id)),
        emit_(std::move(emit)), stop_(stop), addrs_(training.addrs) {
    n_ = (size_t)plan_.at("n_params").as_u64();
    f16_wire_ = training.b200.wire_dtype == "f16";
    sparse_ = training.serializer.sparse;
    sparse_r_ = training.serializer.r;
    exact_ = training.b200.leaky_relu_exact;
    timeout_ms_ = (int)std::min(3.6e6, training.b200.comm_timeout_s * 1000.0);
    for (auto& w : plan_.at("workers").items()) worker_ranks_.push_back((size_t)w.at("rank").as_u64());
    for (size_t i = 0; i < worker_ranks_.size(); ++i)
      if (worker_ranks_[i] == rank_) widx_ = (long)i;
    const Json& wspec = plan_.at("workers")[widx_ >= 0 ? (size_t)widx_ : 0].at("spec").at("trainer");
    max_epochs_ = (size_t)wspec.at("max_epochs").as_u64();
    offline_ = (size_t)wspec.at("offline_epochs").as_u64();
    if (widx_ >= 0) {
      oracle::Dataset d;
      d.x_size = training.dataset.x_size;
      d.y_size = training.dataset.y_size;
      d.samples = std::move(xs);
      d.labels = std::move(ys);
      trainer_ = std::make_unique<oracle::RoundTrainer>(wspec, std::move(d), exact_);
    }
    active_.assign(worker_ranks_.size(), 1);
    resets_progress_ = training.b200.switch_resets_progress;
    ar_phase_ = plan_.at("algorithm").as_string() != "parameter_server";
    policy_ = std::make_unique<SessionPolicy>(worker_ranks_.size());
    if (const Json* es = plan_.find("early_stopping"); es && !es->is_null())
      policy_->enable_early_stopping((size_t)es->at("window").as_u64(), es->at("tolerance").as_double());
    if (plan_.at("algorithm").as_string() == "strategy_switch") {
      const Json& sw = plan_.at("switch");
      policy_->enable_switch((size_t)sw.at("window").as_u64(), sw.at("threshold").as_double());
      can_switch_ = true;
    }
    // ownership table and the optimizer of every owned range
    own_.assign(world_, {});
    Json opt_spec;
    if (plan_.at("algorithm").as_string() == "parameter_server") {
      server_index_.assign(world_, 0);
      size_t si = 0;
      for (auto& s : plan_.at("servers").items()) {
        const size_t r = (size_t)s.at("rank").as_u64();
        for (auto& rg : s.at("ranges").items()) own_[r].push_back({(size_t)rg[0].as_u64(), (size_t)rg[1].as_u64()});
        opt_spec = s.at("spec").at("optimizer");
        server_index_[r] = si++;
        const Json& sy = s.at("spec").at("synchronizer");
        async_ = !(sy.is_string() ? sy.as_string() == "barrier" : sy.find("barrier") != nullptr);
        wild_ = s.at("spec").at("store").as_string() == "wild";
      }
    } else {
      const size_t base = n_ / world_, rem = n_ % world_;
      size_t lo = 0;
      for (size_t r = 0; r < world_; ++r) {
        const size_t cnt = base + (r < rem ? 1 : 0);
        if (cnt) own_[r].push_back({lo, lo + cnt});
        lo += cnt;
      }
      opt_spec = wspec.at("optimizer");
    }
    const oracle::OptimizerSpec os = oracle::OptimizerSpec::from_spec(opt_spec);
    for (auto& rg : own_[rank_]) opts_.emplace_back(os, rg.second - rg.first);
  }

  bool switched() const { return switched_; }

  // Runs the session to its end; the return value is the final parameter vector (every rank holds it).
  std::vector<float> run() {
    connect_mesh();
    share_seed();
    C_.clear();
    for (auto& l : plan_.at("layers").items()) {
      const Json* pg = l.find("param_gen");
      if (!pg || pg->is_null()) continue;
      std::vector<float> part;
      oracle::param_gen_fill(*pg, seed_, part);
      C_.insert(C_.end(), part.begin(), part.end());
    }
    if (C_.size() != n_) throw std::runtime_error("parameter generators do not cover the model");
    W_ = C_;
    R_.assign(n_, 0.f);
    size_t epoch = 0;
    std::string reason = "max_epochs";
    while (epoch < max_epochs_) {
      const size_t nep = std::min(max_epochs_ - epoch, offline_ + 1);
      std::vector<double> losses;
      if (trainer_) {
        oracle::TrainResult tr = trainer_->train(W_.data(), R_.data());
        losses = tr.losses;
        if (losses.size() > nep) losses.resize(nep);
      }
      if (ar_phase_) {
        // all-reduce workers report first and exchange afterwards (worker/src/workers/all_reduce.rs:57-135): a round
        // that ends in a stop or a switch is not applied
        epoch += nep;
        const int decision = decide(losses, nep, reason);
        if (decision == 1) break;
        if (decision == 2 && can_switch_) {
          can_switch_ = false;
          do_switch();
          if (resets_progress_) {            // worker/src/builder.rs:179-181: the rebuilt trainer starts its epochs again
            epoch = 0;
            max_epochs_ = new_max_epochs_;
          }
          continue;
        }
        if (sparse_) exchange_ring_sparse();
        else exchange();
      } else {
        if (async_) exchange_async();
        else if (sparse_) exchange_sparse();
        else exchange();
        epoch += nep;
        if (decide(losses, nep, reason) == 1) break;
      }
    }
    if (async_) publish();      // every rank ends with the owners' final ranges
    // The orchestrator asks node 0 for the result. All-reduce replicas are the run's result through worker 0's copy
    // (orchestrator/src/sessions/session.rs:371-412); under the lossy ring they are not bit-equal, so worker 0's copy
    // travels to rank 0 when another rank hosts that worker.
    if (ar_phase_ && sparse_ && !worker_ranks_.empty() && worker_ranks_[0] != 0) {
      if (rank_ == worker_ranks_[0]) peers_.at(0).send_floats(wire::KIND_PARAMS, C_.data(), C_.size());
      else if (rank_ == 0) {
        wire::Message m = peers_.at(worker_ranks_[0]).recv(timeout_ms_);
        if (m.kind != wire::KIND_PARAMS || m.floats.size() != n_) throw wire::WireError("expected worker 0's replica");
        C_ = std::move(m.floats);
      }
    }
    TrainingEvent done{"complete", 0, {}, reason};
    emit_(done);
    for (auto& p : peers_) p.second.close();
    return C_;
  }

 private:
  struct Range { size_t first, second; };

  // Rank i connects to every lower rank's node address and accepts one connection from every higher rank; the
  // connector names its rank so that the acceptor knows whom it is talking to.
  void connect_mesh() {
    for (size_t j = 0; j < rank_; ++j) {
      const std::string& addr = addrs_[j];
      const size_t c = addr.rfind(':');
      wire::Channel ch;
      for (int attempt = 0;; ++attempt) {
        try {
          ch = wire::connect(addr.substr(0, c), std::stoi(addr.substr(c + 1)), 5000);
          break;
        } catch (const wire::WireError&) {
          if (attempt > 60) throw;
          std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
      }
      ch.connect_as("Worker", node_id_);
      Json hello = Json::object();
      hello.set("rank", Json((unsigned long long)rank_));
      ch.send_command(Json::tagged("hello", hello));
      peers_[j] = std::move(ch);
    }
    for (size_t k = rank_ + 1; k < world_; ++k) {
      pollfd pf{listen_fd_, POLLIN, 0};
      if (::poll(&pf, 1, timeout_ms_) <= 0) throw wire::WireError("a peer rank never connected");
      wire::Channel ch = wire::accept_on(listen_fd_);
      ch.accept_as("Node", node_id_);
      wire::Message m = ch.recv(timeout_ms_);
      const Json* h = m.variant("hello");
      if (!h) throw wire::WireError("expected hello from a peer rank");
      peers_[(size_t)h->at("rank").as_u64()] = std::move(ch);
    }
  }

  // One seed for every rank: the plan's, or one that rank 0 draws and sends around.
  void share_seed() {
    const Json* s = plan_.find("seed");
    if (s && !s->is_null()) { seed_ = s->as_u64(); return; }
    if (rank_ == 0) {
      seed_ = std::random_device{}();
      Json b = Json::object();
      b.set("seed", Json((unsigned long long)seed_));
      for (auto& p : peers_) p.second.send_command(Json::tagged("seed", b));
    } else {
      wire::Message m = peers_.at(0).recv(timeout_ms_);
      const Json* b = m.variant("seed");
      if (!b) throw wire::WireError("expected the seed from rank 0");
      seed_ = b->at("seed").as_u64();
    }
  }

  bool is_worker(size_t r) const {
    for (size_t i = 0; i < worker_ranks_.size(); ++i)
      if (worker_ranks_[i] == r) return active_[i] != 0;
    return false;
  }
  size_t n_active() const { return (size_t)std::count(active_.begin(), active_.end(), (char)1); }

  // All-reduce -> parameter server in place (orchestrator/src/sessions/event_listener.rs:171-219, node/src/router.rs:305-341,
  // worker/src/builder.rs:165-200): the promoted ranks keep the ranges the plan gives them out of the replica every rank
  // holds, stop training and hand their samples to the remaining workers in equal parts; optimizer state restarts.
  void do_switch() {
    const Json& acts = plan_.at("switch").at("post_actions");
    std::vector<size_t> promoted, remaining;           // worker indices
    for (size_t w = 0; w < worker_ranks_.size(); ++w)
      (acts[w].at("action").as_string() == "upgrade" ? promoted : remaining).push_back(w);
    if (rank_ == 0) {
      emit_(TrainingEvent{"switch", 0, {}, ""});
      for (size_t w : promoted) emit_(TrainingEvent{"upgrading", w, {}, ""});
    }
    // the promoted ranks' samples, in equal parts, to the remaining workers (appended in the order of the promoted)
    oracle::Dataset mine;
    if (trainer_) mine = trainer_->dataset();
    const size_t done = trainer_ ? trainer_->epochs_done() : 0;
    for (size_t w : promoted) {
      const size_t pr = worker_ranks_[w];
      if (pr == rank_) {
        auto pieces = mine.partition(remaining.size());
        for (size_t k = 0; k < remaining.size(); ++k) {
          const size_t to = worker_ranks_[remaining[k]];
          if (to == rank_) continue;
          peers_.at(to).send_floats(wire::KIND_PARAMS, pieces[k].samples.data(), pieces[k].samples.size());
          peers_.at(to).send_floats(wire::KIND_PARAMS, pieces[k].labels.data(), pieces[k].labels.size());
        }
      } else if (widx_ >= 0 && acts[(size_t)widx_].at("action").as_string() != "upgrade") {
        wire::Message mx = peers_.at(pr).recv(timeout_ms_), my = peers_.at(pr).recv(timeout_ms_);
        if (mx.kind != wire::KIND_PARAMS || my.kind != wire::KIND_PARAMS) throw wire::WireError("expected a dataset part from a promoted rank");
        oracle::Dataset part;
        part.x_size = mine.x_size;
        part.y_size = mine.y_size;
        part.samples = std::move(mx.floats);
        part.labels = std::move(my.floats);
        mine.append(part);
      }
    }
    // new ownership, fresh optimizer state
    own_.assign(world_, {});
    server_index_.assign(world_, 0);
    Json opt_spec;
    for (size_t w : promoted) {
      const Json& a = acts[w];
      const size_t r = worker_ranks_[w];
      for (auto& rg : a.at("ranges").items()) own_[r].push_back({(size_t)rg[0].as_u64(), (size_t)rg[1].as_u64()});
      server_index_[r] = (size_t)a.at("server_index").as_u64();
      opt_spec = a.at("spec").at("optimizer");
      const Json& sy = a.at("spec").at("synchronizer");
      async_ = !(sy.is_string() ? sy.as_string() == "barrier" : sy.find("barrier") != nullptr);
      wild_ = a.at("spec").at("store").as_string() == "wild";
      active_[w] = 0;
      policy_->worker_left(w);
    }
    opts_.clear();
    const oracle::OptimizerSpec os = oracle::OptimizerSpec::from_spec(opt_spec);
    for (auto& rg : own_[rank_]) opts_.emplace_back(os, rg.second - rg.first);
    // the remaining workers train on with their enlarged partitions; the promoted ranks only serve
    if (widx_ >= 0 && !active_[(size_t)widx_]) {
      trainer_.reset();
      widx_ = -1;
    } else if (widx_ >= 0) {
      const Json& ts = acts[(size_t)widx_].at("trainer_spec");
      trainer_ = std::make_unique<oracle::RoundTrainer>(ts, std::move(mine), exact_);
      if (!resets_progress_) trainer_->set_epochs_done(done);
      offline_ = (size_t)ts.at("offline_epochs").as_u64();
    }
    for (size_t w : remaining) {
      const Json& ts = acts[w].at("trainer_spec");
      new_max_epochs_ = (size_t)ts.at("max_epochs").as_u64();
      offline_ = (size_t)ts.at("offline_epochs").as_u64();
    }
    ar_phase_ = false;
    W_ = C_;
    std::fill(R_.begin(), R_.end(), 0.f);
    if (rank_ == 0)
      for (size_t w : promoted) emit_(TrainingEvent{"upgraded", w, {}, ""});
  }

  void send_range(wire::Channel& ch, const float* p, size_t n, bool f16) {
    if (!f16) { ch.send_floats(wire::KIND_PARAMS, p, n); return; }
    // the reference's dense gradient wire: IEEE f16, two bytes per element (comms/src/handles/compressor.rs:104-118)
    wire::Channel::RawFrame f;
    f.kind = 1;
    f.body.resize(n * 2);
    for (size_t i = 0; i < n; ++i) {
      const uint16_t h = f32_to_f16(p[i]);
      f.body[2 * i] = (char)(h & 0xff);
      f.body[2 * i + 1] = (char)(h >> 8);
    }
    ch.send_raw(f);
  }
  void recv_range(wire::Channel& ch, std::vector<float>& out, size_t n) {
    wire::Message m = ch.recv(timeout_ms_);
    if (m.kind == wire::KIND_PARAMS) {
      if (m.floats.size() != n) throw wire::WireError("a peer sent a range of the wrong length");
      out = std::move(m.floats);
    } else if (m.kind == 1) {
      if (m.raw.size() != 2 * n) throw wire::WireError("a peer sent an f16 range of the wrong length");
      out.resize(n);
      for (size_t i = 0; i < n; ++i)
        out[i] = f16_to_f32((uint16_t)((unsigned char)m.raw[2 * i] | ((unsigned char)m.raw[2 * i + 1] << 8)));
    } else throw wire::WireError("unexpected message during the gradient exchange");
  }

  // Residuals to the owners, averaged update at the owners, fresh parameters to everybody.
  void exchange() {
    const bool me_worker = widx_ >= 0;
    const size_t nw = n_active();
    // a sender thread keeps the sockets draining while this thread receives: nobody blocks on a full send buffer
    std::exception_ptr send_err;
    std::thread sender([&] {
      try {
        if (me_worker)
          for (size_t q = 0; q < world_; ++q)
            if (q != rank_)
              for (auto& rg : own_[q]) send_range(peers_.at(q), R_.data() + rg.first, rg.second - rg.first, f16_wire_);
      } catch (...) { send_err = std::current_exception(); }
    });
    std::vector<std::vector<float>> sums;
    for (auto& rg : own_[rank_]) {
      std::vector<float> s(rg.second - rg.first, 0.f);
      if (me_worker)
        for (size_t i = 0; i < s.size(); ++i) s[i] = f16_wire_ ? f16_round_trip(R_[rg.first + i]) : R_[rg.first + i];
      sums.push_back(std::move(s));
    }
    // fixed order of additions: peers in rank order
    std::vector<float> buf;
    for (size_t q = 0; q < world_; ++q) {
      if (q == rank_ || !is_worker(q)) continue;
      for (size_t k = 0; k < own_[rank_].size(); ++k) {
        recv_range(peers_.at(q), buf, sums[k].size());
        for (size_t i = 0; i < buf.size(); ++i) sums[k][i] += buf[i];
      }
    }
    sender.join();
    if (send_err) std::rethrow_exception(send_err);
    for (size_t k = 0; k < own_[rank_].size(); ++k) {
      const Range rg = own_[rank_][k];
      for (float& v : sums[k]) v /= (float)nw;
      opts_[k].step(C_.data() + rg.first, sums[k].data(), sums[k].size());
    }
    publish();
    std::fill(R_.begin(), R_.end(), 0.f);
  }

  // Every owner sends its fresh ranges to everybody; afterwards every rank holds the whole updated vector.
  void publish() {
    std::exception_ptr send_err;
    std::vector<float> buf;
    std::thread sender2([&] {
      try {
        for (size_t q = 0; q < world_; ++q)
          if (q != rank_)
            for (auto& rg : own_[rank_]) send_range(peers_.at(q), C_.data() + rg.first, rg.second - rg.first, false);
      } catch (...) { send_err = std::current_exception(); }
    });
    for (size_t q = 0; q < world_; ++q) {
      if (q == rank_) continue;
      for (auto& rg : own_[q]) {
        recv_range(peers_.at(q), buf, rg.second - rg.first);
        std::copy(buf.begin(), buf.end(), C_.begin() + (long)rg.first);
      }
    }
    sender2.join();
    if (send_err) std::rethrow_exception(send_err);
    W_ = C_;
  }

  // The sparse serializer (comms/src/handles/compressor.rs:71-98, comms/src/sparse/protocol.rs): per worker and server one
  // message over the server's whole shard (its ranges concatenated): the entries at or above a sampled-quantile
  // threshold as (offset, run of f16) records, or the dense f16 encoding when that is not larger. What was sent leaves
  // the worker's residual, the rest waits for a later round (worker/src/middlewares/server_cluster.rs:85-104).
  void exchange_sparse() {
    const bool me_worker = widx_ >= 0;
    const size_t nw = n_active();
    auto shard_len = [&](size_t q) { size_t n = 0; for (auto& rg : own_[q]) n += rg.second - rg.first; return n; };
    std::map<size_t, Compressed> out;
    std::vector<float> g;
    if (me_worker)
      for (size_t q = 0; q < world_; ++q) {
        if (own_[q].empty()) continue;
        g.clear();
        for (auto& rg : own_[q]) g.insert(g.end(), R_.begin() + (long)rg.first, R_.begin() + (long)rg.second);
        Compressed c = compress_gradient(g.data(), g.size(), true, sparse_r_, seed_ + 31 * (uint64_t)widx_ + server_index_[q]);
        for (auto& rg : own_[q])
          for (size_t i = rg.first; i < rg.second; ++i)
            if (!c.sparse || std::fabs(R_[i]) >= c.threshold) R_[i] = 0.f;
        out[q] = std::move(c);
      }
    auto decode = [&](bool sparse, const uint8_t* bytes, size_t len, size_t n, std::vector<float>& dst) {
      if (sparse) {
        dst.assign(n, 0.f);
        sparse_lift(dst, bytes, len);
        dst.resize(n, 0.f);
      } else {
        if (len != 2 * n) throw wire::WireError("a peer sent an f16 shard of the wrong length");
        dst.resize(n);
        for (size_t i = 0; i < n; ++i) dst[i] = f16_to_f32((uint16_t)(bytes[2 * i] | (bytes[2 * i + 1] << 8)));
      }
    };
    std::exception_ptr send_err;
    std::thread sender([&] {
      try {
        for (auto& kv : out) {
          if (kv.first == rank_) continue;
          wire::Channel::RawFrame f;
          f.kind = kv.second.sparse ? 2 : 1;
          f.body.assign(reinterpret_cast<const char*>(kv.second.bytes.data()), kv.second.bytes.size());
          peers_.at(kv.first).send_raw(f);
        }
      } catch (...) { send_err = std::current_exception(); }
    });
    const size_t mine = shard_len(rank_);
    std::vector<float> sum(mine, 0.f), buf;
    if (mine) {
      if (me_worker) {
        const Compressed& c = out.at(rank_);
        decode(c.sparse, c.bytes.data(), c.bytes.size(), mine, sum);
      }
      for (size_t q = 0; q < world_; ++q) {      // fixed order of additions: peers in rank order
        if (q == rank_ || !is_worker(q)) continue;
        wire::Message m = peers_.at(q).recv(timeout_ms_);
        if (m.kind != 1 && m.kind != 2) throw wire::WireError("unexpected message during the gradient exchange");
        decode(m.kind == 2, reinterpret_cast<const uint8_t*>(m.raw.data()), m.raw.size(), mine, buf);
        for (size_t i = 0; i < mine; ++i) sum[i] += buf[i];
      }
    }
    sender.join();
    if (send_err) std::rethrow_exception(send_err);
    size_t at = 0;
    for (size_t k = 0; k < own_[rank_].size(); ++k) {
      const Range rg = own_[rank_][k];
      const size_t len = rg.second - rg.first;
      for (size_t i = 0; i < len; ++i) sum[at + i] /= (float)nw;
      opts_[k].step(C_.data() + rg.first, sum.data() + at, len);
      at += len;
    }
    publish();
  }

  // The reference's ring all-reduce with the sparse serializer (worker/src/middlewares/worker_ring.rs:112-204,
  // mod.rs:15-59): n - 1 scatter-reduce hops and n - 1 all-gather hops over near-equal chunks, every hop's chunk encoded
  // anew (thresholded (offset, f16 run) records, or dense f16 when that is not larger). In the scatter phase what a worker
  // sent leaves its residual and the rest waits for a later round; in the gather phase a worker keeps of its own copy only
  // what it sent on. Every worker then divides by n and applies its own optimizer to its replica.
  void exchange_ring_sparse() {
    const size_t n = worker_ranks_.size(), w = (size_t)widx_;
    const size_t next = worker_ranks_[(w + 1) % n], prev = worker_ranks_[(w + n - 1) % n];
    auto bounds = [&](size_t c, size_t& lo, size_t& hi) {
      const size_t base = n_ / n, rem = n_ % n;
      lo = base * c + std::min(c, rem);
      hi = lo + base + (c < rem ? 1 : 0);
    };
    // one hop: my chunk goes to the next worker while the previous worker's arrives
    auto hop = [&](const Compressed& c, size_t recv_len, std::vector<float>& got) {
      std::exception_ptr send_err;
      std::thread sender([&] {
        try {
          wire::Channel::RawFrame f;
          f.kind = c.sparse ? 2 : 1;
          f.body.assign(reinterpret_cast<const char*>(c.bytes.data()), c.bytes.size());
          peers_.at(next).send_raw(f);
        } catch (...) { send_err = std::current_exception(); }
      });
      std::exception_ptr recv_err;
      try {
        wire::Message m = peers_.at(prev).recv(timeout_ms_);
        if (m.kind == 2) {
          got.assign(recv_len, 0.f);
          sparse_lift(got, reinterpret_cast<const uint8_t*>(m.raw.data()), m.raw.size());
          got.resize(recv_len, 0.f);
        } else if (m.kind == 1 && m.raw.size() == 2 * recv_len) {
          got.resize(recv_len);
          for (size_t k = 0; k < recv_len; ++k)
            got[k] = f16_to_f32((uint16_t)((unsigned char)m.raw[2 * k] | ((unsigned char)m.raw[2 * k + 1] << 8)));
        } else throw wire::WireError("unexpected message during the ring exchange");
      } catch (...) { recv_err = std::current_exception(); }
      sender.join();
      if (recv_err) std::rethrow_exception(recv_err);
      if (send_err) std::rethrow_exception(send_err);
    };
    std::vector<float> grad(n_, 0.f), got;
    size_t i = w, lo, hi;
    for (size_t st = 0; st + 1 < n; ++st) {                      // scatter-reduce
      bounds(i, lo, hi);
      Compressed c = compress_gradient(R_.data() + lo, hi - lo, true, sparse_r_, seed_ + st * 131 + w);
      for (size_t k = lo; k < hi; ++k)
        if (!c.sparse || std::fabs(R_[k]) >= c.threshold) R_[k] = 0.f;
      i = (i + n - 1) % n;
      bounds(i, lo, hi);
      hop(c, hi - lo, got);
      for (size_t k = lo; k < hi; ++k) R_[k] += got[k - lo];
    }
    i = (w + 1) % n;                                              // all-gather
    bounds(i, lo, hi);
    std::copy(R_.begin() + (long)lo, R_.begin() + (long)hi, grad.begin() + (long)lo);
    for (size_t j = 0; j + 1 < n; ++j) {
      bounds(i, lo, hi);
      Compressed c = compress_gradient(grad.data() + lo, hi - lo, true, sparse_r_, seed_ + 7919 + j * 131 + w);
      if (c.sparse) {
        for (size_t k = lo; k < hi; ++k)
          if (std::fabs(grad[k]) < c.threshold) grad[k] = 0.f;
      } else if (j == 0) {
        std::fill(R_.begin() + (long)lo, R_.begin() + (long)hi, 0.f);
      }
      i = (i + n - 1) % n;
      bounds(i, lo, hi);
      hop(c, hi - lo, got);
      std::copy(got.begin(), got.end(), grad.begin() + (long)lo);
    }
    const float inv = 1.0f / (float)n;
    for (float& g : grad) g *= inv;
    if (!ring_opt_) {
      const Json& wspec = plan_.at("workers")[w].at("spec").at("trainer");
      ring_opt_ = std::make_unique<oracle::Optimizer>(oracle::OptimizerSpec::from_spec(wspec.at("optimizer")), n_);
    }
    ring_opt_->step(C_.data(), grad.data(), n_);
    W_ = C_;
  }

  // Non-blocking synchroniser (parameter_server/src/synchronization/non_blocking.rs; wild store: storage/wild/shard.rs:43-58):
  // an owner applies every worker's push on arrival, alone (blocking store: divided by the number of workers; wild store:
  // as it is), and answers that worker with its shard as it stands then. Three threads per rank and round: a receiver that
  // reads every peer socket and never sends (it applies pushes and files replies), a transmitter that does all the
  // sending in order, and this thread, which encodes its own pushes and waits for both. A receiver that also sent could
  // block on a full socket while its peer does the same.
  void exchange_async() {
    const bool me_worker = widx_ >= 0;
    const size_t nw = n_active();
    auto shard_len = [&](size_t q) { size_t n = 0; for (auto& rg : own_[q]) n += rg.second - rg.first; return n; };
    const size_t mine = shard_len(rank_);
    struct Frame { size_t peer; wire::Channel::RawFrame f; };
    std::mutex tx_mu, shard_mu;
    std::condition_variable tx_cv;
    std::deque<Frame> tx_q;
    bool tx_stop = false;
    std::exception_ptr tx_err, rx_err;
    auto enqueue = [&](size_t peer, wire::Channel::RawFrame f) {
      { std::lock_guard<std::mutex> lk(tx_mu); tx_q.push_back(Frame{peer, std::move(f)}); }
      tx_cv.notify_one();
    };
    std::thread tx([&] {
      try {
        for (;;) {
          Frame fr;
          {
            std::unique_lock<std::mutex> lk(tx_mu);
            tx_cv.wait(lk, [&] { return tx_stop || !tx_q.empty(); });
            if (tx_q.empty()) return;
            fr = std::move(tx_q.front());
            tx_q.pop_front();
          }
          peers_.at(fr.peer).send_raw(fr.f);
        }
      } catch (...) { tx_err = std::current_exception(); }
    });
    auto floats_frame = [](uint32_t kind, const float* p, size_t n) {
      wire::Channel::RawFrame f;
      f.kind = kind;
      f.body.assign(reinterpret_cast<const char*>(p), n * sizeof(float));
      return f;
    };
    // one push, applied alone
    auto apply = [&](const std::vector<float>& grad, std::vector<float>& fresh) {
      std::lock_guard<std::mutex> lk(shard_mu);
      size_t at = 0;
      fresh.clear();
      std::vector<float> g;
      for (size_t k = 0; k < own_[rank_].size(); ++k) {
        const Range rg = own_[rank_][k];
        const size_t len = rg.second - rg.first;
        g.assign(grad.begin() + (long)at, grad.begin() + (long)(at + len));
        if (!wild_) for (float& v : g) v /= (float)nw;
        opts_[k].step(C_.data() + rg.first, g.data(), len);
        fresh.insert(fresh.end(), C_.begin() + (long)rg.first, C_.begin() + (long)rg.second);
        at += len;
      }
    };
    auto decode = [&](const wire::Message& m, size_t n, std::vector<float>& dst) {
      if (m.kind == wire::KIND_PARAMS) {
        if (m.floats.size() != n) throw wire::WireError("a peer sent a shard of the wrong length");
        dst = m.floats;
      } else if (m.kind == 2) {
        dst.assign(n, 0.f);
        sparse_lift(dst, reinterpret_cast<const uint8_t*>(m.raw.data()), m.raw.size());
        dst.resize(n, 0.f);
      } else if (m.kind == 1) {
        if (m.raw.size() != 2 * n) throw wire::WireError("a peer sent an f16 shard of the wrong length");
        dst.resize(n);
        for (size_t i = 0; i < n; ++i)
          dst[i] = f16_to_f32((uint16_t)((unsigned char)m.raw[2 * i] | ((unsigned char)m.raw[2 * i + 1] << 8)));
      } else throw wire::WireError("unexpected message during the gradient exchange");
    };
    // What this rank still expects from each peer this round: a push (the peer is a worker and I own a shard) and / or an
    // answer (the peer owns a shard and I am a worker). A peer that has delivered both is not read any further: its next
    // frames belong to the loss exchange that follows.
    std::map<size_t, int> want_push, want_reply;
    size_t pushes_left = 0, replies_left = 0;
    for (auto& p : peers_) {
      const size_t q = p.first;
      want_push[q] = (mine && is_worker(q)) ? 1 : 0;
      want_reply[q] = (me_worker && !own_[q].empty()) ? 1 : 0;
      pushes_left += (size_t)want_push[q];
      replies_left += (size_t)want_reply[q];
    }
    std::thread rx([&] {
      try {
        std::vector<float> grad, fresh;
        while (pushes_left + replies_left > 0) {
          std::vector<pollfd> pfs;
          std::vector<size_t> who;
          for (auto& p : peers_)
            if (want_push[p.first] + want_reply[p.first] > 0) { pfs.push_back(pollfd{p.second.fd(), POLLIN, 0}); who.push_back(p.first); }
          int r;
          do { r = ::poll(pfs.data(), pfs.size(), timeout_ms_); } while (r < 0 && errno == EINTR);
          if (r <= 0) throw wire::WireError("timed out during the asynchronous exchange");
          for (size_t i = 0; i < pfs.size(); ++i) {
            if (!(pfs[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
            const size_t q = who[i];
            wire::Message m = peers_.at(q).recv(timeout_ms_);
            if (m.kind == wire::KIND_DATACHUNK) {       // an owner's answer: its shard after my push
              size_t at = 0;
              if (m.floats.size() != shard_len(q) || want_reply[q] == 0) throw wire::WireError("unexpected shard from a peer");
              want_reply[q] = 0;
              for (auto& rg : own_[q]) {
                std::copy(m.floats.begin() + (long)at, m.floats.begin() + (long)(at + rg.second - rg.first), W_.begin() + (long)rg.first);
                at += rg.second - rg.first;
              }
              --replies_left;
            } else {                                     // a worker's push for my shard
              if (want_push[q] == 0) throw wire::WireError("unexpected push from a peer");
              want_push[q] = 0;
              decode(m, mine, grad);
              apply(grad, fresh);
              enqueue(q, floats_frame(wire::KIND_DATACHUNK, fresh.data(), fresh.size()));
              --pushes_left;
            }
          }
        }
      } catch (...) { rx_err = std::current_exception(); }
    });
    // my own pushes
    std::vector<float> g, dec, fresh;
    try {
      if (me_worker)
        for (size_t q = 0; q < world_; ++q) {
          if (own_[q].empty()) continue;
          g.clear();
          for (auto& rg : own_[q]) g.insert(g.end(), R_.begin() + (long)rg.first, R_.begin() + (long)rg.second);
          Compressed c;
          const bool coded = sparse_ || f16_wire_;
          if (coded) c = compress_gradient(g.data(), g.size(), sparse_, sparse_r_, seed_ + 31 * (uint64_t)widx_ + server_index_[q]);
          for (auto& rg : own_[q])
            for (size_t i = rg.first; i < rg.second; ++i)
              if (!coded || !c.sparse || std::fabs(R_[i]) >= c.threshold) R_[i] = 0.f;
          if (q == rank_) {          // my own shard: applied here, under the same lock the receiver takes
            if (coded) {
              wire::Message m;
              m.kind = c.sparse ? 2 : 1;
              m.raw.assign(reinterpret_cast<const char*>(c.bytes.data()), c.bytes.size());
              decode(m, mine, dec);
            } else dec = g;
            apply(dec, fresh);
            size_t at = 0;
            for (auto& rg : own_[rank_]) {
              std::copy(fresh.begin() + (long)at, fresh.begin() + (long)(at + rg.second - rg.first), W_.begin() + (long)rg.first);
              at += rg.second - rg.first;
            }
          } else if (coded) {
            wire::Channel::RawFrame f;
            f.kind = c.sparse ? 2 : 1;
            f.body.assign(reinterpret_cast<const char*>(c.bytes.data()), c.bytes.size());
            enqueue(q, std::move(f));
          } else {
            enqueue(q, floats_frame(wire::KIND_PARAMS, g.data(), g.size()));
          }
        }
    } catch (...) { rx_err = rx_err ? rx_err : std::current_exception(); }
    rx.join();
    { std::lock_guard<std::mutex> lk(tx_mu); tx_stop = true; }
    tx_cv.notify_one();
    tx.join();
    if (rx_err) std::rethrow_exception(rx_err);
    if (tx_err) std::rethrow_exception(tx_err);
  }

  // All ranks learn every rank's losses and stop flag and run the same policy on them.
  int decide(const std::vector<double>& losses, size_t nl, std::string& reason) {
    std::vector<float> mine(nl + 1, std::nanf(""));
    for (size_t i = 0; i < losses.size() && i < nl; ++i) mine[i] = (float)losses[i];
    mine[nl] = stop_.load() ? 1.f : 0.f;
    // losses travel as f64 pairs of f32 words to keep the policy's input exact
    std::vector<double> mine_d(nl + 1, std::nan(""));
    for (size_t i = 0; i < losses.size() && i < nl; ++i) mine_d[i] = losses[i];
    mine_d[nl] = stop_.load() ? 1.0 : 0.0;
    std::vector<std::vector<double>> table(world_);
    table[rank_] = mine_d;
    std::exception_ptr send_err;
    std::thread sender([&] {
      try {
        for (auto& p : peers_) p.second.send_floats(wire::KIND_PARAMS, reinterpret_cast<const float*>(mine_d.data()), 2 * mine_d.size());
      } catch (...) { send_err = std::current_exception(); }
    });
    for (auto& p : peers_) {
      wire::Message m = p.second.recv(timeout_ms_);
      if (m.kind != wire::KIND_PARAMS || m.floats.size() != 2 * (nl + 1)) throw wire::WireError("unexpected message during the loss exchange");
      table[p.first].resize(nl + 1);
      std::memcpy(table[p.first].data(), m.floats.data(), (nl + 1) * sizeof(double));
    }
    sender.join();
    if (send_err) std::rethrow_exception(send_err);
    int decision = 0;
    bool stop_req = false;
    for (size_t r = 0; r < world_; ++r) stop_req = stop_req || table[r][nl] > 0;
    for (size_t wi = 0; wi < worker_ranks_.size(); ++wi) {
      std::vector<double> ls;
      for (size_t i = 0; i < nl; ++i)
        if (!std::isnan(table[worker_ranks_[wi]][i])) ls.push_back(table[worker_ranks_[wi]][i]);
      if (ls.empty()) continue;
      for (double v : ls)
        if (!std::isfinite(v)) {
          if (rank_ == 0) emit_(TrainingEvent{"error", wi, {}, "worker reported a non-finite loss"});
          reason = "error";
          return 1;
        }
      if (rank_ == 0) emit_(TrainingEvent{"losses", wi, ls, ""});
      const int d = (int)policy_->on_losses(wi, ls.data(), ls.size());
      if (d == 1) decision = 1;
      else if (d == 2 && decision == 0) decision = 2;
    }
    if (stop_req) { reason = "stopped"; return 1; }
    if (decision == 1) reason = "early_stopping";
    if (decision == 2) switched_ = true;
    return decision;
  }

  Json plan_;
  size_t rank_, world_, n_ = 0, max_epochs_ = 1, offline_ = 0;
  long widx_ = -1;
  int listen_fd_, timeout_ms_ = 300000;
  std::string node_id_;
  Emit emit_;
  std::atomic<bool>& stop_;
  std::vector<std::string> addrs_;
  std::vector<size_t> worker_ranks_;
  std::vector<std::vector<Range>> own_;
  std::vector<oracle::Optimizer> opts_;
  std::unique_ptr<oracle::Optimizer> ring_opt_;      // the whole-replica optimizer of the ring exchange
  std::unique_ptr<oracle::RoundTrainer> trainer_;
  std::unique_ptr<SessionPolicy> policy_;
  std::map<size_t, wire::Channel> peers_;
  std::vector<float> C_, W_, R_;
  uint64_t seed_ = 0;
  bool f16_wire_ = false, exact_ = true, sparse_ = false, async_ = false, wild_ = false;
  bool can_switch_ = false, resets_progress_ = false, switched_ = false, ar_phase_ = false;
  size_t new_max_epochs_ = 1;
  std::vector<char> active_;
  double sparse_r_ = 0.0;
  std::vector<size_t> server_index_;
};

}  // namespace ono
