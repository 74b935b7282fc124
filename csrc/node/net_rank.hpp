// One rank of a multi-process CPU session, natively: the C++ trainer on this node's partition and a TCP mesh to the
// other nodes for the gradient exchange. This is the reference's data plane between node processes
// (node/src/router.rs:166-220, worker/src/middlewares/{worker_ring,server_cluster}.rs, comms/src/connection) rebuilt on
// this runtime's ownership model: every parameter range has one owner; each worker sends the owner its residual for that
// range (f32, or packed f16 with `wire_dtype: "f16"`, the reference's wire), the owner averages, applies the optimizer
// and sends the fresh range to every rank. All-reduce = every rank owns 1/N; parameter server = the server ranks own
// their shards. Decisions (early stop, stop request) are taken by every rank from the same gathered losses, as on the
// GPU ranks, so no extra messaging is needed.
//
// Covered here: all_reduce and parameter_server with the barrier synchroniser and the blocking store. The asynchronous
// synchroniser, the wild store, the sparse serializer and the strategy switch run in a rank process instead (the caller
// checks `NetRank::supports`).
#pragma once
#include <atomic>
#include <cmath>
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
    if (algo == "strategy_switch") return false;
    // the sparse serializer: natively for the parameter server (one thresholded message per worker and server shard, as in
    // comms/src/sparse); the ring all-reduce re-encodes at every hop and stays with the rank processes
    if (training.serializer.sparse && algo != "parameter_server") return false;
    if (algo == "parameter_server")
      for (auto& s : plan.at("servers").items()) {
        const Json& sp = s.at("spec");
        if (sp.at("synchronizer").is_string() ? sp.at("synchronizer").as_string() != "barrier" : !sp.at("synchronizer").find("barrier")) return false;
        if (sp.at("store").as_string() != "blocking") return false;
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
    policy_ = std::make_unique<SessionPolicy>(worker_ranks_.size());
    if (const Json* es = plan_.find("early_stopping"); es && !es->is_null())
      policy_->enable_early_stopping((size_t)es->at("window").as_u64(), es->at("tolerance").as_double());
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
      if (sparse_) exchange_sparse();
      else exchange();
      epoch += nep;
      const int decision = decide(losses, nep, reason);
      if (decision == 1) break;
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

  bool is_worker(size_t r) const { return std::find(worker_ranks_.begin(), worker_ranks_.end(), r) != worker_ranks_.end(); }

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
    const size_t nw = worker_ranks_.size();
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
    const size_t nw = worker_ranks_.size();
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
      decision = std::max(decision, d == 2 ? 0 : d);
    }
    if (stop_req) { reason = "stopped"; return 1; }
    if (decision == 1) reason = "early_stopping";
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
  std::unique_ptr<oracle::RoundTrainer> trainer_;
  std::unique_ptr<SessionPolicy> policy_;
  std::map<size_t, wire::Channel> peers_;
  std::vector<float> C_, W_, R_;
  uint64_t seed_ = 0;
  bool f16_wire_ = false, exact_ = true, sparse_ = false;
  double sparse_r_ = 0.0;
  std::vector<size_t> server_index_;
};

}  // namespace ono
