#include "adapter.hpp"

#include "codec.hpp"

#include <algorithm>
#include <cmath>
#include <map>
#include <numeric>
#include <queue>

namespace ono {

std::vector<std::vector<size_t>> balanced_partitions(const std::vector<size_t>& sizes, size_t k) {
  std::vector<std::vector<size_t>> bins(k);
  if (k == 0) return bins;
  std::vector<size_t> order(sizes.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return sizes[a] > sizes[b]; });
  using Entry = std::pair<size_t, size_t>;  // (load, bin)
  std::priority_queue<Entry, std::vector<Entry>, std::greater<Entry>> heap;
  for (size_t i = 0; i < k; ++i) heap.push({0, i});
  for (size_t item : order) {
    auto [load, bin] = heap.top();
    heap.pop();
    bins[bin].push_back(item);
    heap.push({load + sizes[item], bin});
  }
  return bins;
}

std::vector<std::pair<size_t, size_t>> dataset_partitions(size_t nrows, size_t n) {
  std::vector<std::pair<size_t, size_t>> out;
  if (n == 0) return out;
  const size_t base = nrows / n, rem = nrows % n;
  size_t lo = 0;
  for (size_t i = 0; i < n; ++i) {
    const size_t rows = base + (i < rem ? 1 : 0);
    out.emplace_back(lo, lo + rows);
    lo += rows;
  }
  return out;
}

static Json act_spec(const std::optional<ActFnConfig>& a) { return a ? a->to_json() : Json(); }

static Json triple_j(const std::array<size_t, 3>& t) {
  Json a = Json::array();
  for (size_t v : t) a.push(Json((unsigned long long)v));
  return a;
}

// adapter.rs:1032-1072: (fan_in, limit, fan_out) = (flattened input, weights+biases, flattened output)
static Json param_gen_spec(const ParamGenConfig& init, size_t fan_in, size_t limit, size_t fan_out, size_t offset) {
  Json lim((unsigned long long)limit);
  if (init.kind == ParamGenConfig::Const) {
    Json b = Json::object();
    b.set("value", init.a);
    b.set("limit", lim);
    return Json::tagged("const", b);
  }
  Json dist;
  Json d = Json::object();
  switch (init.kind) {
    case ParamGenConfig::Uniform: d.set("low", init.a); d.set("high", init.b); dist = Json::tagged("uniform", d); break;
    case ParamGenConfig::UniformInclusive: d.set("low", init.a); d.set("high", init.b); dist = Json::tagged("uniform_inclusive", d); break;
    case ParamGenConfig::Normal: d.set("mean", init.a); d.set("std_dev", init.b); dist = Json::tagged("normal", d); break;
    case ParamGenConfig::XavierUniform: d.set("fan_in", Json((unsigned long long)fan_in)); d.set("fan_out", Json((unsigned long long)fan_out)); dist = Json::tagged("xavier_uniform", d); break;
    case ParamGenConfig::LecunUniform: d.set("fan_in", Json((unsigned long long)fan_in)); dist = Json::tagged("lecun_uniform", d); break;
    case ParamGenConfig::Kaiming: d.set("fan_in", Json((unsigned long long)fan_in)); dist = Json::tagged("kaiming", d); break;
    case ParamGenConfig::Xavier: d.set("fan_in", Json((unsigned long long)fan_in)); d.set("fan_out", Json((unsigned long long)fan_out)); dist = Json::tagged("xavier", d); break;
    case ParamGenConfig::Lecun: d.set("fan_in", Json((unsigned long long)fan_in)); dist = Json::tagged("lecun", d); break;
    default: break;
  }
  Json b = Json::object();
  b.set("distribution", dist);
  b.set("limit", lim);
  b.set("index_offset", Json((unsigned long long)offset));
  return Json::tagged("rand", b);
}

void resolve_distribution(const Json& distribution, int& kind, float& a, float& b) {
  const auto& m = distribution.members().at(0);
  const std::string& name = m.first;
  const Json& d = m.second;
  auto f = [&](const char* k) { return (float)d.at(k).as_double(); };
  // machine_learning/src/initialization/random.rs:31-161
  if (name == "uniform") { kind = 0; a = f("low"); b = f("high"); }
  else if (name == "uniform_inclusive") { kind = 1; a = f("low"); b = f("high"); }
  else if (name == "normal") { kind = 2; a = f("mean"); b = f("std_dev"); }
  else if (name == "xavier_uniform") { kind = 1; const float r = std::sqrt(6.0f / (f("fan_in") + f("fan_out"))); a = -r; b = r; }
  else if (name == "lecun_uniform") { kind = 1; const float r = std::sqrt(3.0f / f("fan_in")); a = -r; b = r; }
  else if (name == "kaiming") { kind = 2; a = 0.f; b = std::sqrt(2.0f / f("fan_in")); }
  else if (name == "xavier") { kind = 2; a = 0.f; b = std::sqrt(2.0f / (f("fan_in") + f("fan_out"))); }
  else if (name == "lecun") { kind = 2; a = 0.f; b = std::sqrt(1.0f / f("fan_in")); }
  else throw InvalidConfig("unknown distribution `" + name + "`");
}

std::vector<LayerPlanInfo> adapt_layers(const ModelConfig& model, size_t x_size) {
  std::vector<LayerPlanInfo> out;
  size_t in = x_size, off = 0;
  for (size_t i = 0; i < model.layers.size(); ++i) {
    const LayerConfig& l = model.layers[i];
    LayerPlanInfo p;
    p.index = i;
    p.input_size = in;
    p.output_size = l.out_size();
    p.n_params = l.param_count(in);
    p.offset = off;
    Json body = Json::object();
    switch (l.kind) {
      case LayerConfig::Dense: {
        Json dim = Json::array();
        dim.push(Json((unsigned long long)in));
        dim.push(Json((unsigned long long)l.output_size));
        body.set("dim", dim);
        body.set("act_fn", act_spec(l.act_fn));
        p.layer_spec = Json::tagged("dense", body);
        p.param_gen = param_gen_spec(l.init, in, p.n_params, p.output_size, off);
        break;
      }
      case LayerConfig::Conv:
        body.set("input_dim", triple_j(l.input_dim));
        body.set("kernel_dim", triple_j(l.kernel_dim));
        body.set("stride", Json((unsigned long long)l.stride));
        body.set("padding", Json((unsigned long long)l.padding));
        body.set("act_fn", act_spec(l.act_fn));
        p.layer_spec = Json::tagged("conv", body);
        p.param_gen = param_gen_spec(l.init, in, p.n_params, p.output_size, off);
        break;
      case LayerConfig::MaxPooling:
        body.set("input_dim", triple_j(l.input_dim));
        body.set("filter_size", Json((unsigned long long)l.filter_size));
        body.set("stride", Json((unsigned long long)l.stride));
        body.set("padding", Json((unsigned long long)l.padding));
        body.set("act_fn", act_spec(l.act_fn));
        p.layer_spec = Json::tagged("max_pooling", body);
        break;
    }
    off += p.n_params;
    in = p.output_size;
    out.push_back(std::move(p));
  }
  return out;
}

namespace {

Json optimizer_spec(const OptimizerConfig& o, bool downgrade_to_gd) {
  Json b = Json::object();
  b.set("learning_rate", o.lr);
  if (downgrade_to_gd || o.kind == OptimizerConfig::GradientDescent) return Json::tagged("gradient_descent", b);
  if (o.kind == OptimizerConfig::Momentum) { b.set("momentum", o.mu); return Json::tagged("gradient_descent_with_momentum", b); }
  b.set("beta1", o.b1);
  b.set("beta2", o.b2);
  b.set("epsilon", o.eps);
  return Json::tagged("adam", b);
}

Json usize_array(const std::vector<size_t>& v) {
  Json a = Json::array();
  for (size_t x : v) a.push(Json((unsigned long long)x));
  return a;
}

Json str_array(const std::vector<std::string>& v) {
  Json a = Json::array();
  for (auto& x : v) a.push(x);
  return a;
}

Json ranges_json(const std::vector<std::pair<size_t, size_t>>& r) {
  Json a = Json::array();
  for (auto& [b, e] : r) {
    Json p = Json::array();
    p.push(Json((unsigned long long)b));
    p.push(Json((unsigned long long)e));
    a.push(p);
  }
  return a;
}

Json trainer_spec(const std::vector<LayerPlanInfo>& layers, const TrainingConfig& t, bool ps_worker, size_t batch_size) {
  Json ls = Json::array();
  for (auto& l : layers) ls.push(l.layer_spec);
  Json ds = Json::object();
  ds.set("x_size", Json((unsigned long long)t.dataset.x_size));
  ds.set("y_size", Json((unsigned long long)t.dataset.y_size));
  Json s = Json::object();
  s.set("layers", ls);
  s.set("optimizer", optimizer_spec(t.optimizer, ps_worker));
  s.set("dataset", ds);
  s.set("loss_fn", t.loss_fn == TrainingConfig::Mse ? "mse" : "cross_entropy");
  s.set("offline_epochs", Json((unsigned long long)t.offline_epochs));
  s.set("max_epochs", Json((unsigned long long)t.max_epochs));
  s.set("batch_size", Json((unsigned long long)batch_size));
  s.set("seed", t.seed ? Json(*t.seed) : Json());
  return s;
}

Json serializer_spec(const TrainingConfig& t) {
  if (!t.serializer.sparse) return "base";
  Json b = Json::object();
  b.set("r", t.serializer.r);
  return Json::tagged("sparse_capable", b);
}

struct Sharding {
  std::vector<size_t> server_sizes;                              // parameters owned per server
  std::vector<size_t> server_ordering;                           // weighted layer (relative idx) -> server
  std::vector<std::tuple<size_t, size_t, size_t>> layer_offsets;  // per layer (abs idx): server, start, end (server-local)
  std::vector<std::vector<std::pair<size_t, size_t>>> global_ranges;  // per server, in the flat model vector
  std::vector<std::vector<std::pair<size_t, size_t>>> local_ranges;   // per server, server-local
  std::vector<Json> param_gens;                                  // per server, Chained
};

// adapter.rs:605-687 (layer mode) or an even flat split (B200 extension).
Sharding shard_layers(const std::vector<LayerPlanInfo>& layers, size_t nservers, bool even) {
  Sharding s;
  s.server_sizes.assign(nservers, 0);
  s.global_ranges.resize(nservers);
  s.local_ranges.resize(nservers);
  s.layer_offsets.assign(layers.size(), {0, 0, 0});
  std::vector<size_t> weighted;  // abs idx of layers with parameters
  for (auto& l : layers)
    if (!l.param_gen.is_null()) weighted.push_back(l.index);
  s.server_ordering.assign(weighted.size(), 0);
  const size_t total = layers.empty() ? 0 : layers.back().offset + layers.back().n_params;
  if (even) {
    // Even flat sharding: boundaries at multiples of 4 elements, independent of layer boundaries.
    const size_t units = (total + 3) / 4;
    size_t lo = 0;
    for (size_t i = 0; i < nservers; ++i) {
      const size_t cnt = units / nservers + (i < units % nservers ? 1 : 0);
      const size_t b = lo * 4, e = std::min(total, (lo + cnt) * 4);
      if (e > b) { s.global_ranges[i].push_back({b, e}); s.local_ranges[i].push_back({0, e - b}); }
      s.server_sizes[i] = e > b ? e - b : 0;
      lo += cnt;
    }
    for (size_t i = 0; i < nservers; ++i) {
      Json specs = Json::array();
      Json ch = Json::object();
      ch.set("specs", specs);
      s.param_gens.push_back(Json::tagged("chained", ch));
    }
    return s;
  }
  std::vector<size_t> sizes;
  for (size_t abs : weighted) sizes.push_back(layers[abs].n_params);
  auto bins = balanced_partitions(sizes, nservers);
  for (size_t srv = 0; srv < nservers; ++srv) {
    auto& bin = bins[srv];
    std::sort(bin.begin(), bin.end());  // model order inside a server (rel idx is monotone in abs idx)
    size_t cursor = 0;
    Json specs = Json::array();
    for (size_t rel : bin) {
      const LayerPlanInfo& l = layers[weighted[rel]];
      s.server_ordering[rel] = srv;
      s.layer_offsets[l.index] = {srv, cursor, cursor + l.n_params};
      s.local_ranges[srv].push_back({cursor, cursor + l.n_params});
      auto& gr = s.global_ranges[srv];
      if (!gr.empty() && gr.back().second == l.offset) gr.back().second = l.offset + l.n_params;
      else gr.push_back({l.offset, l.offset + l.n_params});
      cursor += l.n_params;
      specs.push(l.param_gen);
    }
    s.server_sizes[srv] = cursor;
    Json ch = Json::object();
    ch.set("specs", specs);
    s.param_gens.push_back(Json::tagged("chained", ch));
  }
  return s;
}

std::vector<size_t> per_worker_batch(const TrainingConfig& t, size_t nworkers) {
  std::vector<size_t> out(nworkers, t.batch_size);
  if (t.b200.global_batch > 0 && nworkers > 0) {
    const size_t base = t.b200.global_batch / nworkers, rem = t.b200.global_batch % nworkers;
    for (size_t i = 0; i < nworkers; ++i) out[i] = std::max<size_t>(1, base + (i < rem ? 1 : 0));
  }
  return out;
}

}  // namespace

Json adapt_configs(const ModelConfig& model, const TrainingConfig& training, const Calculator& calc) {
  auto layers = adapt_layers(model, training.dataset.x_size);
  if (!training.b200.init_from.empty()) {
    // Warm start: every layer's generator becomes the checkpoint's values for that layer (weight then bias), the way
    // promoted servers receive their parameters inline in the spec (worker/src/workers/all_reduce.rs:87-94).
    std::map<std::string, const NamedTensor*> by_name;
    const std::vector<NamedTensor> tensors = load_safetensors(training.b200.init_from);
    for (auto& t : tensors) by_name[t.name] = &t;
    for (auto& l : layers) {
      if (l.param_gen.is_null()) continue;
      const std::string base = "layer_" + std::to_string(l.index);
      auto w = by_name.find(base + ".weight"), b = by_name.find(base + ".bias");
      if (w == by_name.end() || b == by_name.end())
        throw InvalidConfig("b200.init_from: checkpoint has no tensors for " + base);
      if (w->second->data.size() + b->second->data.size() != l.n_params)
        throw InvalidConfig("b200.init_from: " + base + " holds " + std::to_string(w->second->data.size() + b->second->data.size()) +
                            " values, the model needs " + std::to_string(l.n_params));
      Json vals = Json::array();
      for (float v : w->second->data) vals.push(Json(v));
      for (float v : b->second->data) vals.push(Json(v));
      Json body = Json::object();
      body.set("params", vals);
      l.param_gen = Json::tagged("inline", body);
    }
  }
  const size_t n_params = layers.empty() ? 0 : layers.back().offset + layers.back().n_params;
  const size_t nrows = dataset_rows(training.dataset);
  const auto kind = training.algorithm.kind;
  const bool colocate = training.b200.colocate;
  const bool even = training.b200.sharding == "even";

  std::map<std::string, size_t> rank_of;  // position in training.addrs = rank
  for (size_t i = 0; i < training.addrs.size(); ++i) rank_of[training.addrs[i]] = i;
  auto rank = [&](const std::string& a) { return Json((unsigned long long)rank_of.at(a)); };

  Json plan = Json::object();
  plan.set("algorithm", kind == AlgorithmConfig::AllReduce ? "all_reduce" : kind == AlgorithmConfig::ParameterServer ? "parameter_server" : "strategy_switch");
  plan.set("n_params", Json((unsigned long long)n_params));
  plan.set("n_rows", Json((unsigned long long)nrows));
  Json jl = Json::array();
  for (auto& l : layers) {
    Json o = Json::object();
    o.set("index", Json((unsigned long long)l.index));
    o.set("input_size", Json((unsigned long long)l.input_size));
    o.set("output_size", Json((unsigned long long)l.output_size));
    o.set("n_params", Json((unsigned long long)l.n_params));
    o.set("offset", Json((unsigned long long)l.offset));
    o.set("spec", l.layer_spec);
    o.set("param_gen", l.param_gen);
    jl.push(o);
  }
  plan.set("layers", jl);
  plan.set("serializer", serializer_spec(training));
  plan.set("b200", training.b200.to_json());
  plan.set("seed", training.seed ? Json(*training.seed) : Json());
  if (training.early_stopping_tolerance) {
    Json e = Json::object();
    e.set("window", 3);  // adapter.rs:172-175
    e.set("tolerance", *training.early_stopping_tolerance);
    plan.set("early_stopping", e);
  } else plan.set("early_stopping", Json());

  // Chained generator over the whole model (all-reduce replicas sample all parameters locally).
  Json all_specs = Json::array();
  size_t weighted_layers = 0;
  for (auto& l : layers)
    if (!l.param_gen.is_null()) { all_specs.push(l.param_gen); ++weighted_layers; }
  Json chained_all = Json::object();
  chained_all.set("specs", all_specs);
  const Json model_param_gen = Json::tagged("chained", chained_all);

  std::vector<std::string> server_addrs, worker_addrs;
  if (kind == AlgorithmConfig::AllReduce) {
    worker_addrs = calc.worker_cycle();
  } else if (kind == AlgorithmConfig::ParameterServer) {
    auto roles = calc.node_role_assignment(training.algorithm.nservers);
    server_addrs = roles.server_addrs;
    worker_addrs = colocate ? calc.addrs() : roles.worker_addrs;
  } else {
    server_addrs = calc.node_role_assignment(training.algorithm.nservers).server_addrs;
    worker_addrs = calc.worker_cycle();
  }
  if (worker_addrs.empty()) throw InvalidConfig("no route connects every node: cannot form the worker set");

  const size_t nservers = server_addrs.size();
  // Workers that remain workers after a switch (strategy switch) or the PS worker count.
  const size_t ps_workers = kind == AlgorithmConfig::AllReduce ? 0
                            : colocate ? training.addrs.size() : training.addrs.size() - nservers;
  Sharding sh;
  if (kind != AlgorithmConfig::AllReduce) sh = shard_layers(layers, nservers, even);

  // dataset partitions: over the workers; for the strategy switch over all addresses (adapter.rs:142-143)
  const size_t nparts = kind == AlgorithmConfig::StrategySwitch ? training.addrs.size() : worker_addrs.size();
  const auto parts = dataset_partitions(nrows, nparts);
  const auto batches = per_worker_batch(training, worker_addrs.size());

  auto sync_spec = [&]() -> Json {
    if (training.algorithm.synchronizer == AlgorithmConfig::NonBlocking) return "non_blocking";
    Json b = Json::object();
    b.set("barrier_size", Json((unsigned long long)ps_workers));
    return Json::tagged("barrier", b);
  };
  auto server_spec = [&](size_t i) {
    Json s = Json::object();
    s.set("nworkers", Json((unsigned long long)ps_workers));
    s.set("param_gen", sh.param_gens[i]);
    s.set("optimizer", optimizer_spec(training.optimizer, false));
    s.set("synchronizer", sync_spec());
    s.set("store", training.algorithm.store == AlgorithmConfig::Blocking ? "blocking" : "wild");
    s.set("seed", training.seed ? Json(*training.seed) : Json());
    return s;
  };

  Json servers = Json::array();
  if (kind == AlgorithmConfig::ParameterServer) {
    for (size_t i = 0; i < nservers; ++i) {
      Json s = Json::object();
      s.set("addr", server_addrs[i]);
      s.set("rank", rank(server_addrs[i]));
      s.set("spec", server_spec(i));
      s.set("size", Json((unsigned long long)sh.server_sizes[i]));
      s.set("ranges", ranges_json(sh.global_ranges[i]));
      s.set("local_ranges", ranges_json(sh.local_ranges[i]));
      servers.push(s);
    }
  }
  plan.set("servers", servers);

  Json workers = Json::array();
  for (size_t i = 0; i < worker_addrs.size(); ++i) {
    Json alg;
    if (kind == AlgorithmConfig::ParameterServer) {
      Json b = Json::object();
      b.set("server_addrs", str_array(server_addrs));
      b.set("server_sizes", usize_array(sh.server_sizes));
      b.set("server_ordering", usize_array(sh.server_ordering));
      alg = Json::tagged("parameter_server", b);
    } else {
      Json b = Json::object();
      b.set("pos", Json((unsigned long long)i));
      b.set("worker_addrs", str_array(worker_addrs));
      b.set("param_gen", model_param_gen);
      // adapter.rs:329-331 counts weighted layers for all-reduce, adapter.rs:386 all layers for the switch
      b.set("amount_of_layers", Json((unsigned long long)(kind == AlgorithmConfig::AllReduce ? weighted_layers : layers.size())));
      alg = Json::tagged("all_reduce", b);
    }
    Json spec = Json::object();
    spec.set("trainer", trainer_spec(layers, training, kind == AlgorithmConfig::ParameterServer, batches[i]));
    spec.set("algorithm", alg);
    spec.set("serializer", serializer_spec(training));
    spec.set("seed", training.seed ? Json(*training.seed) : Json());
    Json w = Json::object();
    w.set("addr", worker_addrs[i]);
    w.set("rank", rank(worker_addrs[i]));
    w.set("spec", spec);
    Json part = Json::array();
    part.push(Json((unsigned long long)parts[i].first));
    part.push(Json((unsigned long long)parts[i].second));
    w.set("partition", part);
    workers.push(w);
  }
  plan.set("workers", workers);
  plan.set("server_addrs", str_array(server_addrs));
  plan.set("worker_addrs", str_array(worker_addrs));
  if (kind != AlgorithmConfig::AllReduce) {
    plan.set("server_sizes", usize_array(sh.server_sizes));
    plan.set("server_ordering", usize_array(sh.server_ordering));
    Json lo = Json::array();
    for (auto& [srv, b, e] : sh.layer_offsets) {
      Json t = Json::array();
      t.push(Json((unsigned long long)srv));
      t.push(Json((unsigned long long)b));
      t.push(Json((unsigned long long)e));
      lo.push(t);
    }
    plan.set("layer_offsets", lo);
    Json gr = Json::array();
    for (auto& r : sh.global_ranges) gr.push(ranges_json(r));
    plan.set("server_ranges", gr);
  }

  if (kind == AlgorithmConfig::StrategySwitch) {
    // adapter.rs:229-231, 277-310: one post-action per node, Upgrade for the promoted ones.
    Json actions = Json::array();
    const Json ps_trainer = trainer_spec(layers, training, false, training.batch_size);
    for (auto& addr : worker_addrs) {
      Json a = Json::object();
      a.set("addr", addr);
      a.set("rank", rank(addr));
      auto it = std::find(server_addrs.begin(), server_addrs.end(), addr);
      if (it != server_addrs.end()) {
        const size_t si = (size_t)(it - server_addrs.begin());
        a.set("action", "upgrade");
        a.set("server_index", Json((unsigned long long)si));
        a.set("spec", server_spec(si));
        a.set("ranges", ranges_json(sh.global_ranges[si]));        // global offsets (see header)
        a.set("local_ranges", ranges_json(sh.local_ranges[si]));
      } else {
        a.set("action", "switch");
        a.set("server_addrs", str_array(server_addrs));
        a.set("server_sizes", usize_array(sh.server_sizes));
        a.set("server_ordering", usize_array(sh.server_ordering));
        a.set("trainer_spec", ps_trainer);
      }
      actions.push(a);
    }
    Json sw = Json::object();
    sw.set("post_actions", actions);
    sw.set("metric", training.b200.switch_metric);
    sw.set("window", Json((unsigned long long)training.b200.switch_window));
    sw.set("threshold", training.b200.switch_threshold);
    sw.set("nworkers_after", Json((unsigned long long)ps_workers));
    plan.set("switch", sw);
  } else plan.set("switch", Json());
  return plan;
}

// ---- Calculator -------------------------------------------------------------------------------
Calculator Calculator::uniform(const std::vector<std::string>& addrs) {
  std::map<std::string, std::map<std::string, uint64_t>> st;
  for (auto& a : addrs) {
    auto& row = st[a];
    for (auto& b : addrs)
      if (a != b) row[b] = 1000;
  }
  return Calculator(std::move(st));
}

std::vector<std::string> Calculator::addrs() const {
  std::vector<std::string> v;
  for (auto& kv : stats_) v.push_back(kv.first);
  return v;
}

std::vector<std::tuple<size_t, size_t, uint64_t>> Calculator::edges() const {
  std::map<std::string, size_t> idx;
  size_t i = 0;
  for (auto& kv : stats_) idx[kv.first] = i++;
  std::vector<std::tuple<size_t, size_t, uint64_t>> e;
  i = 0;
  for (auto& kv : stats_) {
    for (auto& [peer, rtt] : kv.second) {
      auto it = idx.find(peer);
      if (it != idx.end()) e.emplace_back(i, it->second, rtt);
    }
    ++i;
  }
  return e;
}

RoleAssignment Calculator::node_role_assignment(size_t servers) const {
  RoleAssignment r;
  auto g = Graph<uint64_t>::make(stats_.size(), edges());
  const auto center = central_vertices(*g, servers);
  size_t i = 0;
  for (auto& kv : stats_) {
    (center.count(i) ? r.server_addrs : r.worker_addrs).push_back(kv.first);
    ++i;
  }
  return r;
}

std::vector<std::string> Calculator::worker_cycle() const {
  auto g = Graph<uint64_t>::make(stats_.size(), edges());
  const auto path = travelling_salesman_cycle(*g);
  const auto a = addrs();
  std::vector<std::string> out;
  for (size_t i : path) out.push_back(a[i]);
  return out;
}

}  // namespace ono
