#include "configs.hpp"

#include <sys/stat.h>

#include <cmath>

namespace ono {

namespace {

// A serde enum value is either "variant" or {"variant": {...}}.
std::pair<std::string, const Json*> variant_of(const Json& j, const char* what) {
  if (j.is_string()) return {j.as_string(), nullptr};
  if (j.is_object() && j.size() == 1) return {j.members()[0].first, &j.members()[0].second};
  throw InvalidConfig(std::string("invalid ") + what + ": expected a string or a single-key object");
}

float f32_field(const Json* body, const char* key, const char* owner) {
  if (!body || !body->is_object() || !body->has(key))
    throw InvalidConfig(std::string(owner) + " is missing field `" + key + "`");
  const Json& v = body->at(key);
  if (!v.is_number()) throw InvalidConfig(std::string(owner) + "." + key + " must be a number");
  return (float)v.as_double();
}

double f64_field(const Json* body, const char* key, const char* owner) {
  if (!body || !body->is_object() || !body->has(key))
    throw InvalidConfig(std::string(owner) + " is missing field `" + key + "`");
  const Json& v = body->at(key);
  if (!v.is_number()) throw InvalidConfig(std::string(owner) + "." + key + " must be a number");
  return v.as_double();
}

size_t nonzero(const Json& v, const char* what) {
  if (!v.is_number()) throw InvalidConfig(std::string(what) + " must be a positive integer");
  long long x;
  try { x = v.as_int(); } catch (const JsonError&) { throw InvalidConfig(std::string(what) + " must be a positive integer"); }
  if (x <= 0) throw InvalidConfig(std::string(what) + " must be a positive integer");
  return (size_t)x;
}

size_t non_negative(const Json& v, const char* what) {
  if (!v.is_number()) throw InvalidConfig(std::string(what) + " must be a non-negative integer");
  long long x;
  try { x = v.as_int(); } catch (const JsonError&) { throw InvalidConfig(std::string(what) + " must be a non-negative integer"); }
  if (x < 0) throw InvalidConfig(std::string(what) + " must be a non-negative integer");
  return (size_t)x;
}

std::array<size_t, 3> triple(const Json& v, const char* what) {
  if (!v.is_array() || v.size() != 3) throw InvalidConfig(std::string(what) + " must be an array of 3 positive integers");
  return {nonzero(v[0], what), nonzero(v[1], what), nonzero(v[2], what)};
}

// comms/src/floats: Float01 in [0,1], FloatPositive > 0, FloatNonNegative >= 0 (and not NaN).
double float01(double v, const char* what) {
  if (!(v >= 0.0 && v <= 1.0)) throw InvalidConfig(std::string(what) + " must be in [0, 1]");
  return v;
}
double float_positive(double v, const char* what) {
  if (!(v > 0.0) || !std::isfinite(v)) throw InvalidConfig(std::string(what) + " must be a positive number");
  return v;
}
double float_non_negative(double v, const char* what) {
  if (!(v >= 0.0)) throw InvalidConfig(std::string(what) + " must be a non-negative number");
  return v;
}

Json triple_json(const std::array<size_t, 3>& t) {
  Json a = Json::array();
  for (size_t v : t) a.push(Json((unsigned long long)v));
  return a;
}

}  // namespace

// ---- ParamGenConfig ---------------------------------------------------------------------------
Json ParamGenConfig::to_json() const {
  Json body = Json::object();
  switch (kind) {
    case Const: body.set("value", a); return Json::tagged("const", body);
    case Uniform: body.set("low", a); body.set("high", b); return Json::tagged("uniform", body);
    case UniformInclusive: body.set("low", a); body.set("high", b); return Json::tagged("uniform_inclusive", body);
    case Normal: body.set("mean", a); body.set("std_dev", b); return Json::tagged("normal", body);
    case XavierUniform: return "xavier_uniform";
    case LecunUniform: return "lecun_uniform";
    case Kaiming: return "kaiming";
    case Xavier: return "xavier";
    case Lecun: return "lecun";
  }
  return Json();
}

ParamGenConfig ParamGenConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "init");
  ParamGenConfig c;
  if (name == "const") { c.kind = Const; c.a = f32_field(body, "value", "const"); }
  else if (name == "uniform") { c.kind = Uniform; c.a = f32_field(body, "low", "uniform"); c.b = f32_field(body, "high", "uniform"); }
  else if (name == "uniform_inclusive") { c.kind = UniformInclusive; c.a = f32_field(body, "low", "uniform_inclusive"); c.b = f32_field(body, "high", "uniform_inclusive"); }
  else if (name == "normal") { c.kind = Normal; c.a = f32_field(body, "mean", "normal"); c.b = f32_field(body, "std_dev", "normal"); }
  else if (name == "xavier_uniform") c.kind = XavierUniform;
  else if (name == "lecun_uniform") c.kind = LecunUniform;
  else if (name == "kaiming") c.kind = Kaiming;
  else if (name == "xavier") c.kind = Xavier;
  else if (name == "lecun") c.kind = Lecun;
  else throw InvalidConfig("unknown initializer `" + name + "`");
  return c;
}

// ---- ActFnConfig ------------------------------------------------------------------------------
const char* ActFnConfig::name() const {
  switch (kind) {
    case Sigmoid: return "sigmoid";
    case Softmax: return "softmax";
    case Tanh: return "tanh";
    case ReLU: return "relu";
    case Gelu: return "gelu";
  }
  return "";
}

Json ActFnConfig::to_json() const {
  Json body = Json::object();
  switch (kind) {
    case Sigmoid: body.set("amp", param); return Json::tagged("sigmoid", body);
    case Tanh: body.set("amp", param); return Json::tagged("tanh", body);
    // serde renders the Rust variant `ReLU` as "re_l_u"; the docs and the TUI say "relu". Both are
    // accepted on input; the documented spelling is written.
    case ReLU: body.set("slope", param); return Json::tagged("relu", body);
    case Softmax: return "softmax";
    case Gelu: return "gelu";
  }
  return Json();
}

ActFnConfig ActFnConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "act_fn");
  ActFnConfig c;
  if (name == "sigmoid") { c.kind = Sigmoid; c.param = f32_field(body, "amp", "sigmoid"); }
  else if (name == "tanh") { c.kind = Tanh; c.param = f32_field(body, "amp", "tanh"); }
  else if (name == "relu" || name == "re_l_u") { c.kind = ReLU; c.param = (float)float01(f32_field(body, "slope", "relu"), "relu.slope"); }
  else if (name == "softmax") c.kind = Softmax;
  else if (name == "gelu") c.kind = Gelu;
  else throw InvalidConfig("unknown activation `" + name + "`");
  return c;
}

// ---- LayerConfig ------------------------------------------------------------------------------
static size_t spatial(size_t in, size_t pad, size_t k, size_t stride) {
  const size_t padded = in + 2 * pad;
  return (padded > k ? padded - k : 0) / stride + 1;
}

size_t LayerConfig::out_size() const {
  switch (kind) {
    case Dense: return output_size;
    case Conv: return spatial(input_dim[1], padding, kernel_dim[2], stride) * spatial(input_dim[2], padding, kernel_dim[2], stride) * kernel_dim[0];
    case MaxPooling: return spatial(input_dim[1], padding, filter_size, stride) * spatial(input_dim[2], padding, filter_size, stride) * input_dim[0];
  }
  return 0;
}

std::optional<size_t> LayerConfig::expected_input_size() const {
  if (kind == Dense) return std::nullopt;
  return input_dim[0] * input_dim[1] * input_dim[2];
}

size_t LayerConfig::param_count(size_t input_size) const {
  switch (kind) {
    case Dense: return (input_size + 1) * output_size;
    case Conv: return kernel_dim[0] * kernel_dim[1] * kernel_dim[2] * kernel_dim[2] + kernel_dim[0];
    case MaxPooling: return 0;
  }
  return 0;
}

Json LayerConfig::to_json() const {
  Json body = Json::object();
  const char* tag = "dense";
  switch (kind) {
    case Dense:
      body.set("output_size", Json((unsigned long long)output_size));
      body.set("init", init.to_json());
      break;
    case Conv:
      tag = "conv";
      body.set("input_dim", triple_json(input_dim));
      body.set("kernel_dim", triple_json(kernel_dim));
      body.set("stride", Json((unsigned long long)stride));
      body.set("padding", Json((unsigned long long)padding));
      body.set("init", init.to_json());
      break;
    case MaxPooling:
      tag = "max_pooling";
      body.set("input_dim", triple_json(input_dim));
      body.set("filter_size", Json((unsigned long long)filter_size));
      body.set("stride", Json((unsigned long long)stride));
      body.set("padding", Json((unsigned long long)padding));
      break;
  }
  body.set("act_fn", act_fn ? act_fn->to_json() : Json());
  return Json::tagged(tag, body);
}

LayerConfig LayerConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "layer");
  if (!body || !body->is_object()) throw InvalidConfig("layer `" + name + "` needs a body object");
  LayerConfig l;
  auto need = [&](const char* k) -> const Json& {
    if (!body->has(k)) throw InvalidConfig(name + " layer is missing field `" + k + "`");
    return body->at(k);
  };
  if (name == "dense") {
    l.kind = Dense;
    l.output_size = nonzero(need("output_size"), "dense.output_size");
    l.init = ParamGenConfig::from_json(need("init"));
  } else if (name == "conv") {
    l.kind = Conv;
    l.input_dim = triple(need("input_dim"), "conv.input_dim");
    l.kernel_dim = triple(need("kernel_dim"), "conv.kernel_dim");
    l.stride = nonzero(need("stride"), "conv.stride");
    l.padding = non_negative(need("padding"), "conv.padding");
    l.init = ParamGenConfig::from_json(need("init"));
  } else if (name == "max_pooling") {
    l.kind = MaxPooling;
    l.input_dim = triple(need("input_dim"), "max_pooling.input_dim");
    l.filter_size = nonzero(need("filter_size"), "max_pooling.filter_size");
    l.stride = nonzero(need("stride"), "max_pooling.stride");
    l.padding = non_negative(need("padding"), "max_pooling.padding");
  } else {
    throw InvalidConfig("unknown layer type `" + name + "`");
  }
  if (const Json* a = body->find("act_fn"); a && !a->is_null()) l.act_fn = ActFnConfig::from_json(*a);
  return l;
}

Json ModelConfig::to_json() const {
  Json arr = Json::array();
  for (auto& l : layers) arr.push(l.to_json());
  Json o = Json::object();
  o.set("layers", arr);
  return o;
}

ModelConfig ModelConfig::from_json(const Json& j) {
  if (!j.is_object() || !j.has("layers") || !j.at("layers").is_array()) throw InvalidConfig("model config needs a `layers` array");
  ModelConfig m;
  for (auto& l : j.at("layers").items()) m.layers.push_back(LayerConfig::from_json(l));
  return m;
}

size_t ModelConfig::param_count(size_t x_size) const {
  size_t in = x_size, total = 0;
  for (auto& l : layers) { total += l.param_count(in); in = l.out_size(); }
  return total;
}

// ---- training ---------------------------------------------------------------------------------
Json OptimizerConfig::to_json() const {
  Json b = Json::object();
  b.set("lr", lr);
  switch (kind) {
    case GradientDescent: return Json::tagged("gradient_descent", b);
    case Momentum: b.set("mu", mu); return Json::tagged("gradient_descent_with_momentum", b);
    case Adam: b.set("b1", b1); b.set("b2", b2); b.set("eps", eps); return Json::tagged("adam", b);
  }
  return Json();
}

OptimizerConfig OptimizerConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "optimizer");
  OptimizerConfig o;
  o.lr = float_positive(f64_field(body, "lr", name.c_str()), "optimizer lr");
  if (name == "gradient_descent") o.kind = GradientDescent;
  else if (name == "gradient_descent_with_momentum") { o.kind = Momentum; o.mu = float01(f64_field(body, "mu", "momentum"), "optimizer mu"); }
  else if (name == "adam") {
    o.kind = Adam;
    o.b1 = float01(f64_field(body, "b1", "adam"), "adam b1");
    o.b2 = float01(f64_field(body, "b2", "adam"), "adam b2");
    o.eps = float_positive(f64_field(body, "eps", "adam"), "adam eps");
  } else throw InvalidConfig("unknown optimizer `" + name + "`");
  return o;
}

Json DatasetConfig::to_json() const {
  Json src_body = Json::object();
  Json src;
  if (is_inline) {
    Json s = Json::array(), l = Json::array();
    for (float v : samples) s.push(Json(v));
    for (float v : labels) l.push(Json(v));
    src_body.set("samples", s);
    src_body.set("labels", l);
    if (rows_hint) src_body.set("rows", Json((unsigned long long)rows_hint));
    src = Json::tagged("inline", src_body);
  } else {
    src_body.set("samples_path", samples_path);
    src_body.set("labels_path", labels_path);
    src = Json::tagged("local", src_body);
  }
  Json o = Json::object();
  o.set("src", src);
  o.set("x_size", Json((unsigned long long)x_size));
  o.set("y_size", Json((unsigned long long)y_size));
  return o;
}

DatasetConfig DatasetConfig::from_json(const Json& j) {
  if (!j.is_object()) throw InvalidConfig("dataset must be an object");
  DatasetConfig d;
  auto [name, body] = variant_of(j.at("src"), "dataset.src");
  if (!body || !body->is_object()) throw InvalidConfig("dataset.src needs a body");
  if (name == "inline") {
    d.is_inline = true;
    for (auto& v : body->at("samples").items()) d.samples.push_back((float)v.as_double());
    for (auto& v : body->at("labels").items()) d.labels.push_back((float)v.as_double());
    if (const Json* r = body->find("rows"); r && !r->is_null()) d.rows_hint = (size_t)r->as_u64();
  } else if (name == "local") {
    d.is_inline = false;
    d.samples_path = body->at("samples_path").as_string();
    d.labels_path = body->at("labels_path").as_string();
  } else throw InvalidConfig("unknown dataset source `" + name + "`");
  d.x_size = nonzero(j.at("x_size"), "dataset.x_size");
  d.y_size = nonzero(j.at("y_size"), "dataset.y_size");
  return d;
}

Json AlgorithmConfig::to_json() const {
  if (kind == AllReduce) return "all_reduce";
  Json b = Json::object();
  b.set("nservers", Json((unsigned long long)nservers));
  b.set("synchronizer", synchronizer == Barrier ? "barrier" : "non_blocking");
  b.set("store", store == Blocking ? "blocking" : "wild");
  return Json::tagged(kind == ParameterServer ? "parameter_server" : "strategy_switch", b);
}

AlgorithmConfig AlgorithmConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "algorithm");
  AlgorithmConfig a;
  if (name == "all_reduce") { a.kind = AllReduce; return a; }
  if (name == "parameter_server") a.kind = ParameterServer;
  else if (name == "strategy_switch") a.kind = StrategySwitch;
  else throw InvalidConfig("unknown algorithm `" + name + "`");
  if (!body || !body->is_object()) throw InvalidConfig(name + " needs nservers, synchronizer and store");
  a.nservers = nonzero(body->at("nservers"), "nservers");
  const std::string s = body->at("synchronizer").as_string();
  if (s == "barrier") a.synchronizer = Barrier;
  else if (s == "non_blocking") a.synchronizer = NonBlocking;
  else throw InvalidConfig("unknown synchronizer `" + s + "`");
  const std::string st = body->at("store").as_string();
  if (st == "blocking") a.store = Blocking;
  else if (st == "wild") a.store = Wild;
  else throw InvalidConfig("unknown store `" + st + "`");
  return a;
}

Json SerializerConfig::to_json() const {
  if (!sparse) return "base";
  Json b = Json::object();
  b.set("r", r);
  return Json::tagged("sparse_capable", b);
}

SerializerConfig SerializerConfig::from_json(const Json& j) {
  auto [name, body] = variant_of(j, "serializer");
  SerializerConfig s;
  if (name == "base") return s;
  if (name != "sparse_capable") throw InvalidConfig("unknown serializer `" + name + "`");
  s.sparse = true;
  s.r = float01(f64_field(body, "r", "sparse_capable"), "serializer r");
  return s;
}

Json B200Config::to_json() const {
  Json o = Json::object();
  o.set("sync_every", sync_every);
  o.set("tile_dtype", tile_dtype);
  o.set("wire_dtype", wire_dtype);
  o.set("wgrad_apply", wgrad_apply);
  o.set("param_pull", param_pull);
  o.set("shard_layout", shard_layout);
  o.set("pre_reduce", pre_reduce);
  o.set("switch_check_every", Json((unsigned long long)switch_check_every));
  o.set("allreduce", allreduce);
  o.set("sharding", sharding);
  o.set("switch_metric", switch_metric);
  o.set("switch_window", Json((unsigned long long)switch_window));
  o.set("switch_threshold", switch_threshold);
  o.set("leaky_relu_exact", leaky_relu_exact);
  o.set("global_batch", Json((unsigned long long)global_batch));
  o.set("switch_resets_progress", switch_resets_progress);
  o.set("colocate", colocate);
  o.set("data", data);
  o.set("probe", probe);
  o.set("phase_timing", phase_timing);
  o.set("grad_stage", grad_stage);
  o.set("grad_push", grad_push);
  o.set("comm_timeout_s", comm_timeout_s);
  o.set("heartbeat_s", heartbeat_s);
  o.set("heartbeat_timeout_s", heartbeat_timeout_s);
  o.set("init_from", init_from);
  o.set("trace_path", trace_path);
  o.set("state_path", state_path);
  o.set("checkpoint_path", checkpoint_path);
  o.set("checkpoint_every", (long long)checkpoint_every);
  o.set("init_state_from", init_state_from);
  o.set("start_epoch", (long long)start_epoch);
  o.set("metrics_path", metrics_path);
  return o;
}

B200Config B200Config::from_json(const Json& j) {
  B200Config c;
  if (!j.is_object()) throw InvalidConfig("b200 must be an object");
  c.present = true;
  auto str = [&](const char* k, std::string& dst, std::initializer_list<const char*> allowed) {
    if (const Json* v = j.find(k)) {
      dst = v->as_string();
      bool ok = false;
      for (const char* a : allowed) ok = ok || dst == a;
      if (!ok) throw InvalidConfig(std::string("b200.") + k + ": unsupported value `" + dst + "`");
    }
  };
  str("sync_every", c.sync_every, {"round", "step"});
  str("tile_dtype", c.tile_dtype, {"tf32", "bf16"});
  str("wire_dtype", c.wire_dtype, {"auto", "f32", "f16", "bf16"});
  str("allreduce", c.allreduce, {"auto", "ring", "oneshot", "twoshot", "nvls", "nccl"});
  str("sharding", c.sharding, {"layer", "even"});
  str("switch_metric", c.switch_metric, {"loss", "grad_norm"});
  str("data", c.data, {"host", "device"});
  str("grad_push", c.grad_push, {"auto", "on", "off", "reduce", "direct"});
  str("wgrad_apply", c.wgrad_apply, {"auto", "off"});
  str("param_pull", c.param_pull, {"auto", "kernel", "staged"});
  str("shard_layout", c.shard_layout, {"striped", "contiguous"});
  str("pre_reduce", c.pre_reduce, {"auto", "on", "off"});
  if (const Json* v = j.find("switch_check_every")) c.switch_check_every = nonzero(*v, "b200.switch_check_every");
  str("grad_stage", c.grad_stage, {"auto", "on", "off"});
  if (const Json* v = j.find("switch_window")) { c.switch_window = nonzero(*v, "b200.switch_window"); if (c.switch_window < 2) throw InvalidConfig("b200.switch_window must be at least 2"); }
  if (const Json* v = j.find("switch_threshold")) c.switch_threshold = float_non_negative(v->as_double(), "b200.switch_threshold");
  if (const Json* v = j.find("leaky_relu_exact")) c.leaky_relu_exact = v->as_bool();
  if (const Json* v = j.find("global_batch")) c.global_batch = non_negative(*v, "b200.global_batch");
  if (const Json* v = j.find("switch_resets_progress")) c.switch_resets_progress = v->as_bool();
  if (const Json* v = j.find("colocate")) c.colocate = v->as_bool();
  if (const Json* v = j.find("probe")) c.probe = v->as_bool();
  if (const Json* v = j.find("phase_timing")) c.phase_timing = v->as_bool();
  if (const Json* v = j.find("comm_timeout_s")) c.comm_timeout_s = float_positive(v->as_double(), "b200.comm_timeout_s");
  if (const Json* v = j.find("heartbeat_s")) c.heartbeat_s = float_non_negative(v->as_double(), "b200.heartbeat_s");
  if (const Json* v = j.find("heartbeat_timeout_s")) c.heartbeat_timeout_s = float_non_negative(v->as_double(), "b200.heartbeat_timeout_s");
  if (const Json* v = j.find("init_from")) c.init_from = v->as_string();
  if (const Json* v = j.find("trace_path")) c.trace_path = v->as_string();
  if (const Json* v = j.find("state_path")) c.state_path = v->as_string();
  if (const Json* v = j.find("checkpoint_path")) c.checkpoint_path = v->as_string();
  if (const Json* v = j.find("checkpoint_every")) {
    c.checkpoint_every = v->as_int();
    if (c.checkpoint_every < 0) throw InvalidConfig("b200.checkpoint_every must be >= 0");
  }
  if (const Json* v = j.find("init_state_from")) c.init_state_from = v->as_string();
  if (const Json* v = j.find("start_epoch")) c.start_epoch = v->as_int();
  if (const Json* v = j.find("metrics_path")) c.metrics_path = v->as_string();
  return c;
}

Json TrainingConfig::to_json(bool with_data) const {
  Json o = Json::object();
  Json a = Json::array();
  for (auto& s : addrs) a.push(s);
  o.set("addrs", a);
  o.set("algorithm", algorithm.to_json());
  o.set("serializer", serializer.to_json());
  if (with_data || !dataset.is_inline) o.set("dataset", dataset.to_json());
  else {
    DatasetConfig d = dataset;
    d.samples.clear();
    d.labels.clear();
    o.set("dataset", d.to_json());
  }
  o.set("optimizer", optimizer.to_json());
  o.set("loss_fn", loss_fn == Mse ? "mse" : "cross_entropy");
  o.set("batch_size", Json((unsigned long long)batch_size));
  o.set("max_epochs", Json((unsigned long long)max_epochs));
  o.set("offline_epochs", Json((unsigned long long)offline_epochs));
  o.set("seed", seed ? Json(*seed) : Json());
  if (early_stopping_tolerance) {
    Json e = Json::object();
    e.set("tolerance", *early_stopping_tolerance);
    o.set("early_stopping", e);
  } else o.set("early_stopping", Json());
  if (b200.present) o.set("b200", b200.to_json());
  return o;
}

TrainingConfig TrainingConfig::from_json(const Json& j) {
  if (!j.is_object()) throw InvalidConfig("training config must be an object");
  TrainingConfig t;
  auto need = [&](const char* k) -> const Json& {
    if (!j.has(k)) throw InvalidConfig(std::string("training config is missing field `") + k + "`");
    return j.at(k);
  };
  try {
    for (auto& a : need("addrs").items()) t.addrs.push_back(a.as_string());
    t.algorithm = AlgorithmConfig::from_json(need("algorithm"));
    if (const Json* s = j.find("serializer"); s && !s->is_null()) t.serializer = SerializerConfig::from_json(*s);
    t.dataset = DatasetConfig::from_json(need("dataset"));
    t.optimizer = OptimizerConfig::from_json(need("optimizer"));
    const std::string loss = need("loss_fn").as_string();
    if (loss == "mse") t.loss_fn = Mse;
    else if (loss == "cross_entropy") t.loss_fn = CrossEntropy;
    else throw InvalidConfig("unknown loss_fn `" + loss + "`");
    t.batch_size = nonzero(need("batch_size"), "batch_size");
    t.max_epochs = nonzero(need("max_epochs"), "max_epochs");
    t.offline_epochs = non_negative(need("offline_epochs"), "offline_epochs");
    if (const Json* s = j.find("seed"); s && !s->is_null()) t.seed = s->as_u64();
    if (const Json* e = j.find("early_stopping"); e && !e->is_null())
      t.early_stopping_tolerance = float_non_negative(e->at("tolerance").as_double(), "early_stopping.tolerance");
    if (const Json* b = j.find("b200"); b && !b->is_null()) t.b200 = B200Config::from_json(*b);
  } catch (const JsonError& e) {
    throw InvalidConfig(std::string("training config: ") + e.what());
  }
  return t;
}

// ---- validation -------------------------------------------------------------------------------
static size_t file_size(const std::string& path, const char* what) {
  struct stat st;
  if (stat(path.c_str(), &st) != 0) throw InvalidConfig(std::string("cannot read dataset ") + what + " file: " + path);
  return (size_t)st.st_size;
}

size_t dataset_rows(const DatasetConfig& d) {
  const size_t row = d.x_size + d.y_size;
  size_t len;
  if (d.is_inline && d.samples.empty() && d.labels.empty() && d.rows_hint) return d.rows_hint;
  if (d.is_inline) len = d.samples.size() + d.labels.size();
  else len = (file_size(d.samples_path, "samples") + file_size(d.labels_path, "labels")) / sizeof(float);
  if (len % row != 0)
    throw InvalidConfig("dataset length (" + std::to_string(len) + ") is not divisible by x_size + y_size (" + std::to_string(row) + ")");
  return len / row;
}

void validate_configs(const ModelConfig& model, const TrainingConfig& training) {
  // validator.rs:104-124 model
  if (model.layers.empty()) throw InvalidConfig("model must have at least one layer");
  for (auto& l : model.layers) {
    if (l.kind == LayerConfig::Dense) continue;
    const size_t k = l.kind == LayerConfig::Conv ? l.kernel_dim[2] : l.filter_size;
    const size_t rh = l.input_dim[1] + 2 * l.padding, rw = l.input_dim[2] + 2 * l.padding;
    if (rh <= k || rw <= k)
      throw InvalidConfig("conv layer input_dim + 2 * padding - kernel_size must be greater than 0 for both height and width");
  }
  // validator.rs:126-203 training
  if (training.addrs.empty()) throw InvalidConfig("at least one network address is required");
  if (training.algorithm.kind != AlgorithmConfig::AllReduce && !training.b200.colocate &&
      training.addrs.size() <= training.algorithm.nservers)
    throw InvalidConfig("the amount of workers must be a positive number");
  if (training.algorithm.kind != AlgorithmConfig::AllReduce && training.b200.colocate &&
      training.algorithm.nservers > training.addrs.size())
    throw InvalidConfig("nservers exceeds the number of addresses");
  const size_t samples = dataset_rows(training.dataset);
  if (samples == 0) throw InvalidConfig("dataset must have at least one sample");
  if (training.batch_size > samples)
    throw InvalidConfig("batch_size (" + std::to_string(training.batch_size) + ") exceeds dataset size (" + std::to_string(samples) + " samples)");
  // validator.rs:35-63 dimensions chain
  size_t in = training.dataset.x_size;
  for (auto& l : model.layers) {
    if (auto exp = l.expected_input_size(); exp && *exp != in)
      throw InvalidConfig("layer expects an input of " + std::to_string(*exp) + " but the incoming size is " + std::to_string(in));
    in = l.out_size();
  }
  if (in != training.dataset.y_size)
    throw InvalidConfig("the model's output size (" + std::to_string(in) + ") must match the dataset's y_size (" + std::to_string(training.dataset.y_size) + ")");
}

}  // namespace ono
