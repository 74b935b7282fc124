// Bindings of the control-plane half of `orchestra._orchestra` (configs, adapter, calculators,
// trackers, codecs, files). See bindings.cpp for the module definition.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "core/adapter.hpp"
#include "core/calculator.hpp"
#include "core/codec.hpp"
#include "core/configs.hpp"
#include "core/dyn_barrier.hpp"
#include "core/trackers.hpp"

namespace py = pybind11;
using namespace ono;
using farray = py::array_t<float, py::array::c_style | py::array::forcecast>;

namespace {

using Edges = std::vector<std::tuple<size_t, size_t, uint64_t>>;

Calculator calculator_from(const TrainingConfig& t, const std::string& stats_json) {
  if (stats_json.empty()) return Calculator::uniform(t.addrs);
  // {"addr": {"peer": max_rtt_ns, ...}, ...}
  Json j = Json::parse(stats_json);
  std::map<std::string, std::map<std::string, uint64_t>> st;
  for (auto& a : t.addrs) st[a];
  for (auto& [addr, peers] : j.members())
    for (auto& [peer, rtt] : peers.members()) st[addr][peer] = rtt.as_u64();
  return Calculator(std::move(st));
}

farray vec_np(const std::vector<float>& v) {
  farray a(v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), sizeof(float) * v.size());
  return a;
}

}  // namespace

void bind_core(py::module_& m) {
  // ---- configs ----
  m.def("normalize_model_config", [](const std::string& js) { return ModelConfig::from_json(Json::parse(js)).to_json().dump(); },
        "Parse model.json text (serde encoding) and re-serialise it canonically; raises ValueError.");
  m.def("normalize_training_config", [](const std::string& js, bool with_data) {
    return TrainingConfig::from_json(Json::parse(js)).to_json(with_data).dump();
  }, py::arg("json"), py::arg("with_data") = true);
  m.def("validate_configs", [](const std::string& model_js, const std::string& training_js) {
    validate_configs(ModelConfig::from_json(Json::parse(model_js)), TrainingConfig::from_json(Json::parse(training_js)));
  });
  m.def("model_param_count", [](const std::string& model_js, size_t x_size) {
    return ModelConfig::from_json(Json::parse(model_js)).param_count(x_size);
  });
  m.def("adapt_configs", [](const std::string& model_js, const std::string& training_js, const std::string& stats_js) {
    const ModelConfig model = ModelConfig::from_json(Json::parse(model_js));
    const TrainingConfig training = TrainingConfig::from_json(Json::parse(training_js));
    validate_configs(model, training);
    return adapt_configs(model, training, calculator_from(training, stats_js)).dump();
  }, py::arg("model_json"), py::arg("training_json"), py::arg("stats_json") = "",
     "Validate and turn the two configs (+ optional RTT statistics) into the run plan (JSON text).");
  m.def("balanced_partitions", &balanced_partitions);
  m.def("dataset_partitions", &dataset_partitions);

  // ---- calculators ----
  m.def("tsp_cycle", [](size_t n, const Edges& edges) {
    auto g = Graph<uint64_t>::make(n, edges);
    if (!g) throw std::invalid_argument("edge names a vertex outside the graph");
    return travelling_salesman_cycle(*g);
  });
  m.def("central_vertices", [](size_t n, const Edges& edges, size_t k) {
    auto g = Graph<uint64_t>::make(n, edges);
    if (!g) throw std::invalid_argument("edge names a vertex outside the graph");
    auto s = central_vertices(*g, k);
    return std::vector<size_t>(s.begin(), s.end());
  });

  // ---- trackers ----
  py::class_<ConvergenceTracker>(m, "ConvergenceTracker")
      .def(py::init<size_t, double>())
      .def("record", &ConvergenceTracker::record)
      .def("converged", &ConvergenceTracker::converged);
  py::class_<SwitchTracker>(m, "SwitchTracker")
      .def(py::init<size_t, double>())
      .def("record", &SwitchTracker::record)
      .def("should_switch", &SwitchTracker::should_switch);
  py::class_<LossRecorder>(m, "LossRecorder")
      .def(py::init<>())
      .def("record", &LossRecorder::record)
      .def("max", &LossRecorder::max)
      .def("mean", &LossRecorder::mean)
      .def("clear", &LossRecorder::clear);
  py::class_<SessionPolicy>(m, "SessionPolicy")
      .def(py::init<size_t>())
      .def("enable_early_stopping", &SessionPolicy::enable_early_stopping)
      .def("enable_switch", &SessionPolicy::enable_switch)
      .def("set_switch_on_metric", &SessionPolicy::set_switch_on_metric)
      .def("on_losses", [](SessionPolicy& p, size_t w, const std::vector<double>& l) { return (int)p.on_losses(w, l.data(), l.size()); })
      .def("on_metric", [](SessionPolicy& p, double v) { return (int)p.on_metric(v); })
      .def("worker_left", &SessionPolicy::worker_left)
      .def("workers_left", &SessionPolicy::workers_left)
      .def("stopped", &SessionPolicy::stopped);
  py::class_<DynBarrier>(m, "DynBarrier")
      .def(py::init<size_t>())
      .def("wait", [](DynBarrier& b) { py::gil_scoped_release rel; return b.wait_with(nullptr); })
      .def("leave", [](DynBarrier& b) { b.leave(nullptr); })
      .def("size", &DynBarrier::size);

  // ---- codecs ----
  m.def("f16_round_trip", [](const farray& a) {
    farray out(a.size());
    for (py::ssize_t i = 0; i < a.size(); ++i) out.mutable_data()[i] = f16_round_trip(a.data()[i]);
    return out;
  });
  m.def("f32_to_f16_bits", [](float f) { return f32_to_f16(f); });
  m.def("sparse_threshold", [](const farray& a, double r, uint64_t seed) { return sparse_threshold(a.data(), (size_t)a.size(), r, seed); });
  m.def("sparse_drop", [](const farray& a, float thr) {
    std::vector<uint8_t> out;
    sparse_drop(out, a.data(), (size_t)a.size(), thr);
    return py::bytes((const char*)out.data(), out.size());
  });
  m.def("sparse_lift", [](py::bytes b, const farray& initial) {
    std::string s = b;
    std::vector<float> g(initial.data(), initial.data() + initial.size());
    sparse_lift(g, (const uint8_t*)s.data(), s.size());
    return vec_np(g);
  }, py::arg("buf"), py::arg("initial") = farray(0));
  m.def("compress_gradient", [](const farray& a, bool sparse, double r, uint64_t seed) {
    Compressed c = compress_gradient(a.data(), (size_t)a.size(), sparse, r, seed);
    return py::make_tuple(c.sparse, c.threshold, py::bytes((const char*)c.bytes.data(), c.bytes.size()));
  });

  // ---- files ----
  m.def("save_safetensors", [](const std::string& path, const std::string& model_js, size_t input_size, const farray& params) {
    std::vector<float> p(params.data(), params.data() + params.size());
    save_safetensors(path, ModelConfig::from_json(Json::parse(model_js)), input_size, p);
  });
  m.def("load_safetensors", [](const std::string& path) {
    py::list out;
    for (auto& t : load_safetensors(path)) out.append(py::make_tuple(t.name, t.shape, vec_np(t.data)));
    return out;
  });
  m.def("ensure_binary_dataset", &ensure_binary_dataset);
  m.def("read_f32_file", [](const std::string& path, size_t off, py::object count) {
    return vec_np(read_f32_file(path, off, count.is_none() ? (size_t)-1 : count.cast<size_t>()));
  }, py::arg("path"), py::arg("offset") = 0, py::arg("count") = py::none());
}
