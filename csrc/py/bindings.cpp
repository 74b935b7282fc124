// pybind11 module `orchestra._orchestra`: the C++ control plane (configs, validation, adapter,
// calculators, trackers, codecs, safetensors, dataset conversion), the CPU oracle engine and the
// in-process CPU cluster, exposed to the Python `orchestra` package. It plays the role of the
// reference's PyO3 glue (orchestra-py/src/lib.rs:16-67); documents cross the boundary as JSON text.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "core/adapter.hpp"
#include "core/calculator.hpp"
#include "core/codec.hpp"
#include "core/configs.hpp"
#include "core/dyn_barrier.hpp"
#include "core/philox.h"
#include "core/trackers.hpp"
#include "oracle/cluster.hpp"
#include "oracle/engine.hpp"

namespace py = pybind11;
using namespace ono;
using farray = py::array_t<float, py::array::c_style | py::array::forcecast>;

namespace {

std::vector<float> to_vec(const farray& a) {
  std::vector<float> v(a.size());
  if (a.size()) std::memcpy(v.data(), a.data(), sizeof(float) * a.size());
  return v;
}

farray to_np(const std::vector<float>& v) {
  farray a(v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), sizeof(float) * v.size());
  return a;
}

struct PySequential {
  oracle::Sequential seq;
  PySequential(const std::string& layer_specs_json, size_t x_size, bool exact) : seq(Json::parse(layer_specs_json), x_size, exact) {}
  farray forward(const farray& params, const farray& x, size_t B) {
    if ((size_t)params.size() < seq.n_params()) throw std::invalid_argument("params too short");
    return to_np(seq.forward(params.data(), x.data(), B));
  }
  farray backward(const farray& params, const farray& d, size_t B) {
    std::vector<float> grad(seq.n_params(), 0.f), dd = to_vec(d);
    seq.backward(params.data(), grad.data(), dd, B);
    return to_np(grad);
  }
};

struct PyOptimizer {
  oracle::Optimizer opt;
  size_t n;
  PyOptimizer(const std::string& spec_json, size_t n_) : opt(oracle::OptimizerSpec::from_spec(Json::parse(spec_json)), n_), n(n_) {}
  farray step(const farray& params, const farray& grad) {
    if ((size_t)params.size() != n || (size_t)grad.size() != n) throw std::invalid_argument("size mismatch");
    std::vector<float> p = to_vec(params);
    opt.step(p.data(), grad.data(), n);
    return to_np(p);
  }
};

oracle::Dataset make_dataset(const farray& xs, const farray& ys, size_t x_size, size_t y_size) {
  oracle::Dataset d;
  d.samples = to_vec(xs);
  d.labels = to_vec(ys);
  d.x_size = x_size;
  d.y_size = y_size;
  if (x_size == 0 || y_size == 0 || d.samples.size() % x_size || d.labels.size() % y_size ||
      d.samples.size() / x_size != d.labels.size() / y_size)
    throw std::invalid_argument("samples/labels do not describe the same number of rows");
  return d;
}

struct PyRoundTrainer {
  oracle::RoundTrainer t;
  PyRoundTrainer(const std::string& spec_json, const farray& xs, const farray& ys, bool exact)
      : t(Json::parse(spec_json),
          make_dataset(xs, ys, (size_t)Json::parse(spec_json).at("dataset").at("x_size").as_u64(),
                       (size_t)Json::parse(spec_json).at("dataset").at("y_size").as_u64()),
          exact) {}
  // returns (params, residual, losses, is_last)
  py::tuple train(const farray& params, const farray& residual) {
    std::vector<float> p = to_vec(params), r = to_vec(residual);
    if (p.size() < t.n_params() || r.size() < t.n_params()) throw std::invalid_argument("buffers too short");
    oracle::TrainResult res;
    {
      py::gil_scoped_release rel;
      res = t.train(p.data(), r.data());
    }
    return py::make_tuple(to_np(p), to_np(r), res.losses, res.is_last);
  }
  py::tuple evaluate(const farray& params, const farray& xs, const farray& ys) {
    auto d = make_dataset(xs, ys, t.dataset().x_size, t.dataset().y_size);
    auto r = t.evaluate(params.data(), d);
    return py::make_tuple(r.first, r.second);
  }
};

struct PyCluster {
  std::unique_ptr<oracle::LocalCluster> c;
  PyCluster(const std::string& plan_json, const farray& xs, const farray& ys, size_t x_size, size_t y_size,
            const std::string& wire, bool sparse, double r, bool exact, bool resets, py::object init_m, py::object init_v,
            float init_b1t, float init_b2t, size_t start_epoch, size_t checkpoint_every) {
    oracle::ClusterOptions o;
    o.wire = wire;
    o.sparse = sparse;
    o.sparse_r = r;
    o.leaky_relu_exact = exact;
    o.switch_resets_progress = resets;
    if (!init_m.is_none()) { auto a = init_m.cast<farray>(); o.init_m.assign(a.data(), a.data() + a.size()); }
    if (!init_v.is_none()) { auto a = init_v.cast<farray>(); o.init_v.assign(a.data(), a.data() + a.size()); }
    o.init_b1t = init_b1t;
    o.init_b2t = init_b2t;
    o.start_epoch = start_epoch;
    o.checkpoint_every = checkpoint_every;
    c = std::make_unique<oracle::LocalCluster>(Json::parse(plan_json), make_dataset(xs, ys, x_size, y_size), o);
  }
  py::object next_event(int timeout_ms) {
    oracle::ClusterEvent ev;
    bool ok;
    {
      py::gil_scoped_release rel;
      ok = c->next_event(ev, timeout_ms);
    }
    if (!ok) return py::none();
    py::dict d;
    d["kind"] = ev.kind;
    d["worker"] = ev.worker;
    d["losses"] = ev.losses;
    d["text"] = ev.text;
    return d;
  }
  void join() {
    py::gil_scoped_release rel;
    c->join();
  }
};

}  // namespace

void bind_core(py::module_& m);

PYBIND11_MODULE(_orchestra, m) {
  m.doc() = "C++ control plane, CPU oracle engine and in-process CPU cluster of the B200 orchestra runtime";
  py::register_exception<InvalidConfig>(m, "InvalidConfig", PyExc_ValueError);
  bind_core(m);

  // ---- oracle engine ----
  py::class_<PySequential>(m, "Sequential")
      .def(py::init<const std::string&, size_t, bool>(), py::arg("layer_specs_json"), py::arg("x_size"), py::arg("leaky_relu_exact") = true)
      .def("forward", &PySequential::forward)
      .def("backward", &PySequential::backward)
      .def_property_readonly("n_params", [](PySequential& s) { return s.seq.n_params(); })
      .def_property_readonly("layer_offsets", [](PySequential& s) { return s.seq.layer_offsets(); });
  m.def("loss_prime", [](const std::string& kind, const farray& yp, const farray& y) {
    std::vector<float> delta;
    const double l = oracle::loss_prime(kind == "mse" ? oracle::Loss::Mse : oracle::Loss::CrossEntropy, yp.data(), y.data(), (size_t)yp.size(), delta);
    return py::make_tuple(l, to_np(delta));
  });
  py::class_<PyOptimizer>(m, "Optimizer").def(py::init<const std::string&, size_t>()).def("step", &PyOptimizer::step);
  m.def("param_gen_fill", [](const std::string& spec_json, uint64_t seed) {
    std::vector<float> v;
    oracle::param_gen_fill(Json::parse(spec_json), seed, v);
    return to_np(v);
  });
  m.def("philox_sample", [](uint64_t index, uint64_t seed, int kind, float a, float b) { return philox_sample(index, seed, kind, a, b); });
  m.def("shuffle_dataset", [](const farray& xs, const farray& ys, size_t x_size, size_t y_size, uint64_t seed, uint64_t epoch) {
    auto d = make_dataset(xs, ys, x_size, y_size);
    d.shuffle(seed, epoch);
    return py::make_tuple(to_np(d.samples), to_np(d.labels));
  });
  py::class_<PyRoundTrainer>(m, "RoundTrainer")
      .def(py::init<const std::string&, const farray&, const farray&, bool>(), py::arg("trainer_spec_json"), py::arg("samples"), py::arg("labels"), py::arg("leaky_relu_exact") = true)
      .def("train", &PyRoundTrainer::train)
      .def("evaluate", &PyRoundTrainer::evaluate)
      .def_property_readonly("n_params", [](PyRoundTrainer& t) { return t.t.n_params(); })
      .def_property_readonly("epochs_done", [](PyRoundTrainer& t) { return t.t.epochs_done(); });
  py::class_<PyCluster>(m, "LocalCluster")
      .def(py::init<const std::string&, const farray&, const farray&, size_t, size_t, const std::string&, bool, double, bool, bool,
                    py::object, py::object, float, float, size_t, size_t>(),
           py::arg("plan_json"), py::arg("samples"), py::arg("labels"), py::arg("x_size"), py::arg("y_size"),
           py::arg("wire") = "f32", py::arg("sparse") = false, py::arg("sparse_r") = 0.0,
           py::arg("leaky_relu_exact") = true, py::arg("switch_resets_progress") = false,
           py::arg("init_m") = py::none(), py::arg("init_v") = py::none(), py::arg("init_b1t") = 1.0f, py::arg("init_b2t") = 1.0f,
           py::arg("start_epoch") = 0, py::arg("checkpoint_every") = 0)
      .def("start", [](PyCluster& c) { c.c->start(); })
      .def("request_stop", [](PyCluster& c) { c.c->request_stop(); })
      .def("next_event", &PyCluster::next_event, py::arg("timeout_ms") = 100)
      .def("join", &PyCluster::join)
      .def("finished", [](PyCluster& c) { return c.c->finished(); })
      .def("switched", [](PyCluster& c) { return c.c->switched(); })
      .def("stop_reason", [](PyCluster& c) { return c.c->stop_reason(); })
      .def("final_params", [](PyCluster& c) { return to_np(c.c->final_params()); })
      .def("pop_checkpoint", [](PyCluster& c) -> py::object {
        std::vector<float> params;
        oracle::ClusterState st;
        if (!c.c->pop_checkpoint(params, st)) return py::none();
        py::dict d;
        d["params"] = to_np(params);
        d["m"] = to_np(st.m);
        d["v"] = to_np(st.v);
        d["adam_pows"] = py::make_tuple(st.b1t, st.b2t);
        d["epochs"] = st.epochs;
        return d;
      })
      .def("final_state", [](PyCluster& c) {
        const auto& st = c.c->final_state();
        py::dict d;
        d["m"] = to_np(st.m);
        d["v"] = to_np(st.v);
        d["adam_pows"] = py::make_tuple(st.b1t, st.b2t);
        d["epochs"] = st.epochs;
        return d;
      });
}
