// ono-orchestrator: headless training run from two JSON documents.
//
//   ono-orchestrator <model.json> <training.json> [--save out.safetensors] [--events] [--quiet]
//
// The counterpart of the reference's headless orchestrator binary (orchestrator/src/main.rs:208-291) with
// the configuration read from the same model.json / training.json documents the terminal UI loads
// (orchestui/src/config/json.rs:29-64). Addresses `cpu:<i>` train in this process; `host:port` addresses
// are nodes that are already listening. Progress goes to stderr as `epoch i/N avg_loss=...` lines
// (orchestra-py/src/session.rs:49-189); `--events` prints every raw event as one JSON line on stdout.
#include <csignal>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>

#include "core/session.hpp"

using namespace ono;

namespace {
std::atomic<bool> g_stop{false};
void on_sigint(int) { g_stop = true; }

std::string slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::ostringstream s;
  s << f.rdbuf();
  return s.str();
}
}  // namespace

int main(int argc, char** argv) {
  std::string model_path, training_path, save_path;
  bool raw_events = false, quiet = false;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--save" && i + 1 < argc) save_path = argv[++i];
    else if (a == "--events") raw_events = true;
    else if (a == "--quiet") quiet = true;
    else if (a == "-h" || a == "--help") {
      std::puts("usage: ono-orchestrator <model.json> <training.json> [--save out.safetensors] [--events] [--quiet]");
      return 0;
    } else if (model_path.empty()) model_path = a;
    else if (training_path.empty()) training_path = a;
    else { std::fprintf(stderr, "unexpected argument %s\n", a.c_str()); return 2; }
  }
  if (model_path.empty() || training_path.empty()) {
    std::fputs("usage: ono-orchestrator <model.json> <training.json> [--save out.safetensors] [--events] [--quiet]\n", stderr);
    return 2;
  }
  try {
    const ModelConfig model = ModelConfig::from_json(Json::parse(slurp(model_path)));
    const TrainingConfig training = TrainingConfig::from_json(Json::parse(slurp(training_path)));
    oracle::Dataset data = load_dataset(training.dataset);
    auto session = start_session(model, training, std::move(data));
    std::signal(SIGINT, on_sigint);
    ProgressAggregator progress(session->n_workers());
    std::string stop_reason = "max_epochs", error;
    bool stop_sent = false;
    auto report = [&](const std::vector<double>& fresh) {
      if (quiet) return;
      for (size_t i = 0; i < fresh.size(); ++i)
        std::fprintf(stderr, "epoch %zu/%zu avg_loss=%.6f\n", progress.history().size() - fresh.size() + i + 1,
                     training.max_epochs, fresh[i]);
    };
    while (true) {
      if (g_stop && !stop_sent) { session->stop(); stop_sent = true; }
      TrainingEvent ev;
      if (!session->next_event(ev, 200)) continue;
      if (raw_events) {
        Json j = Json::object();
        j.set("kind", ev.kind);
        j.set("worker", Json((unsigned long long)ev.worker));
        Json l = Json::array();
        for (double v : ev.losses) l.push(Json(v));
        j.set("losses", l);
        j.set("text", ev.text);
        std::cout << j.dump() << std::endl;
      }
      if (ev.kind == "losses") report(progress.add(ev.worker, ev.losses));
      else if (ev.kind == "upgraded") report(progress.worker_left());
      else if (ev.kind == "switch" && !quiet) std::fputs("switching algorithm to parameter server\n", stderr);
      else if (ev.kind == "error") error = ev.text.empty() ? "worker error" : ev.text;
      else if (ev.kind == "complete") { if (!ev.text.empty()) stop_reason = ev.text; break; }
    }
    report(progress.finish());
    if (stop_reason == "error") {
      std::fprintf(stderr, "training failed: %s\n", error.c_str());
      return 1;
    }
    const std::vector<float> params = session->final_params();
    if (!quiet) std::fprintf(stderr, "training complete: %s, %zu parameters%s\n", stop_reason.c_str(), params.size(),
                             session->switched() ? ", strategy switched" : "");
    if (!save_path.empty()) {
      save_safetensors(save_path, model, training.dataset.x_size, params);
      if (!quiet) std::fprintf(stderr, "saved %s\n", save_path.c_str());
    }
    Json out = Json::object();
    out.set("stop_reason", stop_reason);
    out.set("n_params", Json((unsigned long long)params.size()));
    Json h = Json::array();
    for (double v : progress.history()) h.push(Json(v));
    out.set("loss_history", h);
    out.set("switched", session->switched());
    out.set("metrics", session->run_metrics());
    if (!raw_events) std::cout << out.dump() << std::endl;
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ono-orchestrator: %s\n", e.what());
    return 1;
  }
}
