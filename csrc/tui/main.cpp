// orchestui: terminal front-end of the orchestrator.
//
//   orchestui                                       interactive: menu -> config paths -> dashboard
//   orchestui --render-once <model.json> <training.json> [--size WxH] [--no-save]
//                                                   run to completion without a terminal and print the last frame
//
// Screen flow and panels follow the reference's terminal UI (orchestui/src/ui/screens/mod.rs:21-57,
// orchestui/src/app/run.rs:41-70): a menu, a configuration screen with two path prompts (ghost text shows
// the default), and a training dashboard with header, average and per-worker loss charts, workers table
// with progress bar, log panel, parameter panel and a topology panel (ring / servers+workers / after the
// switch), plus stop / quit / save pop-ups. When a run completes the model is saved to
// `safetensors/<adjective>_<term>.safetensors` (orchestui/src/ui/screens/training.rs:480-493) - that
// directory of auto-named checkpoints is the trained-model repository. Events are consumed without
// blocking the UI (training.rs:302-347).
#include <sys/stat.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "core/session.hpp"
#include "tui/term.hpp"

using namespace ono;
using namespace tui;

namespace {

const char* const kAdjectives[] = {"amber", "brisk", "clever", "dapper", "earnest", "feisty", "glad", "humble", "icy", "jaunty",
                                   "keen", "limber", "mellow", "nimble", "opal", "perky", "quiet", "rosy", "sturdy", "tidy",
                                   "upbeat", "vivid", "wiry", "young", "zippy", "ample", "bright", "cozy", "deft", "elfin"};
const char* const kTerms[] = {"tile", "shard", "replica", "barrier", "residual", "minibatch", "stride", "padding", "filter", "logits",
                              "ring", "server", "worker", "window", "bucket", "epoch", "tensor", "kernel", "layer", "neuron",
                              "gradient", "momentum", "plateau", "descent", "softmax", "sigmoid", "pooling", "dense", "switch", "orchestra"};

std::string random_model_name() {
  uint64_t x = (uint64_t)std::chrono::system_clock::now().time_since_epoch().count() | 1;
  auto next = [&] { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return x; };
  const size_t a = next() % (sizeof kAdjectives / sizeof *kAdjectives), t = next() % (sizeof kTerms / sizeof *kTerms);
  return std::string(kAdjectives[a]) + "_" + kTerms[t] + ".safetensors";
}

std::string slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::ostringstream s;
  s << f.rdbuf();
  return s.str();
}

std::string fmt(const char* f, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, f);
  std::vsnprintf(buf, sizeof buf, f, ap);
  va_end(ap);
  return buf;
}

struct WorkerRow {
  size_t epochs = 0;
  double last = std::nan("");
  std::string state = "training";
  std::vector<double> losses;
};

struct Dashboard {
  ModelConfig model;
  TrainingConfig training;
  Json plan;
  std::unique_ptr<Session> session;
  std::unique_ptr<ProgressAggregator> progress;
  std::vector<WorkerRow> workers;
  std::vector<std::string> log;
  std::vector<float> params;
  std::string stop_reason, error, saved_to;
  bool finished = false, switched = false, stop_requested = false;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  double elapsed_s = 0;

  void say(const std::string& s) {
    log.push_back(s);
    if (log.size() > 200) log.erase(log.begin());
  }

  void start(const std::string& model_path, const std::string& training_path) {
    model = ModelConfig::from_json(Json::parse(slurp(model_path)));
    training = TrainingConfig::from_json(Json::parse(slurp(training_path)));
    if (!training.dataset.is_inline) say("dataset: " + training.dataset.samples_path + " (csv/tsv files are converted to .bin once)");
    oracle::Dataset data = load_dataset(training.dataset);
    say(fmt("dataset loaded: %zu rows, %zu features, %zu outputs", data.rows(), data.x_size, data.y_size));
    session = start_session(model, training, std::move(data), &plan);
    workers.assign(session->n_workers(), WorkerRow{});
    progress = std::make_unique<ProgressAggregator>(session->n_workers());
    say(fmt("%s on %zu node(s), %zu worker(s)", plan.at("algorithm").as_string().c_str(), training.addrs.size(), workers.size()));
  }

  // Drain pending events; returns true when something changed.
  bool pump(int wait_ms) {
    if (!session || finished) return false;
    bool changed = false;
    TrainingEvent ev;
    while (session->next_event(ev, wait_ms)) {
      wait_ms = 0;
      changed = true;
      if (ev.kind == "losses") {
        if (ev.worker < workers.size()) {
          auto& w = workers[ev.worker];
          for (double l : ev.losses) { w.losses.push_back(l); w.last = l; ++w.epochs; }
        }
        for (double m : progress->add(ev.worker, ev.losses))
          say(fmt("epoch %zu/%zu avg_loss=%.6f", progress->history().size(), training.max_epochs, m));
      } else if (ev.kind == "switch") {
        switched = true;
        say("switching algorithm to parameter server");
      } else if (ev.kind == "upgrading") {
        if (ev.worker < workers.size()) workers[ev.worker].state = "upgrading";
      } else if (ev.kind == "upgraded") {
        if (ev.worker < workers.size()) workers[ev.worker].state = "server";
        progress->worker_left();
        say(fmt("worker %zu now serves parameters", ev.worker));
      } else if (ev.kind == "worker_done") {
        if (ev.worker < workers.size() && workers[ev.worker].state == "training") workers[ev.worker].state = "done";
      } else if (ev.kind == "error") {
        error = ev.text.empty() ? "worker error" : ev.text;
        say("error: " + error);
      } else if (ev.kind == "complete") {
        stop_reason = ev.text.empty() ? "max_epochs" : ev.text;
        progress->finish();
        finished = true;
        elapsed_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (stop_reason != "error") params = session->final_params();
        for (auto& w : workers) if (w.state == "training") w.state = "done";
        say("training complete: " + stop_reason);
        break;
      }
    }
    if (!finished) elapsed_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return changed;
  }

  std::string save(std::string path) {
    if (params.empty()) return "";
    if (path.empty()) {
      ::mkdir("safetensors", 0755);
      path = "safetensors/" + random_model_name();
    }
    save_safetensors(path, model, training.dataset.x_size, params);
    saved_to = path;
    say("model saved to " + path);
    return path;
  }

  void draw_topology(Canvas& c, int x, int y, int w, int h) const {
    c.box(x, y, w, h, "topology");
    const std::string algo = plan.is_object() ? plan.at("algorithm").as_string() : "";
    const bool ps_now = algo == "parameter_server" || switched;
    int row = y + 1;
    auto line = [&](const std::string& s, int color = DEFAULT) { if (row < y + h - 1) c.text(x + 2, row++, s, color, false, w - 4); };
    if (!plan.is_object()) return;
    if (!ps_now) {
      std::string ring;
      for (auto& wk : plan.at("workers").items()) ring += fmt("w%llu → ", wk.at("rank").as_u64());
      if (!ring.empty()) ring += fmt("w%llu", plan.at("workers")[0].at("rank").as_u64());
      line("ring all-reduce (order of the tour)", CYAN);
      line(ring);
      line("reduce-scatter ⟶ all-gather ⟶ average ⟶ optimizer on every replica", GREY);
      if (algo == "strategy_switch") line("watching the plateau test: switch promotes servers", YELLOW);
    } else {
      line(switched ? "parameter server (after the switch)" : "parameter server", CYAN);
      std::string servers, wk;
      if (const Json* sv = plan.find("servers"))
        for (auto& s : sv->items()) servers += fmt("[S%llu] ", s.at("rank").as_u64());
      for (auto& w_ : plan.at("workers").items()) {
        const size_t r = (size_t)w_.at("rank").as_u64();
        bool is_server = false;
        if (const Json* sv = plan.find("servers"))
          for (auto& s : sv->items()) is_server = is_server || s.at("rank").as_u64() == r;
        if (!(switched && is_server && !training.b200.colocate)) wk += fmt("(w%zu) ", r);
      }
      line("servers: " + servers, GREEN);
      line("   ⇅ push residual / pull parameters (every worker ↔ every server)", GREY);
      line("workers: " + wk);
    }
  }

  void draw(Canvas& c) const {
    c.clear();
    const int W = c.width(), H = c.height();
    const std::string algo = plan.is_object() ? plan.at("algorithm").as_string() : "-";
    c.box(0, 0, W, 3, "oxidized neural orchestra · B200");
    c.text(2, 1, fmt("strategy %s%s   nodes %zu   batch %zu   epochs %zu   elapsed %.1fs   %s", algo.c_str(), switched ? " → parameter_server" : "",
                     training.addrs.size(), training.batch_size, training.max_epochs, elapsed_s,
                     finished ? ("finished: " + stop_reason).c_str() : stop_requested ? "stopping after this round" : "training"),
           finished ? GREEN : DEFAULT, true, W - 4);
    const int top = 3, bottom_h = std::max(7, H / 3), mid_h = H - top - bottom_h - 1;
    const int left_w = W * 3 / 5;
    // charts
    c.box(0, top, left_w, mid_h, "average loss");
    const auto& hist = progress ? progress->history() : std::vector<double>{};
    if (!hist.empty()) {
      c.chart(2, top + 1, left_w - 4, mid_h - 3, hist, GREEN);
      c.text(2, top + mid_h - 2, fmt("epoch %zu  loss %.6f  (first %.6f)", hist.size(), hist.back(), hist.front()), GREY, false, left_w - 4);
    } else c.text(2, top + 1, "waiting for the first round…", GREY);
    // workers table
    c.box(left_w, top, W - left_w, mid_h, "workers");
    c.text(left_w + 2, top + 1, "id  state      epochs  last loss   trend", CYAN, false, W - left_w - 4);
    for (size_t i = 0; i < workers.size() && (int)i < mid_h - 5; ++i) {
      const auto& w = workers[i];
      c.text(left_w + 2, top + 2 + (int)i, fmt("%-3zu %-10s %-7zu %-11.6f", i, w.state.c_str(), w.epochs, w.last),
             w.state == "server" ? YELLOW : w.state == "done" ? GREEN : DEFAULT, false, 36);
      if (!w.losses.empty() && W - left_w - 42 > 4) c.chart(left_w + 39, top + 2 + (int)i, W - left_w - 42, 1, w.losses, BLUE);
    }
    size_t done_epochs = hist.size();
    c.text(left_w + 2, top + mid_h - 3, fmt("progress %zu/%zu", done_epochs, training.max_epochs), GREY);
    c.bar(left_w + 2, top + mid_h - 2, W - left_w - 4, training.max_epochs ? (double)done_epochs / (double)training.max_epochs : 0.0,
          finished ? GREEN : CYAN);
    // bottom row: log | params | topology
    const int by = top + mid_h, lw = W * 2 / 5, pw = W / 5, tw = W - lw - pw;
    c.box(0, by, lw, bottom_h, "log");
    const int rows = bottom_h - 2;
    for (int i = 0; i < rows; ++i) {
      const int idx = (int)log.size() - rows + i;
      if (idx >= 0) c.text(2, by + 1 + i, log[(size_t)idx], log[(size_t)idx].rfind("error", 0) == 0 ? RED : DEFAULT, false, lw - 4);
    }
    c.box(lw, by, pw, bottom_h, "parameters");
    size_t n_params = plan.is_object() ? (size_t)plan.at("n_params").as_u64() : 0;
    c.text(lw + 2, by + 1, fmt("%zu values", n_params), DEFAULT, false, pw - 4);
    c.text(lw + 2, by + 2, fmt("%zu layers", model.layers.size()), GREY, false, pw - 4);
    if (!params.empty()) {
      double sq = 0;
      for (float v : params) sq += (double)v * v;
      c.text(lw + 2, by + 3, fmt("|θ| = %.4f", std::sqrt(sq)), DEFAULT, false, pw - 4);
      for (int i = 0; i < rows - 4 && (size_t)i < params.size(); ++i) c.text(lw + 2, by + 4 + i, fmt("θ[%d] % .5f", i, params[(size_t)i]), GREY, false, pw - 4);
    }
    if (!saved_to.empty()) c.text(lw + 2, by + bottom_h - 2, "saved", GREEN, true, pw - 4);
    draw_topology(c, lw + pw, by, tw, bottom_h);
    c.text(1, H - 1, finished ? "[w] save as…  [m] menu  [q] quit" : "[s] stop after this round  [q] quit", GREY, false, W - 2);
  }
};

void popup(Canvas& c, const std::string& title, const std::vector<std::string>& lines) {
  int w = (int)title.size() + 6;
  for (auto& l : lines) w = std::max(w, (int)l.size() + 4);
  w = std::min(w, c.width() - 2);
  const int h = (int)lines.size() + 2, x = (c.width() - w) / 2, y = (c.height() - h) / 2;
  for (int j = 0; j < h; ++j) for (int i = 0; i < w; ++i) c.put(x + i, y + j, " ");
  c.box(x, y, w, h, title, YELLOW);
  for (size_t i = 0; i < lines.size(); ++i) c.text(x + 2, y + 1 + (int)i, lines[i], DEFAULT, false, w - 4);
}

int render_once(int argc, char** argv) {
  std::string model_path, training_path;
  int W = 110, H = 34;
  bool save = true;
  for (int i = 2; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--size" && i + 1 < argc) { std::sscanf(argv[++i], "%dx%d", &W, &H); }
    else if (a == "--no-save") save = false;
    else if (model_path.empty()) model_path = a;
    else training_path = a;
  }
  if (training_path.empty()) { std::fputs("usage: orchestui --render-once <model.json> <training.json> [--size WxH] [--no-save]\n", stderr); return 2; }
  Dashboard d;
  d.start(model_path, training_path);
  while (!d.finished) d.pump(200);
  if (save && d.stop_reason != "error") d.save("");
  Canvas c(W, H);
  d.draw(c);
  std::cout << c.plain();
  return d.stop_reason == "error" ? 1 : 0;
}

struct Field {
  std::string label, value, ghost;
};

int interactive() {
  Terminal term;
  if (!term.is_tty()) {
    std::fputs("orchestui needs a terminal (or use --render-once <model.json> <training.json>)\n", stderr);
    return 2;
  }
  enum Screen { MENU, CONFIG, TRAINING } screen = MENU;
  int menu_sel = 0, field_sel = 0;
  Field fields[2] = {{"model config", "", "model.json"}, {"training config", "", "training.json"}};
  std::string config_error;
  std::unique_ptr<Dashboard> dash;
  enum Popup { NONE, CONFIRM_STOP, CONFIRM_QUIT, SAVE_AS } pop = NONE;
  std::string save_path;
  const char* menu_items[] = {"Start training", "Repository", "Quit"};
  while (true) {
    int W, H;
    term.size(W, H);
    Canvas c(W, H);
    if (screen == MENU) {
      c.box(0, 0, W, H, "oxidized neural orchestra");
      c.text(W / 2 - 18, H / 2 - 4, "distributed training on B200 ranks", CYAN, true);
      for (int i = 0; i < 3; ++i) c.text(W / 2 - 10, H / 2 - 1 + i, std::string(i == menu_sel ? "› " : "  ") + menu_items[i], i == menu_sel ? GREEN : DEFAULT, i == menu_sel);
      c.text(2, H - 2, "↑/↓ select   enter confirm   q quit", GREY);
    } else if (screen == CONFIG) {
      c.box(0, 0, W, H, "configuration");
      for (int i = 0; i < 2; ++i) {
        c.text(4, 3 + 4 * i, fields[i].label + ":", i == field_sel ? GREEN : DEFAULT, true);
        c.box(4, 4 + 4 * i, W - 8, 3, "", i == field_sel ? GREEN : GREY);
        if (fields[i].value.empty()) c.text(6, 5 + 4 * i, fields[i].ghost, GREY, false, W - 12);
        else c.text(6, 5 + 4 * i, fields[i].value, DEFAULT, false, W - 12);
      }
      c.text(4, 12, "model.json    { \"layers\": [ { \"dense\": { \"output_size\": 128, \"init\": \"kaiming\", \"act_fn\": { \"relu\": { \"slope\": 0.0 } } } }, … ] }", GREY, false, W - 8);
      c.text(4, 13, "training.json { \"addrs\": [\"gpu:0\", …] | [\"host:port\", …] | [\"cpu:0\", …], \"algorithm\": \"all_reduce\" | { \"parameter_server\": {…} }, … }", GREY, false, W - 8);
      if (!config_error.empty()) c.text(4, 15, config_error, RED, true, W - 8);
      c.text(2, H - 2, "tab/↑/↓ switch field   enter start   esc back", GREY);
    } else {
      dash->pump(0);
      if (dash->finished && dash->saved_to.empty() && dash->stop_reason != "error" && !dash->params.empty()) dash->save("");
      dash->draw(c);
      if (pop == CONFIRM_STOP) popup(c, "stop training", {"Stop after the current round?", "", "[y] yes    [n] no"});
      if (pop == CONFIRM_QUIT) popup(c, "quit", {dash->finished ? "Leave the dashboard?" : "Training is still running. Quit anyway?", "", "[y] yes    [n] no"});
      if (pop == SAVE_AS) popup(c, "save model", {"path: " + save_path + "▏", "", "enter save    esc cancel"});
    }
    term.write(c.ansi());
    const int k = term.read_key(screen == TRAINING ? 100 : 250);
    if (k == KEY_NONE) continue;
    if (screen == MENU) {
      if (k == KEY_UP) menu_sel = (menu_sel + 2) % 3;
      else if (k == KEY_DOWN) menu_sel = (menu_sel + 1) % 3;
      else if (k == 'q') return 0;
      else if (k == KEY_ENTER) {
        if (menu_sel == 0) { screen = CONFIG; config_error.clear(); }
        else if (menu_sel == 1) config_error = "trained models are kept under ./safetensors/";
        else return 0;
      }
    } else if (screen == CONFIG) {
      Field& f = fields[field_sel];
      if (k == KEY_ESC) screen = MENU;
      else if (k == KEY_TAB || k == KEY_UP || k == KEY_DOWN) field_sel ^= 1;
      else if (k == KEY_BACKSPACE) { if (!f.value.empty()) f.value.pop_back(); }
      else if (k == KEY_ENTER) {
        try {
          dash = std::make_unique<Dashboard>();
          dash->start(fields[0].value.empty() ? fields[0].ghost : fields[0].value, fields[1].value.empty() ? fields[1].ghost : fields[1].value);
          screen = TRAINING;
          pop = NONE;
        } catch (const std::exception& e) { config_error = e.what(); dash.reset(); }
      } else if (k >= 32 && k < 127) f.value.push_back((char)k);
    } else {
      if (pop == CONFIRM_STOP) {
        if (k == 'y') { dash->session->stop(); dash->stop_requested = true; dash->say("stop requested"); }
        if (k == 'y' || k == 'n' || k == KEY_ESC) pop = NONE;
      } else if (pop == CONFIRM_QUIT) {
        if (k == 'y') return 0;
        if (k == 'n' || k == KEY_ESC) pop = NONE;
      } else if (pop == SAVE_AS) {
        if (k == KEY_ESC) pop = NONE;
        else if (k == KEY_BACKSPACE) { if (!save_path.empty()) save_path.pop_back(); }
        else if (k == KEY_ENTER) { try { dash->save(save_path); } catch (const std::exception& e) { dash->say(std::string("error: ") + e.what()); } pop = NONE; }
        else if (k >= 32 && k < 127) save_path.push_back((char)k);
      } else {
        if (k == 's' && !dash->finished) pop = CONFIRM_STOP;
        else if (k == 'q') pop = CONFIRM_QUIT;
        else if (k == 'w' && dash->finished) { pop = SAVE_AS; save_path = dash->saved_to; }
        else if (k == 'm' && dash->finished) { screen = MENU; dash.reset(); }
      }
    }
  }
}

}  // namespace

int main(int argc, char** argv) {
  try {
    if (argc >= 2 && std::strcmp(argv[1], "--render-once") == 0) return render_once(argc, argv);
    if (argc >= 2 && (std::strcmp(argv[1], "-h") == 0 || std::strcmp(argv[1], "--help") == 0)) {
      std::puts("usage: orchestui | orchestui --render-once <model.json> <training.json> [--size WxH] [--no-save]");
      return 0;
    }
    return interactive();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "orchestui: %s\n", e.what());
    return 1;
  }
}
