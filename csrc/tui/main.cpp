// orchestui: terminal front-end of the orchestrator.
//
//   orchestui                                       interactive: menu -> config paths -> dashboard
//   orchestui --render-once <model.json> <training.json> [--size WxH] [--no-save]
//                                                   run to completion without a terminal and print the last frame
//   orchestui --script "<keys>" [--size WxH]        drive the interactive screens from a key script instead of a terminal
//                                                   (tokens: <enter> <esc> <up> <down> <left> <right> <tab> <bs> <wait> <dump>);
//                                                   every <dump> prints the current frame as plain text
//
// Screen flow and panels follow the reference's terminal UI (orchestui/src/ui/screens/mod.rs:21-57,
// orchestui/src/app/run.rs:41-70): a menu, a configuration screen with two path prompts (ghost text shows
// the default), and a training dashboard with header, average and per-worker loss charts, workers table
// with progress bar, log panel, parameter panel and a topology panel (ring / servers+workers / after the
// switch), plus stop / quit / save pop-ups. When a run completes the model is saved to
// `safetensors/<adjective>_<term>.safetensors` (orchestui/src/ui/screens/training.rs:480-493) - that
// directory of auto-named checkpoints is the trained-model repository. Events are consumed without
// blocking the UI (training.rs:302-347).
#include <dirent.h>
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
  mutable unsigned frame = 0;      // drives the flow animation of the topology panel
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

  // Topology panel (orchestui/src/ui/components/topology.rs:46-630): the nodes of the current strategy and the traffic
  // between them, animated while training runs. Ring: the workers in tour order with a packet circulating (reduce-scatter
  // then all-gather). Parameter server: servers above, workers below, residuals going up and parameters coming down.
  void draw_topology(Canvas& c, int x, int y, int w, int h) const {
    c.box(x, y, w, h, "topology");
    if (!plan.is_object()) return;
    const std::string algo = plan.at("algorithm").as_string();
    const bool ps_now = algo == "parameter_server" || switched;
    const bool live = !finished;
    const int ix = x + 2, iw = w - 4, iy = y + 1, ih = h - 2;
    if (iw < 12 || ih < 3) return;
    std::vector<size_t> wr, sr;
    for (auto& wk : plan.at("workers").items()) wr.push_back((size_t)wk.at("rank").as_u64());
    if (const Json* sv = plan.find("servers")) for (auto& s_ : sv->items()) sr.push_back((size_t)s_.at("rank").as_u64());
    if (!ps_now) {
      c.text(ix, iy, "ring all-reduce", CYAN, false, iw);
      // nodes laid out on the two long sides of a rectangle, in tour order, arrows along the perimeter
      const size_t n = wr.size();
      const size_t top_n = (n + 1) / 2, bot_n = n - top_n;
      const int step = std::max(5, iw / (int)std::max<size_t>(top_n, 1));
      const int ty = iy + 1, by_ = std::min(iy + ih - 2, iy + 3);
      std::vector<std::pair<int, int>> pos(n);
      for (size_t i = 0; i < top_n; ++i) pos[i] = {ix + (int)i * step, ty};
      for (size_t i = 0; i < bot_n; ++i) pos[top_n + i] = {ix + (int)(top_n - 1 - i) * step - (top_n > bot_n && i == 0 ? 0 : 0), by_};
      const size_t phase = n ? (frame / 2) % (2 * n) : 0;        // 2n hops per round: n-1 scatter, n-1 gather, 2 for the update
      for (size_t i = 0; i < n; ++i) {
        const bool hot = live && (phase % n) == i;
        c.text(pos[i].first, pos[i].second, fmt("w%zu", wr[i]), hot ? YELLOW : DEFAULT, hot, 4);
        const size_t j = (i + 1) % n;
        if (n > 1 && pos[i].second == pos[j].second) {
          const int a = std::min(pos[i].first, pos[j].first) + 3, b = std::max(pos[i].first, pos[j].first) - 1;
          for (int q = a; q <= b; ++q) c.put(q, pos[i].second, pos[i].first < pos[j].first ? "→" : "←", hot ? YELLOW : GREY);
        } else if (n > 1) {
          for (int q = std::min(pos[i].second, pos[j].second) + 1; q < std::max(pos[i].second, pos[j].second); ++q)
            c.put(pos[i].first + 1, q, pos[i].second < pos[j].second ? "↓" : "↑", hot ? YELLOW : GREY);
        }
      }
      if (ih >= 5)
        c.text(ix, iy + ih - 1, !live ? "idle" : phase < n ? "reduce-scatter: partial sums travel the ring" : "all-gather: fresh parameters travel the ring",
               GREY, false, iw);
      if (algo == "strategy_switch" && ih >= 6) c.text(ix, iy + ih - 2, "plateau test armed: switch promotes servers", YELLOW, false, iw);
    } else {
      c.text(ix, iy, switched ? "parameter server (after the switch)" : "parameter server", CYAN, false, iw);
      std::vector<size_t> pure_workers;
      for (size_t r : wr) {
        const bool is_server = std::find(sr.begin(), sr.end(), r) != sr.end();
        if (!(is_server && !training.b200.colocate)) pure_workers.push_back(r);
      }
      const int sstep = std::max(6, iw / (int)std::max<size_t>(sr.size(), 1)), wstep = std::max(5, iw / (int)std::max<size_t>(pure_workers.size(), 1));
      const int sy = iy + 1, wy = std::min(iy + ih - 2, iy + 4);
      for (size_t i = 0; i < sr.size(); ++i) c.text(ix + (int)i * sstep, sy, fmt("[S%zu]", sr[i]), GREEN, true, 6);
      const bool push = (frame / 3) % 2 == 0;
      for (size_t i = 0; i < pure_workers.size(); ++i) {
        const int wx = ix + (int)i * wstep;
        c.text(wx, wy, fmt("(w%zu)", pure_workers[i]), DEFAULT, false, 6);
        if (live) {
          const int span = wy - sy - 1;
          if (span > 0) {
            const int at = push ? wy - 1 - (int)(frame % (unsigned)span) : sy + 1 + (int)(frame % (unsigned)span);
            c.put(wx + 2, at, push ? "↑" : "↓", push ? YELLOW : CYAN);
          }
        }
      }
      if (ih >= 6)
        c.text(ix, iy + ih - 1, !live ? "idle" : push ? "push: residuals to the owners of each shard" : "pull: fresh parameters to every worker", GREY, false, iw);
    }
    ++frame;
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

// The trained-model repository: every *.safetensors under ./safetensors with its size and tensors.
struct RepoEntry {
  std::string name;
  long long bytes = 0;
  std::vector<std::string> tensors;      // "layer_0.weight [784, 128]"
};

std::vector<RepoEntry> scan_repository() {
  std::vector<RepoEntry> out;
  DIR* d = ::opendir("safetensors");
  if (!d) return out;
  while (dirent* e = ::readdir(d)) {
    const std::string n = e->d_name;
    if (n.size() < 13 || n.substr(n.size() - 12) != ".safetensors") continue;
    RepoEntry r;
    r.name = n;
    struct stat st{};
    if (::stat(("safetensors/" + n).c_str(), &st) == 0) r.bytes = (long long)st.st_size;
    try {
      for (auto& t : load_safetensors("safetensors/" + n)) {
        std::string shape;
        for (size_t i = 0; i < t.shape.size(); ++i) shape += (i ? ", " : "") + std::to_string(t.shape[i]);
        r.tensors.push_back(t.name + " [" + shape + "]");
      }
    } catch (const std::exception& ex) { r.tensors.push_back(std::string("unreadable: ") + ex.what()); }
    out.push_back(std::move(r));
  }
  ::closedir(d);
  std::sort(out.begin(), out.end(), [](const RepoEntry& a, const RepoEntry& b) { return a.name < b.name; });
  return out;
}

// Inline examples of the two documents, one pair per strategy (the configuration screen cycles through them).
struct Example { const char* title; std::vector<const char*> lines; };
const Example kExamples[] = {
  {"all-reduce on four GPUs, bf16 tiles, one exchange per step",
   {"model.json     { \"layers\": [ { \"dense\": { \"output_size\": 4096, \"init\": \"kaiming\", \"act_fn\": { \"relu\": { \"slope\": 0.0 } } } },",
    "                               { \"dense\": { \"output_size\": 10, \"init\": \"xavier_uniform\", \"act_fn\": \"softmax\" } } ] }",
    "training.json  { \"addrs\": [\"gpu:0\", \"gpu:1\", \"gpu:2\", \"gpu:3\"], \"algorithm\": \"all_reduce\",",
    "                 \"dataset\": { \"src\": { \"local\": { \"samples_path\": \"x.bin\", \"labels_path\": \"y.bin\" } }, \"x_size\": 784, \"y_size\": 10 },",
    "                 \"optimizer\": { \"adam\": { \"lr\": 0.001 } }, \"loss_fn\": \"cross_entropy\", \"batch_size\": 1024, \"max_epochs\": 10,",
    "                 \"b200\": { \"sync_every\": \"step\", \"tile_dtype\": \"bf16\" } }"}},
  {"parameter server: two servers, blocking store, barrier synchroniser",
   {"training.json  { \"addrs\": [\"host-a:4000\", \"host-b:4000\", \"host-c:4000\", \"host-d:4000\"],",
    "                 \"algorithm\": { \"parameter_server\": { \"nservers\": 2, \"synchronizer\": \"barrier\", \"store\": \"blocking\" } },",
    "                 \"optimizer\": { \"gradient_descent_with_momentum\": { \"lr\": 0.01, \"mu\": 0.9 } }, \"offline_epochs\": 0,",
    "                 \"serializer\": { \"sparse_capable\": { \"r\": 0.01 } }, … }"}},
  {"strategy switch: all-reduce until the loss plateaus, then two ranks become servers",
   {"training.json  { \"addrs\": [\"cpu:0\", \"cpu:1\", \"cpu:2\", \"cpu:3\"],",
    "                 \"algorithm\": { \"strategy_switch\": { \"nservers\": 2, \"synchronizer\": \"barrier\", \"store\": \"blocking\" } },",
    "                 \"early_stopping\": { \"tolerance\": 1e-4 }, \"b200\": { \"switch_window\": 6, \"switch_threshold\": 0.01 }, … }"}},
};

int interactive(Console& term) {
  if (!term.usable()) {
    std::fputs("orchestui needs a terminal (or use --render-once <model.json> <training.json>)\n", stderr);
    return 2;
  }
  enum Screen { MENU, CONFIG, TRAINING, REPOSITORY } screen = MENU;
  int menu_sel = 0, field_sel = 0, repo_sel = 0, example = 0;
  Field fields[2] = {{"model config", "", "model.json"}, {"training config", "", "training.json"}};
  std::string config_error;
  std::unique_ptr<Dashboard> dash;
  std::vector<RepoEntry> repo;
  enum Popup { NONE, CONFIRM_STOP, CONFIRM_QUIT, SAVE_AS } pop = NONE;
  std::string save_path;
  const char* menu_items[] = {"Start training", "Repository", "Quit"};
  const int n_examples = (int)(sizeof kExamples / sizeof *kExamples);
  while (true) {
    int W, H;
    term.size(W, H);
    Canvas c(W, H);
    if (screen == MENU) {
      c.box(0, 0, W, H, "oxidized neural orchestra");
      c.text(W / 2 - 18, H / 2 - 4, "distributed training on B200 ranks", CYAN, true);
      for (int i = 0; i < 3; ++i) c.text(W / 2 - 10, H / 2 - 1 + i, std::string(i == menu_sel ? "› " : "  ") + menu_items[i], i == menu_sel ? GREEN : DEFAULT, i == menu_sel);
      c.text(2, H - 2, "↑/↓ select   enter confirm   q quit", GREY);
    } else if (screen == REPOSITORY) {
      c.box(0, 0, W, H, "trained-model repository · ./safetensors");
      if (repo.empty()) c.text(4, 3, "no saved models yet: a finished run is saved here under a generated name", GREY, false, W - 8);
      const int list_w = std::max(30, W * 2 / 5);
      for (int i = 0; i < (int)repo.size() && i < H - 6; ++i)
        c.text(3, 2 + i, fmt("%s %-28s %9.1f KB", i == repo_sel ? "›" : " ", repo[(size_t)i].name.c_str(), (double)repo[(size_t)i].bytes / 1024.0),
               i == repo_sel ? GREEN : DEFAULT, i == repo_sel, list_w);
      if (!repo.empty()) {
        const RepoEntry& r = repo[(size_t)repo_sel];
        c.box(list_w + 4, 1, W - list_w - 6, H - 4, r.name);
        for (int i = 0; i < (int)r.tensors.size() && i < H - 7; ++i) c.text(list_w + 6, 2 + i, r.tensors[(size_t)i], DEFAULT, false, W - list_w - 10);
      }
      c.text(2, H - 2, "↑/↓ select   esc back", GREY);
    } else if (screen == CONFIG) {
      c.box(0, 0, W, H, "configuration");
      for (int i = 0; i < 2; ++i) {
        c.text(4, 3 + 4 * i, fields[i].label + ":", i == field_sel ? GREEN : DEFAULT, true);
        c.box(4, 4 + 4 * i, W - 8, 3, "", i == field_sel ? GREEN : GREY);
        if (fields[i].value.empty()) c.text(6, 5 + 4 * i, fields[i].ghost, GREY, false, W - 12);
        else c.text(6, 5 + 4 * i, fields[i].value, DEFAULT, false, W - 12);
      }
      const Example& ex = kExamples[example];
      c.text(4, 12, fmt("example %d/%d: %s", example + 1, n_examples, ex.title), CYAN, true, W - 8);
      for (size_t i = 0; i < ex.lines.size() && 13 + (int)i < H - 4; ++i) c.text(4, 13 + (int)i, ex.lines[i], GREY, false, W - 8);
      if (!config_error.empty()) c.text(4, H - 4, config_error, RED, true, W - 8);
      c.text(2, H - 2, "tab/↑/↓ switch field   ←/→ other example   enter start   esc back", GREY);
    } else {
      dash->pump(0);
      if (dash->finished) term.finished_now();
      if (dash->finished && dash->saved_to.empty() && dash->stop_reason != "error" && !dash->params.empty()) dash->save("");
      dash->draw(c);
      if (pop == CONFIRM_STOP) popup(c, "stop training", {"Stop after the current round?", "", "[y] yes    [n] no"});
      if (pop == CONFIRM_QUIT) popup(c, "quit", {dash->finished ? "Leave the dashboard?" : "Training is still running. Quit anyway?", "", "[y] yes    [n] no"});
      if (pop == SAVE_AS) popup(c, "save model", {"path: " + save_path + "▏", "", "enter save    esc cancel"});
    }
    term.write(c.ansi());
    const int k = term.read_key(screen == TRAINING ? 100 : 250);
    if (term.wants_dump()) {
      std::cout << "=== frame ===\n" << c.plain();
      std::cout.flush();
      continue;
    }
    if (k == KEY_NONE) continue;
    if (k == 'Q') return 0;                     // the end of a key script
    if (screen == MENU) {
      if (k == KEY_UP) menu_sel = (menu_sel + 2) % 3;
      else if (k == KEY_DOWN) menu_sel = (menu_sel + 1) % 3;
      else if (k == 'q') return 0;
      else if (k == KEY_ENTER) {
        if (menu_sel == 0) { screen = CONFIG; config_error.clear(); }
        else if (menu_sel == 1) { repo = scan_repository(); repo_sel = 0; screen = REPOSITORY; }
        else return 0;
      }
    } else if (screen == REPOSITORY) {
      if (k == KEY_ESC || k == 'q') screen = MENU;
      else if (k == KEY_UP && !repo.empty()) repo_sel = (repo_sel + (int)repo.size() - 1) % (int)repo.size();
      else if (k == KEY_DOWN && !repo.empty()) repo_sel = (repo_sel + 1) % (int)repo.size();
    } else if (screen == CONFIG) {
      Field& f = fields[field_sel];
      if (k == KEY_ESC) screen = MENU;
      else if (k == KEY_TAB || k == KEY_UP || k == KEY_DOWN) field_sel ^= 1;
      else if (k == KEY_LEFT) example = (example + n_examples - 1) % n_examples;
      else if (k == KEY_RIGHT) example = (example + 1) % n_examples;
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
      std::puts("usage: orchestui | orchestui --render-once <model.json> <training.json> [--size WxH] [--no-save] | orchestui --script \"<keys>\" [--size WxH]");
      return 0;
    }
    if (argc >= 3 && std::strcmp(argv[1], "--script") == 0) {
      int W = 110, H = 34;
      for (int i = 3; i + 1 < argc; ++i) if (std::strcmp(argv[i], "--size") == 0) std::sscanf(argv[i + 1], "%dx%d", &W, &H);
      ScriptConsole sc(argv[2], W, H);
      return interactive(sc);
    }
    Terminal term;
    return interactive(term);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "orchestui: %s\n", e.what());
    return 1;
  }
}
