// ono-node: the role-agnostic node process (node/src/main.rs:27-54, node/src/router.rs:30-342).
//
//   PORT=40000 [HOST=0.0.0.0] [ONO_LOG=info] ono-node [--device cpu|gpu] [--gpu i] [--once]
//
// A node binds HOST:PORT, waits for an orchestrator and learns from the spec it receives what it is
// (worker, parameter server, both). One session at a time; after `disconnect` it listens again.
// It answers the control protocol itself: the connect/accept handshake, `ping`, the all-pairs latency
// probe (`stats_request`, node/src/stat_service.rs:69-152) and `create_node`. The rank it is asked to be
// runs
//   * in this process, on the C++ engine, when the session has a single CPU rank;
//   * in this process as well, as one rank of a TCP mesh between the nodes (node/net_rank.hpp), when the session has
//     several CPU ranks and uses all-reduce or the barrier / blocking parameter server;
//   * otherwise in a child rank process (the PyTorch + CUDA runtime, one per GPU) that this node starts
//     on a loopback port and to which it relays the session's frames in both directions, so that a GPU
//     fault or an out-of-memory in the rank never takes the listener down.
#include <poll.h>
#include <signal.h>
#include <sys/wait.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <thread>

#include "core/session.hpp"
#include "node/net_rank.hpp"

using namespace ono;
using Clock = std::chrono::steady_clock;

namespace {

int g_level = 2;  // 0 error, 1 warn, 2 info, 3 debug
void logf(int level, const char* fmt, ...) {
  if (level > g_level) return;
  static const char* names[] = {"ERROR", "WARN", "INFO", "DEBUG"};
  std::fprintf(stderr, "[ono-node %s] ", names[level]);
  va_list ap;
  va_start(ap, fmt);
  std::vfprintf(stderr, fmt, ap);
  va_end(ap);
  std::fputc('\n', stderr);
}

struct Options {
  std::string host = "127.0.0.1";
  int port = -1;
  std::string device = "cpu";
  int gpu = 0;
  bool once = false;
  std::string python = "python";
};

// ---- latency probe ---------------------------------------------------------------------------------------
struct Stat { double min = 0, max = 0, mean = 0; };

Stat ping_rounds(wire::Channel& ch, size_t rounds) {
  Stat s;
  double sum = 0;
  for (size_t i = 0; i < rounds; ++i) {
    const auto t0 = Clock::now();
    ch.send_command(Json("ping"));
    wire::Message m = ch.recv(10000);
    if (!m.is_command("pong")) throw wire::WireError("expected pong");
    const double ns = (double)std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count();
    s.min = i == 0 ? ns : std::min(s.min, ns);
    s.max = std::max(s.max, ns);
    sum += ns;
  }
  s.mean = rounds ? sum / (double)rounds : 0;
  return s;
}

// Node i connects to addrs[..i] and accepts `incoming` peers; every pair is measured once, by its initiator,
// and the acceptor answers the pings (stat_service.rs:107-152).
Json serve_ping_stats(int listen_fd, const std::string& node_id, const Json& req) {
  const size_t rounds = (size_t)req.at("rounds").as_u64();
  const size_t incoming = (size_t)req.at("incoming").as_u64();
  std::vector<std::thread> ts;
  std::mutex mu;
  Json rtts = Json::object();
  for (size_t k = 0; k < incoming; ++k) {
    ts.emplace_back([&, k] {
      (void)k;
      try {
        pollfd pf{listen_fd, POLLIN, 0};
        if (::poll(&pf, 1, 30000) <= 0) return;
        wire::Channel ch = wire::accept_on(listen_fd);
        ch.accept_as("Node", node_id);
        while (true) {
          wire::Message m = ch.recv(30000);
          if (m.is_command("ping")) ch.send_command(Json("pong"));
          else break;  // disconnect
        }
      } catch (const std::exception& e) { logf(1, "ping responder: %s", e.what()); }
    });
  }
  for (auto& a : req.at("addrs").items()) {
    const std::string addr = a.as_string();
    try {
      const size_t c = addr.rfind(':');
      wire::Channel ch = wire::connect(addr.substr(0, c), std::stoi(addr.substr(c + 1)), 10000);
      ch.connect_as("Node", node_id);
      const Stat s = ping_rounds(ch, rounds);
      ch.send_command(Json("disconnect"));
      Json o = Json::object();
      o.set("min", s.min);
      o.set("max", s.max);
      o.set("mean", s.mean);
      std::lock_guard<std::mutex> lk(mu);
      rtts.set(addr, o);
    } catch (const std::exception& e) { logf(1, "ping %s: %s", addr.c_str(), e.what()); }
  }
  for (auto& t : ts) t.join();
  Json body = Json::object();
  body.set("rtts", rtts);
  Json resp = Json::object();
  resp.set("stats", Json::tagged("ping", body));
  return Json::tagged("stats_response", resp);
}

// ---- a single CPU rank, in this process --------------------------------------------------------------------
void run_local_rank(wire::Channel& ch, const Json& job, std::vector<float> xs, std::vector<float> ys) {
  const ModelConfig model = ModelConfig::from_json(job.at("model"));
  TrainingConfig training = TrainingConfig::from_json(job.at("training"));
  oracle::Dataset data;
  data.x_size = training.dataset.x_size;
  data.y_size = training.dataset.y_size;
  data.samples = std::move(xs);
  data.labels = std::move(ys);
  training.dataset.is_inline = true;
  training.dataset.rows_hint = data.rows();
  Json plan = adapt_configs(model, training, Calculator::uniform(training.addrs));
  LocalSession session(plan, training, std::move(data));
  bool finished = false;
  std::vector<float> params;
  auto send_event = [&](const TrainingEvent& ev) {
    Json e = Json::object();
    e.set("kind", ev.kind);
    e.set("worker", Json((unsigned long long)ev.worker));
    Json l = Json::array();
    for (double v : ev.losses) l.push(Json(v));
    e.set("losses", l);
    e.set("text", ev.text);
    ch.send_command(Json::tagged("event", e));
  };
  while (true) {
    if (!finished) {
      TrainingEvent ev;
      while (session.next_event(ev, 20)) {
        send_event(ev);
        if (ev.kind == "complete") {
          finished = true;
          params = session.final_params();
          ch.send_command(Json("done"));
          break;
        }
      }
    }
    wire::Message m;
    try { m = ch.recv(finished ? -1 : 0); } catch (const wire::WireTimeout&) { continue; }
    if (m.is_command("stop_after_epoch") || m.is_command("abort")) session.stop();
    else if (m.is_command("request_params")) {
      while (!finished) {  // training still running: drain it first
        TrainingEvent ev;
        if (!session.next_event(ev, 100)) continue;
        send_event(ev);
        if (ev.kind == "complete") { finished = true; params = session.final_params(); ch.send_command(Json("done")); }
      }
      ch.send_floats(wire::KIND_PARAMS, params.data(), params.size());
      Json met = Json::object();
      met.set("switched", session.switched());
      send_event(TrainingEvent{"metrics", 0, {}, met.dump()});
    } else if (m.is_command("disconnect")) {
      session.stop();
      return;
    }
  }
}

// ---- one of several CPU ranks, in this process, talking to the other nodes over TCP -----------------------------
void run_net_rank(wire::Channel& ch, const Json& job, const Json& plan, const TrainingConfig& training, int listen_fd,
                  const std::string& node_id, std::vector<float> xs, std::vector<float> ys) {
  const size_t rank = (size_t)job.at("rank").as_u64();
  std::atomic<bool> stop{false}, finished{false};
  std::mutex mu;                       // events leave through the channel from the rank's thread and from this one
  std::vector<float> params;
  std::string failure;
  auto send_event = [&](const TrainingEvent& ev) {
    Json e = Json::object();
    e.set("kind", ev.kind);
    e.set("worker", Json((unsigned long long)ev.worker));
    Json l = Json::array();
    for (double v : ev.losses) l.push(Json(v));
    e.set("losses", l);
    e.set("text", ev.text);
    std::lock_guard<std::mutex> lk(mu);
    ch.send_command(Json::tagged("event", e));
  };
  std::atomic<bool> switched{false};
  std::thread worker([&] {
    try {
      NetRank r(plan, training, rank, listen_fd, node_id, std::move(xs), std::move(ys), send_event, stop);
      params = r.run();
      switched = r.switched();
    } catch (const std::exception& e) {
      failure = e.what();
      logf(1, "rank %zu failed: %s", rank, e.what());
      try {
        send_event(TrainingEvent{"error", 0, {}, std::string("rank ") + std::to_string(rank) + ": " + e.what()});
        send_event(TrainingEvent{"complete", 0, {}, "error"});
      } catch (const std::exception&) {}
    }
    finished = true;
    try {
      std::lock_guard<std::mutex> lk(mu);
      ch.send_command(Json("done"));
    } catch (const std::exception&) {}
  });
  try {
    while (true) {
      wire::Message m;
      try { m = ch.recv(200); } catch (const wire::WireTimeout&) { continue; }
      if (m.is_command("stop_after_epoch") || m.is_command("abort")) stop = true;
      else if (m.is_command("request_params")) {
        while (!finished) std::this_thread::sleep_for(std::chrono::milliseconds(20));
        {
          std::lock_guard<std::mutex> lk(mu);
          ch.send_floats(wire::KIND_PARAMS, params.data(), params.size());
        }
        Json met = Json::object();
        met.set("switched", switched.load());
        met.set("data_plane", "native tcp mesh");
        send_event(TrainingEvent{"metrics", 0, {}, met.dump()});
      } else if (m.is_command("disconnect")) break;
    }
  } catch (const std::exception& e) { logf(1, "orchestrator stream ended: %s", e.what()); }
  stop = true;
  worker.join();
}

// ---- any other rank: a child rank process behind a relay ---------------------------------------------------
void run_child_rank(wire::Channel& up, const Options& opt, const wire::Channel::RawFrame& create_frame) {
  int port = 0;
  { int fd = wire::listen_on("127.0.0.1", 0, &port); ::close(fd); }
  const std::string port_s = std::to_string(port), gpu_s = std::to_string(opt.gpu);
  pid_t pid = ::fork();
  if (pid < 0) throw std::runtime_error("fork failed");
  if (pid == 0) {
    ::execlp(opt.python.c_str(), opt.python.c_str(), "-m", "oxidized_neural_orchestra_b200.runtime.node", "--host", "127.0.0.1",
             "--port", port_s.c_str(), "--device", opt.device.c_str(), "--gpu", gpu_s.c_str(), "--once", (char*)nullptr);
    std::perror("exec rank process");
    ::_exit(127);
  }
  logf(2, "rank process %d on 127.0.0.1:%d (%s %d)", (int)pid, port, opt.device.c_str(), opt.gpu);
  auto reap = [&] {
    int st = 0;
    for (int i = 0; i < 100; ++i) {
      if (::waitpid(pid, &st, WNOHANG) == pid) return;
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    ::kill(pid, SIGKILL);  // exactly the child started above
    ::waitpid(pid, &st, 0);
  };
  wire::Channel down;
  const auto deadline = Clock::now() + std::chrono::seconds(180);  // the first import of the runtime can take a minute
  while (true) {
    try {
      down = wire::connect("127.0.0.1", port, 2000);
      down.connect_as("Orchestrator");
      break;
    } catch (const wire::WireError&) {
      int st = 0;
      if (::waitpid(pid, &st, WNOHANG) == pid) throw std::runtime_error("the rank process exited before it listened");
      if (Clock::now() > deadline) { reap(); throw std::runtime_error("the rank process did not start listening"); }
      std::this_thread::sleep_for(std::chrono::milliseconds(200));
    }
  }
  down.send_raw(create_frame);
  std::atomic<bool> closing{false};
  std::thread back([&] {  // rank -> orchestrator
    try {
      while (true) up.send_raw(down.recv_raw(-1));
    } catch (const std::exception& e) {
      if (!closing) {
        logf(1, "rank process stream ended: %s", e.what());
        try {
          Json ev = Json::object();
          ev.set("kind", "error"); ev.set("worker", 0); ev.set("losses", Json::array());
          ev.set("text", std::string("rank process lost: ") + e.what());
          up.send_command(Json::tagged("event", ev));
          Json c = Json::object();
          c.set("kind", "complete"); c.set("worker", 0); c.set("losses", Json::array()); c.set("text", "error");
          up.send_command(Json::tagged("event", c));
          up.send_command(Json("done"));
        } catch (const std::exception&) {}
      }
    }
  });
  try {
    while (true) {  // orchestrator -> rank
      wire::Channel::RawFrame f = up.recv_raw(-1);
      const bool bye = f.kind == wire::KIND_CONTROL && f.body == "\"disconnect\"";
      try { down.send_raw(f); } catch (const wire::WireError&) {}
      if (bye) break;
    }
  } catch (const std::exception& e) {
    logf(1, "orchestrator stream ended: %s", e.what());
    try { down.send_command(Json("disconnect")); } catch (const wire::WireError&) {}
  }
  closing = true;
  reap();
  down.close();
  back.join();
}

void session(wire::Channel& ch, int listen_fd, const std::string& node_id, const Options& opt) {
  while (true) {
    wire::Channel::RawFrame f = ch.recv_raw(-1);
    if (f.kind != wire::KIND_CONTROL) continue;
    const Json cmd = Json::parse(f.body);
    if (cmd.is_string() && cmd.as_string() == "disconnect") return;
    if (cmd.is_string() && cmd.as_string() == "ping") { ch.send_command(Json("pong")); continue; }
    if (const Json* sr = cmd.find("stats_request")) {
      const Json* ping = sr->find("request") ? sr->at("request").find("ping") : sr->find("ping");
      if (ping) ch.send_command(serve_ping_stats(listen_fd, node_id, *ping));
      else ch.send_command(Json::tagged("stats_response", Json::tagged("stats", Json::array())));
      continue;
    }
    if (const Json* cn = cmd.find("create_node")) {
      const Json& job = cn->at("spec");
      const size_t world = (size_t)job.at("world").as_u64();
      if (opt.device == "cpu" && world == 1) {
        std::vector<float> xs, ys;
        ch.recv_dataset(xs, ys);
        logf(2, "single CPU rank in this process (%zu samples)", job.at("training").at("dataset").at("x_size").as_u64() ? xs.size() / job.at("training").at("dataset").at("x_size").as_u64() : 0);
        run_local_rank(ch, job, std::move(xs), std::move(ys));
        return;
      }
      if (opt.device == "cpu" && std::getenv("ONO_CPU_RANKS_IN_PYTHON") == nullptr) {
        // several CPU ranks: this process is one of them if the strategy is one the native mesh covers
        const ModelConfig model = ModelConfig::from_json(job.at("model"));
        TrainingConfig training = TrainingConfig::from_json(job.at("training"));
        // the same plan on every node: uniform latencies, or the measured ones the orchestrator passed along
        std::map<std::string, std::map<std::string, uint64_t>> stats;
        if (const Json* st = job.find("stats"); st && st->is_object()) {
          for (auto& a : training.addrs) stats[a];
          for (auto& [addr, peers] : st->members())
            for (auto& [peer, rtt] : peers.members()) stats[addr][peer] = rtt.as_u64();
        }
        bool measured = false;
        for (auto& kv : stats) measured = measured || !kv.second.empty();
        Json plan = job.find("plan") && job.at("plan").is_object()
                        ? job.at("plan")
                        : adapt_configs(model, training, measured ? Calculator(std::move(stats)) : Calculator::uniform(training.addrs));
        if (NetRank::supports(plan, training)) {
          std::vector<float> xs, ys;
          ch.recv_dataset(xs, ys);
          logf(2, "rank %llu of %zu in this process (native TCP mesh)", (unsigned long long)job.at("rank").as_u64(), world);
          run_net_rank(ch, job, plan, training, listen_fd, node_id, std::move(xs), std::move(ys));
          return;
        }
      }
      run_child_rank(ch, opt, f);
      return;
    }
  }
}

}  // namespace

int main(int argc, char** argv) {
  Options opt;
  if (const char* h = std::getenv("HOST")) opt.host = h;
  if (const char* p = std::getenv("PORT")) opt.port = std::atoi(p);
  if (const char* py = std::getenv("ONO_PYTHON")) opt.python = py;
  if (const char* l = std::getenv("ONO_LOG")) {
    const std::string s = l;
    g_level = s == "error" ? 0 : s == "warn" ? 1 : s == "debug" || s == "trace" ? 3 : 2;
  }
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--host" && i + 1 < argc) opt.host = argv[++i];
    else if (a == "--port" && i + 1 < argc) opt.port = std::atoi(argv[++i]);
    else if (a == "--device" && i + 1 < argc) opt.device = argv[++i];
    else if (a == "--gpu" && i + 1 < argc) { opt.gpu = std::atoi(argv[++i]); opt.device = "gpu"; }
    else if (a == "--once") opt.once = true;
    else {
      std::fputs("usage: PORT=<port> [HOST=<addr>] ono-node [--device cpu|gpu] [--gpu i] [--once]\n", stderr);
      return a == "-h" || a == "--help" ? 0 : 2;
    }
  }
  if (opt.port < 0) { std::fputs("ono-node: a port is required (--port or the PORT environment variable)\n", stderr); return 2; }
  ::signal(SIGPIPE, SIG_IGN);
  try {
    const std::string node_id = wire::uuid4();
    int bound = 0;
    const int lfd = wire::listen_on(opt.host, opt.port, &bound);
    logf(2, "listening on %s:%d (%s) id %s", opt.host.c_str(), bound, opt.device.c_str(), node_id.c_str());
    while (true) {
      wire::Channel ch = wire::accept_on(lfd);
      try {
        ch.accept_as("Node", node_id);
      } catch (const std::exception&) {
        continue;  // a port probe or a stranger: not a session
      }
      if (ch.peer_entity == "Node") {  // a peer measuring latency outside a stats request: answer its pings
        try {
          while (true) {
            wire::Message m = ch.recv(30000);
            if (m.is_command("ping")) ch.send_command(Json("pong")); else break;
          }
        } catch (const std::exception&) {}
        continue;
      }
      try {
        session(ch, lfd, node_id, opt);
      } catch (const std::exception& e) { logf(1, "session ended: %s", e.what()); }
      if (opt.once) break;
    }
    ::close(lfd);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ono-node: %s\n", e.what());
    return 1;
  }
  return 0;
}
