// Topology calculators of the control plane (orchestrator/src/calculator/{graph,tsp,bipartite,
// node_calculator}.rs): a dense symmetric weight matrix built from the max round-trip time between
// nodes, the exact Held-Karp tour used as the all-reduce ring order, and the k-subset of nodes that
// minimises the worst server<->worker edge, used to place parameter servers.
// On an NVSwitch fabric every pair is equidistant, so ties decide; ties resolve to the lowest indices.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <optional>
#include <set>
#include <string>
#include <tuple>
#include <vector>

namespace ono {

template <class W>
class Graph {
 public:
  // Returns nullopt if an edge names a vertex outside [0, size).
  static std::optional<Graph> make(size_t size, const std::vector<std::tuple<size_t, size_t, W>>& edges) {
    Graph g;
    g.size_ = size;
    g.m_.assign(size * size, std::nullopt);
    for (auto& [i, j, w] : edges) {
      if (i >= size || j >= size) return std::nullopt;
      g.m_[i * size + j] = w;
      g.m_[j * size + i] = w;
    }
    return g;
  }
  std::optional<W> weight(size_t i, size_t j) const {
    if (i < size_ && j < size_) return m_[i * size_ + j];
    return std::nullopt;
  }
  size_t len() const { return size_; }
  bool empty() const { return size_ == 0; }

 private:
  std::vector<std::optional<W>> m_;
  size_t size_ = 0;
};

// Exact minimum Hamiltonian cycle starting at vertex 0 (what tsp.rs:15-37 computes). Empty if none exists.
// A single vertex yields {0}: a ring of one rank (the reference returns an empty tour there, which
// would leave an all-reduce run with no workers).
//
// Bottom-up Held-Karp over one flat table: `cost[S * n + v]` is the cheapest way to leave v, visit every
// vertex outside the visited set S and return to 0. Supersets are numerically larger than their subsets,
// so one descending sweep over S has every successor ready; there is no recursion and no memo lookup.
// Only sets that contain vertex 0 (odd S) are reachable. Among equal costs the lowest next vertex wins,
// which is the order the reference's search settles ties in, so the ring order matches it on an
// equidistant fabric.
template <class W>
std::vector<size_t> travelling_salesman_cycle(const Graph<W>& g) {
  const size_t n = g.len();
  if (n == 0 || n >= 64) return {};
  if (n == 1) return {0};
  if (n > 20) {
    // The exact table needs n * 2^n entries; past 20 ranks take the nearest unvisited neighbour instead.
    std::vector<size_t> path{0};
    uint64_t seen = 1;
    while (path.size() < n) {
      std::optional<W> best;
      size_t pick = n;
      for (size_t w = 1; w < n; ++w) {
        if (seen >> w & 1) continue;
        const auto step = g.weight(path.back(), w);
        if (step && (!best || *step < *best)) { best = step; pick = w; }
      }
      if (pick == n) return {};
      seen |= uint64_t(1) << pick;
      path.push_back(pick);
    }
    return g.weight(path.back(), 0) ? path : std::vector<size_t>{};
  }
  constexpr uint8_t kNone = 0xff;
  const size_t full = (size_t(1) << n) - 1;
  std::vector<W> cost((full + 1) * n);
  std::vector<uint8_t> next((full + 1) * n, kNone);     // next vertex on the best way home, kNone: no way
  std::vector<char> reach((full + 1) * n, 0);
  for (size_t v = 1; v < n; ++v)
    if (auto home = g.weight(v, 0)) { cost[full * n + v] = *home; reach[full * n + v] = 1; }
  for (size_t S = full - 2; S >= 1 && S <= full; S -= 2) {            // odd sets only, descending
    for (size_t v = 0; v < n; ++v) {
      if (!(S >> v & 1) || (v == 0 && S != 1)) continue;            // the walk stands on v; 0 only at the start
      const size_t at = S * n + v;
      for (size_t w = 1; w < n; ++w) {
        if (S >> w & 1) continue;
        const size_t to = (S | size_t(1) << w) * n + w;
        const auto step = g.weight(v, w);
        if (!step || !reach[to]) continue;
        const W total = *step + cost[to];
        if (!reach[at] || total < cost[at]) { cost[at] = total; next[at] = (uint8_t)w; reach[at] = 1; }
      }
    }
    if (S == 1) break;
  }
  if (!reach[1 * n + 0]) return {};
  std::vector<size_t> path{0};
  for (size_t S = 1, v = 0; path.size() < n;) {
    v = next[S * n + v];
    S |= size_t(1) << v;
    path.push_back(v);
  }
  return path;
}

// The k vertices ("servers") minimising the maximum weight of an edge between a chosen and a
// non-chosen vertex (bipartite.rs:16-139); subsets are enumerated in lexicographic order and the
// first best one wins.
template <class W>
std::set<size_t> central_vertices(const Graph<W>& g, size_t k) {
  std::set<size_t> out;
  const size_t n = g.len();
  if (n == 0 || n > 64) return out;
  if (k >= n) { for (size_t i = 0; i < n; ++i) out.insert(i); return out; }
  if (k == 0) return out;
  uint64_t best = 0;
  std::optional<W> best_score;
  bool have = false;
  auto eval = [&](uint64_t center) {
    std::optional<W> mx;
    for (size_t v = 0; v < n; ++v) {
      if (center >> v & 1) continue;
      for (size_t w = 0; w < n; ++w) {
        if (!(center >> w & 1)) continue;
        if (auto wt = g.weight(v, w)) mx = mx ? std::max(*mx, *wt) : *wt;
      }
    }
    return mx;
  };
  struct Bt {
    size_t n, k; decltype(eval)& ev; uint64_t& best; std::optional<W>& best_score; bool& have;
    void run(size_t start, uint64_t center, size_t chosen) {
      if (chosen == k) {
        auto score = ev(center);
        // A subset with no edge to the rest scores "none", which ranks after every real score.
        const bool better = !have || (score && (!best_score || *score < *best_score));
        if (better) { best = center; best_score = score; have = true; }
        return;
      }
      if (k - chosen > n - start) return;
      for (size_t i = start; i < n; ++i) run(i + 1, center | (uint64_t(1) << i), chosen + 1);
    }
  } bt{n, k, eval, best, best_score, have};
  bt.run(0, 0, 0);
  for (size_t i = 0; i < n; ++i)
    if (best >> i & 1) out.insert(i);
  return out;
}

struct RoleAssignment {
  std::vector<std::string> server_addrs, worker_addrs;
};

// node_calculator.rs:42-122. `rtt_max_ns[a][b]` is the max RTT node a measured towards node b;
// addresses are processed in sorted order (the reference keeps them in a BTreeMap).
class Calculator {
 public:
  explicit Calculator(std::map<std::string, std::map<std::string, uint64_t>> rtt_max_ns) : stats_(std::move(rtt_max_ns)) {}
  // All nodes present, every pair at the same distance (an NVSwitch box without a probe).
  static Calculator uniform(const std::vector<std::string>& addrs);
  RoleAssignment node_role_assignment(size_t servers) const;
  std::vector<std::string> worker_cycle() const;
  std::vector<std::string> addrs() const;

 private:
  std::vector<std::tuple<size_t, size_t, uint64_t>> edges() const;
  std::map<std::string, std::map<std::string, uint64_t>> stats_;
};

}  // namespace ono
