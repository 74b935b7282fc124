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

// Exact minimum Hamiltonian cycle starting at vertex 0 (tsp.rs:15-37). Empty if none exists.
// A single vertex yields {0}: a ring of one rank (the reference returns an empty tour there, which
// would leave an all-reduce run with no workers).
template <class W>
std::vector<size_t> travelling_salesman_cycle(const Graph<W>& g) {
  const size_t n = g.len();
  if (n == 0 || n >= 64) return {};
  if (n == 1) return {0};
  const size_t states = n * (size_t(1) << n);
  std::vector<std::optional<W>> mem(states);
  std::vector<std::optional<size_t>> parent(states);
  std::vector<char> done(states, 0);
  // iterative DFS would obscure the recurrence; n is at most a few dozen ranks, depth is n.
  struct Rec {
    const Graph<W>& g; size_t n;
    std::vector<std::optional<W>>& mem; std::vector<std::optional<size_t>>& parent; std::vector<char>& done;
    std::optional<W> run(size_t visited, size_t v) {
      const size_t i = visited * n + v;
      if (done[i]) return mem[i];
      if ((size_t)__builtin_popcountll(visited) == n) return g.weight(v, 0);
      for (size_t w = 1; w < n; ++w) {
        const size_t bit = size_t(1) << w;
        if (visited & bit) continue;
        auto wt = g.weight(v, w);
        if (!wt) continue;
        auto cost = run(visited | bit, w);
        if (!cost) continue;
        const W total = *wt + *cost;
        if (!mem[i] || total < *mem[i]) { mem[i] = total; parent[i] = w; }
      }
      done[i] = 1;
      return mem[i];
    }
  } rec{g, n, mem, parent, done};
  if (!rec.run(1, 0)) return {};
  std::vector<size_t> path{0};
  size_t visited = 1, v = 0;
  while (path.size() < n) {
    const size_t w = *parent[visited * n + v];
    visited |= size_t(1) << w;
    path.push_back(w);
    v = w;
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
