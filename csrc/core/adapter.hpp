// Config -> plan: turns (ModelConfig, TrainingConfig, node statistics) into role assignments and the
// per-node specs, the way orchestrator/src/configs/adapter.rs:60-1202 does:
//   * roles: parameter servers = central vertices, all-reduce ring = TSP tour, strategy switch = both;
//   * per-layer specs with fan_in = flattened input size, fan_out = flattened output size and
//     limit = weights + biases (adapter.rs:1082-1161);
//   * layer -> server assignment by greedy LPT ("largest first into the least-loaded bin",
//     adapter.rs:1189-1202), layers kept in model order inside a server, yielding server_sizes,
//     server_ordering and layer_offsets (adapter.rs:605-687);
//   * the worker-side optimizer is plain gradient descent under a parameter server (adapter.rs:737-758);
//   * contiguous near-equal dataset partitions, the first `rem` partitions one row longer
//     (adapter.rs:889-947).
// Additions of this runtime: a global parameter offset per layer (initialisers are keyed by global
// element index, and upgrades use global offsets - the reference's server-local ranges are only
// right for one server), an "even" flat sharding mode, co-located server/worker ranks, and
// per-worker batch sizes derived from a global batch.
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "calculator.hpp"
#include "configs.hpp"
#include "json.hpp"

namespace ono {

// Greedy LPT: items sorted by descending size (stable), each put into the currently lightest bin
// (ties -> lowest bin index). Returns the item indices of each bin in insertion order.
std::vector<std::vector<size_t>> balanced_partitions(const std::vector<size_t>& sizes, size_t k);

// Row ranges [begin, end) of `nrows` split into `n` contiguous partitions.
std::vector<std::pair<size_t, size_t>> dataset_partitions(size_t nrows, size_t n);

struct LayerPlanInfo {
  size_t index = 0;
  size_t input_size = 0, output_size = 0;
  size_t n_params = 0, offset = 0;   // offset in the flat model vector (layers in model order)
  Json layer_spec;                   // LayerSpec
  Json param_gen;                    // ParamGenSpec or null for weightless layers
};

std::vector<LayerPlanInfo> adapt_layers(const ModelConfig& model, size_t x_size);

// Resolves a distribution spec to (kind, a, b) of the Philox sampler: kind 0 U[a,b), 1 U[a,b], 2 N(a,b).
void resolve_distribution(const Json& distribution, int& kind, float& a, float& b);

// The whole plan as one JSON document (consumed by the session / node runtimes and the bindings).
Json adapt_configs(const ModelConfig& model, const TrainingConfig& training, const Calculator& calc);

}  // namespace ono
