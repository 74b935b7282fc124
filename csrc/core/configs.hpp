// model.json / training.json: the two documents that drive a run, in the reference's serde encoding
// (orchestrator/src/configs/model.rs:9-126, orchestrator/src/configs/training.rs:14-135,
// docs/config-schema.md). Unit enum variants are bare strings, struct variants single-key objects.
// Unknown fields are ignored, which is what lets the additive "b200" block ride in training.json.
#pragma once
#include <array>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.hpp"

namespace ono {

struct InvalidConfig : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// ---- model ------------------------------------------------------------------------------------
struct ParamGenConfig {
  enum Kind { Const, Uniform, UniformInclusive, XavierUniform, LecunUniform, Normal, Kaiming, Xavier, Lecun } kind = Kaiming;
  float a = 0.f, b = 0.f;  // value | low,high | mean,std_dev
  Json to_json() const;
  static ParamGenConfig from_json(const Json& j);
};

struct ActFnConfig {
  enum Kind { Sigmoid, Softmax, Tanh, ReLU, Gelu } kind = ReLU;
  float param = 0.f;  // amp | slope
  Json to_json() const;
  static ActFnConfig from_json(const Json& j);
  const char* name() const;
};

struct LayerConfig {
  enum Kind { Dense, Conv, MaxPooling } kind = Dense;
  size_t output_size = 0;                 // dense
  std::array<size_t, 3> input_dim{};      // conv / pool: (c, h, w)
  std::array<size_t, 3> kernel_dim{};     // conv: (filters, in_channels, k)
  size_t filter_size = 0;                 // pool
  size_t stride = 1, padding = 0;
  ParamGenConfig init;
  std::optional<ActFnConfig> act_fn;
  Json to_json() const;
  static LayerConfig from_json(const Json& j);
  size_t out_size() const;                        // flattened output size (model.rs:64-105)
  std::optional<size_t> expected_input_size() const;
  size_t param_count(size_t input_size) const;    // weights + biases
};

struct ModelConfig {
  std::vector<LayerConfig> layers;
  Json to_json() const;
  static ModelConfig from_json(const Json& j);
  size_t param_count(size_t x_size) const;
};

// ---- training ---------------------------------------------------------------------------------
struct OptimizerConfig {
  enum Kind { GradientDescent, Momentum, Adam } kind = GradientDescent;
  double lr = 0.01, mu = 0.0, b1 = 0.9, b2 = 0.999, eps = 1e-8;
  Json to_json() const;
  static OptimizerConfig from_json(const Json& j);
};

struct DatasetConfig {
  bool is_inline = true;
  std::string samples_path, labels_path;
  std::vector<float> samples, labels;
  size_t x_size = 0, y_size = 0;
  // Inline data may travel outside the document (large arrays stay binary); then `rows` says how
  // many rows the detached arrays hold. Additive key, ignored by the reference's parser.
  size_t rows_hint = 0;
  Json to_json() const;
  static DatasetConfig from_json(const Json& j);
};

struct AlgorithmConfig {
  enum Kind { ParameterServer, AllReduce, StrategySwitch } kind = AllReduce;
  size_t nservers = 0;
  enum Sync { Barrier, NonBlocking } synchronizer = Barrier;
  enum Store { Blocking, Wild } store = Blocking;
  Json to_json() const;
  static AlgorithmConfig from_json(const Json& j);
};

struct SerializerConfig {
  bool sparse = false;
  double r = 0.0;
  Json to_json() const;
  static SerializerConfig from_json(const Json& j);
};

// Additive block understood by this runtime only; every field optional.
struct B200Config {
  std::string sync_every = "round";       // "round" (reference cadence) | "step"
  std::string tile_dtype = "tf32";        // "tf32" | "bf16"
  std::string wire_dtype = "auto";        // "auto" | "f32" | "f16" | "bf16": gradients between ranks (auto: bf16 between GPUs in step cadence, else f32)
  std::string allreduce = "auto";         // "auto" | "ring" | "oneshot" | "twoshot" | "nvls"
  std::string sharding = "layer";         // "layer" (reference LPT) | "even"
  std::string switch_metric = "loss";     // "loss" | "grad_norm"
  size_t switch_window = 6;
  double switch_threshold = 0.01;
  bool leaky_relu_exact = true;
  size_t global_batch = 0;                // 0 = batch_size is per worker (reference)
  bool switch_resets_progress = false;
  bool colocate = false;                  // server ranks also train (B200 extension)
  std::string data = "host";              // "host": per-step H2D from pinned memory | "device"
  bool phase_timing = false;              // run steps uncaptured with CUDA events + NVTX ranges around compute / exchange / refresh
  bool probe = false;                     // measure pairwise node latency before planning (host:port sessions)
  std::string grad_stage = "auto";        // "auto" | "on" | "off": copy peers' finished gradient ranges into local staging during backward
  std::string grad_push = "auto";         // "auto" | "on" | "off" | "reduce": weight-gradient GEMMs store their 16-bit tiles into the owner's slab
                                          // ("reduce": add f32 tiles into the owner's accumulator instead)
  std::string shard_layout = "striped";   // "striped" | "contiguous": equal shares as one slice of every layer per owner (GPU ranks, staged 16-bit push) or as one run
  std::string param_pull = "auto";        // "auto" | "kernel" | "staged": fresh parameters reach the other GPUs from the fused kernel, or by copy engines under the next forward
  std::string pre_reduce = "auto";        // "auto" (4 GPUs and more) | "on" | "off": with fewer owners than ranks, ranks that own nothing sum a part of each owner's share and forward f32 sums
  std::string wgrad_apply = "auto";       // "auto" | "off": on one GPU the weight-gradient GEMMs apply the optimizer in their epilogues
  size_t switch_check_every = 10;         // step cadence: steps between two evaluations of the gradient-norm switch metric
  double comm_timeout_s = 300.0;          // a collective or device wait that exceeds this ends the run with an error
  double heartbeat_s = 2.0;               // period of a node's liveness messages (0 = none)
  double heartbeat_timeout_s = 0.0;       // the orchestrator drops a node that stayed silent this long (0 = never)
  std::string init_from;                  // safetensors checkpoint to start from instead of the initialisers (warm start / resume)
  std::string checkpoint_path;            // GPU ranks: periodic checkpoint (weights here, optimizer state beside it); "{epoch}" is replaced
  long long checkpoint_every = 0;         // epochs between periodic checkpoints (0 = off)
  std::string state_path;                 // GPU ranks and in-process CPU ranks: the optimizer state (m, v, Adam powers) is written here at the end of the run
  long long start_epoch = -1;             // first epoch number for the shuffle sequence (-1: 0, or the epochs recorded in init_state_from)
  std::string init_state_from;            // GPU ranks and in-process CPU ranks: optimizer state to resume from (a file written through state_path)
  std::string trace_path;                 // chrome-trace JSON of the run's phases (empty = off)
  std::string metrics_path;               // JSONL, one record per round / step window (empty = off)
  bool present = false;
  Json to_json() const;
  static B200Config from_json(const Json& j);
};

struct TrainingConfig {
  std::vector<std::string> addrs;
  AlgorithmConfig algorithm;
  SerializerConfig serializer;
  DatasetConfig dataset;
  OptimizerConfig optimizer;
  enum Loss { Mse, CrossEntropy } loss_fn = Mse;
  size_t batch_size = 1, max_epochs = 1, offline_epochs = 0;
  std::optional<unsigned long long> seed;
  std::optional<double> early_stopping_tolerance;
  B200Config b200;
  Json to_json(bool with_data = true) const;
  static TrainingConfig from_json(const Json& j);
};

// Semantic validation (orchestrator/src/configs/validator.rs:28-203). Throws InvalidConfig.
// n_samples_override: used when the dataset is local and its size was read by the caller.
void validate_configs(const ModelConfig& model, const TrainingConfig& training);
size_t dataset_rows(const DatasetConfig& d);

}  // namespace ono
