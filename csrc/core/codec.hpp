// Gradient wire codecs and file formats of the control plane:
//   * f32 <-> f16 (IEEE binary16, round to nearest even): the reference always ships gradients as
//     f16 (comms/src/handles/compressor.rs:106-118, comms/src/handles/worker.rs:84-101);
//   * the sparse "gradient dropping" codec with sampled-quantile threshold
//     (comms/src/sparse/protocol.rs:33-144) and the dense fallback rule (compressor.rs:71-98);
//   * safetensors export/import of a trained model (orchestrator/src/sessions/trained_model.rs:36-121);
//   * csv/tsv -> packed little-endian f32 conversion (orchestrator/src/dataset_format.rs:12-155).
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "configs.hpp"

namespace ono {

uint16_t f32_to_f16(float f);
float f16_to_f32(uint16_t h);
// x -> f16 -> f32, the value the receiver of a dense gradient sees.
inline float f16_round_trip(float f) { return f16_to_f32(f32_to_f16(f)); }

constexpr size_t kSparseSampleMax = 1 << 14;
constexpr float kMinPositiveF16 = 6.103515625e-05f;

// k-th smallest |x| of a random sample of at most 16384 elements, k = floor(sample * (1 - r)),
// floored at the smallest positive normal f16. `seed` drives the sampler (Philox).
float sparse_threshold(const float* residual, size_t n, double r, uint64_t seed);
// [u64 total][u32 offset][u32 len][f16 ...]... little endian; runs of |x| >= threshold.
void sparse_drop(std::vector<uint8_t>& out, const float* residual, size_t n, float threshold);
// Decodes into `grad` (resized to the encoded total, zero filled). Throws std::runtime_error on a
// malformed buffer.
void sparse_lift(std::vector<float>& grad, const uint8_t* buf, size_t len);

struct Compressed {
  bool sparse = false;
  float threshold = 0.f;              // valid when sparse
  std::vector<uint8_t> bytes;         // sparse encoding, or packed f16 when dense
};
// Reference compressor: sparse if enabled and not larger than the dense f16 encoding.
Compressed compress_gradient(const float* residual, size_t n, bool sparse_enabled, double r, uint64_t seed);

// ---- safetensors ------------------------------------------------------------------------------
struct NamedTensor {
  std::string name;
  std::vector<size_t> shape;
  std::vector<float> data;
};
// layer_{i}.weight / layer_{i}.bias in model order; dense weight [in,out], conv [F,C,K,K],
// max-pool layers emit [0]-shaped tensors.
void save_safetensors(const std::string& path, const ModelConfig& model, size_t input_size, const std::vector<float>& params);
std::vector<NamedTensor> load_safetensors(const std::string& path);

// Optimizer-state sidecar of a checkpoint (an addition: the reference exports weights only). A safetensors container with
// `optimizer.m`, `optimizer.v` F32 [n] in the flat parameter order of the weights file, `optimizer.adam_pows` F32 [2]
// (running b1^t, b2^t) and string metadata `optimizer`, `epochs`, `n_params`; the same file the Python runtime writes
// for GPU and CPU ranks. Written to a temporary name and renamed, so a crash never leaves a truncated file.
struct StateSidecar {
  std::vector<float> m, v;
  float b1t = 1.f, b2t = 1.f;
  size_t epochs = 0;
  std::string optimizer;
};
void save_state_sidecar(const std::string& path, const StateSidecar& st);
StateSidecar load_state_sidecar(const std::string& path, size_t n_params);

// ---- dataset files ----------------------------------------------------------------------------
// Converts a .csv/.tsv file to a sibling .bin of packed LE f32 (cached if it exists; a non-numeric
// first row is skipped as a header). Other extensions are returned unchanged.
std::string ensure_binary_dataset(const std::string& path);
std::vector<float> read_f32_file(const std::string& path, size_t offset_elems = 0, size_t count = (size_t)-1);

}  // namespace ono
