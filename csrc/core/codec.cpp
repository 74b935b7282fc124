#include "codec.hpp"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <numeric>
#include <sstream>
#include <stdexcept>

#include "json.hpp"
#include "philox.h"

namespace ono {

uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t exp = (x >> 23) & 0xFFu;
  uint32_t man = x & 0x7FFFFFu;
  if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u | (man >> 13) : 0));  // inf / nan
  int e = (int)exp - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7C00u);  // overflow -> inf
  if (e <= 0) {                                    // subnormal or zero
    if (e < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - e;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)e << 10) | (man >> 13);
  const uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;  // may carry into the exponent, which is correct
  return (uint16_t)(sign | h);
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) x = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) x = sign | 0x7F800000u | (man << 13);
  else x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

float sparse_threshold(const float* residual, size_t n, double r, uint64_t seed) {
  if (n == 0) return 0.0f;
  const size_t sample_size = std::min(kSparseSampleMax, n);
  std::vector<float> sample(sample_size);
  if (sample_size == n) {
    for (size_t i = 0; i < n; ++i) sample[i] = std::fabs(residual[i]);
  } else {
    // sampling without replacement via a partial Fisher-Yates on an index table would cost O(n)
    // memory; stratified sampling (one draw per equal stride) keeps it O(sample) and unbiased.
    const double stride = (double)n / (double)sample_size;
    for (size_t i = 0; i < sample_size; ++i) {
      const Philox4 rnd = philox4x32_10(i, seed);
      const double u = (double)(rnd.v[0] >> 8) * (1.0 / 16777216.0);
      size_t idx = (size_t)(((double)i + u) * stride);
      if (idx >= n) idx = n - 1;
      sample[i] = std::fabs(residual[idx]);
    }
  }
  size_t k = (size_t)((float)sample_size * (1.0f - (float)r));
  k = std::min(k, sample_size - 1);
  std::nth_element(sample.begin(), sample.begin() + k, sample.end());
  return std::max(sample[k], kMinPositiveF16);
}

static void put_le(std::vector<uint8_t>& out, uint64_t v, int bytes) {
  for (int i = 0; i < bytes; ++i) out.push_back((uint8_t)(v >> (8 * i)));
}

void sparse_drop(std::vector<uint8_t>& out, const float* residual, size_t n, float threshold) {
  put_le(out, n, 8);
  size_t last_end = 0, i = 0;
  while (i < n) {
    if (std::fabs(residual[i]) >= threshold) {
      const size_t start = i;
      while (i < n && std::fabs(residual[i]) >= threshold) ++i;
      put_le(out, start - last_end, 4);
      put_le(out, i - start, 4);
      for (size_t j = start; j < i; ++j) put_le(out, f32_to_f16(residual[j]), 2);
      last_end = i;
    } else {
      ++i;
    }
  }
}

void sparse_lift(std::vector<float>& grad, const uint8_t* buf, size_t len) {
  if (len < 8) throw std::runtime_error("The given sparse buffer is smaller than TOTAL_LEN_SIZE");
  auto get = [&](size_t at, int bytes) {
    uint64_t v = 0;
    for (int i = 0; i < bytes; ++i) v |= (uint64_t)buf[at + i] << (8 * i);
    return v;
  };
  const size_t total = (size_t)get(0, 8);
  std::fill(grad.begin(), grad.end(), 0.0f);
  grad.resize(total, 0.0f);
  size_t gi = 0, bi = 8;
  while (bi < len) {
    if (bi + 4 > len) throw std::runtime_error("Missing index bytes at grad lift");
    gi += (size_t)get(bi, 4);
    bi += 4;
    if (bi + 4 > len) throw std::runtime_error("Missing chunk length bytes at grad lift");
    const size_t chunk = (size_t)get(bi, 4);
    bi += 4;
    if (gi > grad.size() || grad.size() - gi < chunk) throw std::runtime_error("Gradient chunk exceeds target vector bounds");
    for (size_t j = 0; j < chunk; ++j) {
      if (bi + 2 > len) throw std::runtime_error("Truncated float data");
      grad[gi + j] = f16_to_f32((uint16_t)get(bi, 2));
      bi += 2;
    }
    gi += chunk;
  }
}

Compressed compress_gradient(const float* residual, size_t n, bool sparse_enabled, double r, uint64_t seed) {
  Compressed c;
  if (sparse_enabled) {
    c.threshold = sparse_threshold(residual, n, r, seed);
    sparse_drop(c.bytes, residual, n, c.threshold);
    if (c.bytes.size() <= n * 2) { c.sparse = true; return c; }
    c.bytes.clear();
  }
  c.bytes.resize(n * 2);
  for (size_t i = 0; i < n; ++i) {
    const uint16_t h = f32_to_f16(residual[i]);
    c.bytes[2 * i] = (uint8_t)h;
    c.bytes[2 * i + 1] = (uint8_t)(h >> 8);
  }
  return c;
}

// ---- safetensors ------------------------------------------------------------------------------
void save_safetensors(const std::string& path, const ModelConfig& model, size_t input_size, const std::vector<float>& params) {
  struct Entry { std::string name; std::vector<size_t> shape; size_t begin, end; };
  std::vector<Entry> entries;
  size_t prev = input_size, off = 0;
  for (size_t i = 0; i < model.layers.size(); ++i) {
    const LayerConfig& l = model.layers[i];
    size_t wc = 0, bc = 0;
    std::vector<size_t> ws{0}, bs{0};
    if (l.kind == LayerConfig::Dense) { wc = prev * l.output_size; bc = l.output_size; ws = {prev, l.output_size}; bs = {l.output_size}; }
    else if (l.kind == LayerConfig::Conv) {
      wc = l.kernel_dim[0] * l.kernel_dim[1] * l.kernel_dim[2] * l.kernel_dim[2];
      bc = l.kernel_dim[0];
      ws = {l.kernel_dim[0], l.kernel_dim[1], l.kernel_dim[2], l.kernel_dim[2]};
      bs = {l.kernel_dim[0]};
    }
    if (off + wc + bc > params.size()) throw std::runtime_error("parameter vector is shorter than the model");
    entries.push_back({"layer_" + std::to_string(i) + ".weight", ws, off, off + wc});
    off += wc;
    entries.push_back({"layer_" + std::to_string(i) + ".bias", bs, off, off + bc});
    off += bc;
    prev = l.out_size();
  }
  // The safetensors crate orders tensors by dtype alignment then name before laying out the data.
  std::vector<size_t> order(entries.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return entries[a].name < entries[b].name; });
  Json header = Json::object();
  size_t cursor = 0;
  std::vector<std::pair<size_t, size_t>> data_pos(entries.size());
  for (size_t idx : order) {
    const Entry& e = entries[idx];
    const size_t bytes = (e.end - e.begin) * 4;
    Json shape = Json::array();
    for (size_t s : e.shape) shape.push(Json((unsigned long long)s));
    Json offs = Json::array();
    offs.push(Json((unsigned long long)cursor));
    offs.push(Json((unsigned long long)(cursor + bytes)));
    Json t = Json::object();
    t.set("dtype", "F32");
    t.set("shape", shape);
    t.set("data_offsets", offs);
    header.set(e.name, t);
    data_pos[idx] = {cursor, bytes};
    cursor += bytes;
  }
  std::string hs = header.dump();
  while (hs.size() % 8) hs.push_back(' ');
  std::ofstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path + " for writing");
  const uint64_t hl = hs.size();
  uint8_t le[8];
  for (int i = 0; i < 8; ++i) le[i] = (uint8_t)(hl >> (8 * i));
  f.write((const char*)le, 8);
  f.write(hs.data(), (std::streamsize)hs.size());
  for (size_t idx : order) {
    const Entry& e = entries[idx];
    if (e.end > e.begin) f.write((const char*)(params.data() + e.begin), (std::streamsize)((e.end - e.begin) * 4));
  }
  if (!f) throw std::runtime_error("short write to " + path);
}

std::vector<NamedTensor> load_safetensors(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  uint8_t le[8];
  f.read((char*)le, 8);
  uint64_t hl = 0;
  for (int i = 0; i < 8; ++i) hl |= (uint64_t)le[i] << (8 * i);
  if (!f || hl > (1ull << 30)) throw std::runtime_error("bad safetensors header");
  std::string hs(hl, '\0');
  f.read(hs.data(), (std::streamsize)hl);
  std::vector<char> data((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  Json header = Json::parse(hs);
  std::vector<NamedTensor> out;
  for (auto& [name, t] : header.members()) {
    if (name == "__metadata__") continue;
    if (t.at("dtype").as_string() != "F32") throw std::runtime_error("only F32 tensors are supported");
    NamedTensor nt;
    nt.name = name;
    for (auto& s : t.at("shape").items()) nt.shape.push_back((size_t)s.as_u64());
    const size_t b = (size_t)t.at("data_offsets")[0].as_u64(), e = (size_t)t.at("data_offsets")[1].as_u64();
    if (e < b || e > data.size()) throw std::runtime_error("tensor data out of bounds");
    nt.data.resize((e - b) / 4);
    if (e > b) std::memcpy(nt.data.data(), data.data() + b, e - b);
    out.push_back(std::move(nt));
  }
  return out;
}

void save_state_sidecar(const std::string& path, const StateSidecar& st) {
  const float pows[2] = {st.b1t, st.b2t};
  const size_t nm = st.m.size() * 4, nv = st.v.size() * 4;
  std::string header = "{\"__metadata__\":{\"optimizer\":\"" + st.optimizer + "\",\"epochs\":\"" + std::to_string(st.epochs) +
                       "\",\"n_params\":\"" + std::to_string(st.m.size()) + "\"}," +
                       "\"optimizer.m\":{\"dtype\":\"F32\",\"shape\":[" + std::to_string(st.m.size()) + "],\"data_offsets\":[0," + std::to_string(nm) + "]}," +
                       "\"optimizer.v\":{\"dtype\":\"F32\",\"shape\":[" + std::to_string(st.v.size()) + "],\"data_offsets\":[" + std::to_string(nm) + "," + std::to_string(nm + nv) + "]}," +
                       "\"optimizer.adam_pows\":{\"dtype\":\"F32\",\"shape\":[2],\"data_offsets\":[" + std::to_string(nm + nv) + "," + std::to_string(nm + nv + 8) + "]}}";
  while (header.size() % 8) header.push_back(' ');
  const std::string tmp = path + ".tmp";
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) throw std::runtime_error("cannot write " + tmp);
    uint8_t le[8];
    const uint64_t hl = header.size();
    for (int i = 0; i < 8; ++i) le[i] = (uint8_t)(hl >> (8 * i));
    f.write((const char*)le, 8);
    f.write(header.data(), (std::streamsize)header.size());
    f.write((const char*)st.m.data(), (std::streamsize)nm);
    f.write((const char*)st.v.data(), (std::streamsize)nv);
    f.write((const char*)pows, 8);
    f.flush();
    if (!f) throw std::runtime_error("short write to " + tmp);
  }
  if (std::rename(tmp.c_str(), path.c_str()) != 0) throw std::runtime_error("cannot rename " + tmp + " to " + path);
}

StateSidecar load_state_sidecar(const std::string& path, size_t n_params) {
  StateSidecar st;
  for (auto& t : load_safetensors(path)) {
    if (t.name == "optimizer.m") st.m = std::move(t.data);
    else if (t.name == "optimizer.v") st.v = std::move(t.data);
    else if (t.name == "optimizer.adam_pows" && t.data.size() == 2) { st.b1t = t.data[0]; st.b2t = t.data[1]; }
  }
  if (st.m.size() != n_params || st.v.size() != n_params)
    throw std::runtime_error(path + ": state of " + std::to_string(st.m.size()) + " parameters does not fit a model of " + std::to_string(n_params));
  // the metadata block: strings
  std::ifstream f(path, std::ios::binary);
  uint8_t le[8];
  f.read((char*)le, 8);
  uint64_t hl = 0;
  for (int i = 0; i < 8; ++i) hl |= (uint64_t)le[i] << (8 * i);
  std::string hs(hl, '\0');
  f.read(hs.data(), (std::streamsize)hl);
  const Json header = Json::parse(hs);
  if (const Json* md = header.find("__metadata__")) {
    if (const Json* e = md->find("epochs"); e && e->is_string()) st.epochs = (size_t)std::strtoull(e->as_string().c_str(), nullptr, 10);
    if (const Json* o = md->find("optimizer"); o && o->is_string()) st.optimizer = o->as_string();
  }
  return st;
}

// ---- dataset files ----------------------------------------------------------------------------
static bool parse_row(const std::string& line, char sep, std::vector<float>& out) {
  size_t start = 0;
  const size_t before = out.size();
  while (true) {
    size_t end = line.find(sep, start);
    std::string field = line.substr(start, end == std::string::npos ? std::string::npos : end - start);
    const size_t a = field.find_first_not_of(" \t\r\n");
    const size_t b = field.find_last_not_of(" \t\r\n");
    if (a == std::string::npos) { out.resize(before); return false; }
    field = field.substr(a, b - a + 1);
    char* endp = nullptr;
    errno = 0;
    const float v = std::strtof(field.c_str(), &endp);
    if (endp == field.c_str() || *endp != '\0') { out.resize(before); return false; }
    out.push_back(v);
    if (end == std::string::npos) break;
    start = end + 1;
  }
  return true;
}

std::string ensure_binary_dataset(const std::string& path) {
  const size_t dot = path.find_last_of('.');
  const std::string ext = dot == std::string::npos ? "" : path.substr(dot + 1);
  if (ext != "csv" && ext != "tsv") return path;
  const std::string out = path.substr(0, dot) + ".bin";
  struct stat st;
  if (stat(out.c_str(), &st) == 0) return out;  // cached
  const char sep = ext == "csv" ? ',' : '\t';
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open dataset file " + path);
  std::ofstream of(out, std::ios::binary);
  if (!of) throw std::runtime_error("cannot create " + out);
  std::string line;
  bool first = true;
  size_t line_no = 0;
  std::vector<float> row;
  while (std::getline(in, line)) {
    ++line_no;
    const size_t a = line.find_first_not_of(" \t\r\n");
    if (a == std::string::npos) continue;
    const size_t b = line.find_last_not_of(" \t\r\n");
    const std::string trimmed = line.substr(a, b - a + 1);
    row.clear();
    const bool ok = parse_row(trimmed, sep, row);
    if (first) {
      first = false;
      if (!ok) continue;  // header row
    } else if (!ok) {
      throw std::runtime_error("line " + std::to_string(line_no) + " of " + path + " is not numeric");
    }
    of.write((const char*)row.data(), (std::streamsize)(row.size() * 4));
  }
  return out;
}

std::vector<float> read_f32_file(const std::string& path, size_t offset_elems, size_t count) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) throw std::runtime_error("cannot open " + path);
  const size_t total = (size_t)f.tellg() / 4;
  if (offset_elems > total) throw std::runtime_error("offset beyond the end of " + path);
  const size_t n = std::min(count, total - offset_elems);
  std::vector<float> v(n);
  f.seekg((std::streamoff)(offset_elems * 4));
  f.read((char*)v.data(), (std::streamsize)(n * 4));
  return v;
}

}  // namespace ono
