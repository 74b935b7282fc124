// Control-plane channel: framed messages over a TCP stream socket (header-only, POSIX sockets).
//
// Frame = u64 BE length | u32 BE kind | body, where length counts the kind word and the body
// (comms/src/codec/sink.rs:37-57, comms/src/codec/source.rs:34-56). Kind 0 carries a JSON command in
// serde's externally tagged snake_case form; kinds 5 and 6 carry raw little-endian f32 payloads
// (parameters, dataset chunks) as in comms/src/protocol/msg.rs:120-191. Gradients never use this
// channel on this runtime: between GPUs they move through NVLink windows.
//
// Handshake (comms/src/connection/connector.rs:175-196, acceptor.rs:52-74): the initiator sends
// connect{id,src}, the acceptor answers accept{id,src}; src names the sender's entity.
#pragma once
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "core/json.hpp"

namespace ono::wire {

constexpr uint32_t KIND_CONTROL = 0, KIND_PARAMS = 5, KIND_DATACHUNK = 6;

struct WireError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct WireTimeout : WireError {
  using WireError::WireError;
};

inline std::string uuid4() {
  static thread_local std::mt19937_64 rng{std::random_device{}()};
  uint64_t a = rng(), b = rng();
  a = (a & 0xffffffffffff0fffULL) | 0x0000000000004000ULL;
  b = (b & 0x3fffffffffffffffULL) | 0x8000000000000000ULL;
  char buf[40];
  std::snprintf(buf, sizeof buf, "%08x-%04x-%04x-%04x-%012llx", (unsigned)(a >> 32), (unsigned)((a >> 16) & 0xffff),
                (unsigned)(a & 0xffff), (unsigned)(b >> 48), (unsigned long long)(b & 0xffffffffffffULL));
  return buf;
}

struct Message {
  uint32_t kind = 0;
  Json command;               // kind 0
  std::vector<float> floats;  // kinds 5, 6
  std::string raw;            // anything else (gradient kinds 1-4)
  bool is_command(const char* unit) const { return kind == KIND_CONTROL && command.is_string() && command.as_string() == unit; }
  const Json* variant(const char* key) const { return kind == KIND_CONTROL ? command.find(key) : nullptr; }
};

class Channel {
 public:
  explicit Channel(int fd = -1) : fd_(fd) {
    if (fd_ >= 0) {
      int one = 1;
      ::setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    }
  }
  Channel(const Channel&) = delete;
  Channel& operator=(const Channel&) = delete;
  Channel(Channel&& o) noexcept : peer_entity(std::move(o.peer_entity)), peer_id(std::move(o.peer_id)), fd_(o.fd_) { o.fd_ = -1; }
  Channel& operator=(Channel&& o) noexcept {
    if (this != &o) { close(); fd_ = o.fd_; o.fd_ = -1; peer_entity = std::move(o.peer_entity); peer_id = std::move(o.peer_id); }
    return *this;
  }
  ~Channel() { close(); }

  bool open() const { return fd_ >= 0; }
  int fd() const { return fd_; }
  void close() {
    if (fd_ >= 0) { ::shutdown(fd_, SHUT_RDWR); ::close(fd_); fd_ = -1; }
  }

  void send_command(const Json& cmd) {
    const std::string body = cmd.dump();
    send_frame(KIND_CONTROL, body.data(), body.size());
  }
  void send_floats(uint32_t kind, const float* p, size_t n) { send_frame(kind, p, n * sizeof(float)); }

  // timeout_ms < 0 waits forever; a timeout throws WireTimeout before any byte of a frame was consumed.
  Message recv(int timeout_ms = -1) {
    if (timeout_ms >= 0) {
      pollfd pf{fd_, POLLIN, 0};
      int r;
      do { r = ::poll(&pf, 1, timeout_ms); } while (r < 0 && errno == EINTR);
      if (r == 0) throw WireTimeout("timed out waiting for a message");
      if (r < 0) throw WireError(std::string("poll: ") + std::strerror(errno));
    }
    unsigned char head[12];
    recv_exact(head, 12);
    uint64_t len = 0;
    for (int i = 0; i < 8; ++i) len = (len << 8) | head[i];
    uint32_t kind = ((uint32_t)head[8] << 24) | ((uint32_t)head[9] << 16) | ((uint32_t)head[10] << 8) | head[11];
    if (len < 4 || len > (1ull << 36)) throw WireError("bad frame length");
    const size_t body = (size_t)(len - 4);
    Message m;
    m.kind = kind;
    if (kind == KIND_PARAMS || kind == KIND_DATACHUNK) {
      if (body % 4) throw WireError("float payload is not a multiple of 4 bytes");
      m.floats.resize(body / 4);
      recv_exact(m.floats.data(), body);
    } else {
      m.raw.resize(body);
      recv_exact(m.raw.data(), body);
      if (kind == KIND_CONTROL) {
        // serde_json writes NaN losses as null (comms/src/protocol/msg.rs:201-229); tolerate a bare NaN too
        size_t at = 0;
        while ((at = m.raw.find("NaN", at)) != std::string::npos) m.raw.replace(at, 3, "null");
        m.command = Json::parse(m.raw);
      } else if (kind < 1 || kind > 4) {
        throw WireError("Received an invalid kind byte " + std::to_string(kind));
      }
    }
    return m;
  }

  // Undecoded frames, for relays that forward a session to another process.
  struct RawFrame { uint32_t kind = 0; std::string body; };
  RawFrame recv_raw(int timeout_ms = -1) {
    if (timeout_ms >= 0) {
      pollfd pf{fd_, POLLIN, 0};
      int r;
      do { r = ::poll(&pf, 1, timeout_ms); } while (r < 0 && errno == EINTR);
      if (r == 0) throw WireTimeout("timed out waiting for a message");
      if (r < 0) throw WireError(std::string("poll: ") + std::strerror(errno));
    }
    unsigned char head[12];
    recv_exact(head, 12);
    uint64_t len = 0;
    for (int i = 0; i < 8; ++i) len = (len << 8) | head[i];
    RawFrame f;
    f.kind = ((uint32_t)head[8] << 24) | ((uint32_t)head[9] << 16) | ((uint32_t)head[10] << 8) | head[11];
    if (len < 4 || len > (1ull << 36)) throw WireError("bad frame length");
    f.body.resize((size_t)(len - 4));
    recv_exact(f.body.data(), f.body.size());
    return f;
  }
  void send_raw(const RawFrame& f) { send_frame(f.kind, f.body.data(), f.body.size()); }

  std::string connect_as(const std::string& entity, std::string my_id = "") {
    if (my_id.empty()) my_id = uuid4();
    Json b = Json::object();
    b.set("id", my_id);
    b.set("src", entity);
    send_command(Json::tagged("connect", b));
    Message m = recv(30000);
    const Json* a = m.variant("accept");
    if (!a) throw WireError("expected accept");
    peer_id = a->at("id").as_string();
    peer_entity = a->at("src").as_string();
    return my_id;
  }
  void accept_as(const std::string& entity, const std::string& my_id) {
    Message m = recv(30000);
    const Json* c = m.variant("connect");
    if (!c) throw WireError("expected connect");
    peer_id = c->at("id").as_string();
    peer_entity = c->at("src").as_string();
    Json b = Json::object();
    b.set("id", my_id);
    b.set("src", entity);
    send_command(Json::tagged("accept", b));
  }

  // Dataset streaming (comms/src/share_dataset/send_dataset.rs:18-90, recv_dataset.rs:17-69): for xs then ys,
  // share_dataset_size{size} -> data chunks -> eof.
  void send_dataset(const float* xs, size_t nx, const float* ys, size_t ny, size_t chunk_bytes = 1 << 20) {
    const std::pair<const float*, size_t> parts[2] = {{xs, nx}, {ys, ny}};
    for (auto& pr : parts) {
      Json b = Json::object();
      b.set("size", Json((unsigned long long)pr.second));
      send_command(Json::tagged("share_dataset_size", b));
      const size_t step = std::max<size_t>(1, chunk_bytes / 4);
      for (size_t lo = 0; lo < pr.second; lo += step) send_floats(KIND_DATACHUNK, pr.first + lo, std::min(step, pr.second - lo));
      send_command(Json("eof"));
    }
  }
  void recv_dataset(std::vector<float>& xs, std::vector<float>& ys) {
    std::vector<float>* outs[2] = {&xs, &ys};
    for (auto* out : outs) {
      Message m = recv(300000);
      const Json* s = m.variant("share_dataset_size");
      if (!s) throw WireError("expected share_dataset_size");
      out->clear();
      out->reserve((size_t)s->at("size").as_u64());
      const size_t want = (size_t)s->at("size").as_u64();
      while (true) {
        Message c = recv(300000);
        if (c.is_command("eof")) break;
        if (c.kind != KIND_DATACHUNK) throw WireError("unexpected message while receiving a dataset");
        out->insert(out->end(), c.floats.begin(), c.floats.end());
      }
      if (out->size() != want) throw WireError("dataset stream shorter than announced");
    }
  }

  std::string peer_entity, peer_id;

 private:
  void send_all(const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n) {
      ssize_t k = ::send(fd_, c, n, MSG_NOSIGNAL);
      if (k < 0) {
        if (errno == EINTR) continue;
        throw WireError(std::string("send: ") + std::strerror(errno));
      }
      c += k;
      n -= (size_t)k;
    }
  }
  void send_frame(uint32_t kind, const void* body, size_t n) {
    unsigned char head[12];
    const uint64_t len = (uint64_t)n + 4;
    for (int i = 0; i < 8; ++i) head[i] = (unsigned char)(len >> (56 - 8 * i));
    for (int i = 0; i < 4; ++i) head[8 + i] = (unsigned char)(kind >> (24 - 8 * i));
    send_all(head, 12);
    if (n) send_all(body, n);
  }
  void recv_exact(void* p, size_t n) {
    char* c = static_cast<char*>(p);
    while (n) {
      ssize_t k = ::recv(fd_, c, n, 0);
      if (k == 0) throw WireError("peer closed the connection");
      if (k < 0) {
        if (errno == EINTR) continue;
        throw WireError(std::string("recv: ") + std::strerror(errno));
      }
      c += k;
      n -= (size_t)k;
    }
  }
  int fd_;
};

inline Channel connect(const std::string& host, int port, int timeout_ms = 30000) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  if (::getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res)
    throw WireError("cannot resolve " + host);
  int fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
  if (fd < 0) { ::freeaddrinfo(res); throw WireError("socket failed"); }
  timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
  ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
  int rc = ::connect(fd, res->ai_addr, res->ai_addrlen);
  ::freeaddrinfo(res);
  if (rc != 0) {
    ::close(fd);
    throw WireError("cannot connect to " + host + ":" + std::to_string(port) + ": " + std::strerror(errno));
  }
  timeval none{0, 0};
  ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &none, sizeof none);
  return Channel(fd);
}

// Listening socket on host:port (port 0 = any); returns the fd and stores the bound port.
inline int listen_on(const std::string& host, int port, int* bound_port = nullptr) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) throw WireError("socket failed");
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (host.empty() || host == "0.0.0.0") a.sin_addr.s_addr = INADDR_ANY;
  else if (::inet_pton(AF_INET, host == "localhost" ? "127.0.0.1" : host.c_str(), &a.sin_addr) != 1) {
    ::close(fd);
    throw WireError("bad listen address " + host);
  }
  if (::bind(fd, (sockaddr*)&a, sizeof a) != 0 || ::listen(fd, 64) != 0) {
    ::close(fd);
    throw WireError(std::string("cannot listen on ") + host + ":" + std::to_string(port) + ": " + std::strerror(errno));
  }
  if (bound_port) {
    socklen_t l = sizeof a;
    ::getsockname(fd, (sockaddr*)&a, &l);
    *bound_port = ntohs(a.sin_port);
  }
  return fd;
}

inline Channel accept_on(int listen_fd) {
  int fd;
  do { fd = ::accept(listen_fd, nullptr, nullptr); } while (fd < 0 && errno == EINTR);
  if (fd < 0) throw WireError(std::string("accept: ") + std::strerror(errno));
  return Channel(fd);
}

}  // namespace ono::wire
