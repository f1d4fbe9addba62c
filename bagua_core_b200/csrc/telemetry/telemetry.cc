#include "telemetry.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <random>

namespace bagua {

namespace {

std::string u128_to_string(unsigned __int128 v) {
  if (v == 0) return "0";
  char buf[40];
  int i = 40;
  while (v > 0) {
    buf[--i] = (char)('0' + (int)(v % 10));
    v /= 10;
  }
  return std::string(buf + i, buf + 40);
}

std::string json_escape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 2);
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) {
          char b[8];
          std::snprintf(b, sizeof(b), "\\u%04x", c);
          o += b;
        } else {
          o += (char)c;
        }
    }
  }
  return o;
}

unsigned __int128 random_trace_id() {
  static thread_local std::mt19937_64 rng{std::random_device{}()};
  return ((unsigned __int128)rng() << 64) | rng();
}

}  // namespace

Telemetry& Telemetry::instance() {
  static Telemetry* t = new Telemetry();  // leaked: the flusher thread may outlive static destruction
  return *t;
}

Telemetry::~Telemetry() { shutdown(); }

void Telemetry::init(const std::string& addr) {
  std::lock_guard<std::mutex> g(mu_);
  if (enabled_.load()) return;
  auto colon = addr.rfind(':');
  host_ = colon == std::string::npos ? addr : addr.substr(0, colon);
  port_ = colon == std::string::npos ? 80 : std::atoi(addr.c_str() + colon + 1);
  stop_ = false;
  thread_ = std::thread([this] { run(); });
  enabled_.store(true, std::memory_order_release);
}

void Telemetry::init_from_env_once() {
  std::call_once(env_once_, [this] {
    const char* addr = std::getenv("AUTO_TUNE_SERVER_ADDR");
    if (addr && *addr) {
      BAGUA_LOG(Info, "detected auto tuning server, connecting");
      init(addr);
    } else {
      BAGUA_LOG(Warn, "auto tuning server not detected, may experience degraded performance");
    }
  });
}

void Telemetry::record(const std::string& action, const std::string& tensor_name, uint64_t start_ms,
                       uint64_t end_ms) {
  if (!enabled()) return;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (queue_.size() > 65536) queue_.pop_front();  // never grow without bound if the server is down
    queue_.push_back(Span{random_trace_id(), action, tensor_name, start_ms, end_ms});
  }
  cv_.notify_one();
}

std::string Telemetry::to_json(const std::vector<Span>& batch) {
  std::string s = "{\"spans\":[";
  for (size_t i = 0; i < batch.size(); ++i) {
    const Span& sp = batch[i];
    if (i) s += ",";
    s += "{\"trace_id\":" + u128_to_string(sp.trace_id) + ",\"action\":\"" + json_escape(sp.action) +
         "\",\"tensor_name\":\"" + json_escape(sp.tensor_name) + "\",\"start_time\":" + std::to_string(sp.start_ms) +
         ",\"end_time\":" + std::to_string(sp.end_ms) + "}";
  }
  s += "]}";
  return s;
}

bool Telemetry::post(const std::string& body) {
  struct addrinfo hints;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo* res = nullptr;
  if (getaddrinfo(host_.c_str(), std::to_string(port_).c_str(), &hints, &res) != 0 || !res) return false;
  int fd = -1;
  for (auto* p = res; p; p = p->ai_next) {
    fd = ::socket(p->ai_family, p->ai_socktype, p->ai_protocol);
    if (fd < 0) continue;
    struct timeval tv {2, 0};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    if (::connect(fd, p->ai_addr, p->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return false;
  std::string req = "POST /api/v1/report_tensor_execution_order HTTP/1.1\r\nHost: " + host_ + ":" +
                    std::to_string(port_) + "\r\nContent-Type: application/json\r\nContent-Length: " +
                    std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
  size_t off = 0;
  while (off < req.size()) {
    ssize_t n = ::send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
    if (n <= 0) {
      ::close(fd);
      return false;
    }
    off += (size_t)n;
  }
  char buf[256];
  ssize_t n = ::recv(fd, buf, sizeof(buf) - 1, 0);
  ::close(fd);
  if (n <= 0) return false;
  buf[n] = 0;
  // "HTTP/1.1 200 OK"
  const char* sp = std::strchr(buf, ' ');
  return sp && std::atoi(sp + 1) == 200;
}

void Telemetry::run() {
  for (;;) {
    std::vector<Span> batch;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, std::chrono::milliseconds(500), [&] { return stop_ || queue_.size() >= 512; });
      if (queue_.empty()) {
        drained_.notify_all();
        if (stop_) return;
        continue;
      }
      while (!queue_.empty() && batch.size() < 512) {
        batch.push_back(std::move(queue_.front()));
        queue_.pop_front();
      }
      busy_ = true;
    }
    const bool ok = post(to_json(batch));
    if (ok) {
      exported_ += batch.size();
    } else {
      failed_++;
      BAGUA_LOG(Warn, "upload bagua span failed (" << batch.size() << " spans dropped)");
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      busy_ = false;
      if (queue_.empty()) drained_.notify_all();
    }
  }
}

uint64_t Telemetry::flush(int timeout_ms) {
  if (enabled()) {
    cv_.notify_one();
    std::unique_lock<std::mutex> lk(mu_);
    auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (!(queue_.empty() && !busy_)) {
      cv_.notify_one();
      if (drained_.wait_until(lk, std::min(deadline, std::chrono::steady_clock::now() + std::chrono::milliseconds(50))) ==
              std::cv_status::timeout &&
          std::chrono::steady_clock::now() >= deadline)
        break;
    }
  }
  return exported_.load();
}

void Telemetry::shutdown() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!enabled_.load()) return;
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
  enabled_.store(false);
}

}  // namespace bagua
