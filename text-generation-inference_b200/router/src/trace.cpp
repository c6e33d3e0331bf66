#include "trace.hpp"

#include <arpa/inet.h>
#include <netdb.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <memory>
#include <random>
#include <sstream>

namespace trace {

namespace {

bool is_hex(const std::string& s) {
  for (char c : s)
    if (!((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'))) return false;
  return !s.empty();
}

bool all_zero(const std::string& s) {
  for (char c : s)
    if (c != '0') return false;
  return true;
}

std::string json_escape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 2);
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += static_cast<char>(c); }
    else if (c == '\n') o += "\\n";
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
    else o += static_cast<char>(c);
  }
  return o;
}

std::unique_ptr<Exporter> g_exporter;
thread_local Context t_current;

}  // namespace

void set_current(const Context& c) { t_current = c; }
const Context& current() { return t_current; }

Context parse_traceparent(const std::string& header) {
  Context c;
  // version-traceid-parentid-flags, lower-case hex, version ff is invalid, all-zero ids are invalid
  if (header.size() < 55 || header[2] != '-' || header[35] != '-' || header[52] != '-') return c;
  const std::string ver = header.substr(0, 2), tid = header.substr(3, 32), sid = header.substr(36, 16),
                    fl = header.substr(53, 2);
  if (!is_hex(ver) || ver == "ff" || !is_hex(tid) || !is_hex(sid) || !is_hex(fl)) return c;
  if (all_zero(tid) || all_zero(sid)) return c;
  if (ver == "00" && header.size() != 55) return c;
  c.trace_id = tid;
  c.span_id = sid;
  c.sampled = (std::stoi(fl, nullptr, 16) & 1) != 0;
  return c;
}

std::string format_traceparent(const Context& c) {
  return "00-" + c.trace_id + "-" + c.span_id + (c.sampled ? "-01" : "-00");
}

std::string random_hex(size_t digits) {
  static thread_local std::mt19937_64 rng(std::random_device{}() ^
                                          static_cast<uint64_t>(std::chrono::steady_clock::now().time_since_epoch().count()));
  static const char* hex = "0123456789abcdef";
  std::string s(digits, '0');
  bool nonzero = false;
  while (!nonzero) {
    for (size_t i = 0; i < digits; ++i) {
      s[i] = hex[rng() & 15];
      nonzero = nonzero || s[i] != '0';
    }
  }
  return s;
}

uint64_t now_ns() {
  return static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
}

std::string encode_otlp(const std::vector<Span>& spans, const std::string& service_name) {
  std::ostringstream o;
  o << "{\"resourceSpans\":[{\"resource\":{\"attributes\":[{\"key\":\"service.name\",\"value\":{\"stringValue\":\""
    << json_escape(service_name) << "\"}}]},\"scopeSpans\":[{\"scope\":{\"name\":\"tgi_b200.router\"},\"spans\":[";
  bool first = true;
  for (const Span& s : spans) {
    if (!first) o << ',';
    first = false;
    o << "{\"traceId\":\"" << s.trace_id << "\",\"spanId\":\"" << s.span_id << "\"";
    if (!s.parent_span_id.empty()) o << ",\"parentSpanId\":\"" << s.parent_span_id << "\"";
    o << ",\"name\":\"" << json_escape(s.name) << "\",\"kind\":" << s.kind << ",\"startTimeUnixNano\":\"" << s.start_ns
      << "\",\"endTimeUnixNano\":\"" << s.end_ns << "\",\"attributes\":[";
    bool fa = true;
    for (const auto& kv : s.str_attrs) {
      if (!fa) o << ',';
      fa = false;
      o << "{\"key\":\"" << json_escape(kv.first) << "\",\"value\":{\"stringValue\":\"" << json_escape(kv.second) << "\"}}";
    }
    for (const auto& kv : s.int_attrs) {
      if (!fa) o << ',';
      fa = false;
      o << "{\"key\":\"" << json_escape(kv.first) << "\",\"value\":{\"intValue\":\"" << kv.second << "\"}}";
    }
    o << "],\"status\":{\"code\":" << (s.error ? 2 : 1) << "}}";
  }
  o << "]}]}]}";
  return o.str();
}

Exporter::Exporter(const std::string& endpoint, const std::string& service_name) : service_(service_name) {
  std::string rest = endpoint;
  const std::string scheme = "http://";
  if (rest.rfind(scheme, 0) == 0) rest = rest.substr(scheme.size());
  size_t slash = rest.find('/');
  path_ = slash == std::string::npos ? "" : rest.substr(slash);
  std::string hostport = slash == std::string::npos ? rest : rest.substr(0, slash);
  if (path_.empty() || path_ == "/") path_ = "/v1/traces";
  size_t colon = hostport.rfind(':');
  if (colon != std::string::npos) {
    port_ = std::atoi(hostport.c_str() + colon + 1);
    hostport = hostport.substr(0, colon);
  }
  host_ = hostport;
  thread_ = std::thread([this] { loop(); });
}

Exporter::~Exporter() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

void Exporter::submit(Span&& s) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (queue_.size() >= 4096) {   // collector gone or slow: keep memory bounded
      ++dropped_;
      return;
    }
    queue_.push_back(std::move(s));
  }
  cv_.notify_one();
}

void Exporter::loop() {
  for (;;) {
    std::vector<Span> batch;
    bool stopping;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, std::chrono::milliseconds(500), [this] { return stop_ || queue_.size() >= 64; });
      while (!queue_.empty() && batch.size() < 512) {
        batch.push_back(std::move(queue_.front()));
        queue_.pop_front();
      }
      stopping = stop_ && queue_.empty();
    }
    if (!batch.empty()) {
      if (post(encode_otlp(batch, service_))) exported_ += batch.size();
      else dropped_ += batch.size();
    }
    if (stopping) return;
  }
}

bool Exporter::post(const std::string& body) { return http_post_json(host_, port_, path_, body); }

bool http_post_json(const std::string& host_, int port_, const std::string& path_, const std::string& body) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host_.c_str(), std::to_string(port_).c_str(), &hints, &res) != 0 || res == nullptr) return false;
  int fd = -1;
  for (addrinfo* a = res; a != nullptr; a = a->ai_next) {
    fd = ::socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    timeval tv{2, 0};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
    if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return false;
  std::string req = "POST " + path_ + " HTTP/1.1\r\nHost: " + host_ + ":" + std::to_string(port_) +
                    "\r\nContent-Type: application/json\r\nContent-Length: " + std::to_string(body.size()) +
                    "\r\nConnection: close\r\n\r\n" + body;
  size_t off = 0;
  bool ok = true;
  while (off < req.size()) {
    ssize_t w = ::send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
    if (w <= 0) { ok = false; break; }
    off += static_cast<size_t>(w);
  }
  if (ok) {
    char buf[256];
    ssize_t r = ::recv(fd, buf, sizeof buf - 1, 0);
    ok = r > 12 && std::strncmp(buf, "HTTP/1.", 7) == 0 && buf[9] == '2';   // any 2xx
  }
  ::close(fd);
  return ok;
}

void init(const std::string& endpoint, const std::string& service_name) {
  if (endpoint.empty()) return;
  g_exporter.reset(new Exporter(endpoint, service_name));
}

Exporter* exporter() { return g_exporter.get(); }

void shutdown() { g_exporter.reset(); }

}  // namespace trace
