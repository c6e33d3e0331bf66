#include "http.hpp"

#include "trace.hpp"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace http {

const char* status_text(int s) {
  switch (s) {
    case 200: return "OK";
    case 204: return "No Content";
    case 400: return "Bad Request";
    case 401: return "Unauthorized";
    case 404: return "Not Found";
    case 405: return "Method Not Allowed";
    case 413: return "Payload Too Large";
    case 422: return "Unprocessable Entity";
    case 424: return "Failed Dependency";
    case 429: return "Too Many Requests";
    case 500: return "Internal Server Error";
    case 503: return "Service Unavailable";
    default: return "Unknown";
  }
}

bool Response::write_all(const char* p, size_t n) {
  while (n && alive_) {
    ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
    if (w <= 0) {
      alive_ = false;
      return false;
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return alive_;
}

bool Response::send(int status, const std::string& content_type, const std::string& body) {
  status_ = status;
  started_ = true;
  std::string head = "HTTP/1.1 " + std::to_string(status) + " " + status_text(status) + "\r\n";
  head += "content-type: " + content_type + "\r\ncontent-length: " + std::to_string(body.size()) + "\r\n";
  for (auto& h : headers_) head += h.first + ": " + h.second + "\r\n";
  head += keep_alive ? "connection: keep-alive\r\n\r\n" : "connection: close\r\n\r\n";
  return write_all(head.data(), head.size()) && write_all(body.data(), body.size());
}

bool Response::begin_stream(int status, const std::string& content_type) {
  status_ = status;
  started_ = true;
  std::string head = "HTTP/1.1 " + std::to_string(status) + " " + status_text(status) + "\r\n";
  head += "content-type: " + content_type + "\r\ntransfer-encoding: chunked\r\ncache-control: no-cache\r\n";
  for (auto& h : headers_) head += h.first + ": " + h.second + "\r\n";
  head += keep_alive ? "connection: keep-alive\r\n\r\n" : "connection: close\r\n\r\n";
  return write_all(head.data(), head.size());
}

bool Response::write_chunk(const std::string& data) {
  if (data.empty()) return alive_;
  char len[32];
  int n = snprintf(len, sizeof len, "%zx\r\n", data.size());
  return write_all(len, static_cast<size_t>(n)) && write_all(data.data(), data.size()) && write_all("\r\n", 2);
}

bool Response::end_stream() { return write_all("0\r\n\r\n", 5); }

bool Response::client_gone() {
  if (!alive_) return true;
  pollfd p{fd_, POLLIN | POLLRDHUP, 0};
  if (::poll(&p, 1, 0) > 0) {
    if (p.revents & (POLLHUP | POLLERR | POLLRDHUP)) alive_ = false;
    else if (p.revents & POLLIN) {
      char c;
      ssize_t r = ::recv(fd_, &c, 1, MSG_PEEK | MSG_DONTWAIT);
      if (r == 0) alive_ = false;
    }
  }
  return !alive_;
}

Server::Server(const std::string& host, int port, size_t payload_limit)
    : host_(host), port_(port), payload_limit_(payload_limit) {}

Server::~Server() { stop(); }

void Server::route(const std::string& method, const std::string& path, Handler h) {
  routes_[method + " " + path] = std::move(h);
}

int Server::start() {
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) throw std::runtime_error("socket() failed");
  int one = 1;
  ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port_));
  if (host_.empty() || host_ == "0.0.0.0") addr.sin_addr.s_addr = INADDR_ANY;
  else if (::inet_pton(AF_INET, host_.c_str(), &addr.sin_addr) != 1) throw std::runtime_error("bad listen address " + host_);
  if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0)
    throw std::runtime_error("cannot bind port " + std::to_string(port_));
  if (::listen(listen_fd_, 1024) != 0) throw std::runtime_error("listen() failed");
  socklen_t len = sizeof addr;
  ::getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &len);
  port_ = ntohs(addr.sin_port);
  return port_;
}

void Server::serve_forever() {
  while (!stop_.load()) {
    pollfd p{listen_fd_, POLLIN, 0};
    int r = ::poll(&p, 1, 200);
    if (r <= 0) continue;
    int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    ++active_;
    std::thread([this, fd] {
      connection(fd);
      ::close(fd);
      --active_;
    }).detach();
  }
  // graceful shutdown: let in-flight requests finish (bounded)
  for (int i = 0; i < 100 && active_.load() > 0; ++i) ::usleep(100000);
}

void Server::stop() {
  stop_.store(true);
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
}

bool Server::read_request(int fd, std::string& buf, Request& req, int& error_status) {
  error_status = 0;
  size_t header_end;
  while ((header_end = buf.find("\r\n\r\n")) == std::string::npos) {
    if (buf.size() > (1 << 16)) { error_status = 400; return false; }
    pollfd p{fd, POLLIN, 0};
    int pr = ::poll(&p, 1, 1000);
    if (stop_.load()) return false;
    if (pr == 0) continue;
    char tmp[8192];
    ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
    if (r <= 0) return false;
    buf.append(tmp, static_cast<size_t>(r));
  }
  std::string head = buf.substr(0, header_end);
  buf.erase(0, header_end + 4);
  size_t line_end = head.find("\r\n");
  std::string request_line = head.substr(0, line_end);
  size_t sp1 = request_line.find(' '), sp2 = request_line.rfind(' ');
  if (sp1 == std::string::npos || sp2 == sp1) { error_status = 400; return false; }
  req.method = request_line.substr(0, sp1);
  std::string target = request_line.substr(sp1 + 1, sp2 - sp1 - 1);
  size_t q = target.find('?');
  req.path = target.substr(0, q);
  req.query = q == std::string::npos ? "" : target.substr(q + 1);
  req.headers.clear();
  size_t pos = line_end == std::string::npos ? head.size() : line_end + 2;
  while (pos < head.size()) {
    size_t e = head.find("\r\n", pos);
    if (e == std::string::npos) e = head.size();
    std::string line = head.substr(pos, e - pos);
    size_t c = line.find(':');
    if (c != std::string::npos) {
      std::string k = line.substr(0, c), v = line.substr(c + 1);
      std::transform(k.begin(), k.end(), k.begin(), ::tolower);
      size_t b = v.find_first_not_of(" \t");
      v = b == std::string::npos ? "" : v.substr(b);
      while (!v.empty() && (v.back() == ' ' || v.back() == '\t')) v.pop_back();
      req.headers[k] = v;
    }
    pos = e + 2;
  }
  size_t content_length = 0;
  std::string cl = req.header("content-length");
  if (!cl.empty()) content_length = static_cast<size_t>(strtoull(cl.c_str(), nullptr, 10));
  if (content_length > payload_limit_) { error_status = 413; return false; }
  while (buf.size() < content_length) {
    char tmp[65536];
    ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
    if (r <= 0) return false;
    buf.append(tmp, static_cast<size_t>(r));
  }
  req.body = buf.substr(0, content_length);
  buf.erase(0, content_length);
  return true;
}

void Server::connection(int fd) {
  std::string buf;
  while (!stop_.load()) {
    Request req;
    int err = 0;
    if (!read_request(fd, buf, req, err)) {
      if (err) {
        Response r(fd);
        r.keep_alive = false;
        r.send(err, "application/json", std::string("{\"error\":\"") + status_text(err) + "\",\"error_type\":\"validation\"}");
      }
      return;
    }
    Response resp(fd);
    std::string conn = req.header("connection");
    std::transform(conn.begin(), conn.end(), conn.begin(), ::tolower);
    resp.keep_alive = conn != "close";
    if (req.method == "OPTIONS") {   // CORS pre-flight
      resp.set_header("access-control-allow-origin", "*");
      resp.set_header("access-control-allow-headers", "*");
      resp.set_header("access-control-allow-methods", "GET, POST, OPTIONS");
      resp.send(204, "text/plain", "");
      continue;
    }
    if (middleware_ && !middleware_(req, resp)) {
      if (!resp.keep_alive) return;
      continue;
    }
    auto it = routes_.find(req.method + " " + req.path);
    // one server span per request; its parent is the caller's span when a valid `traceparent` came in
    trace::Span span;
    const bool traced = trace::exporter() != nullptr && it != routes_.end() && req.path != "/health" &&
                        req.path != "/metrics";
    if (traced) {
      const trace::Context parent = trace::parse_traceparent(req.header("traceparent"));
      span.trace_id = parent.valid() ? parent.trace_id : trace::random_hex(32);
      span.parent_span_id = parent.valid() ? parent.span_id : "";
      span.span_id = trace::random_hex(16);
      span.name = req.method + " " + req.path;
      span.start_ns = trace::now_ns();
      trace::set_current(trace::Context{span.trace_id, span.span_id, true});
    }
    auto finish_span = [&](bool failed) {
      if (!traced) return;
      trace::set_current(trace::Context{});
      span.end_ns = trace::now_ns();
      span.error = failed || resp.status() >= 500;
      span.str_attrs.emplace_back("http.method", req.method);
      span.str_attrs.emplace_back("http.route", req.path);
      span.int_attrs.emplace_back("http.status_code", resp.status());
      span.int_attrs.emplace_back("http.request_content_length", static_cast<long long>(req.body.size()));
      trace::exporter()->submit(std::move(span));
    };
    try {
      if (it != routes_.end()) it->second(req, resp);
      else if (fallback_) fallback_(req, resp);
      else resp.send(404, "application/json", "{\"error\":\"Not Found\",\"error_type\":\"not_found\"}");
      finish_span(false);
    } catch (const std::exception& e) {
      finish_span(true);
      if (!resp.started()) {
        std::string msg = e.what();
        for (auto& c : msg) if (c == '"' || c == '\\' || c == '\n') c = ' ';
        resp.send(500, "application/json", "{\"error\":\"" + msg + "\",\"error_type\":\"internal\"}");
      } else {
        return;
      }
    }
    if (!resp.keep_alive) return;
  }
}

}  // namespace http
