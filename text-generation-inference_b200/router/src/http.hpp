// Minimal HTTP/1.1 server: one thread per connection, keep-alive, request bodies by
// Content-Length, responses either whole or as a chunked stream (Server-Sent Events).
// It carries the router's REST surface (reference: axum routes, router/src/server.rs:2203-2288).
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <string>
#include <thread>
#include <vector>

namespace http {

struct Request {
  std::string method, path, query, body;
  std::map<std::string, std::string> headers;   // lower-case names
  std::string header(const std::string& name) const {
    auto it = headers.find(name);
    return it == headers.end() ? "" : it->second;
  }
};

// Handed to handlers; either `send` once, or `begin_stream` + `write_chunk`* + `end_stream`.
class Response {
 public:
  explicit Response(int fd) : fd_(fd) {}
  void set_header(const std::string& k, const std::string& v) { headers_.emplace_back(k, v); }
  bool send(int status, const std::string& content_type, const std::string& body);
  bool begin_stream(int status, const std::string& content_type);
  bool write_chunk(const std::string& data);   // false once the client is gone
  bool end_stream();
  bool client_gone();                           // non-blocking probe of the socket
  bool started() const { return started_; }
  int status() const { return status_; }        // status line sent so far (0: nothing yet)
  bool keep_alive = true;

 private:
  bool write_all(const char* p, size_t n);
  int fd_;
  bool started_ = false;
  int status_ = 0;
  bool alive_ = true;
  std::vector<std::pair<std::string, std::string>> headers_;
};

using Handler = std::function<void(const Request&, Response&)>;

class Server {
 public:
  Server(const std::string& host, int port, size_t payload_limit);
  ~Server();
  void route(const std::string& method, const std::string& path, Handler h);
  void set_fallback(Handler h) { fallback_ = std::move(h); }
  void set_middleware(std::function<bool(const Request&, Response&)> m) { middleware_ = std::move(m); }
  // binds and listens; returns the bound port (useful with port 0)
  int start();
  void serve_forever();
  void stop();

 private:
  void connection(int fd);
  bool read_request(int fd, std::string& buf, Request& req, int& error_status);
  std::string host_;
  int port_;
  size_t payload_limit_;
  int listen_fd_ = -1;
  std::atomic<bool> stop_{false};
  std::map<std::string, Handler> routes_;
  Handler fallback_;
  std::function<bool(const Request&, Response&)> middleware_;
  std::atomic<int> active_{0};
};

const char* status_text(int status);

}  // namespace http
