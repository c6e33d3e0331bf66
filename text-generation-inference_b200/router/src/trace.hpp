// Request tracing of the router: W3C trace-context parsing, one server span per HTTP request and an
// OTLP/HTTP JSON exporter on a background thread.
//
// Reference: `router/src/logging.rs:22-136` (OTLP exporter set-up, `traceparent` extraction middleware)
// and `backends/grpc-metadata/src/lib.rs:1-41` (context propagation).  The exporter speaks the JSON
// encoding of OTLP over plain HTTP (`POST /v1/traces`), which every collector accepts; no SDK is linked.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace trace {

// `traceparent: 00-<32 hex trace id>-<16 hex parent span id>-<2 hex flags>`
struct Context {
  std::string trace_id, span_id;
  bool sampled = true;
  bool valid() const { return trace_id.size() == 32 && span_id.size() == 16; }
};
Context parse_traceparent(const std::string& header);   // invalid input -> !valid()
std::string format_traceparent(const Context& c);
std::string random_hex(size_t digits);
uint64_t now_ns();                                      // wall clock, ns since the epoch

struct Span {
  std::string name, trace_id, span_id, parent_span_id;
  uint64_t start_ns = 0, end_ns = 0;
  int kind = 2;                                         // SPAN_KIND_SERVER
  bool error = false;
  std::vector<std::pair<std::string, std::string>> str_attrs;
  std::vector<std::pair<std::string, long long>> int_attrs;
};

// POST `body` as application/json over plain HTTP (2 s socket timeouts); true on a 2xx answer.
bool http_post_json(const std::string& host, int port, const std::string& path, const std::string& body);

// One OTLP ExportTraceServiceRequest (JSON) for a batch of spans.
std::string encode_otlp(const std::vector<Span>& spans, const std::string& service_name);

class Exporter {
 public:
  // endpoint: http://host:port[/path]; a path-less endpoint gets /v1/traces
  Exporter(const std::string& endpoint, const std::string& service_name);
  ~Exporter();                                          // flushes what is queued
  void submit(Span&& s);
  uint64_t exported() const { return exported_; }
  uint64_t dropped() const { return dropped_; }

 private:
  void loop();
  bool post(const std::string& body);
  std::string host_, path_, service_;
  int port_ = 4318;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Span> queue_;
  bool stop_ = false;
  std::atomic<uint64_t> exported_{0}, dropped_{0};
  std::thread thread_;
};

// The span of the HTTP request that the calling thread is serving (invalid outside a traced request).
// The scheduler copies it into the queue entry so that the shard calls made for that request
// continue its trace (role of backends/grpc-metadata/src/lib.rs:1-41 in the reference).
void set_current(const Context& c);
const Context& current();

// process-wide exporter; null until `init` is called with a non-empty endpoint
void init(const std::string& endpoint, const std::string& service_name);
Exporter* exporter();
void shutdown();

}  // namespace trace
