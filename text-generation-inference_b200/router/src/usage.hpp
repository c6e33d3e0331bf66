// Usage statistics of the router: the events the reference reports (start, ping, stop, error) with the same payload
// (a random id for the run, the reduced launch arguments, a description of the host), delivered to a sink the
// operator names.
//
// Reference: `router/src/usage_stats.rs:1-414` (payload, container detection, host probes) and
// `router/src/server.rs:1745-1870` (when events are sent).  The reference posts to a fixed address of its vendor;
// this router sends nothing anywhere unless `--usage-stats-endpoint http://host:port/path` names a collector, and
// otherwise appends the events as JSON lines to `--usage-stats-file` when that is given.  Levels as in the
// reference: `on` (error events carry the message), `no-stack` (error events carry "unknown_error"), `off`.
#pragma once
#include <atomic>
#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>

#include "json.hpp"

namespace usage {

bool is_container();                       // /.dockerenv, or a container runtime named in /proc/self/cgroup
json::Value host_description();            // cpu, memory, platform, accelerator names (read-only probes)

class Reporter {
 public:
  // level: on | no-stack | off.  endpoint / file may be empty.
  Reporter(const std::string& level, const std::string& endpoint, const std::string& file, json::Value args);
  ~Reporter();
  bool enabled() const { return level_ != "off"; }
  std::string event(const std::string& type, const std::string& error_reason = "") const;   // the JSON document
  void send(const std::string& type, const std::string& error_reason = "");
  void start_pings(int interval_s);        // a Ping event every interval until the reporter is destroyed

 private:
  std::string level_, host_, path_, file_, uid_;
  int port_ = 80;
  json::Value args_, env_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::thread ping_;
};

}  // namespace usage
