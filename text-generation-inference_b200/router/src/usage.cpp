#include "usage.hpp"

#include <sys/utsname.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "trace.hpp"

namespace usage {

namespace {

std::string first_line_after(const std::string& path, const std::string& key) {
  std::ifstream f(path);
  std::string line;
  while (std::getline(f, line)) {
    if (line.rfind(key, 0) != 0) continue;
    size_t colon = line.find(':');
    if (colon == std::string::npos) continue;
    size_t b = line.find_first_not_of(" \t", colon + 1);
    return b == std::string::npos ? "" : line.substr(b);
  }
  return "";
}

// output of a read-only query tool, or "" when the tool is missing (2 KB at most)
std::string run_query(const char* cmd) {
  std::string out;
  FILE* p = popen(cmd, "r");
  if (p == nullptr) return out;
  char buf[256];
  while (out.size() < 2048 && fgets(buf, sizeof buf, p) != nullptr) out += buf;
  pclose(p);
  while (!out.empty() && (out.back() == '\n' || out.back() == '\r')) out.pop_back();
  return out;
}

// version-4 UUID from the tracing module's random source
std::string uuid4() {
  std::string h = trace::random_hex(32);
  h[12] = '4';
  h[16] = "89ab"[(h[16] >= 'a' ? h[16] - 'a' + 10 : h[16] - '0') & 3];
  return h.substr(0, 8) + "-" + h.substr(8, 4) + "-" + h.substr(12, 4) + "-" + h.substr(16, 4) + "-" + h.substr(20, 12);
}

}  // namespace

bool is_container() {
  if (access("/.dockerenv", F_OK) == 0) return true;
  std::ifstream f("/proc/self/cgroup");
  std::string line;
  while (std::getline(f, line))
    for (const char* marker : {"docker", "kubepods", "containerd", "lxc"})
      if (line.find(marker) != std::string::npos) return true;
  return false;
}

json::Value host_description() {
  json::Value env = json::Value::object();
  const char* sha = std::getenv("GIT_SHA");
  const char* label = std::getenv("DOCKER_LABEL");
  env.set("git_sha", sha ? sha : "unknown");
  env.set("docker_label", label ? label : "unknown");
  env.set("cpu_count", static_cast<long>(sysconf(_SC_NPROCESSORS_ONLN)));
  env.set("cpu_type", first_line_after("/proc/cpuinfo", "model name"));
  const std::string mem = first_line_after("/proc/meminfo", "MemTotal");        // "<n> kB"
  env.set("total_memory", static_cast<long long>(std::strtoll(mem.c_str(), nullptr, 10)) * 1024);
  utsname u{};
  if (uname(&u) == 0) {
    env.set("architecture", std::string(u.machine));
    env.set("platform", std::string(u.sysname) + "-" + u.release);
  }
  env.set("is_container", is_container());
  // accelerator names as the vendor's query tool prints them (a read of the inventory, nothing is changed)
  const std::string gpus = run_query("nvidia-smi --query-gpu=name,driver_version,memory.total --format=csv,noheader 2>/dev/null");
  json::Value list = json::Value::array();
  std::stringstream ss(gpus);
  std::string line;
  while (std::getline(ss, line))
    if (!line.empty()) list.push(line);
  env.set("nvidia_info", list);
  return env;
}

Reporter::Reporter(const std::string& level, const std::string& endpoint, const std::string& file, json::Value args)
    : level_(level == "on" || level == "no-stack" ? level : "off"), file_(file), uid_(uuid4()), args_(std::move(args)) {
  if (!enabled()) return;
  env_ = host_description();
  std::string rest = endpoint;
  const std::string scheme = "http://";
  if (rest.rfind(scheme, 0) == 0) rest = rest.substr(scheme.size());
  if (!rest.empty()) {
    size_t slash = rest.find('/');
    path_ = slash == std::string::npos ? "/" : rest.substr(slash);
    std::string hostport = slash == std::string::npos ? rest : rest.substr(0, slash);
    size_t colon = hostport.rfind(':');
    if (colon != std::string::npos) {
      port_ = std::atoi(hostport.c_str() + colon + 1);
      hostport = hostport.substr(0, colon);
    }
    host_ = hostport;
  }
}

Reporter::~Reporter() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (ping_.joinable()) ping_.join();
}

std::string Reporter::event(const std::string& type, const std::string& error_reason) const {
  json::Value ua = json::Value::object();
  ua.set("uid", uid_);
  ua.set("args", args_);
  ua.set("env", env_);
  json::Value ev = json::Value::object();
  ev.set("user_agent", ua);
  ev.set("event_type", type);
  if (type == "Error") ev.set("error_reason", level_ == "on" ? error_reason : std::string("unknown_error"));
  return ev.dump();
}

void Reporter::send(const std::string& type, const std::string& error_reason) {
  if (!enabled()) return;
  const std::string body = event(type, error_reason);
  if (!host_.empty()) trace::http_post_json(host_, port_, path_, body);
  if (!file_.empty()) {
    std::lock_guard<std::mutex> g(mu_);
    std::ofstream f(file_, std::ios::app);
    f << body << "\n";
  }
}

void Reporter::start_pings(int interval_s) {
  if (!enabled() || interval_s <= 0 || ping_.joinable()) return;
  ping_ = std::thread([this, interval_s] {
    std::unique_lock<std::mutex> lk(mu_);
    while (!stop_) {
      if (cv_.wait_for(lk, std::chrono::seconds(interval_s), [this] { return stop_; })) break;
      lk.unlock();
      send("Ping");
      lk.lock();
    }
  });
}

}  // namespace usage
