#include "shard_client.hpp"

#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <future>
#include <stdexcept>
#include <thread>

namespace sched {

namespace {
enum Method : uint8_t { kInfo = 0, kServiceDiscovery, kClearCache, kFilterBatch, kWarmup, kPrefill, kDecode, kHealth };

void write_all(int fd, const char* p, size_t n) {
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w <= 0) throw std::runtime_error("shard connection: write failed");
    p += w;
    n -= static_cast<size_t>(w);
  }
}
void read_all(int fd, char* p, size_t n) {
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r <= 0) throw std::runtime_error("shard connection: closed by peer");
    p += r;
    n -= static_cast<size_t>(r);
  }
}
}  // namespace

FramedConnection::FramedConnection(const std::string& path) : path_(path) { connect_once(); }
FramedConnection::~FramedConnection() {
  if (fd_ >= 0) ::close(fd_);
}

void FramedConnection::connect_once() {
  fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd_ < 0) throw std::runtime_error("socket() failed");
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  if (path_.size() >= sizeof(addr.sun_path)) throw std::runtime_error("unix socket path too long");
  std::strcpy(addr.sun_path, path_.c_str());
  if (::connect(fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0) {
    ::close(fd_);
    fd_ = -1;
    throw std::runtime_error("cannot connect to shard at " + path_);
  }
}

std::string FramedConnection::call(uint8_t method, const std::string& payload, const std::string& traceparent) {
  std::lock_guard<std::mutex> g(m_);
  if (fd_ < 0) connect_once();
  const bool with_trace = traceparent.size() == 55;
  char head[5];
  head[0] = static_cast<char>(with_trace ? (method | 0x80) : method);
  const uint32_t n = static_cast<uint32_t>(payload.size());
  std::memcpy(head + 1, &n, 4);
  std::string body;
  char rh[5];
  try {
    write_all(fd_, head, 5);
    if (with_trace) write_all(fd_, traceparent.data(), 55);
    write_all(fd_, payload.data(), payload.size());
    read_all(fd_, rh, 5);
    uint32_t rn;
    std::memcpy(&rn, rh + 1, 4);
    body.assign(rn, '\0');
    if (rn) read_all(fd_, body.data(), rn);
  } catch (const std::runtime_error&) {
    // a transport failure leaves the stream out of sync: drop the socket, the next call reconnects
    ::close(fd_);
    fd_ = -1;
    throw;
  }
  if (rh[0] != 0) throw std::runtime_error(body);   // the shard answered with an error message
  return body;
}

std::shared_ptr<ShardedClient> ShardedClient::connect(const std::string& uds_path, int timeout_s) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout_s);
  std::unique_ptr<FramedConnection> first;
  while (true) {
    try {
      first = std::make_unique<FramedConnection>(uds_path + "-0.raw");
      break;
    } catch (const std::exception&) {
      if (std::chrono::steady_clock::now() > deadline) throw;
      std::this_thread::sleep_for(std::chrono::milliseconds(200));
    }
  }
  auto urls = pb::decode_service_discovery(first->call(kServiceDiscovery, ""));
  first.reset();
  std::vector<std::string> paths;
  for (auto& u : urls) {
    std::string p = u;
    const std::string prefix = "unix://";
    if (p.compare(0, prefix.size(), prefix) == 0) p = p.substr(prefix.size());
    paths.push_back(p + ".raw");
  }
  if (paths.empty()) paths.push_back(uds_path + "-0.raw");
  return std::make_shared<ShardedClient>(paths);
}

ShardedClient::ShardedClient(std::vector<std::string> paths) {
  for (auto& p : paths) conns_.push_back(std::make_unique<FramedConnection>(p));
}

std::vector<std::string> ShardedClient::all(uint8_t method, const std::string& payload) {
  std::vector<std::string> out(conns_.size());
  if (conns_.size() == 1) {
    out[0] = conns_[0]->call(method, payload, traceparent_);
    return out;
  }
  const std::string tp = traceparent_;
  std::vector<std::future<std::string>> fs;
  for (auto& c : conns_) fs.push_back(std::async(std::launch::async, [&c, method, &payload, &tp] { return c->call(method, payload, tp); }));
  std::exception_ptr err;
  for (size_t i = 0; i < fs.size(); ++i) {
    try {
      out[i] = fs[i].get();
    } catch (...) {
      err = std::current_exception();
    }
  }
  if (err) std::rethrow_exception(err);
  return out;
}

pb::InfoResponse ShardedClient::info() { return pb::InfoResponse::decode(all(kInfo, "")[0]); }
void ShardedClient::health() { all(kHealth, ""); }
void ShardedClient::clear_cache(std::optional<uint64_t> id) { all(kClearCache, pb::encode_clear_cache_request(id)); }

pb::CachedBatch ShardedClient::filter_batch(uint64_t batch_id, const std::vector<uint64_t>& ids) {
  return pb::decode_filter_response(all(kFilterBatch, pb::encode_filter_request(batch_id, ids))[0]);
}

pb::WarmupResponse ShardedClient::warmup(const pb::Batch& batch, std::optional<uint32_t> max_input_tokens,
                                         uint32_t max_prefill_tokens, std::optional<uint32_t> max_total_tokens) {
  auto raw = all(kWarmup, pb::encode_warmup_request(batch, max_input_tokens, max_prefill_tokens, max_total_tokens));
  pb::WarmupResponse out = pb::WarmupResponse::decode(raw[0]);
  for (size_t i = 1; i < raw.size(); ++i) {   // every limit is the minimum over the shards
    auto r = pb::WarmupResponse::decode(raw[i]);
    if (r.max_supported_total_tokens &&
        (!out.max_supported_total_tokens || *r.max_supported_total_tokens < *out.max_supported_total_tokens))
      out.max_supported_total_tokens = r.max_supported_total_tokens;
    out.max_input_tokens = std::min(out.max_input_tokens, r.max_input_tokens);
    out.max_total_tokens = std::min(out.max_total_tokens, r.max_total_tokens);
  }
  return out;
}

pb::StepResponse ShardedClient::merge(std::vector<std::string>& raw) {
  pb::StepResponse out = pb::StepResponse::decode(raw[0]);
  for (size_t i = 1; i < raw.size(); ++i) {
    auto r = pb::StepResponse::decode(raw[i]);
    for (auto& g : r.generations) out.generations.push_back(std::move(g));
    if (r.total_ns > out.total_ns) {   // report the slowest shard
      out.forward_ns = r.forward_ns;
      out.decode_ns = r.decode_ns;
      out.total_ns = r.total_ns;
      out.concat_ns = r.concat_ns;
    }
  }
  return out;
}

pb::StepResponse ShardedClient::prefill(const pb::Batch& batch, const pb::CachedBatch* cached) {
  auto raw = all(kPrefill, pb::encode_prefill_request(batch, cached));
  return merge(raw);
}

pb::StepResponse ShardedClient::decode(const std::vector<pb::CachedBatch>& batches) {
  auto raw = all(kDecode, pb::encode_decode_request(batches));
  return merge(raw);
}

}  // namespace sched
