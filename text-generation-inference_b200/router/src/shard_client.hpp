// Transport to the shard processes: the generate.v3 protobuf messages in length-prefixed frames
// over unix sockets (see serve_framed in server/server.py).  `ShardedClient` fans every call out to
// all shards in parallel, concatenates their generations and keeps the slowest shard's timings,
// like the reference's ShardedClient (backends/v3/src/client/sharded_client.rs:103-258).
#pragma once
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "scheduler.hpp"

namespace sched {

class FramedConnection {
 public:
  explicit FramedConnection(const std::string& path);
  ~FramedConnection();
  // throws std::runtime_error on transport errors and on an error status from the shard
  // A non-empty `traceparent` (55 characters, W3C trace context) travels in the frame header.
  std::string call(uint8_t method, const std::string& payload, const std::string& traceparent = "");

 private:
  void connect_once();
  std::string path_;
  int fd_ = -1;
  std::mutex m_;
};

class ShardedClient : public ShardClient {
 public:
  // `uds_path` is the path of shard 0 without the rank suffix (e.g. /tmp/text-generation-server)
  static std::shared_ptr<ShardedClient> connect(const std::string& uds_path, int timeout_s = 600);
  explicit ShardedClient(std::vector<std::string> paths);

  pb::InfoResponse info() override;
  void health() override;
  void clear_cache(std::optional<uint64_t> batch_id) override;
  pb::CachedBatch filter_batch(uint64_t batch_id, const std::vector<uint64_t>& request_ids) override;
  pb::WarmupResponse warmup(const pb::Batch& batch, std::optional<uint32_t> max_input_tokens,
                            uint32_t max_prefill_tokens, std::optional<uint32_t> max_total_tokens) override;
  pb::StepResponse prefill(const pb::Batch& batch, const pb::CachedBatch* cached) override;
  pb::StepResponse decode(const std::vector<pb::CachedBatch>& batches) override;
  void set_traceparent(const std::string& tp) override { traceparent_ = tp; }
  size_t num_shards() const { return conns_.size(); }

 private:
  std::vector<std::string> all(uint8_t method, const std::string& payload);
  static pb::StepResponse merge(std::vector<std::string>& raw);
  std::vector<std::unique_ptr<FramedConnection>> conns_;
  std::string traceparent_;   // written and read by the scheduler thread only
};

}  // namespace sched
