// Continuous-batching scheduler: request queue, batch builder, and the batching loop that drives
// the shards (Prefill / Decode / FilterBatch / ClearCache).
//
// Covers the reference's `Queue` + `State::next_batch` (backends/v3/src/queue.rs:22-504) and
// `BackendV3` batching task (backends/v3/src/backend.rs:129-554): token budgets, block allocation
// per admitted request, splitting the last admitted prompt to exactly fill the prefill budget when
// the shards support chunking, back-off when blocks run out, dropping cancelled requests, filtering
// finished requests out of the running batch, and failing a whole batch on a shard error.
//
// Threading: one scheduler thread owns the queue, the allocator and the entries; HTTP threads hand
// requests over through a mutex-protected inbox and read results from a per-request stream.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "pb.hpp"
#include "radix.hpp"
#include "trace.hpp"

namespace sched {

using Clock = std::chrono::steady_clock;

// ---- what flows back to the HTTP layer -------------------------------------------------------
struct Token {
  uint32_t id = 0;
  std::string text;
  float logprob = 0.f;
  bool special = false;
};

struct StreamEvent {
  enum Kind { Prefill, Intermediate, End, Error } kind = Intermediate;
  std::vector<Token> prefill_tokens;               // Prefill
  Token token;                                     // Intermediate / End
  std::vector<Token> top_tokens;
  std::optional<pb::GeneratedText> generated_text; // End
  Clock::time_point queued, start;                 // End
  std::string error, error_type;                   // Error
};

// Thread-safe single-consumer stream of events for one request.
class ResponseStream {
 public:
  void push(StreamEvent ev) {
    {
      std::lock_guard<std::mutex> g(m_);
      q_.push_back(std::move(ev));
    }
    cv_.notify_one();
  }
  // false on timeout
  bool pop(StreamEvent& out, int timeout_ms) {
    std::unique_lock<std::mutex> g(m_);
    if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !q_.empty(); })) return false;
    out = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  void close() { closed_.store(true); }          // consumer went away (client disconnected)
  bool is_closed() const { return closed_.load(); }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  std::deque<StreamEvent> q_;
  std::atomic<bool> closed_{false};
};

// ---- validated request ------------------------------------------------------------------------
struct ValidRequest {
  std::string inputs;
  std::vector<pb::InputChunk> chunks;
  std::vector<uint32_t> input_ids;      // empty when the tokenizer is not available to the router
  uint32_t input_length = 0;
  uint32_t truncate = 0;
  bool add_special_tokens = true;
  bool decoder_input_details = false;
  pb::NextTokenChooserParameters parameters;
  pb::StoppingCriteriaParameters stopping;
  uint32_t top_n_tokens = 0;
  std::optional<std::string> adapter_id;
};

struct Entry {
  ValidRequest request;
  std::shared_ptr<ResponseStream> stream;
  Clock::time_point queue_time;
  std::optional<Clock::time_point> batch_time;
  std::optional<BlockAllocation> allocation;
  // set once the shards returned the first generated token: from then on the KV of the whole prompt
  // exists and its blocks may enter the prefix cache when the entry is released
  bool prefill_done = false;
  trace::Context trace;   // span of the HTTP request, when it is traced
};

struct NextBatch {
  pb::Batch batch;
  std::vector<uint64_t> ids;
};

struct QueueConfig {
  bool requires_padding = false;
  uint32_t block_size = 16;
  bool prefix_caching = true;
  std::optional<uint32_t> window_size;
  uint32_t speculate = 0;
  bool support_chunking = true;
  uint32_t max_batch_total_tokens = 0;
};

// The pending-request FIFO and the batch builder.  Not thread-safe: owned by the scheduler thread.
class Queue {
 public:
  explicit Queue(const QueueConfig& cfg);

  uint64_t append(Entry e);
  size_t size() const { return entries_.size(); }
  BlockAllocator* allocator() { return allocator_.get(); }

  // Entries admitted by the last next_batch() are moved into `running`.
  std::optional<NextBatch> next_batch(std::optional<size_t> min_size, std::optional<size_t> max_size,
                                      uint32_t prefill_token_budget, uint32_t token_budget,
                                      std::unordered_map<uint64_t, Entry>& running);
  void release(Entry& e);   // give the entry's blocks back

  uint64_t dropped = 0;

 private:
  QueueConfig cfg_;
  std::deque<std::pair<uint64_t, Entry>> entries_;
  std::unique_ptr<BlockAllocator> allocator_;
  uint64_t next_id_ = 0;
  uint64_t next_batch_id_ = 0;
};

// ---- shard transport ---------------------------------------------------------------------------
class ShardClient {
 public:
  virtual ~ShardClient() = default;
  virtual pb::InfoResponse info() = 0;
  virtual void health() = 0;
  virtual void clear_cache(std::optional<uint64_t> batch_id) = 0;
  virtual pb::CachedBatch filter_batch(uint64_t batch_id, const std::vector<uint64_t>& request_ids) = 0;
  virtual pb::WarmupResponse warmup(const pb::Batch& batch, std::optional<uint32_t> max_input_tokens,
                                    uint32_t max_prefill_tokens, std::optional<uint32_t> max_total_tokens) = 0;
  virtual pb::StepResponse prefill(const pb::Batch& batch, const pb::CachedBatch* cached) = 0;
  virtual pb::StepResponse decode(const std::vector<pb::CachedBatch>& batches) = 0;
  // W3C `traceparent` sent along with the following calls of this thread's owner ("" = none)
  virtual void set_traceparent(const std::string&) {}
};

struct Metrics;   // metrics.hpp

struct BackendConfig {
  uint32_t waiting_served_ratio_x100 = 30;   // 0.3
  uint32_t max_batch_prefill_tokens = 4096;
  uint32_t max_batch_total_tokens = 16384;
  uint32_t max_waiting_tokens = 20;
  std::optional<size_t> max_batch_size;
};

// The batching loop.  `schedule()` may be called from any thread.
class Backend {
 public:
  Backend(std::shared_ptr<ShardClient> client, const QueueConfig& qcfg, const BackendConfig& bcfg,
          Metrics* metrics = nullptr);
  ~Backend();

  std::shared_ptr<ResponseStream> schedule(ValidRequest req);
  bool health(bool current_health);
  void stop();
  // one pass of the loop body; exposed so tests can drive the scheduler deterministically
  bool step_once();
  size_t queue_size();

 private:
  void run();
  void drain_inbox();
  std::optional<pb::CachedBatch> prefill(NextBatch& nb, const pb::CachedBatch* cached);
  std::optional<pb::CachedBatch> decode(std::vector<pb::CachedBatch>& batches);
  std::optional<pb::CachedBatch> after_step(pb::StepResponse& resp, const char* method);
  void fail_entries(const std::vector<uint64_t>& ids, const std::string& msg);
  void send_generation(Entry& e, pb::Generation& g, bool& finished);
  // Opens the span of one shard step as a child of the first traced request among `ids`, hands its
  // `traceparent` to the shard client and returns the span (name empty when nothing is traced).
  trace::Span begin_step_span(const char* name, const std::vector<uint64_t>& ids);
  void end_step_span(trace::Span& span, bool failed);

  std::shared_ptr<ShardClient> client_;
  QueueConfig qcfg_;
  BackendConfig bcfg_;
  Metrics* metrics_;
  Queue queue_;
  std::unordered_map<uint64_t, Entry> running_;
  std::optional<pb::CachedBatch> cached_;
  uint32_t waiting_tokens_ = 1;

  std::mutex inbox_m_;
  std::condition_variable inbox_cv_;
  std::deque<Entry> inbox_;
  std::atomic<bool> stop_{false};
  std::thread thread_;
  bool threaded_ = false;

 public:
  void start_thread();
};

}  // namespace sched
