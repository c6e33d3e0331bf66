#include "scheduler.hpp"

#include <algorithm>
#include <cmath>

#include "metrics.hpp"

namespace sched {

// ------------------------------------------------------------------------------------------------
// Queue
// ------------------------------------------------------------------------------------------------
Queue::Queue(const QueueConfig& cfg) : cfg_(cfg) {
  if (!cfg.requires_padding) {
    const uint32_t blocks = (cfg.max_batch_total_tokens + cfg.block_size - 1) / cfg.block_size;
    allocator_ = std::make_unique<BlockAllocator>(std::max<uint32_t>(blocks, 2), cfg.block_size, cfg.prefix_caching,
                                                  cfg.window_size);
  }
}

uint64_t Queue::append(Entry e) {
  const uint64_t id = next_id_++;
  entries_.emplace_back(id, std::move(e));
  return id;
}

void Queue::release(Entry& e) {
  if (e.allocation && allocator_) {
    // an entry that never ran, or whose prefill failed or was cut short, has no KV beyond the prefix it
    // found in the cache: nothing of it may be inserted into the trie
    allocator_->free(e.allocation->blocks, e.allocation->allocation_id, e.prefill_done ? UINT32_MAX : 0);
    e.allocation.reset();
  }
}

std::optional<NextBatch> Queue::next_batch(std::optional<size_t> min_size, std::optional<size_t> max_size,
                                           uint32_t prefill_token_budget, uint32_t token_budget,
                                           std::unordered_map<uint64_t, Entry>& running) {
  if (entries_.empty()) return std::nullopt;
  if (min_size && entries_.size() < *min_size) return std::nullopt;
  if (max_size && *max_size == 0) return std::nullopt;
  // the prefill budget is rounded up to whole blocks
  prefill_token_budget = (prefill_token_budget + cfg_.block_size - 1) / cfg_.block_size * cfg_.block_size;

  struct Picked {
    uint64_t id;
    Entry entry;
    std::optional<uint32_t> chunk_len;
  };
  std::vector<Picked> batch;
  uint32_t max_input_length = 0, prefill_tokens = 0, decode_tokens = 0, max_blocks = 0;

  while (!entries_.empty()) {
    auto [id, entry] = std::move(entries_.front());
    entries_.pop_front();
    if (entry.stream->is_closed()) {   // the client went away while the request was queued
      ++dropped;
      continue;
    }
    const auto& rq = entry.request;
    std::optional<uint32_t> chunk_len;
    if (!allocator_) {
      // padded models: every row is as long as the longest prompt
      max_input_length = std::max(max_input_length, rq.input_length);
      prefill_tokens = static_cast<uint32_t>(batch.size() + 1) * max_input_length;
      decode_tokens += rq.stopping.max_new_tokens;
      const uint32_t total = prefill_tokens + decode_tokens + cfg_.speculate;
      if (prefill_tokens > prefill_token_budget || total > token_budget) {
        entries_.emplace_front(id, std::move(entry));
        break;
      }
    } else {
      // prompt logprobs need every prompt token recomputed: no prefix re-use for such requests
      const std::vector<uint32_t>* ids =
          (rq.decoder_input_details || rq.input_ids.empty()) ? nullptr : &rq.input_ids;
      const uint32_t tokens = rq.input_length + rq.stopping.max_new_tokens + cfg_.speculate - 1;
      auto alloc = allocator_->allocate(tokens, ids);
      if (!alloc) {   // out of blocks: try again once running requests finish
        entries_.emplace_front(id, std::move(entry));
        break;
      }
      max_blocks = std::max<uint32_t>(max_blocks, static_cast<uint32_t>(alloc->blocks.size()));
      if (alloc->prefix_len >= rq.input_length && rq.input_length > 0) {
        // the whole prompt is cached; the forward pass still needs one token to produce logits
        alloc->prefix_len = rq.input_length - 1;
      }
      const uint32_t postfix = rq.input_length - alloc->prefix_len;
      entry.allocation = std::move(alloc);
      if (prefill_tokens + postfix > prefill_token_budget) {
        if (cfg_.support_chunking) {
          const uint32_t room = prefill_token_budget > prefill_tokens ? prefill_token_budget - prefill_tokens : 0;
          if (room > 0) {
            batch.push_back(Picked{id, std::move(entry), room});
          } else {
            release(entry);
            entries_.emplace_front(id, std::move(entry));
          }
        } else {
          release(entry);
          entries_.emplace_front(id, std::move(entry));
        }
        break;
      }
      prefill_tokens += postfix;
    }
    batch.push_back(Picked{id, std::move(entry), chunk_len});
    if (max_size && batch.size() == *max_size) break;
  }
  if (batch.empty()) return std::nullopt;
  if (min_size && batch.size() < *min_size) {
    for (auto it = batch.rbegin(); it != batch.rend(); ++it) {
      release(it->entry);
      entries_.emplace_front(it->id, std::move(it->entry));
    }
    return std::nullopt;
  }
  (void)token_budget;
  NextBatch nb;
  nb.batch.id = next_batch_id_++;
  nb.batch.size = static_cast<uint32_t>(batch.size());
  nb.batch.max_blocks = max_blocks;
  uint32_t max_tokens = 0;
  const auto now = Clock::now();
  for (auto& p : batch) {
    const auto& rq = p.entry.request;
    pb::Request r;
    r.id = p.id;
    r.inputs = rq.inputs;
    r.input_chunks = rq.chunks;
    r.truncate = rq.truncate;
    r.add_special_tokens = rq.add_special_tokens;
    r.parameters = rq.parameters;
    r.stopping_parameters = rq.stopping;
    r.prefill_logprobs = rq.decoder_input_details;
    r.top_n_tokens = rq.top_n_tokens;
    r.adapter_id = rq.adapter_id;
    if (p.entry.allocation) {
      r.blocks = p.entry.allocation->blocks;
      r.slots = p.entry.allocation->slots;
      r.cache_len = p.entry.allocation->prefix_len;
    }
    r.chunk_len = p.chunk_len;
    max_tokens += rq.input_length + rq.stopping.max_new_tokens;
    nb.batch.requests.push_back(std::move(r));
    nb.ids.push_back(p.id);
    p.entry.batch_time = now;
    running.emplace(p.id, std::move(p.entry));
  }
  nb.batch.max_tokens = max_tokens;
  return nb;
}

// ------------------------------------------------------------------------------------------------
// Backend
// ------------------------------------------------------------------------------------------------
Backend::Backend(std::shared_ptr<ShardClient> client, const QueueConfig& qcfg, const BackendConfig& bcfg,
                 Metrics* metrics)
    : client_(std::move(client)), qcfg_(qcfg), bcfg_(bcfg), metrics_(metrics), queue_(qcfg) {}

Backend::~Backend() { stop(); }

void Backend::start_thread() {
  threaded_ = true;
  thread_ = std::thread([this] { run(); });
}

void Backend::stop() {
  stop_.store(true);
  inbox_cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

std::shared_ptr<ResponseStream> Backend::schedule(ValidRequest req) {
  Entry e;
  e.request = std::move(req);
  e.stream = std::make_shared<ResponseStream>();
  e.queue_time = Clock::now();
  e.trace = trace::current();
  auto stream = e.stream;
  {
    std::lock_guard<std::mutex> g(inbox_m_);
    inbox_.push_back(std::move(e));
  }
  inbox_cv_.notify_one();
  return stream;
}

size_t Backend::queue_size() {
  std::lock_guard<std::mutex> g(inbox_m_);
  return inbox_.size() + queue_.size();
}

void Backend::drain_inbox() {
  std::deque<Entry> got;
  {
    std::lock_guard<std::mutex> g(inbox_m_);
    got.swap(inbox_);
  }
  for (auto& e : got) queue_.append(std::move(e));
  if (metrics_) metrics_->gauge_set("tgi_queue_size", static_cast<double>(queue_.size()));
}

void Backend::run() {
  while (!stop_.load()) {
    const bool worked = step_once();
    if (!worked) {
      std::unique_lock<std::mutex> g(inbox_m_);
      inbox_cv_.wait_for(g, std::chrono::milliseconds(50), [&] { return stop_.load() || !inbox_.empty(); });
    }
  }
}

bool Backend::step_once() {
  drain_inbox();
  if (!cached_) {
    auto nb = queue_.next_batch(std::nullopt, bcfg_.max_batch_size, bcfg_.max_batch_prefill_tokens,
                                bcfg_.max_batch_total_tokens, running_);
    if (!nb) return false;
    cached_ = prefill(*nb, nullptr);
    waiting_tokens_ = 1;
    return true;
  }
  // a batch is running: try to admit more requests, then decode
  const uint32_t batch_size = cached_->size;
  const uint32_t batch_max_tokens = cached_->max_tokens;
  const uint32_t current_tokens = cached_->current_tokens;
  if (metrics_) {
    metrics_->gauge_set("tgi_batch_current_size", batch_size);
    metrics_->gauge_set("tgi_batch_current_max_tokens", batch_max_tokens);
  }
  const uint32_t token_budget =
      bcfg_.max_batch_total_tokens > batch_max_tokens ? bcfg_.max_batch_total_tokens - batch_max_tokens : 0;
  std::optional<size_t> min_size, max_size;
  uint32_t prefill_budget;
  if (qcfg_.support_chunking) {
    if (bcfg_.max_batch_size) max_size = *bcfg_.max_batch_size > batch_size ? *bcfg_.max_batch_size - batch_size : 0;
    prefill_budget =
        bcfg_.max_batch_prefill_tokens > current_tokens ? bcfg_.max_batch_prefill_tokens - current_tokens : 0;
  } else {
    // without chunking a new prefill stalls the running batch: only worth it for enough requests,
    // unless the queue has been waiting too long
    if (waiting_tokens_ < bcfg_.max_waiting_tokens)
      min_size = static_cast<size_t>(std::ceil(batch_size * bcfg_.waiting_served_ratio_x100 / 100.0));
    if (bcfg_.max_batch_size) max_size = *bcfg_.max_batch_size > batch_size ? *bcfg_.max_batch_size - batch_size : 0;
    prefill_budget = bcfg_.max_batch_prefill_tokens;
  }
  std::vector<pb::CachedBatch> batches;
  bool merged = false;
  if (prefill_budget > 0) {
    auto nb = queue_.next_batch(min_size, max_size, prefill_budget, token_budget, running_);
    if (nb) {
      if (metrics_) {
        const char* reason = qcfg_.support_chunking ? "chunking" : (min_size ? "backpressure" : "wait_exceeded");
        metrics_->counter_inc("tgi_batch_concat", {{"reason", reason}});
      }
      if (qcfg_.support_chunking) {
        // the shards concatenate the new requests to the running batch and run one forward for both
        pb::CachedBatch running_batch = *cached_;
        cached_ = prefill(*nb, &running_batch);
        merged = true;
      } else {
        auto fresh = prefill(*nb, nullptr);
        waiting_tokens_ = 1;
        if (fresh) batches.push_back(*fresh);
      }
    }
  }
  if (merged) return true;
  if (cached_) batches.insert(batches.begin(), *cached_);
  if (batches.empty()) {
    cached_.reset();
    return true;
  }
  cached_ = decode(batches);
  ++waiting_tokens_;
  return true;
}

void Backend::fail_entries(const std::vector<uint64_t>& ids, const std::string& msg) {
  for (uint64_t id : ids) {
    auto it = running_.find(id);
    if (it == running_.end()) continue;
    StreamEvent ev;
    ev.kind = StreamEvent::Error;
    ev.error = msg;
    ev.error_type = "generation";
    it->second.stream->push(std::move(ev));
    queue_.release(it->second);
    running_.erase(it);
  }
}

trace::Span Backend::begin_step_span(const char* name, const std::vector<uint64_t>& ids) {
  trace::Span span;
  for (uint64_t id : ids) {
    auto it = running_.find(id);
    if (it == running_.end() || !it->second.trace.valid()) continue;
    span.name = name;
    span.trace_id = it->second.trace.trace_id;
    span.parent_span_id = it->second.trace.span_id;
    span.span_id = trace::random_hex(16);
    span.kind = 3;   // SPAN_KIND_CLIENT
    span.start_ns = trace::now_ns();
    span.int_attrs.emplace_back("batch.size", static_cast<long long>(ids.size()));
    break;
  }
  client_->set_traceparent(span.name.empty() ? std::string()
                                             : trace::format_traceparent(trace::Context{span.trace_id, span.span_id, true}));
  return span;
}

void Backend::end_step_span(trace::Span& span, bool failed) {
  client_->set_traceparent("");
  if (span.name.empty() || trace::exporter() == nullptr) return;
  span.end_ns = trace::now_ns();
  span.error = failed;
  trace::exporter()->submit(std::move(span));
}

std::optional<pb::CachedBatch> Backend::prefill(NextBatch& nb, const pb::CachedBatch* cached) {
  const auto t0 = Clock::now();
  if (metrics_) metrics_->counter_inc("tgi_batch_inference_count", {{"method", "prefill"}});
  trace::Span span = begin_step_span("prefill", nb.ids);
  try {
    pb::StepResponse resp = client_->prefill(nb.batch, cached);
    end_step_span(span, false);
    if (metrics_) {
      metrics_->observe("tgi_batch_forward_duration", resp.forward_ns * 1e-9, {{"method", "prefill"}});
      metrics_->observe("tgi_batch_decode_duration", resp.decode_ns * 1e-9, {{"method", "prefill"}});
      metrics_->observe("tgi_batch_inference_duration",
                        std::chrono::duration<double>(Clock::now() - t0).count(), {{"method", "prefill"}});
      metrics_->counter_inc("tgi_batch_inference_success", {{"method", "prefill"}});
    }
    return after_step(resp, "prefill");
  } catch (const std::exception& e) {
    end_step_span(span, true);
    std::vector<uint64_t> ids = nb.ids;
    if (cached) ids.insert(ids.end(), cached->request_ids.begin(), cached->request_ids.end());
    try {
      client_->clear_cache(nb.batch.id);
      if (cached) client_->clear_cache(cached->id);
    } catch (...) {
    }
    if (metrics_) metrics_->counter_inc("tgi_batch_inference_failure", {{"method", "prefill"}});
    fail_entries(ids, e.what());
    return std::nullopt;
  }
}

std::optional<pb::CachedBatch> Backend::decode(std::vector<pb::CachedBatch>& batches) {
  const auto t0 = Clock::now();
  if (metrics_) metrics_->counter_inc("tgi_batch_inference_count", {{"method", "decode"}});
  std::vector<uint64_t> step_ids;
  for (auto& b : batches) step_ids.insert(step_ids.end(), b.request_ids.begin(), b.request_ids.end());
  trace::Span span = begin_step_span("decode", step_ids);
  try {
    pb::StepResponse resp = client_->decode(batches);
    end_step_span(span, false);
    if (metrics_) {
      metrics_->observe("tgi_batch_forward_duration", resp.forward_ns * 1e-9, {{"method", "decode"}});
      metrics_->observe("tgi_batch_decode_duration", resp.decode_ns * 1e-9, {{"method", "decode"}});
      if (resp.concat_ns) metrics_->observe("tgi_batch_concat_duration", *resp.concat_ns * 1e-9, {{"method", "decode"}});
      metrics_->observe("tgi_batch_inference_duration",
                        std::chrono::duration<double>(Clock::now() - t0).count(), {{"method", "decode"}});
      metrics_->counter_inc("tgi_batch_inference_success", {{"method", "decode"}});
    }
    return after_step(resp, "decode");
  } catch (const std::exception& e) {
    end_step_span(span, true);
    std::vector<uint64_t> ids;
    for (auto& b : batches) {
      ids.insert(ids.end(), b.request_ids.begin(), b.request_ids.end());
      try {
        client_->clear_cache(b.id);
      } catch (...) {
      }
    }
    if (metrics_) metrics_->counter_inc("tgi_batch_inference_failure", {{"method", "decode"}});
    fail_entries(ids, e.what());
    return std::nullopt;
  }
}

void Backend::send_generation(Entry& e, pb::Generation& g, bool& finished) {
  finished = false;
  if (e.stream->is_closed()) {   // client disconnected: stop generating for it
    finished = true;
    return;
  }
  if (g.prefill_tokens && !g.prefill_tokens->ids.empty()) {
    StreamEvent ev;
    ev.kind = StreamEvent::Prefill;
    const auto& pt = *g.prefill_tokens;
    for (size_t i = 0; i < pt.ids.size(); ++i) {
      Token t;
      t.id = pt.ids[i];
      t.text = i < pt.texts.size() ? pt.texts[i] : "";
      t.logprob = i < pt.logprobs.size() ? pt.logprobs[i] : 0.f;
      ev.prefill_tokens.push_back(std::move(t));
    }
    e.stream->push(std::move(ev));
  }
  const size_t n = g.tokens.ids.size();
  if (n > 0) e.prefill_done = true;
  if (metrics_ && n > 0) metrics_->histogram_value("tgi_request_skipped_tokens", static_cast<double>(n - 1));   // speculated tokens accepted
  for (size_t i = 0; i < n; ++i) {
    StreamEvent ev;
    ev.token.id = g.tokens.ids[i];
    ev.token.text = i < g.tokens.texts.size() ? g.tokens.texts[i] : "";
    ev.token.logprob = i < g.tokens.logprobs.size() ? g.tokens.logprobs[i] : 0.f;
    ev.token.special = i < g.tokens.is_special.size() ? g.tokens.is_special[i] : false;
    if (i < g.top_tokens.size()) {
      const auto& tt = g.top_tokens[i];
      for (size_t k = 0; k < tt.ids.size(); ++k) {
        Token t;
        t.id = tt.ids[k];
        t.text = k < tt.texts.size() ? tt.texts[k] : "";
        t.logprob = k < tt.logprobs.size() ? tt.logprobs[k] : 0.f;
        t.special = k < tt.is_special.size() ? tt.is_special[k] : false;
        ev.top_tokens.push_back(std::move(t));
      }
    }
    const bool last = (i + 1 == n) && g.generated_text.has_value();
    if (last) {
      ev.kind = StreamEvent::End;
      ev.generated_text = g.generated_text;
      ev.queued = e.queue_time;
      ev.start = e.batch_time.value_or(e.queue_time);
      finished = true;
    } else {
      ev.kind = StreamEvent::Intermediate;
    }
    e.stream->push(std::move(ev));
  }
}

std::optional<pb::CachedBatch> Backend::after_step(pb::StepResponse& resp, const char* method) {
  const auto t0 = Clock::now();
  for (auto& g : resp.generations) {
    auto it = running_.find(g.request_id);
    if (it == running_.end()) continue;
    bool finished = false;
    send_generation(it->second, g, finished);
    if (finished) {
      queue_.release(it->second);
      running_.erase(it);
    }
  }
  std::optional<pb::CachedBatch> next = resp.batch;
  if (next) {
    // drop requests that finished or whose client disconnected from the shard-side batch
    std::vector<uint64_t> keep;
    for (uint64_t id : next->request_ids) {
      auto it = running_.find(id);
      if (it == running_.end()) continue;
      if (it->second.stream->is_closed()) {
        queue_.release(it->second);
        running_.erase(it);
        continue;
      }
      keep.push_back(id);
    }
    if (keep.size() != next->request_ids.size()) {
      try {
        if (keep.empty()) {
          client_->clear_cache(next->id);
          next.reset();
        } else {
          next = client_->filter_batch(next->id, keep);
        }
      } catch (const std::exception& e) {
        fail_entries(keep, std::string("filter_batch failed: ") + e.what());
        next.reset();
      }
    }
  } else {
    // the shards consider every request finished; anything we still track is an error
    if (!running_.empty() && !cached_) {
      std::vector<uint64_t> ids;
      for (auto& kv : running_) ids.push_back(kv.first);
      // entries of other (not yet merged) batches do not exist in this design: all running belong here
      fail_entries(ids, "request disappeared from the running batch");
    }
  }
  if (metrics_) {
    metrics_->observe("tgi_batch_filter_duration", std::chrono::duration<double>(Clock::now() - t0).count(),
                      {{"method", method}});
    metrics_->histogram_value("tgi_batch_next_size", next ? next->size : 0);
  }
  return next;
}

bool Backend::health(bool current_health) {
  if (current_health) {
    try {
      client_->health();
      return true;
    } catch (...) {
      return false;
    }
  }
  // after a failure: prove the shards can run a model step on the reserved block 0
  try {
    pb::Batch b;
    b.id = UINT64_MAX;
    b.size = 1;
    b.max_tokens = 2;
    b.max_blocks = 1;
    pb::Request r;
    r.id = UINT64_MAX;
    r.inputs = "liveness";
    pb::InputChunk c;
    c.text = "liveness";
    r.input_chunks.push_back(c);
    r.truncate = 10;
    r.parameters.temperature = 1.f;
    r.parameters.top_p = 1.f;
    r.parameters.typical_p = 1.f;
    r.parameters.repetition_penalty = 1.f;
    r.stopping_parameters.max_new_tokens = 1;
    r.blocks = {0};
    for (uint32_t s = 0; s < qcfg_.block_size; ++s) r.slots.push_back(s);
    r.add_special_tokens = true;
    b.requests.push_back(r);
    auto resp = client_->prefill(b, nullptr);
    if (resp.batch) client_->clear_cache(resp.batch->id);
    return true;
  } catch (...) {
    return false;
  }
}

}  // namespace sched
