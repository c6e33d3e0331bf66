#include "api.hpp"
#include "images.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <ctime>
#include <sstream>

namespace api {

using json::Value;
using sched::Clock;

namespace {

double seconds_since(Clock::time_point t) { return std::chrono::duration<double>(Clock::now() - t).count(); }

double num_or(const Value& obj, const char* key, double dflt) {
  const Value* v = obj.find(key);
  return (v && v->is_number()) ? v->as_double() : dflt;
}
bool bool_or(const Value& obj, const char* key, bool dflt) {
  const Value* v = obj.find(key);
  return (v && v->is_bool()) ? v->as_bool() : dflt;
}

Value token_json(const sched::Token& t, bool with_special) {
  Value o = Value::object();
  o.set("id", t.id);
  o.set("text", t.text);
  if (std::isnan(t.logprob)) o.set("logprob", Value());
  else o.set("logprob", static_cast<double>(t.logprob));
  if (with_special) o.set("special", t.special);
  return o;
}

std::string sse(const Value& v) { return "data:" + v.dump() + "\n\n"; }

}  // namespace

std::string finish_reason_str(uint32_t r, bool openai) {
  switch (r) {
    case 0: return "length";
    case 1: return openai ? "stop" : "eos_token";
    default: return openai ? "stop" : "stop_sequence";
  }
}

Router::Router(std::shared_ptr<sched::Backend> backend, TextServices text, RouterConfig cfg, sched::Metrics* metrics)
    : backend_(std::move(backend)), text_(std::move(text)), cfg_(std::move(cfg)), metrics_(metrics) {}

std::unique_ptr<Router::Permit> Router::acquire() {
  // limit of requests in flight; beyond it the client gets 429 instead of an ever longer queue
  size_t now = ++in_flight_;
  if (now > cfg_.max_concurrent_requests) {
    --in_flight_;
    if (metrics_) metrics_->counter_inc("tgi_request_failure", {{"err", "overloaded"}});
    throw ApiError(429, "overloaded", "Model is overloaded");
  }
  auto p = std::make_unique<Permit>();
  p->counter = &in_flight_;
  return p;
}

void Router::send_error(http::Response& resp, const ApiError& e) {
  Value o = Value::object();
  o.set("error", std::string(e.what()));
  o.set("error_type", e.type);
  if (!resp.started()) resp.send(e.status, "application/json", o.dump());
}

// ------------------------------------------------------------------------------------------------
// validation (ranges as in the reference: router/src/validation.rs:204-447)
// ------------------------------------------------------------------------------------------------
GenerateParams Router::validate(const std::string& inputs, const Value& p) {
  GenerateParams g;
  if (inputs.empty()) throw validation_error("`inputs` cannot be empty");
  auto& v = g.valid;
  const double best_of = num_or(p, "best_of", 1);
  if (best_of < 1) throw validation_error("`best_of` must be strictly positive");
  if (best_of > cfg_.max_best_of)
    throw validation_error("`best_of` must be > 0 and <= " + std::to_string(cfg_.max_best_of) + ". Given: " +
                           std::to_string(static_cast<int>(best_of)));
  if (best_of > 1) g.best_of = static_cast<uint32_t>(best_of);

  const double temperature = num_or(p, "temperature", 1.0);
  if (p.has("temperature") && temperature <= 0) throw validation_error("`temperature` must be strictly positive");
  const double rep = num_or(p, "repetition_penalty", 1.0);
  if (rep <= 0) throw validation_error("`repetition_penalty` must be strictly positive");
  const double freq = num_or(p, "frequency_penalty", 0.0);
  if (freq < -2.0 || freq > 2.0) throw validation_error("`frequency_penalty` must be >= -2.0 and <= 2.0");
  double top_p = 1.0;
  if (p.has("top_p")) {
    top_p = p["top_p"].as_double();
    if (top_p <= 0.0 || top_p >= 1.0) throw validation_error("`top_p` must be > 0.0 and < 1.0");
  }
  double typical_p = 1.0;
  if (p.has("typical_p")) {
    typical_p = p["typical_p"].as_double();
    if (typical_p <= 0.0 || typical_p >= 1.0) throw validation_error("`typical_p` must be > 0.0 and < 1.0");
  }
  uint32_t top_k = 0;
  if (p.has("top_k")) {
    if (p["top_k"].as_double() <= 0) throw validation_error("`top_k` must be strictly positive");
    top_k = static_cast<uint32_t>(p["top_k"].as_int());
  }
  const bool do_sample = bool_or(p, "do_sample", false);
  if (g.best_of) {
    const bool sampling = do_sample || temperature != 1.0 || top_k != 0 || top_p < 1.0 || typical_p < 1.0;
    if (!sampling) throw validation_error("you must use sampling when `best_of` is > 1");
    if (p.has("seed")) throw validation_error("`seed` must not be set when `best_of` > 1");
  }
  uint32_t top_n = 0;
  if (p.has("top_n_tokens")) {
    const double t = p["top_n_tokens"].as_double();
    if (t < 0 || t > cfg_.max_top_n_tokens)
      throw validation_error("`top_n_tokens` must be >= 0 and <= " + std::to_string(cfg_.max_top_n_tokens));
    top_n = static_cast<uint32_t>(t);
  }
  std::vector<std::string> stops;
  if (p.has("stop")) {
    for (const auto& s : p["stop"].items())
      if (s.is_string()) stops.push_back(s.as_string());
    if (stops.size() > cfg_.max_stop_sequences)
      throw validation_error("`stop` supports up to " + std::to_string(cfg_.max_stop_sequences) +
                             " stop sequences. Given: " + std::to_string(stops.size()));
  }
  uint32_t truncate = 0;
  if (p.has("truncate")) {
    const double t = p["truncate"].as_double();
    if (t <= 0 || t > cfg_.max_input_tokens)
      throw validation_error("`truncate` must be strictly positive and less than " +
                             std::to_string(cfg_.max_input_tokens));
    truncate = static_cast<uint32_t>(t);
  }
  if (p.has("max_new_tokens")) {
    const double m = p["max_new_tokens"].as_double();
    if (m <= 0) throw validation_error("`max_new_tokens` must be strictly positive");
    g.max_new_tokens = static_cast<uint32_t>(m);
  }
  // tokenise (the scheduler needs the ids for prefix caching and the length for its budgets)
  const bool add_special = bool_or(p, "add_special_tokens", true);
  std::vector<images::Piece> pieces;
  if (images::tokens_per_image(cfg_.model_config, 1, 1) > 0) pieces = images::split_markdown(inputs);
  bool has_image = false;
  for (const auto& pc : pieces) has_image = has_image || pc.is_image;
  if (has_image) {
    // vision-language request: text pieces are tokenised on their own, every image contributes
    // placeholder ids (derived from its bytes, so the prefix cache tells images apart)
    if (truncate) throw validation_error("`truncate` cannot be combined with image inputs");
    bool first_text = true;
    bool after_image = false;     // the previous piece was an image: Idefics2 lets adjacent images share a marker
    for (const auto& pc : pieces) {
      pb::InputChunk c;
      if (!pc.is_image) {
        if (pc.text.empty()) continue;
        after_image = false;
        const bool wrap = cfg_.model_config.is_object() && cfg_.model_config.has("_text_wrap");
        auto ids = wrap ? text_.encode(cfg_.model_config["_text_wrap"]["prefix"].as_string() + pc.text +
                                           cfg_.model_config["_text_wrap"]["suffix"].as_string(), false, 0)
                        : text_.encode(pc.text, add_special && first_text, 0);
        first_text = false;
        v.input_ids.insert(v.input_ids.end(), ids.begin(), ids.end());
        c.text = pc.text;
      } else {
        images::Fetched img;
        try {
          img = images::fetch(pc.text, cfg_.max_image_bytes);
        } catch (const std::exception& e) {
          throw validation_error(std::string("invalid image: ") + e.what());
        }
        uint32_t n = images::tokens_per_image(cfg_.model_config, img.width, img.height);
        if (after_image && cfg_.model_config.has("_idefics2") && n > 0) --n;
        after_image = true;
        for (uint32_t i = 0; i < n; ++i) v.input_ids.push_back(images::placeholder_id(img.data, i));
        c.is_image = true;
        c.data = std::move(img.data);
        c.mimetype = img.mimetype;
      }
      v.chunks.push_back(std::move(c));
    }
  } else {
    v.input_ids = text_.encode(inputs, add_special, truncate);
  }
  v.input_length = static_cast<uint32_t>(v.input_ids.size());
  if (v.input_length == 0) throw validation_error("`inputs` cannot be empty");
  if (v.input_length > cfg_.max_input_tokens)
    throw validation_error("`inputs` must have less than " + std::to_string(cfg_.max_input_tokens) +
                           " tokens. Given: " + std::to_string(v.input_length));
  uint32_t max_new;
  if (g.max_new_tokens) {
    max_new = *g.max_new_tokens;
    g.max_total_new_tokens = max_new;
  } else {
    // default: whatever the context still holds, served in legs of at most 1024 tokens
    const uint32_t room = cfg_.max_total_tokens > v.input_length ? cfg_.max_total_tokens - v.input_length : 0;
    g.max_total_new_tokens = room;
    max_new = std::min<uint32_t>(room, 1024);
  }
  if (max_new == 0 || v.input_length + max_new > cfg_.max_total_tokens)
    throw validation_error("`inputs` tokens + `max_new_tokens` must be <= " + std::to_string(cfg_.max_total_tokens) +
                           ". Given: " + std::to_string(v.input_length) + " `inputs` tokens and " +
                           std::to_string(max_new) + " `max_new_tokens`");
  v.inputs = inputs;
  if (!has_image) {
    pb::InputChunk chunk;
    chunk.text = inputs;
    v.chunks.push_back(chunk);
  }
  v.truncate = truncate;
  v.add_special_tokens = add_special;
  v.top_n_tokens = top_n;
  v.decoder_input_details = bool_or(p, "decoder_input_details", false);
  v.parameters.temperature = static_cast<float>(temperature);
  v.parameters.top_k = top_k;
  v.parameters.top_p = static_cast<float>(top_p);
  v.parameters.typical_p = static_cast<float>(typical_p);
  v.parameters.do_sample = do_sample;
  v.parameters.repetition_penalty = static_cast<float>(rep);
  v.parameters.frequency_penalty = static_cast<float>(freq);
  v.parameters.watermark = bool_or(p, "watermark", false);
  if (p.has("seed")) {
    v.parameters.seed = p["seed"].as_u64();
  } else {
    std::lock_guard<std::mutex> lk(rng_m_);
    v.parameters.seed = rng_();
  }
  if (p.has("grammar")) {
    if (cfg_.disable_grammar_support) throw validation_error("grammar is not supported");
    const Value& gr = p["grammar"];
    if (!gr.has("type") || gr.find("value") == nullptr) throw validation_error("`grammar` needs `type` and `value`");
    auto compiled = text_.compile_grammar(gr["type"].as_string(), gr["value"]);
    v.parameters.grammar = compiled.first;
    v.parameters.grammar_type = compiled.second;
  }
  if (p.has("adapter_id") && p["adapter_id"].is_string()) v.adapter_id = p["adapter_id"].as_string();
  v.stopping.max_new_tokens = max_new;
  v.stopping.stop_sequences = stops;
  v.stopping.ignore_eos_token = false;
  g.return_full_text = bool_or(p, "return_full_text", false);
  g.details = bool_or(p, "details", false);
  g.decoder_input_details = v.decoder_input_details;
  return g;
}

// ------------------------------------------------------------------------------------------------
// generation orchestration
// ------------------------------------------------------------------------------------------------
// Streams one request; when a leg stops for length before the request's own budget is used up,
// the request is re-submitted with the text generated so far (what the reference's Infer does to
// serve `max_new_tokens = None` in 1024-token legs, router/src/infer/mod.rs:164-188).
void Router::stream_tokens(GenerateParams p,
                           const std::function<bool(const sched::StreamEvent&, const std::string&)>& on_event) {
  std::string text_so_far;
  uint32_t generated_total = 0;
  while (true) {
    auto stream = backend_->schedule(p.valid);
    bool again = false;
    while (true) {
      sched::StreamEvent ev;
      if (!stream->pop(ev, 200)) continue;
      if (ev.kind == sched::StreamEvent::Error) {
        healthy_.store(false);
        stream->close();
        throw ApiError(424, "generation", "Request failed during generation: " + ev.error);
      }
      if (ev.kind == sched::StreamEvent::Prefill) {
        if (!on_event(ev, text_so_far)) { stream->close(); return; }
        continue;
      }
      ++generated_total;
      if (!ev.token.special) text_so_far += ev.token.text;
      if (ev.kind == sched::StreamEvent::End) {
        const bool more = ev.generated_text->finish_reason == 0 && !p.max_new_tokens &&
                          generated_total < p.max_total_new_tokens;
        if (more) {
          // continue: next leg starts from the prompt plus everything generated so far
          sched::StreamEvent mid = ev;
          mid.kind = sched::StreamEvent::Intermediate;
          mid.generated_text.reset();
          if (!on_event(mid, text_so_far)) { stream->close(); return; }
          p.valid.inputs += ev.generated_text->text;
          p.valid.chunks.clear();
          pb::InputChunk c;
          c.text = p.valid.inputs;
          p.valid.chunks.push_back(c);
          p.valid.input_ids = text_.encode(p.valid.inputs, p.valid.add_special_tokens, 0);
          p.valid.input_length = static_cast<uint32_t>(p.valid.input_ids.size());
          const uint32_t left = p.max_total_new_tokens - generated_total;
          p.valid.stopping.max_new_tokens = std::min<uint32_t>(left, 1024);
          again = p.valid.input_length + p.valid.stopping.max_new_tokens <= cfg_.max_total_tokens;
          if (!again) {
            ev.generated_text->generated_tokens = generated_total;
            ev.generated_text->text = text_so_far;
            on_event(ev, text_so_far);
          }
          break;
        }
        ev.generated_text->generated_tokens = generated_total;
        on_event(ev, text_so_far);
        return;
      }
      if (!on_event(ev, text_so_far)) { stream->close(); return; }
    }
    if (!again) return;
  }
}

Collected Router::generate(GenerateParams p) {
  Collected c;
  c.input_length = p.valid.input_length;
  const auto t0 = Clock::now();
  bool done = false;
  Clock::time_point queued = t0, started = t0;
  stream_tokens(p, [&](const sched::StreamEvent& ev, const std::string& text) {
    if (ev.kind == sched::StreamEvent::Prefill) {
      c.prefill = ev.prefill_tokens;
      return true;
    }
    c.tokens.push_back(ev.token);
    c.top_tokens.push_back(ev.top_tokens);
    if (ev.kind == sched::StreamEvent::End) {
      c.generated_text = *ev.generated_text;
      c.output_text = p.max_new_tokens ? ev.generated_text->text : text;
      if (c.output_text.empty()) c.output_text = ev.generated_text->text;
      queued = ev.queued;
      started = ev.start;
      done = true;
    }
    return true;
  });
  if (!done) throw ApiError(500, "incomplete_generation", "Incomplete generation");
  c.total_s = seconds_since(t0);
  c.queue_s = std::chrono::duration<double>(started - queued).count();
  c.inference_s = seconds_since(started);
  return c;
}

}  // namespace api
