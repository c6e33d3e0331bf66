// Native routes: /generate, /generate_stream, /, /tokenize, /info, /health, /metrics, /v1/models,
// /invocations (SageMaker) and /vertex.  (Reference: router/src/server.rs:126-679, 1317-1340,
// sagemaker.rs, vertex.rs.)
#include <chrono>
#include <cmath>

#include "api.hpp"

namespace api {

using json::Value;
using sched::Clock;

namespace {
Value token_json(const sched::Token& t, bool with_special) {
  Value o = Value::object();
  o.set("id", t.id);
  o.set("text", t.text);
  if (std::isnan(t.logprob)) o.set("logprob", Value());
  else o.set("logprob", static_cast<double>(t.logprob));
  if (with_special) o.set("special", t.special);
  return o;
}
Value parse_body(const http::Request& req) {
  try {
    Value v = Value::parse(req.body);
    if (!v.is_object()) throw validation_error("request body must be a JSON object");
    return v;
  } catch (const std::runtime_error& e) {
    throw ApiError(422, "validation", std::string("Failed to parse the request body as JSON: ") + e.what());
  }
}
std::string ms(double seconds) { return std::to_string(static_cast<long long>(seconds * 1000.0)); }
}  // namespace

Value Router::info_json() const {
  Value o = Value::object();
  o.set("model_id", cfg_.model_id);
  o.set("model_sha", cfg_.model_sha.empty() ? Value() : Value(cfg_.model_sha));
  o.set("model_pipeline_tag", cfg_.model_pipeline_tag);
  o.set("max_concurrent_requests", static_cast<unsigned long long>(cfg_.max_concurrent_requests));
  o.set("max_best_of", cfg_.max_best_of);
  o.set("max_stop_sequences", cfg_.max_stop_sequences);
  o.set("max_input_tokens", cfg_.max_input_tokens);
  o.set("max_total_tokens", cfg_.max_total_tokens);
  o.set("validation_workers", cfg_.validation_workers);
  o.set("max_client_batch_size", cfg_.max_client_batch_size);
  o.set("router", "tgi-b200-router");
  o.set("version", cfg_.version);
  o.set("sha", Value());
  o.set("docker_label", cfg_.docker_label.empty() ? Value() : Value(cfg_.docker_label));
  return o;
}

static Value details_json(const Collected& c, const GenerateParams& p, bool sampling) {
  Value d = Value::object();
  d.set("finish_reason", finish_reason_str(c.generated_text.finish_reason, false));
  d.set("generated_tokens", c.generated_text.generated_tokens);
  d.set("seed", (sampling && c.generated_text.seed) ? Value(static_cast<unsigned long long>(*c.generated_text.seed))
                                                    : Value());
  Value prefill = Value::array();
  if (p.decoder_input_details)
    for (auto& t : c.prefill) prefill.push(token_json(t, false));
  d.set("prefill", prefill);
  Value toks = Value::array();
  for (auto& t : c.tokens) toks.push(token_json(t, true));
  d.set("tokens", toks);
  if (p.valid.top_n_tokens > 0) {
    Value tt = Value::array();
    for (auto& row : c.top_tokens) {
      Value r = Value::array();
      for (auto& t : row) r.push(token_json(t, true));
      tt.push(r);
    }
    d.set("top_tokens", tt);
  }
  return d;
}

void Router::generate_response(const std::string& inputs, const Value& params, http::Response& resp, bool as_array) {
  const auto t0 = Clock::now();
  if (metrics_) metrics_->counter_inc("tgi_request_count");
  auto permit = acquire();
  GenerateParams p;
  try {
    p = validate(inputs, params);
  } catch (const ApiError&) {
    if (metrics_) metrics_->counter_inc("tgi_request_failure", {{"err", "validation"}});
    throw;
  }
  const double validation_s = std::chrono::duration<double>(Clock::now() - t0).count();
  const uint32_t n = p.best_of.value_or(1);
  std::vector<Collected> outs;
  try {
    for (uint32_t i = 0; i < n; ++i) {
      GenerateParams pi = p;
      if (i > 0) {
        std::lock_guard<std::mutex> lk(rng_m_);
        pi.valid.parameters.seed = rng_();
      }
      outs.push_back(generate(pi));
    }
  } catch (const ApiError&) {
    if (metrics_) metrics_->counter_inc("tgi_request_failure", {{"err", "generation"}});
    throw;
  }
  // best_of: keep the sequence with the highest mean log-probability
  size_t best = 0;
  double best_score = -1e300;
  for (size_t i = 0; i < outs.size(); ++i) {
    double s = 0;
    for (auto& t : outs[i].tokens) s += t.logprob;
    s /= std::max<size_t>(1, outs[i].tokens.size());
    if (s > best_score) { best_score = s; best = i; }
  }
  Collected& c = outs[best];
  const bool sampling = p.valid.parameters.do_sample || p.valid.parameters.temperature != 1.f ||
                        p.valid.parameters.top_k != 0 || p.valid.parameters.top_p < 1.f ||
                        p.valid.parameters.typical_p < 1.f;
  Value out = Value::object();
  out.set("generated_text", p.return_full_text ? inputs + c.output_text : c.output_text);
  if (p.details) {
    Value d = details_json(c, p, sampling);
    if (outs.size() > 1) {
      Value others = Value::array();
      for (size_t i = 0; i < outs.size(); ++i) {
        if (i == best) continue;
        Value b = details_json(outs[i], p, sampling);
        b.set("generated_text", p.return_full_text ? inputs + outs[i].output_text : outs[i].output_text);
        others.push(b);
      }
      d.set("best_of_sequences", others);
    }
    out.set("details", d);
  }
  const double total_s = std::chrono::duration<double>(Clock::now() - t0).count();
  const double per_token = c.inference_s / std::max<uint32_t>(1, c.generated_text.generated_tokens);
  resp.set_header("x-compute-type", cfg_.device_type.empty() ? "gpu+optimized" : cfg_.device_type);
  resp.set_header("x-compute-time", std::to_string(total_s));
  resp.set_header("x-compute-characters", std::to_string(inputs.size()));
  resp.set_header("x-total-time", ms(total_s));
  resp.set_header("x-validation-time", ms(validation_s));
  resp.set_header("x-queue-time", ms(c.queue_s));
  resp.set_header("x-inference-time", ms(c.inference_s));
  resp.set_header("x-time-per-token", ms(per_token));
  resp.set_header("x-prompt-tokens", std::to_string(c.input_length));
  resp.set_header("x-generated-tokens", std::to_string(c.generated_text.generated_tokens));
  if (metrics_) {
    metrics_->counter_inc("tgi_request_success");
    metrics_->observe("tgi_request_duration", total_s);
    metrics_->observe("tgi_request_validation_duration", validation_s);
    metrics_->observe("tgi_request_queue_duration", c.queue_s);
    metrics_->observe("tgi_request_inference_duration", c.inference_s);
    metrics_->observe("tgi_request_mean_time_per_token_duration", per_token);
    metrics_->histogram_value("tgi_request_input_length", c.input_length);
    metrics_->histogram_value("tgi_request_generated_tokens", c.generated_text.generated_tokens);
    metrics_->histogram_value("tgi_request_max_new_tokens", p.valid.stopping.max_new_tokens);
  }
  if (as_array) {
    Value arr = Value::array();
    arr.push(out);
    resp.send(200, "application/json", arr.dump());
  } else {
    resp.send(200, "application/json", out.dump());
  }
}

void Router::generate_stream_response(const std::string& inputs, const Value& params, http::Response& resp) {
  const auto t0 = Clock::now();
  if (metrics_) metrics_->counter_inc("tgi_request_count");
  resp.set_header("x-accel-buffering", "no");
  resp.set_header("x-compute-type", cfg_.device_type.empty() ? "gpu+optimized" : cfg_.device_type);
  resp.set_header("x-compute-characters", std::to_string(inputs.size()));
  auto sse_error = [&](const ApiError& e) {
    Value o = Value::object();
    o.set("error", std::string(e.what()));
    o.set("error_type", e.type);
    if (!resp.started()) resp.begin_stream(200, "text/event-stream");
    resp.write_chunk("data:" + o.dump() + "\n\n");
    resp.end_stream();
  };
  try {
    auto permit = acquire();
    GenerateParams p = validate(inputs, params);
    if (p.best_of) throw validation_error("`best_of` != 1 is not supported when streaming tokens");
    if (p.decoder_input_details)
      throw validation_error("`decoder_input_details` == true is not supported when streaming tokens");
    resp.begin_stream(200, "text/event-stream");
    uint32_t index = 0;
    const bool sampling = p.valid.parameters.do_sample || p.valid.parameters.temperature != 1.f ||
                          p.valid.parameters.top_k != 0 || p.valid.parameters.top_p < 1.f ||
                          p.valid.parameters.typical_p < 1.f;
    stream_tokens(p, [&](const sched::StreamEvent& ev, const std::string& text) {
      if (ev.kind == sched::StreamEvent::Prefill) return true;
      Value o = Value::object();
      o.set("index", index++);
      o.set("token", token_json(ev.token, true));
      if (p.valid.top_n_tokens > 0) {
        Value tt = Value::array();
        for (auto& t : ev.top_tokens) tt.push(token_json(t, true));
        o.set("top_tokens", tt);
      }
      if (ev.kind == sched::StreamEvent::End) {
        const std::string& gen = p.max_new_tokens ? ev.generated_text->text : text;
        o.set("generated_text", p.return_full_text ? inputs + gen : gen);
        Value d = Value();
        if (p.details) {
          d = Value::object();
          d.set("finish_reason", finish_reason_str(ev.generated_text->finish_reason, false));
          d.set("generated_tokens", ev.generated_text->generated_tokens);
          d.set("seed", (sampling && ev.generated_text->seed)
                            ? Value(static_cast<unsigned long long>(*ev.generated_text->seed)) : Value());
          d.set("input_length", p.valid.input_length);
        }
        o.set("details", d);
      } else {
        o.set("generated_text", Value());
        o.set("details", Value());
      }
      return resp.write_chunk("data:" + o.dump() + "\n\n") && !resp.client_gone();
    });
    resp.end_stream();
    if (metrics_) {
      metrics_->counter_inc("tgi_request_success");
      metrics_->observe("tgi_request_duration", std::chrono::duration<double>(Clock::now() - t0).count());
    }
  } catch (const ApiError& e) {
    if (metrics_) metrics_->counter_inc("tgi_request_failure", {{"err", e.type}});
    sse_error(e);
  }
}

void Router::h_generate(const http::Request& req, http::Response& resp) {
  try {
    Value body = parse_body(req);
    if (!body.has("inputs") || !body["inputs"].is_string()) throw validation_error("`inputs` must be a string");
    generate_response(body["inputs"].as_string(), body["parameters"].is_object() ? body["parameters"] : Value::object(),
                      resp, false);
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_generate_stream(const http::Request& req, http::Response& resp) {
  try {
    Value body = parse_body(req);
    if (!body.has("inputs") || !body["inputs"].is_string()) throw validation_error("`inputs` must be a string");
    generate_stream_response(body["inputs"].as_string(),
                             body["parameters"].is_object() ? body["parameters"] : Value::object(), resp);
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_compat(const http::Request& req, http::Response& resp) {
  try {
    Value body = parse_body(req);
    if (!body.has("inputs") || !body["inputs"].is_string()) throw validation_error("`inputs` must be a string");
    Value params = body["parameters"].is_object() ? body["parameters"] : Value::object();
    if (body["stream"].is_bool() && body["stream"].as_bool())
      generate_stream_response(body["inputs"].as_string(), params, resp);
    else
      generate_response(body["inputs"].as_string(), params, resp, true);
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_tokenize(const http::Request& req, http::Response& resp) {
  try {
    Value body = parse_body(req);
    if (!body.has("inputs") || !body["inputs"].is_string()) throw validation_error("`inputs` must be a string");
    const bool add = !(body["add_special_tokens"].is_bool() && !body["add_special_tokens"].as_bool());
    Value r = text_.encode_with_offsets(body["inputs"].as_string(), add);
    resp.send(200, "application/json", r.dump());
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_invocations(const http::Request& req, http::Response& resp) {
  // SageMaker: one endpoint for the three request kinds, told apart by their fields
  try {
    Value body = parse_body(req);
    if (body.has("messages")) return h_chat(req, resp);
    if (body.has("prompt")) return h_completions(req, resp);
    return h_compat(req, resp);
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_vertex(const http::Request& req, http::Response& resp) {
  // Vertex AI: {"instances": [{inputs, parameters} | chat request]} -> {"predictions": [...]}
  try {
    Value body = parse_body(req);
    if (!body["instances"].is_array()) throw validation_error("`instances` must be a list");
    Value preds = Value::array();
    for (const auto& inst : body["instances"].items()) {
      if (!inst.has("inputs")) throw validation_error("every instance needs `inputs`");
      GenerateParams p = validate(inst["inputs"].as_string(),
                                  inst["parameters"].is_object() ? inst["parameters"] : Value::object());
      auto permit = acquire();
      Collected c = generate(p);
      preds.push(Value(c.output_text));
    }
    Value out = Value::object();
    out.set("predictions", preds);
    resp.send(200, "application/json", out.dump());
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::install(http::Server& s) {
  using namespace std::placeholders;
  s.set_middleware([this](const http::Request& req, http::Response& resp) {
    // CORS: any origin by default, else only the configured ones (reference: --cors-allow-origin)
    if (cfg_.cors_allow_origin.empty()) {
      resp.set_header("access-control-allow-origin", "*");
    } else {
      const std::string origin = req.header("origin");
      for (const auto& o : cfg_.cors_allow_origin)
        if (o == origin || o == "*") resp.set_header("access-control-allow-origin", o == "*" ? "*" : origin);
    }
    if (cfg_.api_key.empty()) return true;
    const bool open = req.path == "/health" || req.path == "/ping" || req.path == "/" || req.path == "/metrics";
    if (open && req.method == "GET") return true;
    if (req.header("authorization") == "Bearer " + cfg_.api_key) return true;
    resp.send(401, "application/json", "{\"error\":\"Unauthorized\",\"error_type\":\"unauthorized\"}");
    return false;
  });
  s.route("POST", "/generate", std::bind(&Router::h_generate, this, _1, _2));
  s.route("POST", "/generate_stream", std::bind(&Router::h_generate_stream, this, _1, _2));
  s.route("POST", "/", std::bind(&Router::h_compat, this, _1, _2));
  s.route("POST", "/v1/chat/completions", std::bind(&Router::h_chat, this, _1, _2));
  s.route("POST", "/v1/completions", std::bind(&Router::h_completions, this, _1, _2));
  s.route("POST", "/tokenize", std::bind(&Router::h_tokenize, this, _1, _2));
  s.route("POST", "/chat_tokenize", std::bind(&Router::h_chat_tokenize, this, _1, _2));
  s.route("POST", "/invocations", std::bind(&Router::h_invocations, this, _1, _2));
  s.route("POST", "/vertex", std::bind(&Router::h_vertex, this, _1, _2));
  s.set_fallback(std::bind(&Router::h_kserve, this, _1, _2));   // parameterised /v2/models/{name}/versions/{v}/... paths
  auto info = [this](const http::Request&, http::Response& r) { r.send(200, "application/json", info_json().dump()); };
  s.route("GET", "/info", info);
  s.route("GET", "/", [this](const http::Request&, http::Response& r) {
    const bool ok = backend_->health(healthy_.load());
    healthy_.store(ok);
    if (ok) r.send(200, "application/json", "{}");
    else r.send(503, "application/json", "{\"error\":\"unhealthy\",\"error_type\":\"healthcheck\"}");
  });
  auto health = [this](const http::Request&, http::Response& r) {
    const bool ok = backend_->health(healthy_.load());
    healthy_.store(ok);
    if (ok) r.send(200, "application/json", "{}");
    else r.send(503, "application/json", "{\"error\":\"unhealthy\",\"error_type\":\"healthcheck\"}");
  };
  s.route("GET", "/health", health);
  s.route("GET", "/ping", health);
  s.route("GET", "/metrics", [this](const http::Request&, http::Response& r) {
    r.send(200, "text/plain; version=0.0.4", metrics_ ? metrics_->render() : "");
  });
  s.route("GET", "/v1/models", [this](const http::Request&, http::Response& r) {
    Value m = Value::object();
    m.set("id", cfg_.model_id);
    m.set("object", "model");
    m.set("created", 0);
    m.set("owned_by", cfg_.model_id);
    Value data = Value::array();
    data.push(m);
    Value o = Value::object();
    o.set("object", "list");
    o.set("data", data);
    r.send(200, "application/json", o.dump());
  });
  s.route("GET", "/api-doc/openapi.json", [this](const http::Request&, http::Response& r) {
    r.send(200, "application/json", openapi_schema(cfg_.version).dump());
  });
  s.route("GET", "/docs", [](const http::Request&, http::Response& r) { r.send(200, "text/html", openapi_html()); });
}

}  // namespace api
