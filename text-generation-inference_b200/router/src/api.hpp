// Request pipeline and REST routes of the router: validation, tokenisation, chat templating, tool
// grammars, generation orchestration (concurrency limit, best_of, continuation past 1024 new
// tokens), OpenAI-compatible and native responses, SSE streaming, Prometheus metrics.
//
// Reference counterparts: router/src/validation.rs (rules :204-447), router/src/infer/mod.rs
// (`Infer`, :100-364), router/src/server.rs (handlers), router/src/lib.rs (schemas, chat ->
// generate conversion :941-1036), router/src/infer/tool_grammar.rs, router/src/chat.rs.
#pragma once
#include <atomic>
#include <functional>
#include <memory>
#include <optional>
#include <random>
#include <string>

#include "http.hpp"
#include "json.hpp"
#include "metrics.hpp"
#include "scheduler.hpp"

namespace api {

struct ApiError : std::runtime_error {
  int status;
  std::string type;
  ApiError(int s, std::string t, const std::string& msg) : std::runtime_error(msg), status(s), type(std::move(t)) {}
};
inline ApiError validation_error(const std::string& m) { return ApiError(422, "validation", m); }

// Tokenizer / template services; the production implementation calls the embedded Python bridge,
// tests plug in fakes.
struct TextServices {
  // returns token ids (after truncation from the left when `truncate` > 0)
  std::function<std::vector<uint32_t>(const std::string& text, bool add_special_tokens, uint32_t truncate)> encode;
  std::function<json::Value(const std::string& text, bool add_special_tokens)> encode_with_offsets;
  std::function<std::string(const json::Value& messages, const json::Value& tools, const std::string& tool_prompt)>
      chat_template;
  // {type,value} -> (grammar, grammar_type)
  std::function<std::pair<std::string, uint32_t>(const std::string& type, const json::Value& value)> compile_grammar;
};

struct RouterConfig {
  size_t max_concurrent_requests = 128;
  uint32_t max_best_of = 2;
  uint32_t max_stop_sequences = 4;
  uint32_t max_top_n_tokens = 5;
  uint32_t max_input_tokens = 1024;
  uint32_t max_total_tokens = 2048;
  uint32_t max_client_batch_size = 4;
  bool disable_grammar_support = false;
  std::string api_key;
  std::string model_id = "model";
  std::string model_sha;
  std::string model_pipeline_tag = "text-generation";
  std::string version = "0.1.0";
  std::string docker_label;
  // engine facts for /info
  std::string dtype, device_type;
  uint32_t waiting_served_ratio_x100 = 30;
  uint32_t max_batch_total_tokens = 0, max_waiting_tokens = 20;
  std::optional<size_t> max_batch_size;
  uint32_t validation_workers = 2;
  // config.json of the checkpoint (null when unknown): decides whether `inputs` may carry images and
  // how many placeholder tokens an image costs
  json::Value model_config;
  size_t max_image_bytes = 20u << 20;
  std::vector<std::string> cors_allow_origin;   // empty: any origin
};

struct GenerateParams {   // the `parameters` object of /generate, already range-checked
  std::optional<uint32_t> best_of;
  std::optional<uint32_t> max_new_tokens;
  bool return_full_text = false, details = false, decoder_input_details = false, stream = false;
  sched::ValidRequest valid;
  uint32_t max_total_new_tokens = 0;   // budget for continuation legs
};

struct Collected {   // outcome of a non-streaming generation
  std::vector<sched::Token> prefill, tokens;
  std::vector<std::vector<sched::Token>> top_tokens;
  pb::GeneratedText generated_text;
  double queue_s = 0, inference_s = 0, total_s = 0, validation_s = 0;
  uint32_t input_length = 0;
  std::string output_text;
};

class Router {
 public:
  Router(std::shared_ptr<sched::Backend> backend, TextServices text, RouterConfig cfg, sched::Metrics* metrics);
  void install(http::Server& server);

  // exposed for tests
  GenerateParams validate(const std::string& inputs, const json::Value& parameters);
  Collected generate(GenerateParams p);
  json::Value chat_to_generate(const json::Value& chat_request, std::string& inputs_out, bool& using_tools);
  json::Value info_json() const;

 private:
  struct Permit {
    std::atomic<size_t>* counter = nullptr;
    ~Permit() { if (counter) --*counter; }
  };
  std::unique_ptr<Permit> acquire();
  void stream_tokens(GenerateParams p, const std::function<bool(const sched::StreamEvent&, const std::string& text_so_far)>& on_event);

  void h_generate(const http::Request&, http::Response&);
  void h_generate_stream(const http::Request&, http::Response&);
  void h_compat(const http::Request&, http::Response&);
  void h_chat(const http::Request&, http::Response&);
  void h_completions(const http::Request&, http::Response&);
  void h_tokenize(const http::Request&, http::Response&);
  void h_chat_tokenize(const http::Request&, http::Response&);
  void h_invocations(const http::Request&, http::Response&);
  void h_vertex(const http::Request&, http::Response&);
  void h_kserve(const http::Request&, http::Response&);   // every /v2/... path (KServe open inference protocol)
  void generate_response(const std::string& inputs, const json::Value& params, http::Response& resp, bool as_array);
  void generate_stream_response(const std::string& inputs, const json::Value& params, http::Response& resp);
  void send_error(http::Response& resp, const ApiError& e);

  std::shared_ptr<sched::Backend> backend_;
  TextServices text_;
  RouterConfig cfg_;
  sched::Metrics* metrics_;
  std::atomic<size_t> in_flight_{0};
  std::atomic<bool> healthy_{true};
  std::mt19937_64 rng_{std::random_device{}()};
  std::mutex rng_m_;
};

// Tool calling helpers (exposed for tests)
json::Value tools_to_grammar_schema(const json::Value& tools, const json::Value& tool_choice);
std::string finish_reason_str(uint32_t r, bool openai);

// OpenAPI document of the HTTP surface (openapi.cpp) and a self-contained page that renders it
json::Value openapi_schema(const std::string& version);
std::string openapi_html();

}  // namespace api
