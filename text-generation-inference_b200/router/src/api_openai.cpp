// OpenAI-compatible routes: /v1/chat/completions (with tools and streaming), /v1/completions,
// /chat_tokenize.  Reference: router/src/lib.rs:492-1036 (schemas, chat -> generate conversion),
// router/src/infer/tool_grammar.rs:20-122, router/src/chat.rs (stream state machine),
// router/src/server.rs:715-1302.
#include <chrono>
#include <cmath>
#include <ctime>

#include "api.hpp"

#include <exception>
#include <mutex>
#include <thread>

namespace api {

using json::Value;

namespace {
Value parse_body(const http::Request& req) {
  try {
    Value v = Value::parse(req.body);
    if (!v.is_object()) throw validation_error("request body must be a JSON object");
    return v;
  } catch (const std::runtime_error& e) {
    throw ApiError(422, "validation", std::string("Failed to parse the request body as JSON: ") + e.what());
  }
}
long long unix_now() { return static_cast<long long>(std::time(nullptr)); }

const char* kDefaultToolPrompt =
    "\nGiven the functions available, please respond with a JSON for a function call with its proper arguments "
    "that best answers the given prompt. Respond in the format {name: function name, parameters: dictionary of "
    "argument name and its value}.Do not use variables.\n";
}  // namespace

// Tools -> one JSON schema: an `anyOf` over the functions, each with a constant `_name` property
// next to its own parameters, plus a `no_tool` escape hatch carrying free-text `content`.
Value tools_to_grammar_schema(const Value& tools, const Value& tool_choice) {
  std::string only;   // restrict to one function when tool_choice names it
  if (tool_choice.is_object() && tool_choice["function"].is_object())
    only = tool_choice["function"]["name"].as_string();
  else if (tool_choice.is_string() && tool_choice.as_string() != "auto" && tool_choice.as_string() != "required" &&
           tool_choice.as_string() != "none")
    only = tool_choice.as_string();
  const bool required = tool_choice.is_string() && tool_choice.as_string() == "required";
  Value defs = Value::object();
  Value any_of = Value::array();
  auto add = [&](const std::string& name, const std::string& description, const Value& parameters) {
    Value props = Value::object();
    Value name_prop = Value::object();
    name_prop.set("type", "string");
    name_prop.set("const", name);
    props.set("_name", name_prop);
    Value req = Value::array();
    req.push("_name");
    if (parameters.is_object()) {
      if (parameters["properties"].is_object())
        for (auto& kv : parameters["properties"].members()) props.set(kv.first, kv.second);
      if (parameters["required"].is_array())
        for (auto& r : parameters["required"].items()) req.push(r);
    }
    Value def = Value::object();
    def.set("type", "object");
    if (!description.empty()) def.set("description", description);
    def.set("properties", props);
    def.set("required", req);
    defs.set(name, def);
    Value ref = Value::object();
    ref.set("$ref", "#/$functions/" + name);
    any_of.push(ref);
  };
  bool found = false;
  for (const auto& t : tools.items()) {
    const Value& f = t["function"];
    if (!f.is_object()) continue;
    const std::string name = f["name"].as_string();
    if (!only.empty() && name != only) continue;
    found = true;
    add(name, f["description"].is_string() ? f["description"].as_string() : "",
        f.has("arguments") ? f["arguments"] : f["parameters"]);
  }
  if (!only.empty() && !found) throw validation_error("Tool with name " + only + " not found");
  if (only.empty() && !required) {
    Value params = Value::object();
    Value props = Value::object();
    Value content = Value::object();
    content.set("type", "string");
    content.set("description", "The response content");
    props.set("content", content);
    params.set("properties", props);
    Value req = Value::array();
    req.push("content");
    params.set("required", req);
    add("no_tool", "Open ended response with no specific tool selected", params);
  }
  Value schema = Value::object();
  schema.set("$functions", defs);
  Value properties = Value::object();
  Value fn = Value::object();
  fn.set("anyOf", any_of);
  properties.set("function", fn);
  schema.set("properties", properties);
  Value req = Value::array();
  req.push("function");
  schema.set("required", req);
  schema.set("type", "object");
  return schema;
}

// Chat request -> (inputs, /generate parameters).
Value Router::chat_to_generate(const Value& chat, std::string& inputs_out, bool& using_tools) {
  if (!chat["messages"].is_array() || chat["messages"].items().empty())
    throw validation_error("`messages` must be a non-empty list");
  if (chat.has("logit_bias") && chat["logit_bias"].is_object() && !chat["logit_bias"].members().empty())
    throw validation_error("`logit_bias` is not supported");
  Value params = Value::object();
  const Value& tool_choice = chat["tool_choice"];
  const bool tools_off = tool_choice.is_string() && tool_choice.as_string() == "none";
  using_tools = chat["tools"].is_array() && !chat["tools"].items().empty() && !tools_off;
  if (chat.has("response_format") && using_tools)
    throw validation_error("`response_format` and `tools` cannot both be used");
  Value tools = using_tools ? chat["tools"] : Value();
  const std::string tool_prompt = chat["tool_prompt"].is_string() ? chat["tool_prompt"].as_string() : kDefaultToolPrompt;
  inputs_out = text_.chat_template(chat["messages"], tools, tool_prompt);
  if (using_tools) {
    Value g = Value::object();
    g.set("type", "json");
    g.set("value", tools_to_grammar_schema(chat["tools"], tool_choice));
    params.set("grammar", g);
  } else if (chat["response_format"].is_object()) {
    const Value& rf = chat["response_format"];
    Value g = Value::object();
    const std::string type = rf["type"].as_string();
    if (type == "json_schema") {
      g.set("type", "json_schema");
      g.set("value", rf.has("json_schema") ? rf["json_schema"] : rf["value"]);
      params.set("grammar", g);
    } else if (type == "json_object" || type == "json") {
      g.set("type", "json");
      g.set("value", rf.has("schema") ? rf["schema"] : rf["value"]);
      params.set("grammar", g);
    } else if (type == "regex") {
      g.set("type", "regex");
      g.set("value", rf["value"]);
      params.set("grammar", g);
    }
  }
  // temperature 0 means greedy; presence_penalty is served as a repetition penalty shifted by 2
  bool do_sample = true;
  if (chat.has("temperature")) {
    const double t = chat["temperature"].as_double();
    if (t == 0.0) do_sample = false;
    else params.set("temperature", t);
  }
  params.set("do_sample", do_sample);
  if (chat.has("presence_penalty")) params.set("repetition_penalty", chat["presence_penalty"].as_double() + 2.0);
  if (chat.has("frequency_penalty")) params.set("frequency_penalty", chat["frequency_penalty"]);
  if (chat.has("top_p")) params.set("top_p", chat["top_p"]);
  if (chat.has("seed")) params.set("seed", chat["seed"]);
  if (chat.has("max_completion_tokens")) params.set("max_new_tokens", chat["max_completion_tokens"]);
  else if (chat.has("max_tokens")) params.set("max_new_tokens", chat["max_tokens"]);
  if (chat.has("stop")) {
    if (chat["stop"].is_string()) {
      Value a = Value::array();
      a.push(chat["stop"]);
      params.set("stop", a);
    } else {
      params.set("stop", chat["stop"]);
    }
  }
  if (chat.has("top_logprobs")) params.set("top_n_tokens", chat["top_logprobs"]);
  params.set("details", true);
  params.set("add_special_tokens", false);   // the template already wrote the special tokens
  if (chat["model"].is_string() && chat["model"].as_string() != "tgi" && chat["model"].as_string() != cfg_.model_id &&
      !chat["model"].as_string().empty())
    params.set("adapter_id", chat["model"]);
  return params;
}

namespace {
// Result of parsing a finished tool-grammar generation.
struct ToolOutcome {
  bool is_tool = false;
  std::string name, arguments, content;
};
ToolOutcome parse_tool_output(const std::string& text) {
  ToolOutcome out;
  Value v;
  try {
    v = Value::parse(text);
  } catch (const std::runtime_error&) {
    throw ApiError(500, "incomplete_generation", "the model did not produce a complete tool call");
  }
  const Value& f = v["function"];
  if (!f.is_object() || !f["_name"].is_string())
    throw ApiError(500, "incomplete_generation", "the tool call has no function name");
  out.name = f["_name"].as_string();
  if (out.name == "no_tool") {
    out.content = f["content"].is_string() ? f["content"].as_string() : "";
    return out;
  }
  out.is_tool = true;
  Value args = Value::object();
  for (auto& kv : f.members())
    if (kv.first != "_name") args.set(kv.first, kv.second);
  out.arguments = args.dump();
  return out;
}

Value logprobs_json(const std::vector<sched::Token>& tokens, const std::vector<std::vector<sched::Token>>& top) {
  Value content = Value::array();
  for (size_t i = 0; i < tokens.size(); ++i) {
    Value t = Value::object();
    t.set("token", tokens[i].text);
    t.set("logprob", static_cast<double>(tokens[i].logprob));
    Value tl = Value::array();
    if (i < top.size())
      for (auto& x : top[i]) {
        Value e = Value::object();
        e.set("token", x.text);
        e.set("logprob", static_cast<double>(x.logprob));
        tl.push(e);
      }
    t.set("top_logprobs", tl);
    content.push(t);
  }
  Value o = Value::object();
  o.set("content", content);
  return o;
}
}  // namespace

void Router::h_chat(const http::Request& req, http::Response& resp) {
  try {
    Value chat = parse_body(req);
    if (metrics_) metrics_->counter_inc("tgi_request_count");
    std::string inputs;
    bool using_tools = false;
    Value params;
    try {
      params = chat_to_generate(chat, inputs, using_tools);
    } catch (const ApiError& e) {
      if (metrics_) metrics_->counter_inc("tgi_request_failure", {{"err", e.type == "template_error" ? "template" : "validation"}});
      throw;
    }
    const bool want_logprobs = chat["logprobs"].is_bool() && chat["logprobs"].as_bool();
    const bool stream = chat["stream"].is_bool() && chat["stream"].as_bool();
    const bool include_usage = chat["stream_options"].is_object() && chat["stream_options"]["include_usage"].is_bool() &&
                               chat["stream_options"]["include_usage"].as_bool();
    const std::string fingerprint = cfg_.version + "-" + (cfg_.docker_label.empty() ? "native" : cfg_.docker_label);
    const std::string model = chat["model"].is_string() ? chat["model"].as_string() : cfg_.model_id;
    auto permit = acquire();
    GenerateParams p = validate(inputs, params);
    const std::string id = "chatcmpl-" + std::to_string(p.valid.parameters.seed % 1000000007ull);

    if (!stream) {
      Collected c = generate(p);
      Value message = Value::object();
      message.set("role", "assistant");
      if (using_tools) {
        ToolOutcome t = parse_tool_output(c.output_text);
        if (t.is_tool) {
          Value fn = Value::object();
          fn.set("name", t.name);
          fn.set("arguments", t.arguments);
          Value call = Value::object();
          call.set("id", "0");
          call.set("type", "function");
          call.set("function", fn);
          Value calls = Value::array();
          calls.push(call);
          message.set("tool_calls", calls);
        } else {
          message.set("content", t.content);
        }
      } else {
        message.set("content", c.output_text);
      }
      Value choice = Value::object();
      choice.set("index", 0);
      choice.set("message", message);
      choice.set("logprobs", want_logprobs ? logprobs_json(c.tokens, c.top_tokens) : Value());
      choice.set("finish_reason", finish_reason_str(c.generated_text.finish_reason, true));
      Value choices = Value::array();
      choices.push(choice);
      Value usage = Value::object();
      usage.set("prompt_tokens", c.input_length);
      usage.set("completion_tokens", c.generated_text.generated_tokens);
      usage.set("total_tokens", c.input_length + c.generated_text.generated_tokens);
      Value out = Value::object();
      out.set("id", id);
      out.set("object", "chat.completion");
      out.set("created", unix_now());
      out.set("model", model);
      out.set("system_fingerprint", fingerprint);
      out.set("choices", choices);
      out.set("usage", usage);
      if (metrics_) metrics_->counter_inc("tgi_request_success");
      resp.send(200, "application/json", out.dump());
      return;
    }

    // ---- streaming ----
    resp.set_header("x-accel-buffering", "no");
    resp.begin_stream(200, "text/event-stream");
    auto chunk = [&](const Value& delta, const Value& finish, const Value& logprobs) {
      Value choice = Value::object();
      choice.set("index", 0);
      choice.set("delta", delta);
      choice.set("logprobs", logprobs);
      choice.set("finish_reason", finish);
      Value choices = Value::array();
      choices.push(choice);
      Value o = Value::object();
      o.set("id", id);
      o.set("object", "chat.completion.chunk");
      o.set("created", unix_now());
      o.set("model", model);
      o.set("system_fingerprint", fingerprint);
      o.set("choices", choices);
      return resp.write_chunk("data:" + o.dump() + "\n\n");
    };
    // Tool calls stream as JSON text constrained by the grammar.  The text is buffered until the
    // function name is known; a `no_tool` answer then streams its `content` string, a real tool
    // streams its name first and the argument text after it.
    std::string buffered;
    uint32_t prompt_tokens = p.valid.input_length, completion_tokens = 0;
    stream_tokens(p, [&](const sched::StreamEvent& ev, const std::string& text) {
      if (ev.kind == sched::StreamEvent::Prefill) return true;
      ++completion_tokens;
      const bool end = ev.kind == sched::StreamEvent::End;
      Value finish = end ? Value(finish_reason_str(ev.generated_text->finish_reason, true)) : Value();
      Value lp = Value();
      if (want_logprobs) lp = logprobs_json({ev.token}, {ev.top_tokens});
      if (!using_tools) {
        Value delta = Value::object();
        delta.set("role", "assistant");
        delta.set("content", ev.token.special ? "" : ev.token.text);
        return chunk(delta, finish, lp) && !resp.client_gone();
      }
      buffered = text;
      if (!end) return !resp.client_gone();
      ToolOutcome t = parse_tool_output(buffered);
      Value delta = Value::object();
      delta.set("role", "assistant");
      if (t.is_tool) {
        Value fn = Value::object();
        fn.set("name", t.name);
        fn.set("arguments", t.arguments);
        Value call = Value::object();
        call.set("index", 0);
        call.set("id", "");
        call.set("type", "function");
        call.set("function", fn);
        Value calls = Value::array();
        calls.push(call);
        delta.set("tool_calls", calls);
      } else {
        delta.set("content", t.content);
      }
      return chunk(delta, finish, lp);
    });
    if (include_usage) {
      Value usage = Value::object();
      usage.set("prompt_tokens", prompt_tokens);
      usage.set("completion_tokens", completion_tokens);
      usage.set("total_tokens", prompt_tokens + completion_tokens);
      Value o = Value::object();
      o.set("id", id);
      o.set("object", "chat.completion.chunk");
      o.set("created", unix_now());
      o.set("model", model);
      o.set("system_fingerprint", fingerprint);
      o.set("choices", Value::array());
      o.set("usage", usage);
      resp.write_chunk("data:" + o.dump() + "\n\n");
    }
    resp.write_chunk("data: [DONE]\n\n");
    resp.end_stream();
    if (metrics_) metrics_->counter_inc("tgi_request_success");
  } catch (const ApiError& e) {
    if (resp.started()) {
      Value o = Value::object();
      o.set("error", std::string(e.what()));
      o.set("error_type", e.type);
      resp.write_chunk("data:" + o.dump() + "\n\n");
      resp.end_stream();
    } else {
      send_error(resp, e);
    }
  }
}

void Router::h_chat_tokenize(const http::Request& req, http::Response& resp) {
  try {
    Value chat = parse_body(req);
    std::string inputs;
    bool using_tools = false;
    chat_to_generate(chat, inputs, using_tools);
    Value toks = text_.encode_with_offsets(inputs, false);
    Value out = Value::object();
    out.set("tokenize_response", toks);
    out.set("templated_text", inputs);
    resp.send(200, "application/json", out.dump());
  } catch (const ApiError& e) {
    send_error(resp, e);
  }
}

void Router::h_completions(const http::Request& req, http::Response& resp) {
  try {
    Value body = parse_body(req);
    if (body.has("suffix")) throw validation_error("Suffix is not supported and can be achieved by preprocessing the prompt.");
    std::vector<std::string> prompts;
    if (body["prompt"].is_string()) prompts.push_back(body["prompt"].as_string());
    else if (body["prompt"].is_array())
      for (auto& pr : body["prompt"].items()) prompts.push_back(pr.as_string());
    if (prompts.empty()) throw validation_error("`prompt` must be a string or a list of strings");
    if (prompts.size() > cfg_.max_client_batch_size)
      throw validation_error("Number of prompts exceeds the maximum allowed batch size of " +
                             std::to_string(cfg_.max_client_batch_size));
    Value params = Value::object();
    bool do_sample = true;
    if (body.has("temperature")) {
      if (body["temperature"].as_double() == 0.0) do_sample = false;
      else params.set("temperature", body["temperature"]);
    }
    params.set("do_sample", do_sample);
    if (body.has("top_p")) params.set("top_p", body["top_p"]);
    if (body.has("seed")) params.set("seed", body["seed"]);
    if (body.has("max_tokens")) params.set("max_new_tokens", body["max_tokens"]);
    if (body.has("repetition_penalty")) params.set("repetition_penalty", body["repetition_penalty"]);
    if (body.has("frequency_penalty")) params.set("frequency_penalty", body["frequency_penalty"]);
    if (body.has("stop")) params.set("stop", body["stop"]);
    params.set("details", true);
    const bool stream = body["stream"].is_bool() && body["stream"].as_bool();
    const std::string model = body["model"].is_string() ? body["model"].as_string() : cfg_.model_id;
    const std::string fingerprint = cfg_.version + "-" + (cfg_.docker_label.empty() ? "native" : cfg_.docker_label);
    if (!stream) {
      Value choices = Value::array();
      uint32_t prompt_tokens = 0, completion_tokens = 0;
      // the prompts of one request run side by side, so the scheduler batches them (server.rs joins their futures)
      std::vector<GenerateParams> ps;
      for (const auto& pr : prompts) ps.push_back(validate(pr, params));
      std::vector<Collected> done(prompts.size());
      std::vector<std::exception_ptr> failed(prompts.size());
      {
        std::vector<std::thread> workers;
        for (size_t i = 1; i < prompts.size(); ++i)
          workers.emplace_back([&, i] {
            try {
              auto permit = acquire();
              done[i] = generate(ps[i]);
            } catch (...) {
              failed[i] = std::current_exception();
            }
          });
        try {
          auto permit = acquire();
          done[0] = generate(ps[0]);
        } catch (...) {
          failed[0] = std::current_exception();
        }
        for (auto& w : workers) w.join();
      }
      for (auto& f : failed)
        if (f) std::rethrow_exception(f);
      for (size_t i = 0; i < prompts.size(); ++i) {
        Collected& c = done[i];
        Value choice = Value::object();
        choice.set("index", static_cast<unsigned>(i));
        choice.set("text", c.output_text);
        choice.set("logprobs", Value());
        choice.set("finish_reason", finish_reason_str(c.generated_text.finish_reason, true));
        choices.push(choice);
        prompt_tokens += c.input_length;
        completion_tokens += c.generated_text.generated_tokens;
      }
      Value usage = Value::object();
      usage.set("prompt_tokens", prompt_tokens);
      usage.set("completion_tokens", completion_tokens);
      usage.set("total_tokens", prompt_tokens + completion_tokens);
      Value out = Value::object();
      out.set("id", "");
      out.set("object", "text_completion");
      out.set("created", unix_now());
      out.set("model", model);
      out.set("system_fingerprint", fingerprint);
      out.set("choices", choices);
      out.set("usage", usage);
      resp.send(200, "application/json", out.dump());
      return;
    }
    // all prompts are validated before the first byte goes out (a bad one is a plain 422); their token streams are
    // interleaved on the one response, every chunk tagged with the index of its prompt
    std::vector<GenerateParams> ps;
    for (const auto& pr : prompts) ps.push_back(validate(pr, params));
    resp.set_header("x-accel-buffering", "no");
    resp.begin_stream(200, "text/event-stream");
    std::mutex write_mu;
    std::vector<std::exception_ptr> failed(prompts.size());
    auto run_one = [&](size_t i) {
      auto permit = acquire();
      stream_tokens(ps[i], [&, i](const sched::StreamEvent& ev, const std::string&) {
        if (ev.kind == sched::StreamEvent::Prefill) return true;
        Value choice = Value::object();
        choice.set("index", static_cast<unsigned>(i));
        choice.set("text", ev.token.special ? "" : ev.token.text);
        choice.set("logprobs", Value());
        choice.set("finish_reason", ev.kind == sched::StreamEvent::End
                                        ? Value(finish_reason_str(ev.generated_text->finish_reason, true)) : Value());
        Value choices = Value::array();
        choices.push(choice);
        Value o = Value::object();
        o.set("id", "");
        o.set("object", "text_completion");
        o.set("created", unix_now());
        o.set("model", model);
        o.set("system_fingerprint", fingerprint);
        o.set("choices", choices);
        std::lock_guard<std::mutex> g(write_mu);
        return resp.write_chunk("data:" + o.dump() + "\n\n") && !resp.client_gone();
      });
    };
    {
      std::vector<std::thread> workers;
      for (size_t i = 1; i < prompts.size(); ++i)
        workers.emplace_back([&, i] {
          try {
            run_one(i);
          } catch (...) {
            failed[i] = std::current_exception();
          }
        });
      try {
        run_one(0);
      } catch (...) {
        failed[0] = std::current_exception();
      }
      for (auto& w : workers) w.join();
    }
    for (auto& f : failed)
      if (f) std::rethrow_exception(f);
    resp.write_chunk("data: [DONE]\n\n");
    resp.end_stream();
  } catch (const ApiError& e) {
    if (resp.started()) {
      Value o = Value::object();
      o.set("error", std::string(e.what()));
      o.set("error_type", e.type);
      resp.write_chunk("data:" + o.dump() + "\n\n");
      resp.end_stream();
    } else {
      send_error(resp, e);
    }
  }
}

}  // namespace api
