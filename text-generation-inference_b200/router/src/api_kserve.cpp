// KServe "open inference protocol" (v2) routes.
//
// Reference: router/src/kserve.rs:70-169 (health, server and model metadata, model ready, infer).
// The paths carry the model name and version, so they are served from the HTTP server's fallback
// handler and parsed here.  An infer request holds text inputs as BYTES tensors; every element is one
// prompt; the answer carries one BYTES tensor per prompt whose data is the generated text as a list
// of byte values (what the reference emits).
#include <sstream>

#include "api.hpp"

namespace api {

using json::Value;

namespace {

std::vector<std::string> split_path(const std::string& path) {
  std::vector<std::string> parts;
  std::stringstream ss(path);
  std::string item;
  while (std::getline(ss, item, '/'))
    if (!item.empty()) parts.push_back(item);
  return parts;
}

void not_found(http::Response& resp) {
  resp.send(404, "application/json", "{\"error\":\"Not Found\",\"error_type\":\"not_found\"}");
}

}  // namespace

void Router::h_kserve(const http::Request& req, http::Response& resp) {
  const std::vector<std::string> parts = split_path(req.path);
  if (parts.empty() || parts[0] != "v2") return not_found(resp);
  try {
    if (req.method == "GET" && parts.size() == 1) {   // server metadata
      Value o = Value::object();
      o.set("name", "text-generation-inference");
      o.set("version", cfg_.version);
      Value ext = Value::array();
      ext.push(Value("health"));
      ext.push(Value("models"));
      ext.push(Value("metrics"));
      o.set("extensions", ext);
      return (void)resp.send(200, "application/json", o.dump());
    }
    if (req.method == "GET" && parts.size() == 3 && parts[1] == "health" && (parts[2] == "live" || parts[2] == "ready")) {
      bool ok = true;
      if (parts[2] == "ready") {
        ok = backend_->health(healthy_.load());
        healthy_.store(ok);
      }
      Value o = Value::object();
      o.set("live", ok);
      return (void)resp.send(ok ? 200 : 503, "application/json", o.dump());
    }
    // /v2/models/{name}[/versions/{version}][/ready|/infer]
    if (parts.size() < 3 || parts[1] != "models") return not_found(resp);
    const std::string model = parts[2];
    size_t i = 3;
    std::string version = "1";
    if (parts.size() >= 5 && parts[3] == "versions") {
      version = parts[4];
      i = 5;
    }
    const std::string action = i < parts.size() ? parts[i] : "";
    if (req.method == "GET" && action.empty()) {   // model metadata
      Value o = Value::object();
      o.set("name", model);
      Value versions = Value::array();
      versions.push(Value(version));
      o.set("versions", versions);
      o.set("platform", "tgi");
      auto tensor = [](const char* name) {
        Value t = Value::object();
        t.set("name", name);
        t.set("datatype", "BYTES");
        Value shape = Value::array();
        shape.push(Value(-1));
        t.set("shape", shape);
        return t;
      };
      Value ins = Value::array();
      ins.push(tensor("text_input"));
      Value outs = Value::array();
      outs.push(tensor("generated_text"));
      o.set("inputs", ins);
      o.set("outputs", outs);
      return (void)resp.send(200, "application/json", o.dump());
    }
    if (req.method == "GET" && action == "ready") {
      Value o = Value::object();
      o.set("name", model);
      o.set("ready", true);
      return (void)resp.send(200, "application/json", o.dump());
    }
    if (req.method == "POST" && action == "infer") {
      Value body = Value::parse(req.body);
      if (!body.is_object() || !body.has("inputs") || !body["inputs"].is_array() || body["inputs"].items().empty())
        throw validation_error("`inputs` must be a non-empty list of tensors");
      const Value params = body.has("parameters") && body["parameters"].is_object() ? body["parameters"] : Value::object();
      std::vector<std::string> prompts;
      for (const auto& t : body["inputs"].items()) {
        if (!t.is_object() || !t.has("data") || !t["data"].is_array()) throw validation_error("every input tensor needs `data`");
        for (const auto& d : t["data"].items()) {
          if (!d.is_string()) throw validation_error("input tensors must hold strings (datatype BYTES)");
          prompts.push_back(d.as_string());
        }
      }
      if (prompts.empty()) throw validation_error("no prompt in `inputs`");
      if (prompts.size() > cfg_.max_client_batch_size)
        throw validation_error("batch size exceeds the maximum of " + std::to_string(cfg_.max_client_batch_size));
      Value outputs = Value::array();
      for (const auto& prompt : prompts) {
        GenerateParams p = validate(prompt, params);
        auto permit = acquire();
        Collected c = generate(p);
        Value t = Value::object();
        t.set("name", "generated_text");
        t.set("datatype", "BYTES");
        Value shape = Value::array();
        shape.push(Value(static_cast<long long>(c.output_text.size())));
        t.set("shape", shape);
        Value data = Value::array();
        for (unsigned char ch : c.output_text) data.push(Value(static_cast<int>(ch)));
        t.set("data", data);
        outputs.push(t);
      }
      Value o = Value::object();
      o.set("model_name", model);
      o.set("model_version", version);
      o.set("id", body.has("id") && body["id"].is_string() ? body["id"] : Value(std::string("")));
      o.set("outputs", outputs);
      return (void)resp.send(200, "application/json", o.dump());
    }
    not_found(resp);
  } catch (const ApiError& e) {
    send_error(resp, e);
  } catch (const std::exception& e) {
    send_error(resp, validation_error(std::string("invalid request: ") + e.what()));
  }
}

}  // namespace api
