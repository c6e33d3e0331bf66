// OpenAPI description of the HTTP surface, served at /api-doc/openapi.json, rendered at /docs and printed by
// `tgi-b200-router print-schema`.
//
// Reference: the utoipa `ApiDoc` of `router/src/server.rs:1502-1620` (paths + component schemas) and
// `text-generation-router print-schema` (`backends/v3/src/main.rs:128-134`).
#include "api.hpp"

namespace api {

namespace {

const char* kSchema = R"JSON({
 "openapi": "3.0.3",
 "info": {"title": "Text Generation Inference (B200)", "version": "0",
          "description": "Text generation server: continuous batching over paged KV, OpenAI-compatible routes",
          "license": {"name": "Apache 2.0"}},
 "paths": {
  "/generate": {"post": {"tags": ["Text Generation Inference"], "summary": "Generate tokens",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/GenerateRequest"}}}},
    "responses": {"200": {"description": "Generated text", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/GenerateResponse"}}}},
                  "422": {"description": "Input validation error", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ErrorResponse"}}}},
                  "424": {"description": "Generation error", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ErrorResponse"}}}},
                  "429": {"description": "Model is overloaded", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ErrorResponse"}}}},
                  "500": {"description": "Incomplete generation", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ErrorResponse"}}}}}}},
  "/generate_stream": {"post": {"tags": ["Text Generation Inference"], "summary": "Generate a stream of tokens (server-sent events)",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/GenerateRequest"}}}},
    "responses": {"200": {"description": "Stream of StreamResponse events", "content": {"text/event-stream": {"schema": {"$ref": "#/components/schemas/StreamResponse"}}}}}}},
  "/": {"post": {"tags": ["Text Generation Inference"], "summary": "Generate tokens if `stream == false`, or a stream of tokens if `stream == true`",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/CompatGenerateRequest"}}}},
    "responses": {"200": {"description": "Generated text or event stream"}}},
   "get": {"summary": "Health probe of the root path", "responses": {"200": {"description": "OK"}}}},
  "/v1/chat/completions": {"post": {"tags": ["Text Generation Inference"], "summary": "Generate chat completions (OpenAI schema)",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ChatRequest"}}}},
    "responses": {"200": {"description": "chat.completion object or chat.completion.chunk events"}}}},
  "/v1/completions": {"post": {"tags": ["Text Generation Inference"], "summary": "Generate completions (OpenAI schema)",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/CompletionRequest"}}}},
    "responses": {"200": {"description": "text_completion object or events"}}}},
  "/v1/models": {"get": {"summary": "Model served", "responses": {"200": {"description": "list object"}}}},
  "/tokenize": {"post": {"summary": "Tokenize inputs",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/GenerateRequest"}}}},
    "responses": {"200": {"description": "Tokens", "content": {"application/json": {"schema": {"type": "array", "items": {"$ref": "#/components/schemas/SimpleToken"}}}}}}}},
  "/chat_tokenize": {"post": {"summary": "Template and tokenize a chat request",
    "requestBody": {"required": true, "content": {"application/json": {"schema": {"$ref": "#/components/schemas/ChatRequest"}}}},
    "responses": {"200": {"description": "tokenize_response and templated_text"}}}},
  "/info": {"get": {"summary": "Model and router limits", "responses": {"200": {"description": "Info", "content": {"application/json": {"schema": {"$ref": "#/components/schemas/Info"}}}}}}},
  "/health": {"get": {"summary": "Backend health probe", "responses": {"200": {"description": "Healthy"}, "503": {"description": "Unhealthy"}}}},
  "/ping": {"get": {"summary": "Alias of /health", "responses": {"200": {"description": "Healthy"}}}},
  "/metrics": {"get": {"summary": "Prometheus metrics (text exposition format)", "responses": {"200": {"description": "Metrics"}}}},
  "/invocations": {"post": {"summary": "SageMaker: generate, chat or completion request by shape", "responses": {"200": {"description": "Response of the matching route"}}}},
  "/vertex": {"post": {"summary": "Vertex AI: `instances` of generate / chat / completion requests", "responses": {"200": {"description": "predictions"}}}},
  "/v2/health/live": {"get": {"summary": "KServe liveness", "responses": {"200": {"description": "live"}}}},
  "/v2/health/ready": {"get": {"summary": "KServe readiness", "responses": {"200": {"description": "ready"}}}},
  "/v2/models/{model_name}/versions/{model_version}/infer": {"post": {"summary": "KServe v2 inference", "responses": {"200": {"description": "outputs"}}}}
 },
 "components": {"schemas": {
  "GenerateRequest": {"type": "object", "required": ["inputs"], "properties": {
    "inputs": {"type": "string", "example": "My name is Olivier and I"},
    "parameters": {"$ref": "#/components/schemas/GenerateParameters"}}},
  "CompatGenerateRequest": {"type": "object", "required": ["inputs"], "properties": {
    "inputs": {"type": "string"}, "parameters": {"$ref": "#/components/schemas/GenerateParameters"},
    "stream": {"type": "boolean", "default": false}}},
  "GenerateParameters": {"type": "object", "properties": {
    "best_of": {"type": "integer", "minimum": 1, "nullable": true},
    "temperature": {"type": "number", "exclusiveMinimum": 0, "nullable": true},
    "repetition_penalty": {"type": "number", "exclusiveMinimum": 0, "nullable": true},
    "frequency_penalty": {"type": "number", "minimum": -2, "maximum": 2, "nullable": true},
    "top_k": {"type": "integer", "exclusiveMinimum": 0, "nullable": true},
    "top_p": {"type": "number", "exclusiveMinimum": 0, "exclusiveMaximum": 1, "nullable": true},
    "typical_p": {"type": "number", "exclusiveMinimum": 0, "exclusiveMaximum": 1, "nullable": true},
    "do_sample": {"type": "boolean", "default": false},
    "max_new_tokens": {"type": "integer", "minimum": 0, "nullable": true},
    "return_full_text": {"type": "boolean", "nullable": true},
    "stop": {"type": "array", "items": {"type": "string"}, "maxItems": 4},
    "truncate": {"type": "integer", "nullable": true},
    "watermark": {"type": "boolean", "default": false},
    "details": {"type": "boolean", "default": false},
    "decoder_input_details": {"type": "boolean", "default": false},
    "seed": {"type": "integer", "minimum": 0, "nullable": true},
    "top_n_tokens": {"type": "integer", "minimum": 0, "maximum": 5, "nullable": true},
    "grammar": {"$ref": "#/components/schemas/GrammarType"},
    "adapter_id": {"type": "string", "nullable": true}}},
  "GrammarType": {"type": "object", "required": ["type", "value"], "properties": {
    "type": {"type": "string", "enum": ["json", "json_schema", "regex"]}, "value": {}}},
  "GenerateResponse": {"type": "object", "required": ["generated_text"], "properties": {
    "generated_text": {"type": "string"}, "details": {"$ref": "#/components/schemas/Details"}}},
  "Details": {"type": "object", "required": ["finish_reason", "generated_tokens", "prefill", "tokens"], "properties": {
    "finish_reason": {"$ref": "#/components/schemas/FinishReason"},
    "generated_tokens": {"type": "integer"}, "seed": {"type": "integer", "nullable": true},
    "prefill": {"type": "array", "items": {"$ref": "#/components/schemas/PrefillToken"}},
    "tokens": {"type": "array", "items": {"$ref": "#/components/schemas/Token"}},
    "top_tokens": {"type": "array", "items": {"type": "array", "items": {"$ref": "#/components/schemas/Token"}}},
    "best_of_sequences": {"type": "array", "items": {"$ref": "#/components/schemas/BestOfSequence"}}}},
  "BestOfSequence": {"type": "object", "properties": {
    "generated_text": {"type": "string"}, "finish_reason": {"$ref": "#/components/schemas/FinishReason"},
    "generated_tokens": {"type": "integer"}, "seed": {"type": "integer", "nullable": true},
    "prefill": {"type": "array", "items": {"$ref": "#/components/schemas/PrefillToken"}},
    "tokens": {"type": "array", "items": {"$ref": "#/components/schemas/Token"}}}},
  "FinishReason": {"type": "string", "enum": ["length", "eos_token", "stop_sequence"]},
  "Token": {"type": "object", "required": ["id", "text", "logprob", "special"], "properties": {
    "id": {"type": "integer"}, "text": {"type": "string"}, "logprob": {"type": "number"}, "special": {"type": "boolean"}}},
  "PrefillToken": {"type": "object", "required": ["id", "text", "logprob"], "properties": {
    "id": {"type": "integer"}, "text": {"type": "string"}, "logprob": {"type": "number", "nullable": true}}},
  "SimpleToken": {"type": "object", "properties": {
    "id": {"type": "integer"}, "text": {"type": "string"}, "start": {"type": "integer"}, "stop": {"type": "integer"}}},
  "StreamResponse": {"type": "object", "required": ["index", "token"], "properties": {
    "index": {"type": "integer"}, "token": {"$ref": "#/components/schemas/Token"},
    "top_tokens": {"type": "array", "items": {"$ref": "#/components/schemas/Token"}},
    "generated_text": {"type": "string", "nullable": true},
    "details": {"$ref": "#/components/schemas/StreamDetails"}}},
  "StreamDetails": {"type": "object", "nullable": true, "properties": {
    "finish_reason": {"$ref": "#/components/schemas/FinishReason"}, "generated_tokens": {"type": "integer"},
    "seed": {"type": "integer", "nullable": true}, "input_length": {"type": "integer"}}},
  "ErrorResponse": {"type": "object", "required": ["error", "error_type"], "properties": {
    "error": {"type": "string"}, "error_type": {"type": "string"}}},
  "Message": {"type": "object", "required": ["role"], "properties": {
    "role": {"type": "string"}, "name": {"type": "string", "nullable": true},
    "content": {"oneOf": [{"type": "string"}, {"type": "array", "items": {"$ref": "#/components/schemas/MessageChunk"}}]},
    "tool_calls": {"type": "array", "items": {"type": "object"}}}},
  "MessageChunk": {"type": "object", "required": ["type"], "properties": {
    "type": {"type": "string", "enum": ["text", "image_url"]}, "text": {"type": "string"},
    "image_url": {"type": "object", "properties": {"url": {"type": "string"}}}}},
  "ChatRequest": {"type": "object", "required": ["messages"], "properties": {
    "model": {"type": "string", "nullable": true, "description": "anything but \"tgi\" selects the LoRA adapter of that name"},
    "messages": {"type": "array", "items": {"$ref": "#/components/schemas/Message"}},
    "frequency_penalty": {"type": "number", "nullable": true}, "presence_penalty": {"type": "number", "nullable": true},
    "logit_bias": {"type": "array", "items": {"type": "number"}, "nullable": true},
    "logprobs": {"type": "boolean", "nullable": true}, "top_logprobs": {"type": "integer", "minimum": 0, "maximum": 5, "nullable": true},
    "max_tokens": {"type": "integer", "nullable": true}, "max_completion_tokens": {"type": "integer", "nullable": true},
    "n": {"type": "integer", "nullable": true}, "stop": {"type": "array", "items": {"type": "string"}, "nullable": true},
    "stream": {"type": "boolean", "default": false}, "seed": {"type": "integer", "nullable": true},
    "temperature": {"type": "number", "nullable": true}, "top_p": {"type": "number", "nullable": true},
    "tools": {"type": "array", "items": {"type": "object"}, "nullable": true}, "tool_prompt": {"type": "string", "nullable": true},
    "tool_choice": {"nullable": true}, "response_format": {"$ref": "#/components/schemas/GrammarType"},
    "stream_options": {"type": "object", "properties": {"include_usage": {"type": "boolean"}}}}},
  "CompletionRequest": {"type": "object", "required": ["prompt"], "properties": {
    "model": {"type": "string", "nullable": true},
    "prompt": {"oneOf": [{"type": "string"}, {"type": "array", "items": {"type": "string"}}]},
    "max_tokens": {"type": "integer", "nullable": true}, "temperature": {"type": "number", "nullable": true},
    "top_p": {"type": "number", "nullable": true}, "stream": {"type": "boolean", "default": false},
    "seed": {"type": "integer", "nullable": true}, "suffix": {"type": "string", "nullable": true},
    "repetition_penalty": {"type": "number", "nullable": true}, "frequency_penalty": {"type": "number", "nullable": true},
    "stop": {"type": "array", "items": {"type": "string"}, "nullable": true}}},
  "Info": {"type": "object", "properties": {
    "model_id": {"type": "string"}, "model_sha": {"type": "string", "nullable": true}, "model_pipeline_tag": {"type": "string", "nullable": true},
    "max_concurrent_requests": {"type": "integer"}, "max_best_of": {"type": "integer"}, "max_stop_sequences": {"type": "integer"},
    "max_input_tokens": {"type": "integer"}, "max_total_tokens": {"type": "integer"}, "validation_workers": {"type": "integer"},
    "max_client_batch_size": {"type": "integer"}, "router": {"type": "string"}, "version": {"type": "string"},
    "sha": {"type": "string", "nullable": true}, "docker_label": {"type": "string", "nullable": true}}}
 }}
})JSON";

}  // namespace

json::Value openapi_schema(const std::string& version) {
  json::Value doc = json::Value::parse(kSchema);
  json::Value info = doc["info"];
  info.set("version", version);
  doc.set("info", info);
  return doc;
}

// Self-contained page (no external scripts): lists every path of the schema with its summary and request type.
std::string openapi_html() {
  return R"HTML(<!doctype html><html><head><meta charset="utf-8"><title>Text Generation Inference (B200) API</title>
<style>body{font-family:sans-serif;margin:2em;max-width:60em}code{background:#eee;padding:1px 4px}
.m{display:inline-block;width:4em;font-weight:bold}.post{color:#0a6}.get{color:#06c}li{margin:.4em 0}</style></head>
<body><h1>Text Generation Inference (B200) API</h1><p>Schema: <a href="/api-doc/openapi.json">/api-doc/openapi.json</a></p>
<ul id="paths"></ul><h2>Schemas</h2><pre id="schemas"></pre>
<script>fetch('/api-doc/openapi.json').then(r=>r.json()).then(d=>{const ul=document.getElementById('paths');
for(const [p,ms] of Object.entries(d.paths))for(const [m,o] of Object.entries(ms)){const li=document.createElement('li');
const rb=o.requestBody&&o.requestBody.content['application/json'].schema['$ref'];
li.innerHTML='<span class="m '+m+'">'+m.toUpperCase()+'</span><code>'+p+'</code> '+(o.summary||'')+(rb?' &mdash; body: <code>'+rb.split('/').pop()+'</code>':'');
ul.appendChild(li);}document.getElementById('schemas').textContent=JSON.stringify(d.components.schemas,null,1);});</script>
</body></html>)HTML";
}

}  // namespace api
