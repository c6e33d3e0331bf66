// tgi-b200-router: HTTP front + scheduler process.  Connects to the shard processes, warms them
// up, derives the serving limits and serves the REST API.
// (Reference: backends/v3/src/main.rs:9-196 flags and checks, backends/v3/src/lib.rs:48-169
// connect_backend, router/src/server.rs:1502-1867 run.)
#include <csignal>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <map>

#include "trace.hpp"
#include "usage.hpp"
#include "api.hpp"
#include "http.hpp"
#include "metrics.hpp"
#include "pybridge.hpp"
#include "scheduler.hpp"
#include "shard_client.hpp"

namespace {

http::Server* g_server = nullptr;
void on_signal(int) {
  if (g_server) g_server->stop();
}

struct Args {
  std::map<std::string, std::string> kv;
  // --flag value | --flag=value | env FLAG (upper case, dashes -> underscores)
  Args(int argc, char** argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.rfind("--", 0) != 0) continue;
      a = a.substr(2);
      size_t eq = a.find('=');
      if (eq != std::string::npos) kv[a.substr(0, eq)] = a.substr(eq + 1);
      else if (i + 1 < argc && std::strncmp(argv[i + 1], "--", 2) != 0) kv[a] = argv[++i];
      else kv[a] = "true";
    }
  }
  std::string get(const std::string& name, const std::string& dflt = "") const {
    auto it = kv.find(name);
    if (it != kv.end()) return it->second;
    std::string env = name;
    for (auto& c : env) c = c == '-' ? '_' : static_cast<char>(toupper(c));
    const char* e = std::getenv(env.c_str());
    return e ? e : dflt;
  }
  long num(const std::string& name, long dflt) const {
    std::string v = get(name);
    return v.empty() ? dflt : std::strtol(v.c_str(), nullptr, 10);
  }
  bool flag(const std::string& name) const {
    std::string v = get(name);
    return v == "true" || v == "1";
  }
  bool has(const std::string& name) const { return !get(name).empty(); }
};

api::TextServices python_text_services() {
  api::TextServices t;
  t.encode = [](const std::string& text, bool add, uint32_t truncate) {
    json::Value a = json::Value::object();
    a.set("text", text);
    a.set("add_special_tokens", add);
    if (truncate) a.set("truncate", truncate);
    json::Value r = bridge::call("encode", a);
    std::vector<uint32_t> ids;
    for (auto& v : r["ids"].items()) ids.push_back(static_cast<uint32_t>(v.as_int()));
    return ids;
  };
  t.encode_with_offsets = [](const std::string& text, bool add) {
    json::Value a = json::Value::object();
    a.set("text", text);
    a.set("add_special_tokens", add);
    a.set("offsets", true);
    return bridge::call("encode", a)["tokens"];
  };
  t.chat_template = [](const json::Value& messages, const json::Value& tools, const std::string& tool_prompt) {
    json::Value a = json::Value::object();
    a.set("messages", messages);
    if (!tools.is_null()) a.set("tools", tools);
    a.set("tool_prompt", tool_prompt);
    json::Value r = bridge::call("apply_chat_template", a);
    if (!r["ok"].as_bool()) throw api::ApiError(422, r["error_type"].as_string(), r["error"].as_string());
    return r["text"].as_string();
  };
  t.compile_grammar = [](const std::string& type, const json::Value& value) {
    json::Value a = json::Value::object();
    a.set("type", type);
    a.set("value", value);
    json::Value r = bridge::call("compile_grammar", a);
    if (!r["ok"].as_bool()) throw api::validation_error(r["error"].as_string());
    return std::make_pair(r["grammar"].as_string(), static_cast<uint32_t>(r["grammar_type"].as_int()));
  };
  return t;
}

// Worst-case batch for the memory probe of the shards: full-length prompts up to the prefill
// budget, all sampling stages on, prompt logprobs and top tokens requested.
pb::Batch warmup_batch(uint32_t max_input_tokens, uint32_t max_prefill_tokens, uint32_t max_total_tokens,
                       uint32_t block_size) {
  pb::Batch b;
  uint32_t n_tokens = 0;
  uint64_t id = 0;
  while (n_tokens < max_prefill_tokens) {
    const uint32_t len = std::min(max_input_tokens, max_prefill_tokens - n_tokens);
    pb::Request r;
    r.id = id++;
    std::string text;
    for (uint32_t i = 0; i < len; ++i) text += "_test ";
    r.inputs = text;
    pb::InputChunk c;
    c.text = text;
    r.input_chunks.push_back(c);
    r.truncate = len;
    r.add_special_tokens = true;
    r.prefill_logprobs = true;
    r.top_n_tokens = 20;
    r.parameters.temperature = 0.9f;
    r.parameters.top_k = 10;
    r.parameters.top_p = 0.9f;
    r.parameters.typical_p = 0.9f;
    r.parameters.do_sample = false;
    r.parameters.repetition_penalty = 1.2f;
    r.parameters.frequency_penalty = 0.1f;
    r.stopping_parameters.max_new_tokens = max_total_tokens > len ? max_total_tokens - len : 1;
    r.stopping_parameters.ignore_eos_token = true;
    b.requests.push_back(r);
    n_tokens += len;
  }
  b.id = 0;
  b.size = static_cast<uint32_t>(b.requests.size());
  b.max_tokens = max_input_tokens * b.size;
  b.max_blocks = (max_total_tokens + block_size - 1) / block_size;
  return b;
}

}  // namespace

int main(int argc, char** argv) {
  Args args(argc, argv);
  if (argc > 1 && std::string(argv[1]) == "print-schema") {   // OpenAPI document on stdout, nothing else started
    std::cout << api::openapi_schema("0").dump() << std::endl;
    return 0;
  }
  if (args.flag("help")) {
    std::cout << "tgi-b200-router --master-shard-uds-path PATH --tokenizer-name DIR [--port 3000] [--hostname 0.0.0.0]\n"
                 "  [--max-concurrent-requests 128] [--max-best-of 2] [--max-stop-sequences 4] [--max-top-n-tokens 5]\n"
                 "  [--max-input-tokens N] [--max-total-tokens N] [--max-batch-prefill-tokens N] [--max-batch-total-tokens N]\n"
                 "  [--waiting-served-ratio 0.3] [--max-waiting-tokens 20] [--max-batch-size N] [--max-client-batch-size 4]\n"
                 "  [--api-key KEY] [--payload-limit BYTES] [--disable-grammar-support] [--repo-root DIR]\n";
    return 0;
  }
  std::unique_ptr<usage::Reporter> usage_reporter;   // outlives the try block: fatal errors are reported too
  try {
    const std::string uds = args.get("master-shard-uds-path", "/tmp/text-generation-server");
    const std::string tokenizer = args.get("tokenizer-name", args.get("model-id"));
    std::string repo_root = args.get("repo-root");
    if (repo_root.empty()) {
      // the binary lives in <repo>/text-generation-inference_b200/router/
      std::string self = argv[0];
      size_t p = self.rfind('/');
      repo_root = (p == std::string::npos ? std::string(".") : self.substr(0, p)) + "/../..";
    }
    bridge::init(repo_root);
    json::Value la = json::Value::object();
    la.set("tokenizer_name", tokenizer);
    json::Value loaded = bridge::call("load", la);
    if (!loaded["ok"].as_bool()) throw std::runtime_error("tokenizer load failed");

    std::cerr << "[router] connecting to shards at " << uds << std::endl;
    auto client = sched::ShardedClient::connect(uds, static_cast<int>(args.num("shard-connect-timeout", 1800)));
    client->clear_cache(std::nullopt);
    pb::InfoResponse info = client->info();

    uint32_t max_input = static_cast<uint32_t>(args.num("max-input-tokens", 0));
    uint32_t max_total = static_cast<uint32_t>(args.num("max-total-tokens", 0));
    uint32_t max_prefill = static_cast<uint32_t>(args.num("max-batch-prefill-tokens", 4096));
    if (max_input && max_total && max_input >= max_total)
      throw std::runtime_error("`max_input_tokens` must be < `max_total_tokens`");
    const uint32_t probe_input = max_input ? max_input : std::min<uint32_t>(max_prefill, 4095);
    const uint32_t probe_total = max_total ? max_total : probe_input + 1;
    if (!info.support_chunking && max_prefill < probe_input)
      throw std::runtime_error("`max_batch_prefill_tokens` must be >= `max_input_tokens`");
    std::cerr << "[router] warming up shards" << std::endl;
    pb::WarmupResponse w = client->warmup(warmup_batch(probe_input, max_prefill, probe_total, std::max(1u, info.block_size)),
                                          max_input ? std::optional<uint32_t>(max_input) : std::nullopt, max_prefill,
                                          max_total ? std::optional<uint32_t>(max_total) : std::nullopt);
    if (!max_input) max_input = w.max_input_tokens;
    if (!max_total) max_total = w.max_total_tokens;
    uint32_t max_batch_total = static_cast<uint32_t>(args.num("max-batch-total-tokens", 0));
    if (w.max_supported_total_tokens) {
      if (max_batch_total && max_batch_total > *w.max_supported_total_tokens)
        std::cerr << "[router] `--max-batch-total-tokens` is larger than what the shards support; clamping" << std::endl;
      if (!max_batch_total || max_batch_total > *w.max_supported_total_tokens)
        max_batch_total = *w.max_supported_total_tokens;
    } else if (!max_batch_total) {
      max_batch_total = std::max<uint32_t>(16000, std::max(max_total, max_prefill));
    }
    if (max_total > max_batch_total)
      throw std::runtime_error("`max_total_tokens` must be <= `max_batch_total_tokens`");
    std::cerr << "[router] max_input_tokens=" << max_input << " max_total_tokens=" << max_total
              << " max_batch_total_tokens=" << max_batch_total << " block_size=" << info.block_size << std::endl;

    sched::Metrics metrics(max_input, max_total);
    metrics.gauge_set("tgi_batch_max_total_tokens", max_batch_total);
    metrics.gauge_set("tgi_batch_total_tokens", max_batch_total);
    sched::QueueConfig qc;
    qc.requires_padding = info.requires_padding;
    qc.block_size = std::max(1u, info.block_size);
    qc.prefix_caching = info.use_prefix_caching && !args.flag("disable-prefix-caching");
    qc.window_size = info.window_size;
    qc.speculate = info.speculate;
    qc.support_chunking = info.support_chunking;
    qc.max_batch_total_tokens = max_batch_total;
    sched::BackendConfig bc;
    bc.max_batch_prefill_tokens = max_prefill;
    bc.max_batch_total_tokens = max_batch_total;
    bc.max_waiting_tokens = static_cast<uint32_t>(args.num("max-waiting-tokens", 20));
    bc.waiting_served_ratio_x100 = static_cast<uint32_t>(std::atof(args.get("waiting-served-ratio", "0.3").c_str()) * 100);
    if (args.has("max-batch-size")) bc.max_batch_size = static_cast<size_t>(args.num("max-batch-size", 0));
    auto backend = std::make_shared<sched::Backend>(client, qc, bc, &metrics);
    backend->start_thread();

    api::RouterConfig rc;
    rc.max_concurrent_requests = static_cast<size_t>(args.num("max-concurrent-requests", 128));
    rc.max_best_of = static_cast<uint32_t>(args.num("max-best-of", 2));
    rc.max_stop_sequences = static_cast<uint32_t>(args.num("max-stop-sequences", 4));
    rc.max_top_n_tokens = static_cast<uint32_t>(args.num("max-top-n-tokens", 5));
    rc.max_input_tokens = max_input;
    rc.max_total_tokens = max_total;
    rc.max_client_batch_size = static_cast<uint32_t>(args.num("max-client-batch-size", 4));
    rc.disable_grammar_support = args.flag("disable-grammar-support");
    // largest image a request may carry or point at (reference: --max-image-fetch-size, 1 GiB by default)
    rc.max_image_bytes = static_cast<size_t>(args.num("max-image-fetch-size", 1073741824L));
    rc.api_key = args.get("api-key");
    {
      std::stringstream origins(args.get("cors-allow-origin"));
      std::string o;
      while (std::getline(origins, o, ','))
        if (!o.empty()) rc.cors_allow_origin.push_back(o);
    }
    rc.model_id = args.get("model-id", tokenizer);
    rc.dtype = info.dtype;
    rc.device_type = info.device_type;
    rc.max_batch_total_tokens = max_batch_total;
    {
      // the checkpoint's config.json tells whether this is a vision-language model
      std::ifstream cf(tokenizer + "/config.json");
      if (cf) {
        std::stringstream ss;
        ss << cf.rdbuf();
        try {
          rc.model_config = json::Value::parse(ss.str());
        } catch (const std::exception&) {
        }
      }
    }
    api::TextServices text_services = python_text_services();
    if (rc.model_config.is_object() && rc.model_config.has("model_type") &&
        rc.model_config["model_type"].as_string() == "idefics3") {
      // Image splitting of Idefics3 / SmolVLM: the prompt of a split image contains marker tokens.  When the tokenizer
      // has them, the token count of an image follows the shard's layout (models/idefics3.py); the settings come
      // from the checkpoint's preprocessor_config.json.
      try {
        const auto fake = text_services.encode("<fake_token_around_image>", false, 0);
        const auto glob = text_services.encode("<global-img>", false, 0);
        const auto rc11 = text_services.encode("<row_1_col_1>", false, 0);
        if (fake.size() == 1 && glob.size() == 1 && rc11.size() == 1) {
          const json::Value& vis = rc.model_config["vision_config"];
          const double tile = vis.is_object() && vis.has("image_size") ? vis["image_size"].as_double() : 364;
          double longest = 4 * tile;
          bool split = true;
          std::ifstream pf(tokenizer + "/preprocessor_config.json");
          if (pf) {
            std::stringstream ss;
            ss << pf.rdbuf();
            try {
              json::Value pc = json::Value::parse(ss.str());
              if (pc.has("size") && pc["size"].is_object() && pc["size"].has("longest_edge"))
                longest = pc["size"]["longest_edge"].as_double();
              if (pc.has("do_image_splitting")) split = pc["do_image_splitting"].as_bool();
            } catch (const std::exception&) {
            }
          }
          json::Value sp = json::Value::object();
          sp.set("tile", tile);
          sp.set("longest_edge", longest);
          sp.set("split", split);
          sp.set("nl", static_cast<long>(text_services.encode("\n", false, 0).size()));
          sp.set("nlnl", static_cast<long>(text_services.encode("\n\n", false, 0).size()));
          rc.model_config.set("_idefics3", sp);
        }
      } catch (const std::exception& e) {
        std::cerr << "[router] idefics3 marker probe failed: " << e.what() << std::endl;
      }
    }
    if (rc.model_config.is_object() && rc.model_config.has("model_type") &&
        rc.model_config["model_type"].as_string() == "paligemma" && loaded.has("bos_token") &&
        loaded["bos_token"].is_string() && !loaded["bos_token"].as_string().empty()) {
      // PaliGemma: every text piece is bos + text + "\n", tokenised as it stands (the shard does the same)
      json::Value w = json::Value::object();
      w.set("prefix", loaded["bos_token"].as_string());
      w.set("suffix", "\n");
      rc.model_config.set("_text_wrap", w);
    }
    if (rc.model_config.is_object() && rc.model_config.has("model_type") &&
        rc.model_config["model_type"].as_string() == "gemma3" && rc.model_config.has("vision_config") &&
        loaded.has("is_hf_tokenizer") && loaded["is_hf_tokenizer"].as_bool()) {
      const size_t pad = text_services.encode("\n\n", false, 0).size();
      if (pad > 0 && pad <= 2) {
        json::Value g = json::Value::object();
        g.set("pad", static_cast<long>(pad));
        rc.model_config.set("_gemma3", g);
      }
    }
    if (rc.model_config.is_object() && rc.model_config.has("model_type") &&
        rc.model_config["model_type"].as_string() == "idefics2") {
      try {
        if (text_services.encode("<fake_token_around_image>", false, 0).size() == 1) {
          bool split = false;
          std::ifstream pf(tokenizer + "/preprocessor_config.json");
          if (pf) {
            std::stringstream ss;
            ss << pf.rdbuf();
            try {
              json::Value pc = json::Value::parse(ss.str());
              if (pc.has("do_image_splitting")) split = pc["do_image_splitting"].as_bool();
            } catch (const std::exception&) {
            }
          }
          json::Value sp = json::Value::object();
          sp.set("split", split);
          rc.model_config.set("_idefics2", sp);
        }
      } catch (const std::exception& e) {
        std::cerr << "[router] idefics2 marker probe failed: " << e.what() << std::endl;
      }
    }
    api::Router router(backend, text_services, rc, &metrics);

    http::Server server(args.get("hostname", "0.0.0.0"), static_cast<int>(args.num("port", 3000)),
                        static_cast<size_t>(args.num("payload-limit", 2000000)));
    router.install(server);
    // request spans go to an OTLP/HTTP collector when one is configured
    trace::init(args.get("otlp-endpoint"), args.get("otlp-service-name", "text-generation-inference.router"));
    // usage statistics (off unless asked for; events go to the operator's collector or file, nowhere else)
    json::Value uargs = json::Value::object();
    uargs.set("model_config", rc.model_config.is_object() && rc.model_config.has("model_type")
                                  ? json::Value(rc.model_config["model_type"].as_string()) : json::Value());
    uargs.set("tokenizer_class", json::Value());
    uargs.set("validation_workers", args.num("validation-workers", 2));
    uargs.set("max_concurrent_requests", static_cast<long>(rc.max_concurrent_requests));
    uargs.set("max_best_of", static_cast<long>(rc.max_best_of));
    uargs.set("max_stop_sequences", static_cast<long>(rc.max_stop_sequences));
    uargs.set("max_top_n_tokens", static_cast<long>(rc.max_top_n_tokens));
    uargs.set("max_input_tokens", static_cast<long>(rc.max_input_tokens));
    uargs.set("max_total_tokens", static_cast<long>(rc.max_total_tokens));
    uargs.set("max_batch_total_tokens", static_cast<long>(rc.max_batch_total_tokens));
    uargs.set("max_client_batch_size", static_cast<long>(rc.max_client_batch_size));
    uargs.set("disable_grammar_support", rc.disable_grammar_support);
    uargs.set("usage_stats_level", args.get("usage-stats", "off"));
    usage_reporter = std::make_unique<usage::Reporter>(args.get("usage-stats", "off"), args.get("usage-stats-endpoint"),
                                                       args.get("usage-stats-file"), uargs);
    g_server = &server;
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    std::signal(SIGPIPE, SIG_IGN);
    const int port = server.start();
    std::cerr << "[router] Connected; listening on port " << port << std::endl;
    usage_reporter->send("Start");
    usage_reporter->start_pings(static_cast<int>(args.num("usage-stats-ping-seconds", 900)));
    // optional second listener that only serves the Prometheus text format (reference: --prometheus-port)
    std::unique_ptr<http::Server> prom;
    std::thread prom_thread;
    if (args.num("prometheus-port", 0) > 0) {
      prom = std::make_unique<http::Server>(args.get("hostname", "0.0.0.0"), static_cast<int>(args.num("prometheus-port", 0)),
                                            static_cast<size_t>(1 << 16));
      prom->route("GET", "/metrics", [&metrics](const http::Request&, http::Response& r) {
        r.send(200, "text/plain; version=0.0.4", metrics.render());
      });
      const int pport = prom->start();
      std::cerr << "[router] Prometheus metrics on port " << pport << std::endl;
      prom_thread = std::thread([&prom] { prom->serve_forever(); });
    }
    server.serve_forever();
    if (prom) {
      prom->stop();
      if (prom_thread.joinable()) prom_thread.join();
    }
    backend->stop();
    usage_reporter->send("Stop");
    trace::shutdown();   // flushes the spans still queued
    std::cerr << "[router] shut down" << std::endl;
    return 0;
  } catch (const std::exception& e) {
    std::cerr << "[router] fatal: " << e.what() << std::endl;
    if (usage_reporter) usage_reporter->send("Error", e.what());
    return 1;
  }
}
