// tgi-b200-launcher: reads the model config, decides the serving limits, starts one shard process
// per GPU and the router, forwards their logs and supervises them.
//
// Reference: launcher/src/main.rs — flags (:582-914), `resolve_attention` (:131-200), `find_num_shards`
// (:1374-1413), FLOP/VRAM based default for max_batch_prefill_tokens (:28-89, 261-352, 2114-2154),
// `download_convert_model` (:1434-1577), `shard_manager` (:923-1249) with `log_lines` (:1294-1372),
// `spawn_webserver` (:1831-2013), `terminate` (:2015-2036), supervision loop (:2333-2361).
//
// Order of a start: weights are fetched / converted by `text-generation-server download-weights` before any
// shard exists; the shards start with --json-output and their records are re-emitted at their own level under
// the shard's name; the router starts once every shard's socket is there; any child that exits brings the
// deployment down.
#include <fcntl.h>
#include <signal.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "json.hpp"

namespace {

volatile sig_atomic_t g_stop = 0;
void on_signal(int) { g_stop = 1; }

struct Args {
  std::map<std::string, std::string> kv;
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
  bool has(const std::string& n) const { return !get(n).empty(); }
  long num(const std::string& n, long d) const { return has(n) ? std::strtol(get(n).c_str(), nullptr, 10) : d; }
};

struct Child {
  pid_t pid = -1;
  std::string name;
};

// Model facts used for the automatic limits.
struct ModelFacts {
  double flops_per_token = 0;     // forward FLOPs per token
  double weight_bytes = 0;        // bytes of parameters at the serving dtype
  double kv_bytes_per_token = 0;
  long max_position_embeddings = 0;
  bool ok = false;
};

ModelFacts read_model(const std::string& model_dir, double bytes_per_param, double kv_bytes) {
  ModelFacts f;
  std::ifstream in(model_dir + "/config.json");
  if (!in) return f;
  std::stringstream ss;
  ss << in.rdbuf();
  json::Value c;
  try {
    c = json::Value::parse(ss.str());
  } catch (...) {
    return f;
  }
  if (c["text_config"].is_object()) c = c["text_config"];
  auto num = [&](const char* k, double d) { return c[k].is_number() ? c[k].as_double() : d; };
  const double H = num("hidden_size", 0), L = num("num_hidden_layers", 0), nh = num("num_attention_heads", 0);
  if (H == 0 || L == 0 || nh == 0) return f;
  const double hd = num("head_dim", H / nh), nkv = num("num_key_value_heads", nh);
  const double I = num("intermediate_size", 4 * H), V = num("vocab_size", 32000);
  const double experts_active = num("num_experts_per_tok", 1), experts = num("num_local_experts", num("num_experts", 1));
  const double attn = H * (nh * hd) + 2 * H * (nkv * hd) + (nh * hd) * H;
  const double mlp = 3 * H * I;
  f.flops_per_token = 2 * (L * (attn + mlp * experts_active) + V * H);
  f.weight_bytes = (L * (attn + mlp * experts) + 2 * V * H) * bytes_per_param;
  f.kv_bytes_per_token = 2 * L * nkv * hd * kv_bytes;
  f.max_position_embeddings = static_cast<long>(num("max_position_embeddings", 4096));
  f.ok = true;
  return f;
}

int count_gpus() {
  const char* vis = std::getenv("CUDA_VISIBLE_DEVICES");
  if (vis == nullptr) vis = std::getenv("NVIDIA_VISIBLE_DEVICES");
  if (vis != nullptr && std::string(vis) != "all" && std::string(vis) != "") {
    int n = 1;
    for (const char* p = vis; *p; ++p) n += *p == ',';
    return n;
  }
  FILE* p = popen("nvidia-smi --list-gpus 2>/dev/null | wc -l", "r");
  int n = 0;
  if (p) {
    if (fscanf(p, "%d", &n) != 1) n = 0;
    pclose(p);
  }
  return n;
}

double gpu_memory_bytes() {
  FILE* p = popen("nvidia-smi --query-gpu=memory.total --format=csv,noheader,nounits 2>/dev/null | head -1", "r");
  double mib = 0;
  if (p) {
    if (fscanf(p, "%lf", &mib) != 1) mib = 0;
    pclose(p);
  }
  return mib * 1024.0 * 1024.0;
}

// ---- logging -----------------------------------------------------------------------------------
bool g_json_output = false;
std::mutex g_log_mutex;

std::string json_escape(const std::string& s) {
  std::string o;
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += static_cast<char>(c); }
    else if (c == '\n') o += "\\n";
    else if (c == '\t') o += "\\t";
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
    else o += static_cast<char>(c);
  }
  return o;
}

void log_line(const std::string& level, const std::string& target, const std::string& message) {
  std::lock_guard<std::mutex> g(g_log_mutex);
  if (g_json_output) {
    const auto now = std::chrono::duration_cast<std::chrono::milliseconds>(
                         std::chrono::system_clock::now().time_since_epoch()).count();
    std::cout << "{\"timestamp\":" << now << ",\"level\":\"" << level << "\",\"target\":\"" << json_escape(target)
              << "\",\"message\":\"" << json_escape(message) << "\"}" << std::endl;
  } else {
    std::cerr << "[" << target << "] " << level << " " << message << std::endl;
  }
}

// One output line of a child.  Shards write JSON records when started with --json-output (the launcher always
// starts them so): those are re-emitted at their own level under the child's name, like the reference's
// `log_lines` (launcher/src/main.rs:1294-1372).  Anything else (tracebacks, library chatter, the router's plain
// text) is passed on as an INFO line.
void forward_child_line(const std::string& name, const std::string& line) {
  if (line.empty()) return;
  if (line[0] == '{') {
    try {
      json::Value v = json::Value::parse(line);
      if (v.is_object() && v["message"].is_string()) {
        std::string level = v["level"].is_string() ? v["level"].as_string() : "INFO";
        for (auto& c : level) c = static_cast<char>(toupper(c));
        if (level == "WARN") level = "WARNING";
        log_line(level, name, v["message"].as_string());
        return;
      }
    } catch (const std::exception&) {
    }
  }
  log_line("INFO", name, line);
}

struct Spawned {
  pid_t pid = -1;
  int out_fd = -1;   // read end of the child's stdout + stderr
};

Spawned spawn(const std::vector<std::string>& argv, const std::map<std::string, std::string>& env, bool capture) {
  int fds[2] = {-1, -1};
  if (capture && pipe(fds) != 0) capture = false;
  pid_t pid = fork();
  if (pid != 0) {
    Spawned s;
    s.pid = pid;
    if (capture) {
      close(fds[1]);
      s.out_fd = fds[0];
    }
    return s;
  }
  setpgid(0, 0);
  if (capture) {
    dup2(fds[1], STDOUT_FILENO);
    dup2(fds[1], STDERR_FILENO);
    close(fds[0]);
    close(fds[1]);
  }
  for (auto& kv : env) setenv(kv.first.c_str(), kv.second.c_str(), 1);
  std::vector<char*> a;
  for (auto& s : argv) a.push_back(const_cast<char*>(s.c_str()));
  a.push_back(nullptr);
  execvp(a[0], a.data());
  std::perror("exec");
  _exit(127);
}

// Reads the child's output until it closes and forwards it line by line.
std::thread log_pump(const std::string& name, int fd) {
  return std::thread([name, fd] {
    std::string buf;
    char chunk[4096];
    while (true) {
      const ssize_t n = read(fd, chunk, sizeof chunk);
      if (n <= 0) break;
      buf.append(chunk, static_cast<size_t>(n));
      size_t nl;
      while ((nl = buf.find('\n')) != std::string::npos) {
        forward_child_line(name, buf.substr(0, nl));
        buf.erase(0, nl + 1);
      }
    }
    if (!buf.empty()) forward_child_line(name, buf);
    close(fd);
  });
}

void terminate(std::vector<Child>& children, int grace_s) {
  for (auto& c : children)
    if (c.pid > 0) kill(c.pid, SIGTERM);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(grace_s);
  for (auto& c : children) {
    while (c.pid > 0) {
      int st;
      if (waitpid(c.pid, &st, WNOHANG) == c.pid) { c.pid = -1; break; }
      if (std::chrono::steady_clock::now() > deadline) {
        kill(c.pid, SIGKILL);
        waitpid(c.pid, &st, 0);
        c.pid = -1;
        break;
      }
      usleep(100000);
    }
  }
}

// Dense bf16 tensor rate of one GPU by product name (reference: ComputeType::f16_flop, launcher/src/main.rs:
// 1753-1811); `--peak-flops` / PEAK_FLOPS overrides it, an unknown card counts as 1e15.
double peak_flops_per_gpu(const Args& args) {
  if (args.has("peak-flops")) return std::atof(args.get("peak-flops").c_str());
  std::string name;
  FILE* p = popen("nvidia-smi --query-gpu=name --format=csv,noheader 2>/dev/null | head -1", "r");
  if (p) {
    char b[256];
    if (fgets(b, sizeof b, p)) name = b;
    pclose(p);
  }
  for (auto& c : name) c = static_cast<char>(tolower(c));
  struct { const char* key; double flops; } table[] = {
      {"b200", 2.25e15}, {"b100", 1.8e15}, {"gb200", 2.5e15}, {"h200", 0.99e15}, {"h100", 0.99e15}, {"h20", 0.148e15},
      {"a100", 0.312e15}, {"l40s", 0.362e15}, {"l40", 0.181e15}, {"l4", 0.121e15}, {"a10g", 0.125e15}, {"a10", 0.125e15},
      {"t4", 0.065e15}};
  for (auto& t : table)
    if (name.find(t.key) != std::string::npos) return t.flops;
  return 1e15;
}

// Prefix caching is switched off for models whose prompts are not plain token sequences, as the reference's
// `resolve_attention` does (launcher/src/main.rs:131-200): vision-language models, encoder-decoder models, and
// deployments with LoRA adapters (the cached KV depends on the adapter).  PREFIX_CACHING in the environment wins.
std::string resolve_prefix_caching(const std::string& model_dir, const Args& args) {
  if (const char* e = std::getenv("PREFIX_CACHING")) return e;
  std::ifstream in(model_dir + "/config.json");
  if (in) {
    std::stringstream ss;
    ss << in.rdbuf();
    try {
      json::Value c = json::Value::parse(ss.str());
      if (c["vision_config"].is_object()) {
        log_line("INFO", "launcher", "Disabling prefix caching because of VLM model");
        return "0";
      }
      if (c["is_encoder_decoder"].is_bool() && c["is_encoder_decoder"].as_bool()) {
        log_line("INFO", "launcher", "Disabling prefix caching because of seq2seq model");
        return "0";
      }
    } catch (const std::exception&) {
    }
  }
  if (args.has("lora-adapters")) {
    log_line("INFO", "launcher", "Disabling prefix caching because of lora adapters");
    return "0";
  }
  return "1";
}

}  // namespace

int main(int argc, char** argv) {
  Args args(argc, argv);
  if (args.has("help") || !args.has("model-id")) {
    std::cout <<
        "tgi-b200-launcher --model-id ID_OR_DIR [options]   (every option also reads the upper-case environment variable)\n"
        "  model:     --revision R --quantize fp8|gptq|awq|eetq|exl2|marlin|bitsandbytes[-nf4|-fp4]|compressed-tensors\n"
        "             --dtype bfloat16|float16 --kv-cache-dtype fp8_e4m3fn|fp8_e5m2 --speculate N --trust-remote-code\n"
        "             --lora-adapters a,b --rope-scaling linear|dynamic --rope-factor F --tokenizer-config-path P\n"
        "             --huggingface-hub-cache DIR --weights-cache-override DIR --disable-custom-kernels\n"
        "  shards:    --sharded true|false --num-shard N --shard-uds-path /tmp/text-generation-server --master-addr 127.0.0.1\n"
        "             --master-port 29500 --cuda-graphs 1,2,4,... --cuda-memory-fraction 1.0 --peak-flops F\n"
        "  limits:    --max-input-tokens N (--max-input-length) --max-total-tokens N --max-batch-prefill-tokens N\n"
        "             --max-batch-total-tokens N --max-batch-size N --max-concurrent-requests 128 --max-best-of 2\n"
        "             --max-stop-sequences 4 --max-top-n-tokens 5 --max-waiting-tokens 20 --waiting-served-ratio 0.3\n"
        "             --max-client-batch-size 4 --payload-limit 2000000 --validation-workers 2\n"
        "  serving:   --hostname 0.0.0.0 --port 3000 --prometheus-port 9000 --api-key KEY --cors-allow-origin a,b\n"
        "             --disable-grammar-support --enable-prefill-logprobs --watermark-gamma G --watermark-delta D\n"
        "  operation: --json-output --otlp-endpoint URL --otlp-service-name NAME --usage-stats on|off|no-stack --usage-stats-endpoint URL --usage-stats-file PATH --max-image-fetch-size BYTES\n"
        "             --graceful-termination-timeout 90 --env --python python\n";
    return args.has("help") ? 0 : 2;
  }
  g_json_output = args.has("json-output");
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  signal(SIGPIPE, SIG_IGN);
  if (args.has("ngrok")) {
    log_line("ERROR", "launcher", "ngrok tunnels are not supported");
    return 2;
  }
  const std::string model = args.get("model-id");
  int num_shard = static_cast<int>(args.num("num-shard", 0));
  if (args.has("sharded") && args.get("sharded") == "false") {
    if (num_shard > 1) {
      log_line("ERROR", "launcher", "`sharded` is false but `num_shard` > 1");
      return 2;
    }
    num_shard = 1;
  }
  if (num_shard <= 0) num_shard = std::max(1, count_gpus());
  if (args.has("sharded") && args.get("sharded") == "true" && num_shard < 2) {
    log_line("ERROR", "launcher", "`sharded` is true but only one GPU is visible");
    return 2;
  }
  const std::string quantize = args.get("quantize");
  const std::string uds = args.get("shard-uds-path", "/tmp/text-generation-server");
  const int grace = static_cast<int>(args.num("graceful-termination-timeout", 90));
  const std::string python = args.get("python", "python");
  if (args.has("env")) {
    if (system("nvidia-smi") != 0) log_line("WARNING", "launcher", "nvidia-smi is not available");
  }
  if (args.has("usage-stats") && args.get("usage-stats") != "off" && !args.has("usage-stats-endpoint") &&
      !args.has("usage-stats-file"))
    log_line("INFO", "launcher", "usage statistics have no sink: name one with --usage-stats-endpoint or --usage-stats-file");

  // environment shared by the weight download and the shards
  std::map<std::string, std::string> base_env;
  if (args.has("huggingface-hub-cache")) base_env["HUGGINGFACE_HUB_CACHE"] = args.get("huggingface-hub-cache");
  if (args.has("weights-cache-override")) base_env["WEIGHTS_CACHE_OVERRIDE"] = args.get("weights-cache-override");
  if (args.has("disable-custom-kernels")) base_env["DISABLE_CUSTOM_KERNELS"] = "True";

  // ---- weights: fetch (and convert) before any shard starts (launcher/src/main.rs:1434-1577) ----
  std::vector<std::thread> pumps;
  {
    std::vector<std::string> cmd = {python, "-m", "tgi_b200.server.cli", "download-weights", model, "--extension",
                                    ".safetensors", "--json-output"};
    if (args.has("revision")) { cmd.push_back("--revision"); cmd.push_back(args.get("revision")); }
    if (args.has("merge-lora")) cmd.push_back("--merge-lora");
    log_line("INFO", "launcher", "Starting check and download process for " + model);
    Spawned d = spawn(cmd, base_env, true);
    std::thread pump = log_pump("download", d.out_fd);
    int status = 0;
    while (true) {
      const pid_t w = waitpid(d.pid, &status, WNOHANG);
      if (w == d.pid) break;
      if (g_stop) {
        kill(d.pid, SIGTERM);
        waitpid(d.pid, &status, 0);
        pump.join();
        return 0;
      }
      usleep(100000);
    }
    pump.join();
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) {
      log_line("ERROR", "launcher", "Download encountered an error (status " + std::to_string(status) + ")");
      return 1;
    }
    log_line("INFO", "launcher", "Successfully downloaded weights for " + model);
  }

  // ---- automatic limits: prefill budget from FLOPs, token limits from the KV memory left ----
  const double bytes_per_param = (quantize == "fp8" || quantize == "eetq" || quantize == "bitsandbytes") ? 1.0
                                 : (quantize == "gptq" || quantize == "awq" || quantize.find("nf4") != std::string::npos) ? 0.5 : 2.0;
  const double kv_bytes = args.get("kv-cache-dtype").rfind("fp8", 0) == 0 ? 1.0 : 2.0;
  ModelFacts facts = read_model(model, bytes_per_param, kv_bytes);
  long max_prefill = args.num("max-batch-prefill-tokens", 0);
  if (max_prefill == 0) {
    max_prefill = 4096;
    if (facts.ok) {
      // tokens one forward can take in about a fifth of a second at the tensor rate of the node
      const double flops = peak_flops_per_gpu(args) * 0.6 * num_shard;
      long by_flops = static_cast<long>(flops * 0.2 / facts.flops_per_token);
      const double mem = gpu_memory_bytes() * num_shard;
      long by_mem = mem > facts.weight_bytes ? static_cast<long>((mem * 0.9 - facts.weight_bytes) / facts.kv_bytes_per_token) : 4096;
      long v = std::min({by_flops, by_mem > 0 ? by_mem : by_flops, facts.max_position_embeddings > 0 ? facts.max_position_embeddings * 8 : by_flops});
      v = std::max(256L, std::min(v, 65536L));
      max_prefill = v / 256 * 256;
    }
  }
  long max_input = args.num("max-input-tokens", args.num("max-input-length", 0)), max_total = args.num("max-total-tokens", 0);
  if (max_input && max_total && max_input >= max_total) {
    log_line("ERROR", "launcher", "`max_input_tokens` must be < `max_total_tokens`");
    return 2;
  }
  const std::string prefix_caching = resolve_prefix_caching(model, args);

  // ---- shards ----
  std::vector<Child> children;
  for (int r = 0; r < num_shard; ++r) unlink((uds + "-" + std::to_string(r)).c_str());
  for (int r = 0; r < num_shard; ++r) {
    std::vector<std::string> cmd = {python, "-m", "tgi_b200.server.cli", "serve", model, "--uds-path", uds, "--json-output"};
    if (num_shard > 1) cmd.push_back("--sharded");
    if (!quantize.empty()) { cmd.push_back("--quantize"); cmd.push_back(quantize); }
    for (const char* f : {"dtype", "kv-cache-dtype", "speculate", "revision"})
      if (args.has(f)) { cmd.push_back(std::string("--") + f); cmd.push_back(args.get(f)); }
    if (max_input) { cmd.push_back("--max-input-tokens"); cmd.push_back(std::to_string(max_input)); }
    if (args.has("trust-remote-code")) cmd.push_back("--trust-remote-code");
    if (args.has("otlp-endpoint")) {   // shards and router export to the same collector under their own service names
      cmd.push_back("--otlp-endpoint");
      cmd.push_back(args.get("otlp-endpoint"));
      cmd.push_back("--otlp-service-name");
      cmd.push_back(args.get("otlp-service-name", "text-generation-inference") + ".server");
    }
    std::map<std::string, std::string> env = base_env;
    env["RANK"] = std::to_string(r);
    env["LOCAL_RANK"] = std::to_string(r);
    env["WORLD_SIZE"] = std::to_string(num_shard);
    env["MASTER_ADDR"] = args.get("master-addr", "127.0.0.1");
    env["MASTER_PORT"] = args.get("master-port", "29500");
    env["TORCH_NCCL_AVOID_RECORD_STREAMS"] = "1";
    env["PREFIX_CACHING"] = prefix_caching;
    if (args.has("cuda-graphs")) env["CUDA_GRAPHS"] = args.get("cuda-graphs");
    if (args.has("cuda-memory-fraction")) env["CUDA_MEMORY_FRACTION"] = args.get("cuda-memory-fraction");
    if (args.has("lora-adapters")) env["LORA_ADAPTERS"] = args.get("lora-adapters");
    if (args.has("rope-scaling")) env["ROPE_SCALING"] = args.get("rope-scaling");
    if (args.has("rope-factor")) env["ROPE_FACTOR"] = args.get("rope-factor");
    if (args.has("watermark-gamma")) env["WATERMARK_GAMMA"] = args.get("watermark-gamma");
    if (args.has("watermark-delta")) env["WATERMARK_DELTA"] = args.get("watermark-delta");
    if (args.has("enable-prefill-logprobs")) env["REQUEST_LOGPROBS"] = "1";
    Child c;
    c.name = "shard-" + std::to_string(r);
    Spawned sp = spawn(cmd, env, true);
    c.pid = sp.pid;
    pumps.push_back(log_pump(c.name, sp.out_fd));
    log_line("INFO", "launcher", "Starting " + c.name + " (pid " + std::to_string(c.pid) + ")");
    children.push_back(c);
  }
  auto join_pumps = [&pumps] {
    for (auto& t : pumps)
      if (t.joinable()) t.join();
  };
  // a shard is ready when its socket exists
  for (int r = 0; r < num_shard && !g_stop; ++r) {
    const std::string sock = uds + "-" + std::to_string(r) + ".raw";
    struct stat st;
    while (!g_stop && stat(sock.c_str(), &st) != 0) {
      int status;
      for (auto& c : children)
        if (c.pid > 0 && waitpid(c.pid, &status, WNOHANG) == c.pid) {
          log_line("ERROR", "launcher", c.name + " failed to start (status " + std::to_string(status) + ")");
          c.pid = -1;
          terminate(children, grace);
          join_pumps();
          return 1;
        }
      usleep(100000);
    }
    if (!g_stop) log_line("INFO", "launcher", "Shard " + std::to_string(r) + " ready");
  }
  if (g_stop) {
    terminate(children, grace);
    join_pumps();
    return 0;
  }

  // ---- router ----
  std::string self = argv[0];
  size_t slash = self.rfind('/');
  const std::string dir = slash == std::string::npos ? "." : self.substr(0, slash);
  std::vector<std::string> rcmd = {dir + "/tgi-b200-router", "--master-shard-uds-path", uds, "--tokenizer-name",
                                   args.get("tokenizer-name", model), "--model-id", model,
                                   "--max-batch-prefill-tokens", std::to_string(max_prefill)};
  for (const char* f : {"port", "hostname", "max-concurrent-requests", "max-best-of", "max-stop-sequences",
                        "max-top-n-tokens", "max-total-tokens", "max-batch-total-tokens",
                        "waiting-served-ratio", "max-waiting-tokens", "max-batch-size", "max-client-batch-size",
                        "api-key", "payload-limit", "max-image-fetch-size", "repo-root", "prometheus-port", "cors-allow-origin",
                        "tokenizer-config-path", "validation-workers", "revision"})
    if (args.has(f)) { rcmd.push_back(std::string("--") + f); rcmd.push_back(args.get(f)); }
  if (max_input) { rcmd.push_back("--max-input-tokens"); rcmd.push_back(std::to_string(max_input)); }
  if (args.has("disable-grammar-support")) rcmd.push_back("--disable-grammar-support");
  if (prefix_caching == "0" || prefix_caching == "false") rcmd.push_back("--disable-prefix-caching");
  if (g_json_output) rcmd.push_back("--json-output");
  if (args.has("otlp-endpoint")) {
    rcmd.push_back("--otlp-endpoint");
    rcmd.push_back(args.get("otlp-endpoint"));
    rcmd.push_back("--otlp-service-name");
    rcmd.push_back(args.get("otlp-service-name", "text-generation-inference") + ".router");
  }
  for (const char* f : {"usage-stats", "usage-stats-endpoint", "usage-stats-file", "usage-stats-ping-seconds"})
    if (args.has(f)) { rcmd.push_back(std::string("--") + f); rcmd.push_back(args.get(f)); }
  Child router;
  router.name = "router";
  {
    Spawned sp = spawn(rcmd, {}, true);
    router.pid = sp.pid;
    pumps.push_back(log_pump(router.name, sp.out_fd));
  }
  log_line("INFO", "launcher", "Starting router (pid " + std::to_string(router.pid) + ")");
  children.push_back(router);

  // ---- supervise: any child exiting brings the deployment down ----
  int exit_code = 0;
  while (!g_stop) {
    int status;
    bool dead = false;
    for (auto& c : children) {
      if (c.pid > 0 && waitpid(c.pid, &status, WNOHANG) == c.pid) {
        log_line("ERROR", "launcher", c.name + " exited (status " + std::to_string(status) + "); shutting down");
        c.pid = -1;
        dead = true;
        exit_code = 1;
      }
    }
    if (dead) break;
    usleep(100000);
  }
  // router first so it stops accepting requests, then the shards
  std::vector<Child> r1 = {children.back()};
  children.pop_back();
  terminate(r1, grace);
  terminate(children, grace);
  join_pumps();
  return exit_code;
}
