// tgi-b200-launcher: reads the model config, decides the serving limits, starts one shard process
// per GPU and the router, forwards their logs and supervises them.
//
// Reference: launcher/src/main.rs — flags (:582-914), `find_num_shards` (:1374-1413), FLOP/VRAM based
// default for max_batch_prefill_tokens (:28-89, 261-352, 2114-2154), `shard_manager` (:923-1249),
// `spawn_webserver` (:1831-2013), `terminate` (:2015-2036), supervision loop (:2333-2361).
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

pid_t spawn(const std::vector<std::string>& argv, const std::map<std::string, std::string>& env) {
  pid_t pid = fork();
  if (pid != 0) return pid;
  setpgid(0, 0);
  for (auto& kv : env) setenv(kv.first.c_str(), kv.second.c_str(), 1);
  std::vector<char*> a;
  for (auto& s : argv) a.push_back(const_cast<char*>(s.c_str()));
  a.push_back(nullptr);
  execvp(a[0], a.data());
  std::perror("exec");
  _exit(127);
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

}  // namespace

int main(int argc, char** argv) {
  Args args(argc, argv);
  if (args.has("help") || !args.has("model-id")) {
    std::cout << "tgi-b200-launcher --model-id DIR [--num-shard N] [--quantize fp8|gptq|awq|eetq|bitsandbytes...]\n"
                 "  [--dtype bfloat16|float16] [--kv-cache-dtype fp8_e4m3fn] [--speculate N] [--port 3000] [--hostname 0.0.0.0]\n"
                 "  [--max-input-tokens N] [--max-total-tokens N] [--max-batch-prefill-tokens N] [--max-batch-total-tokens N]\n"
                 "  [--max-concurrent-requests 128] [--max-batch-size N] [--cuda-graphs 1,2,4,...] [--cuda-memory-fraction 1.0]\n"
                 "  [--shard-uds-path /tmp/text-generation-server] [--master-addr 127.0.0.1] [--master-port 29500]\n"
                 "  [--lora-adapters a,b] [--api-key KEY] [--graceful-termination-timeout 90] [--env]\n";
    return args.has("help") ? 0 : 2;
  }
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  const std::string model = args.get("model-id");
  int num_shard = static_cast<int>(args.num("num-shard", 0));
  if (num_shard <= 0) num_shard = std::max(1, count_gpus());
  const std::string quantize = args.get("quantize");
  const std::string uds = args.get("shard-uds-path", "/tmp/text-generation-server");
  const int grace = static_cast<int>(args.num("graceful-termination-timeout", 90));
  if (args.has("env")) {
    if (system("nvidia-smi") != 0) std::cerr << "nvidia-smi is not available" << std::endl;
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
      // tokens one forward can take in ~ a fifth of a second at the bf16 tensor rate of the node
      const double flops = 1.4e15 * num_shard;
      long by_flops = static_cast<long>(flops * 0.2 / facts.flops_per_token);
      const double mem = gpu_memory_bytes() * num_shard;
      long by_mem = mem > facts.weight_bytes ? static_cast<long>((mem * 0.9 - facts.weight_bytes) / facts.kv_bytes_per_token) : 4096;
      long v = std::min({by_flops, by_mem > 0 ? by_mem : by_flops, facts.max_position_embeddings > 0 ? facts.max_position_embeddings * 8 : by_flops});
      v = std::max(256L, std::min(v, 65536L));
      max_prefill = v / 256 * 256;
    }
  }
  long max_input = args.num("max-input-tokens", 0), max_total = args.num("max-total-tokens", 0);
  if (max_input && max_total && max_input >= max_total) {
    std::cerr << "`max_input_tokens` must be < `max_total_tokens`" << std::endl;
    return 2;
  }

  // ---- shards ----
  std::vector<Child> children;
  const std::string python = args.get("python", "python");
  for (int r = 0; r < num_shard; ++r) unlink((uds + "-" + std::to_string(r)).c_str());
  for (int r = 0; r < num_shard; ++r) {
    std::vector<std::string> cmd = {python, "-m", "tgi_b200.server.cli", "serve", model, "--uds-path", uds};
    if (num_shard > 1) cmd.push_back("--sharded");
    if (!quantize.empty()) { cmd.push_back("--quantize"); cmd.push_back(quantize); }
    for (const char* f : {"dtype", "kv-cache-dtype", "speculate", "revision", "max-input-tokens"})
      if (args.has(f)) { cmd.push_back(std::string("--") + f); cmd.push_back(args.get(f)); }
    if (args.has("trust-remote-code")) cmd.push_back("--trust-remote-code");
    if (args.has("otlp-endpoint")) {   // shards and router export to the same collector under their own service names
      cmd.push_back("--otlp-endpoint");
      cmd.push_back(args.get("otlp-endpoint"));
      cmd.push_back("--otlp-service-name");
      cmd.push_back(args.get("otlp-service-name", "text-generation-inference") + ".server");
    }
    std::map<std::string, std::string> env = {
        {"RANK", std::to_string(r)}, {"LOCAL_RANK", std::to_string(r)}, {"WORLD_SIZE", std::to_string(num_shard)},
        {"MASTER_ADDR", args.get("master-addr", "127.0.0.1")}, {"MASTER_PORT", args.get("master-port", "29500")},
        {"TORCH_NCCL_AVOID_RECORD_STREAMS", "1"}};
    if (args.has("cuda-graphs")) env["CUDA_GRAPHS"] = args.get("cuda-graphs");
    if (args.has("cuda-memory-fraction")) env["CUDA_MEMORY_FRACTION"] = args.get("cuda-memory-fraction");
    if (args.has("lora-adapters")) env["LORA_ADAPTERS"] = args.get("lora-adapters");
    if (args.has("rope-scaling")) env["ROPE_SCALING"] = args.get("rope-scaling");
    if (args.has("rope-factor")) env["ROPE_FACTOR"] = args.get("rope-factor");
    Child c;
    c.name = "shard-" + std::to_string(r);
    c.pid = spawn(cmd, env);
    std::cerr << "[launcher] started " << c.name << " (pid " << c.pid << ")" << std::endl;
    children.push_back(c);
  }
  // a shard is ready when its socket exists
  for (int r = 0; r < num_shard && !g_stop; ++r) {
    const std::string sock = uds + "-" + std::to_string(r) + ".raw";
    struct stat st;
    while (!g_stop && stat(sock.c_str(), &st) != 0) {
      int status;
      for (auto& c : children)
        if (c.pid > 0 && waitpid(c.pid, &status, WNOHANG) == c.pid) {
          std::cerr << "[launcher] " << c.name << " failed to start (status " << status << ")" << std::endl;
          c.pid = -1;
          terminate(children, grace);
          return 1;
        }
      usleep(100000);
    }
    if (!g_stop) std::cerr << "[launcher] shard " << r << " ready" << std::endl;
  }
  if (g_stop) {
    terminate(children, grace);
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
                        "max-top-n-tokens", "max-input-tokens", "max-total-tokens", "max-batch-total-tokens",
                        "waiting-served-ratio", "max-waiting-tokens", "max-batch-size", "max-client-batch-size",
                        "api-key", "payload-limit", "disable-grammar-support", "repo-root"})
    if (args.has(f)) { rcmd.push_back(std::string("--") + f); rcmd.push_back(args.get(f)); }
  if (args.has("otlp-endpoint")) {
    rcmd.push_back("--otlp-endpoint");
    rcmd.push_back(args.get("otlp-endpoint"));
    rcmd.push_back("--otlp-service-name");
    rcmd.push_back(args.get("otlp-service-name", "text-generation-inference") + ".router");
  }
  Child router;
  router.name = "router";
  router.pid = spawn(rcmd, {});
  std::cerr << "[launcher] started router (pid " << router.pid << ")" << std::endl;
  children.push_back(router);

  // ---- supervise: any child exiting brings the deployment down ----
  int exit_code = 0;
  while (!g_stop) {
    int status;
    bool dead = false;
    for (auto& c : children) {
      if (c.pid > 0 && waitpid(c.pid, &status, WNOHANG) == c.pid) {
        std::cerr << "[launcher] " << c.name << " exited (status " << status << "); shutting down" << std::endl;
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
  return exit_code;
}
