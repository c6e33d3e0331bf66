// tgi-b200-benchmark: shard-level prefill / decode microbenchmark.
//
// Talks to the shard processes directly (no router, no HTTP), like the reference's
// `text-generation-benchmark` (benchmark/src/generation.rs:64-238, lib.rs:19-160, table.rs): for every
// batch size it runs warm-up rounds and then `--runs` timed rounds of one prefill of
// `--sequence-length` tokens per request followed by `--decode-length` decode steps with
// `ignore_eos_token`, and reports latency and throughput of both phases as avg / min / max /
// p50 / p90 / p99.  Output is a plain-text table per phase (or `--json` for one JSON document);
// the reference's terminal UI is not reproduced.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <map>
#include <numeric>
#include <sstream>
#include <string>
#include <vector>

#include "json.hpp"
#include "shard_client.hpp"

namespace {

using Clock = std::chrono::steady_clock;

struct Options {
  std::string uds = "/tmp/text-generation-server";
  std::vector<uint32_t> batch_sizes = {1, 2, 4, 8, 16, 32};
  uint32_t sequence_length = 10, decode_length = 8, runs = 10, warmups = 1;
  uint32_t top_n_tokens = 0, block_size = 16;
  float temperature = 1.f, top_p = 1.f, typical_p = 1.f, repetition_penalty = 1.f, frequency_penalty = 0.f;
  uint32_t top_k = 0;
  bool do_sample = false, watermark = false, json = false;
};

struct Series {
  std::vector<double> latency_ms, throughput;
};

struct Summary {
  double avg = 0, lo = 0, hi = 0, p50 = 0, p90 = 0, p99 = 0;
};

Summary summarize(std::vector<double> v) {
  Summary s;
  if (v.empty()) return s;
  std::sort(v.begin(), v.end());
  auto pct = [&](double p) {
    const double pos = p * (v.size() - 1);
    const size_t i = static_cast<size_t>(pos);
    const double frac = pos - i;
    return i + 1 < v.size() ? v[i] * (1 - frac) + v[i + 1] * frac : v[i];
  };
  s.avg = std::accumulate(v.begin(), v.end(), 0.0) / v.size();
  s.lo = v.front();
  s.hi = v.back();
  s.p50 = pct(0.5);
  s.p90 = pct(0.9);
  s.p99 = pct(0.99);
  return s;
}

std::vector<uint32_t> parse_list(const std::string& s) {
  std::vector<uint32_t> out;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, ',')) {
    if (!item.empty()) out.push_back(static_cast<uint32_t>(std::stoul(item)));
  }
  return out;
}

void usage() {
  std::cerr << "tgi-b200-benchmark [--master-shard-uds-path PATH] [--batch-size 1,2,4] [--sequence-length 10]\n"
               "  [--decode-length 8] [--runs 10] [--warmups 1] [--temperature T] [--top-k K] [--top-p P]\n"
               "  [--typical-p P] [--repetition-penalty R] [--frequency-penalty F] [--watermark] [--do-sample]\n"
               "  [--top-n-tokens N] [--json]\n";
}

bool parse(int argc, char** argv, Options& o) {
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> std::string {
      if (i + 1 >= argc) throw std::runtime_error("missing value for " + a);
      return argv[++i];
    };
    if (a == "--master-shard-uds-path" || a == "-m") o.uds = next();
    else if (a == "--batch-size" || a == "-b") o.batch_sizes = parse_list(next());
    else if (a == "--sequence-length" || a == "-s") o.sequence_length = std::stoul(next());
    else if (a == "--decode-length" || a == "-d") o.decode_length = std::stoul(next());
    else if (a == "--runs" || a == "-r") o.runs = std::stoul(next());
    else if (a == "--warmups" || a == "-w") o.warmups = std::stoul(next());
    else if (a == "--temperature") o.temperature = std::stof(next());
    else if (a == "--top-k") o.top_k = std::stoul(next());
    else if (a == "--top-p") o.top_p = std::stof(next());
    else if (a == "--typical-p") o.typical_p = std::stof(next());
    else if (a == "--repetition-penalty") o.repetition_penalty = std::stof(next());
    else if (a == "--frequency-penalty") o.frequency_penalty = std::stof(next());
    else if (a == "--top-n-tokens") o.top_n_tokens = std::stoul(next());
    else if (a == "--watermark") o.watermark = true;
    else if (a == "--do-sample") o.do_sample = true;
    else if (a == "--json") o.json = true;
    else if (a == "--help" || a == "-h") { usage(); return false; }
    else throw std::runtime_error("unknown argument " + a);
  }
  return true;
}

// A batch of `n` identical requests whose input text tokenises to about `sequence_length` tokens;
// `truncate` pins the exact length (the shard keeps the last `truncate` tokens).
pb::Batch make_batch(uint64_t id, uint32_t n, const Options& o) {
  pb::Batch b;
  b.id = id;
  b.size = n;
  std::string text;
  for (uint32_t i = 0; i < o.sequence_length; ++i) text += "_test ";
  const uint32_t total = o.sequence_length + o.decode_length;
  const uint32_t blocks_per = (total + o.block_size - 1) / o.block_size + 1;
  uint32_t cursor = 1;   // block 0 belongs to the health probe
  for (uint32_t r = 0; r < n; ++r) {
    pb::Request q;
    q.id = r;
    q.inputs = text;
    pb::InputChunk c;
    c.text = text;
    q.input_chunks.push_back(c);
    q.truncate = o.sequence_length;
    q.add_special_tokens = true;
    q.parameters.temperature = o.temperature;
    q.parameters.top_k = o.top_k;
    q.parameters.top_p = o.top_p;
    q.parameters.typical_p = o.typical_p;
    q.parameters.do_sample = o.do_sample;
    q.parameters.repetition_penalty = o.repetition_penalty;
    q.parameters.frequency_penalty = o.frequency_penalty;
    q.parameters.watermark = o.watermark;
    q.stopping_parameters.max_new_tokens = o.decode_length;
    q.stopping_parameters.ignore_eos_token = true;
    q.top_n_tokens = o.top_n_tokens;
    for (uint32_t k = 0; k < blocks_per; ++k) {
      q.blocks.push_back(cursor + k);
      for (uint32_t s = 0; s < o.block_size; ++s) q.slots.push_back((cursor + k) * o.block_size + s);
    }
    cursor += blocks_per;
    b.requests.push_back(std::move(q));
  }
  b.max_tokens = n * total;
  b.max_blocks = cursor;
  return b;
}

struct RunResult {
  double prefill_ms = 0, decode_ms = 0;
  uint32_t decode_steps = 0;
};

RunResult one_run(sched::ShardedClient& client, uint64_t id, uint32_t n, const Options& o) {
  RunResult r;
  pb::Batch batch = make_batch(id, n, o);
  auto t0 = Clock::now();
  pb::StepResponse resp = client.prefill(batch, nullptr);
  r.prefill_ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
  auto t1 = Clock::now();
  while (resp.batch.has_value()) {
    std::vector<pb::CachedBatch> cached{*resp.batch};
    resp = client.decode(cached);
    ++r.decode_steps;
    if (r.decode_steps > o.decode_length + 4) break;   // a shard that ignores max_new_tokens must not loop forever
  }
  r.decode_ms = std::chrono::duration<double, std::milli>(Clock::now() - t1).count();
  client.clear_cache(std::nullopt);
  return r;
}

void print_table(const std::string& title, const std::vector<uint32_t>& sizes, const std::map<uint32_t, Series>& data,
                 bool latency) {
  std::printf("\n%s\n", title.c_str());
  std::printf("| %-6s | %-10s | %-10s | %-10s | %-10s | %-10s | %-10s |\n", "batch", "avg", "min", "max", "p50", "p90", "p99");
  std::printf("|--------|------------|------------|------------|------------|------------|------------|\n");
  for (uint32_t n : sizes) {
    auto it = data.find(n);
    if (it == data.end()) continue;
    const Summary s = summarize(latency ? it->second.latency_ms : it->second.throughput);
    std::printf("| %-6u | %10.2f | %10.2f | %10.2f | %10.2f | %10.2f | %10.2f |\n", n, s.avg, s.lo, s.hi, s.p50, s.p90, s.p99);
  }
}

json::Value series_json(const Series& s) {
  auto one = [](const std::vector<double>& v) {
    const Summary m = summarize(v);
    json::Value o = json::Value::object();
    o.set("avg", m.avg);
    o.set("min", m.lo);
    o.set("max", m.hi);
    o.set("p50", m.p50);
    o.set("p90", m.p90);
    o.set("p99", m.p99);
    return o;
  };
  json::Value o = json::Value::object();
  o.set("latency_ms", one(s.latency_ms));
  o.set("throughput_tokens_per_s", one(s.throughput));
  return o;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  try {
    if (!parse(argc, argv, o)) return 0;
    auto client = sched::ShardedClient::connect(o.uds, 60);
    const pb::InfoResponse info = client->info();
    if (info.block_size) o.block_size = info.block_size;
    std::map<uint32_t, Series> prefill, decode;
    uint64_t id = 0;
    for (uint32_t n : o.batch_sizes) {
      for (uint32_t w = 0; w < o.warmups; ++w) one_run(*client, id++, n, o);
      for (uint32_t r = 0; r < o.runs; ++r) {
        const RunResult res = one_run(*client, id++, n, o);
        prefill[n].latency_ms.push_back(res.prefill_ms);
        prefill[n].throughput.push_back(n * o.sequence_length / (res.prefill_ms / 1e3));
        if (res.decode_steps > 0) {
          // latency of one decode step (inter-token latency); throughput in generated tokens per second
          decode[n].latency_ms.push_back(res.decode_ms / res.decode_steps);
          decode[n].throughput.push_back(n * res.decode_steps / (res.decode_ms / 1e3));
        }
      }
      if (!o.json) std::fprintf(stderr, "batch size %u done\n", n);
    }
    if (o.json) {
      json::Value root = json::Value::object();
      json::Value cfg = json::Value::object();
      cfg.set("sequence_length", static_cast<double>(o.sequence_length));
      cfg.set("decode_length", static_cast<double>(o.decode_length));
      cfg.set("runs", static_cast<double>(o.runs));
      cfg.set("shards", static_cast<double>(client->num_shards()));
      cfg.set("dtype", info.dtype);
      cfg.set("attention_impl", info.attention_impl);
      root.set("config", cfg);
      json::Value res = json::Value::array();
      for (uint32_t n : o.batch_sizes) {
        json::Value e = json::Value::object();
        e.set("batch_size", static_cast<double>(n));
        e.set("prefill", series_json(prefill[n]));
        e.set("decode", series_json(decode[n]));
        res.push(e);
      }
      root.set("results", res);
      std::cout << root.dump() << std::endl;
    } else {
      std::printf("shards=%zu dtype=%s attention=%s sequence_length=%u decode_length=%u runs=%u\n", client->num_shards(),
                  info.dtype.c_str(), info.attention_impl.c_str(), o.sequence_length, o.decode_length, o.runs);
      print_table("Prefill latency (ms)", o.batch_sizes, prefill, true);
      print_table("Prefill throughput (tokens/s)", o.batch_sizes, prefill, false);
      print_table("Decode latency per token (ms)", o.batch_sizes, decode, true);
      print_table("Decode throughput (tokens/s)", o.batch_sizes, decode, false);
    }
  } catch (const std::exception& e) {
    std::cerr << "benchmark failed: " << e.what() << std::endl;
    usage();
    return 1;
  }
  return 0;
}
