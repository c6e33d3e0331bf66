// proto3 wire codec for the `generate.v3` router<->shard contract, written by hand
// (no protoc in the build environment).  Field numbers follow proto/v3/generate.proto of the
// reference (messages at lines 25-289).  Only what the router sends or receives is modelled.
#pragma once
#include <cstdint>
#include <cstring>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace pb {

// ---- wire primitives ----------------------------------------------------------------------
class Writer {
 public:
  std::string out;
  void varint(uint64_t v) {
    while (v >= 0x80) {
      out.push_back(static_cast<char>(v | 0x80));
      v >>= 7;
    }
    out.push_back(static_cast<char>(v));
  }
  void tag(uint32_t field, uint32_t wt) { varint((static_cast<uint64_t>(field) << 3) | wt); }
  void u64(uint32_t f, uint64_t v) { if (v) { tag(f, 0); varint(v); } }
  void u64_always(uint32_t f, uint64_t v) { tag(f, 0); varint(v); }
  void boolean(uint32_t f, bool v) { if (v) { tag(f, 0); varint(1); } }
  void f32(uint32_t f, float v) {
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    if (bits) { tag(f, 5); out.append(reinterpret_cast<const char*>(&bits), 4); }
  }
  void bytes(uint32_t f, const std::string& s) { if (!s.empty()) { tag(f, 2); varint(s.size()); out += s; } }
  void bytes_always(uint32_t f, const std::string& s) { tag(f, 2); varint(s.size()); out += s; }
  void packed_u32(uint32_t f, const std::vector<uint32_t>& v) {
    if (v.empty()) return;
    Writer w;
    for (uint32_t x : v) w.varint(x);
    bytes_always(f, w.out);
  }
  void packed_u64(uint32_t f, const std::vector<uint64_t>& v) {
    if (v.empty()) return;
    Writer w;
    for (uint64_t x : v) w.varint(x);
    bytes_always(f, w.out);
  }
};

class Reader {
 public:
  Reader(const char* p, size_t n) : p_(p), end_(p + n) {}
  explicit Reader(const std::string& s) : Reader(s.data(), s.size()) {}
  bool done() const { return p_ >= end_; }
  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (true) {
      if (p_ >= end_ || shift > 63) throw std::runtime_error("pb: truncated varint");
      uint8_t b = static_cast<uint8_t>(*p_++);
      v |= static_cast<uint64_t>(b & 0x7F) << shift;
      if (!(b & 0x80)) return v;
      shift += 7;
    }
  }
  // returns field number, sets wire type
  uint32_t tag(uint32_t& wt) {
    uint64_t t = varint();
    wt = static_cast<uint32_t>(t & 7);
    return static_cast<uint32_t>(t >> 3);
  }
  std::string bytes() {
    uint64_t n = varint();
    if (static_cast<uint64_t>(end_ - p_) < n) throw std::runtime_error("pb: truncated bytes");
    std::string s(p_, n);
    p_ += n;
    return s;
  }
  float f32() {
    if (end_ - p_ < 4) throw std::runtime_error("pb: truncated fixed32");
    float v;
    std::memcpy(&v, p_, 4);
    p_ += 4;
    return v;
  }
  void skip(uint32_t wt) {
    switch (wt) {
      case 0: varint(); break;
      case 1: if (end_ - p_ < 8) throw std::runtime_error("pb: truncated"); p_ += 8; break;
      case 2: bytes(); break;
      case 5: if (end_ - p_ < 4) throw std::runtime_error("pb: truncated"); p_ += 4; break;
      default: throw std::runtime_error("pb: unsupported wire type");
    }
  }
 private:
  const char* p_;
  const char* end_;
};

// ---- messages -----------------------------------------------------------------------------
struct InfoResponse {
  bool requires_padding = false;
  std::string dtype, device_type, attention_impl;
  std::optional<uint32_t> window_size;
  uint32_t speculate = 0, block_size = 0;
  bool support_chunking = false, use_prefix_caching = false;
  static InfoResponse decode(const std::string& s);
};

struct NextTokenChooserParameters {
  float temperature = 1.f;
  uint32_t top_k = 0;
  float top_p = 1.f, typical_p = 1.f;
  bool do_sample = false;
  uint64_t seed = 0;
  float repetition_penalty = 1.f, frequency_penalty = 0.f;
  bool watermark = false;
  std::string grammar;
  uint32_t grammar_type = 0;  // 0 none, 1 json, 2 regex
  void encode(Writer& w) const;
};

struct StoppingCriteriaParameters {
  uint32_t max_new_tokens = 0;
  std::vector<std::string> stop_sequences;
  bool ignore_eos_token = false;
  void encode(Writer& w) const;
};

struct InputChunk {
  bool is_image = false;
  std::string text;       // text chunk
  std::string data;       // image bytes
  std::string mimetype;
};

struct Request {
  uint64_t id = 0;
  std::vector<InputChunk> input_chunks;
  std::string inputs;
  uint32_t truncate = 0;
  NextTokenChooserParameters parameters;
  StoppingCriteriaParameters stopping_parameters;
  bool prefill_logprobs = false;
  uint32_t top_n_tokens = 0;
  std::vector<uint32_t> blocks, slots;
  std::optional<std::string> adapter_id;
  uint32_t cache_len = 0;
  bool add_special_tokens = true;
  std::optional<uint32_t> chunk_len;
  void encode(Writer& w) const;
};

struct Batch {
  uint64_t id = 0;
  std::vector<Request> requests;
  uint32_t size = 0, max_tokens = 0, max_blocks = 0;
  void encode(Writer& w) const;
};

struct CachedBatch {
  uint64_t id = 0;
  std::vector<uint64_t> request_ids;
  uint32_t size = 0, max_tokens = 0, current_tokens = 0;
  void encode(Writer& w) const;
  static CachedBatch decode(const std::string& s);
};

struct Tokens {
  std::vector<uint32_t> ids;
  std::vector<float> logprobs;
  std::vector<std::string> texts;
  std::vector<bool> is_special;
  static Tokens decode(const std::string& s);
};

struct GeneratedText {
  std::string text;
  uint32_t generated_tokens = 0;
  uint32_t finish_reason = 0;  // 0 length, 1 eos, 2 stop sequence
  std::optional<uint64_t> seed;
  static GeneratedText decode(const std::string& s);
};

struct Generation {
  uint64_t request_id = 0;
  std::optional<Tokens> prefill_tokens;
  Tokens tokens;
  std::optional<GeneratedText> generated_text;
  std::vector<Tokens> top_tokens;
  static Generation decode(const std::string& s);
};

struct StepResponse {  // PrefillResponse and DecodeResponse share their layout
  std::vector<Generation> generations;
  std::optional<CachedBatch> batch;
  uint64_t forward_ns = 0, decode_ns = 0, total_ns = 0;
  std::optional<uint64_t> concat_ns;
  static StepResponse decode(const std::string& s);
};

struct WarmupResponse {
  std::optional<uint32_t> max_supported_total_tokens;
  uint32_t max_input_tokens = 0, max_total_tokens = 0;
  static WarmupResponse decode(const std::string& s);
};

std::string encode_prefill_request(const Batch& batch, const CachedBatch* cached);
std::string encode_decode_request(const std::vector<CachedBatch>& batches);
std::string encode_filter_request(uint64_t batch_id, const std::vector<uint64_t>& request_ids);
std::string encode_clear_cache_request(const std::optional<uint64_t>& id);
std::string encode_warmup_request(const Batch& batch, std::optional<uint32_t> max_input_tokens,
                                  uint32_t max_prefill_tokens, std::optional<uint32_t> max_total_tokens);
CachedBatch decode_filter_response(const std::string& s);
std::vector<std::string> decode_service_discovery(const std::string& s);

}  // namespace pb
