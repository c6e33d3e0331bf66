#include "pb.hpp"

namespace pb {

namespace {
template <class F>
void parse(const std::string& s, F&& on_field) {
  Reader r(s);
  while (!r.done()) {
    uint32_t wt;
    uint32_t f = r.tag(wt);
    if (!on_field(f, wt, r)) r.skip(wt);
  }
}
std::vector<uint32_t> unpack_u32(Reader& r, uint32_t wt) {
  std::vector<uint32_t> v;
  if (wt == 2) {
    std::string b = r.bytes();
    Reader rr(b);
    while (!rr.done()) v.push_back(static_cast<uint32_t>(rr.varint()));
  } else {
    v.push_back(static_cast<uint32_t>(r.varint()));
  }
  return v;
}
}  // namespace

InfoResponse InfoResponse::decode(const std::string& s) {
  InfoResponse m;
  parse(s, [&](uint32_t f, uint32_t wt, Reader& r) {
    switch (f) {
      case 1: m.requires_padding = r.varint(); return true;
      case 2: m.dtype = r.bytes(); return true;
      case 3: m.device_type = r.bytes(); return true;
      case 4: m.window_size = static_cast<uint32_t>(r.varint()); return true;
      case 5: m.speculate = static_cast<uint32_t>(r.varint()); return true;
      case 6: m.support_chunking = r.varint(); return true;
      case 7: m.use_prefix_caching = r.varint(); return true;
      case 8: m.attention_impl = r.bytes(); return true;
      case 9: m.block_size = static_cast<uint32_t>(r.varint()); return true;
    }
    (void)wt;
    return false;
  });
  return m;
}

void NextTokenChooserParameters::encode(Writer& w) const {
  w.f32(1, temperature);
  w.u64(2, top_k);
  w.f32(3, top_p);
  w.f32(4, typical_p);
  w.boolean(5, do_sample);
  w.u64(6, seed);
  w.f32(7, repetition_penalty);
  w.boolean(8, watermark);
  w.f32(9, frequency_penalty);
  w.bytes(10, grammar);
  w.u64(11, grammar_type);
}

void StoppingCriteriaParameters::encode(Writer& w) const {
  w.u64(1, max_new_tokens);
  for (const auto& s : stop_sequences) w.bytes_always(2, s);
  w.boolean(3, ignore_eos_token);
}

void Request::encode(Writer& w) const {
  w.u64(1, id);
  w.bytes(2, inputs);
  w.u64(3, truncate);
  {
    Writer p;
    parameters.encode(p);
    w.bytes_always(4, p.out);
  }
  {
    Writer p;
    stopping_parameters.encode(p);
    w.bytes_always(5, p.out);
  }
  w.boolean(6, prefill_logprobs);
  w.u64(7, top_n_tokens);
  if (!input_chunks.empty()) {
    Writer in;
    for (const auto& c : input_chunks) {
      Writer ch;
      if (c.is_image) {
        Writer img;
        img.bytes(1, c.data);
        img.bytes(2, c.mimetype);
        ch.bytes_always(2, img.out);
      } else {
        ch.bytes_always(1, c.text);
      }
      in.bytes_always(1, ch.out);
    }
    w.bytes_always(8, in.out);
  }
  w.packed_u32(9, blocks);
  w.packed_u32(10, slots);
  if (adapter_id) w.bytes_always(11, *adapter_id);
  w.u64(12, cache_len);
  w.boolean(13, add_special_tokens);
  if (chunk_len) w.u64_always(14, *chunk_len);
}

void Batch::encode(Writer& w) const {
  w.u64(1, id);
  for (const auto& r : requests) {
    Writer p;
    r.encode(p);
    w.bytes_always(2, p.out);
  }
  w.u64(3, size);
  w.u64(4, max_tokens);
  w.u64(5, max_blocks);
}

void CachedBatch::encode(Writer& w) const {
  w.u64(1, id);
  w.packed_u64(2, request_ids);
  w.u64(3, size);
  w.u64(4, max_tokens);
  w.u64(5, current_tokens);
}

CachedBatch CachedBatch::decode(const std::string& s) {
  CachedBatch m;
  parse(s, [&](uint32_t f, uint32_t wt, Reader& r) {
    switch (f) {
      case 1: m.id = r.varint(); return true;
      case 2:
        if (wt == 2) {
          std::string b = r.bytes();
          Reader rr(b);
          while (!rr.done()) m.request_ids.push_back(rr.varint());
        } else {
          m.request_ids.push_back(r.varint());
        }
        return true;
      case 3: m.size = static_cast<uint32_t>(r.varint()); return true;
      case 4: m.max_tokens = static_cast<uint32_t>(r.varint()); return true;
      case 5: m.current_tokens = static_cast<uint32_t>(r.varint()); return true;
    }
    return false;
  });
  return m;
}

Tokens Tokens::decode(const std::string& s) {
  Tokens m;
  parse(s, [&](uint32_t f, uint32_t wt, Reader& r) {
    switch (f) {
      case 1: {
        auto v = unpack_u32(r, wt);
        m.ids.insert(m.ids.end(), v.begin(), v.end());
        return true;
      }
      case 2:
        if (wt == 2) {
          std::string b = r.bytes();
          for (size_t i = 0; i + 4 <= b.size(); i += 4) {
            float v;
            std::memcpy(&v, b.data() + i, 4);
            m.logprobs.push_back(v);
          }
        } else {
          m.logprobs.push_back(r.f32());
        }
        return true;
      case 3: m.texts.push_back(r.bytes()); return true;
      case 4: {
        auto v = unpack_u32(r, wt);
        for (uint32_t x : v) m.is_special.push_back(x != 0);
        return true;
      }
    }
    return false;
  });
  return m;
}

GeneratedText GeneratedText::decode(const std::string& s) {
  GeneratedText m;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    switch (f) {
      case 1: m.text = r.bytes(); return true;
      case 2: m.generated_tokens = static_cast<uint32_t>(r.varint()); return true;
      case 3: m.finish_reason = static_cast<uint32_t>(r.varint()); return true;
      case 4: m.seed = r.varint(); return true;
    }
    return false;
  });
  return m;
}

Generation Generation::decode(const std::string& s) {
  Generation m;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    switch (f) {
      case 1: m.request_id = r.varint(); return true;
      case 2: m.prefill_tokens = Tokens::decode(r.bytes()); return true;
      case 3: m.tokens = Tokens::decode(r.bytes()); return true;
      case 4: m.generated_text = GeneratedText::decode(r.bytes()); return true;
      case 5: m.top_tokens.push_back(Tokens::decode(r.bytes())); return true;
    }
    return false;
  });
  return m;
}

StepResponse StepResponse::decode(const std::string& s) {
  StepResponse m;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    switch (f) {
      case 1: m.generations.push_back(Generation::decode(r.bytes())); return true;
      case 2: m.batch = CachedBatch::decode(r.bytes()); return true;
      case 3: m.forward_ns = r.varint(); return true;
      case 4: m.decode_ns = r.varint(); return true;
      case 5: m.total_ns = r.varint(); return true;
      case 6: m.concat_ns = r.varint(); return true;
    }
    return false;
  });
  return m;
}

WarmupResponse WarmupResponse::decode(const std::string& s) {
  WarmupResponse m;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    switch (f) {
      case 1: m.max_supported_total_tokens = static_cast<uint32_t>(r.varint()); return true;
      case 2: m.max_input_tokens = static_cast<uint32_t>(r.varint()); return true;
      case 3: m.max_total_tokens = static_cast<uint32_t>(r.varint()); return true;
    }
    return false;
  });
  return m;
}

std::string encode_prefill_request(const Batch& batch, const CachedBatch* cached) {
  Writer w, b;
  batch.encode(b);
  w.bytes_always(1, b.out);
  if (cached) {
    Writer c;
    cached->encode(c);
    w.bytes_always(2, c.out);
  }
  return w.out;
}

std::string encode_decode_request(const std::vector<CachedBatch>& batches) {
  Writer w;
  for (const auto& cb : batches) {
    Writer c;
    cb.encode(c);
    w.bytes_always(1, c.out);
  }
  return w.out;
}

std::string encode_filter_request(uint64_t batch_id, const std::vector<uint64_t>& request_ids) {
  Writer w;
  w.u64(1, batch_id);
  w.packed_u64(2, request_ids);
  return w.out;
}

std::string encode_clear_cache_request(const std::optional<uint64_t>& id) {
  Writer w;
  if (id) w.u64_always(1, *id);
  return w.out;
}

std::string encode_warmup_request(const Batch& batch, std::optional<uint32_t> max_input_tokens,
                                  uint32_t max_prefill_tokens, std::optional<uint32_t> max_total_tokens) {
  Writer w, b;
  batch.encode(b);
  w.bytes_always(1, b.out);
  if (max_input_tokens) w.u64_always(2, *max_input_tokens);
  w.u64(3, max_prefill_tokens);
  if (max_total_tokens) w.u64_always(4, *max_total_tokens);
  return w.out;
}

CachedBatch decode_filter_response(const std::string& s) {
  CachedBatch out;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    if (f == 1) {
      out = CachedBatch::decode(r.bytes());
      return true;
    }
    return false;
  });
  return out;
}

std::vector<std::string> decode_service_discovery(const std::string& s) {
  std::vector<std::string> urls;
  parse(s, [&](uint32_t f, uint32_t, Reader& r) {
    if (f == 1) {
      urls.push_back(r.bytes());
      return true;
    }
    return false;
  });
  return urls;
}

}  // namespace pb
