// pybind11 bindings of the router core, used only by the unit tests (tests/test_router_*.py):
// block allocator / radix trie, batch builder, the batching loop against a scripted fake shard,
// request validation, tool grammar and the protobuf codec.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "api.hpp"
#include "images.hpp"
#include "trace.hpp"
#include "json.hpp"
#include "pb.hpp"
#include "radix.hpp"
#include "scheduler.hpp"

namespace py = pybind11;

namespace {

// A shard that answers from Python callbacks: prefill(batch_bytes, cached_bytes|None) -> bytes etc.
class PyShard : public sched::ShardClient {
 public:
  py::object obj;
  explicit PyShard(py::object o) : obj(std::move(o)) {}
  pb::InfoResponse info() override { return pb::InfoResponse(); }
  void health() override {
    py::gil_scoped_acquire g;
    obj.attr("health")();
  }
  void clear_cache(std::optional<uint64_t> id) override {
    py::gil_scoped_acquire g;
    obj.attr("clear_cache")(id);
  }
  pb::CachedBatch filter_batch(uint64_t id, const std::vector<uint64_t>& keep) override {
    py::gil_scoped_acquire g;
    std::string raw = obj.attr("filter_batch")(py::bytes(pb::encode_filter_request(id, keep))).cast<std::string>();
    return pb::decode_filter_response(raw);
  }
  pb::WarmupResponse warmup(const pb::Batch&, std::optional<uint32_t>, uint32_t, std::optional<uint32_t>) override {
    return pb::WarmupResponse();
  }
  pb::StepResponse prefill(const pb::Batch& b, const pb::CachedBatch* c) override {
    py::gil_scoped_acquire g;
    std::string raw = obj.attr("prefill")(py::bytes(pb::encode_prefill_request(b, c))).cast<std::string>();
    return pb::StepResponse::decode(raw);
  }
  pb::StepResponse decode(const std::vector<pb::CachedBatch>& bs) override {
    py::gil_scoped_acquire g;
    std::string raw = obj.attr("decode")(py::bytes(pb::encode_decode_request(bs))).cast<std::string>();
    return pb::StepResponse::decode(raw);
  }
};

sched::ValidRequest make_request(uint32_t input_length, uint32_t max_new_tokens, std::vector<uint32_t> ids,
                                 bool decoder_input_details) {
  sched::ValidRequest r;
  r.inputs = "x";
  r.input_length = input_length;
  r.input_ids = std::move(ids);
  r.stopping.max_new_tokens = max_new_tokens;
  r.decoder_input_details = decoder_input_details;
  return r;
}

py::dict event_to_dict(const sched::StreamEvent& ev) {
  py::dict d;
  const char* kinds[] = {"prefill", "token", "end", "error"};
  d["kind"] = kinds[ev.kind];
  d["token_id"] = ev.token.id;
  d["text"] = ev.token.text;
  d["error"] = ev.error;
  if (ev.generated_text) {
    d["generated_text"] = ev.generated_text->text;
    d["finish_reason"] = ev.generated_text->finish_reason;
    d["generated_tokens"] = ev.generated_text->generated_tokens;
  }
  return d;
}

}  // namespace

PYBIND11_MODULE(_router_test, m) {
  m.def("tokens_per_image", [](const std::string& config_json, uint32_t width, uint32_t height) {
    return images::tokens_per_image(json::Value::parse(config_json), width, height);
  });
  m.def("parse_traceparent", [](const std::string& h) {
    const trace::Context c = trace::parse_traceparent(h);
    return py::make_tuple(c.valid(), c.trace_id, c.span_id, c.sampled);
  });
  py::class_<sched::BlockAllocation>(m, "BlockAllocation")
      .def_readonly("allocation_id", &sched::BlockAllocation::allocation_id)
      .def_readonly("blocks", &sched::BlockAllocation::blocks)
      .def_readonly("slots", &sched::BlockAllocation::slots)
      .def_readonly("prefix_len", &sched::BlockAllocation::prefix_len);

  py::class_<sched::BlockAllocator>(m, "BlockAllocator")
      .def(py::init<uint32_t, uint32_t, bool, std::optional<uint32_t>>(), py::arg("num_blocks"), py::arg("block_size"),
           py::arg("prefix_caching"), py::arg("window") = std::nullopt)
      .def("allocate",
           [](sched::BlockAllocator& a, uint32_t tokens, std::optional<std::vector<uint32_t>> prompt) {
             return a.allocate(tokens, prompt ? &*prompt : nullptr);
           },
           py::arg("tokens"), py::arg("prompt") = std::nullopt)
      .def("free", &sched::BlockAllocator::free, py::arg("blocks"), py::arg("allocation_id"),
           py::arg("computed_tokens") = UINT32_MAX)
      .def("free_blocks", &sched::BlockAllocator::free_blocks)
      .def("cached_blocks", [](sched::BlockAllocator& a) { return a.trie().cached_blocks(); })
      .def("check", [](sched::BlockAllocator& a) { return a.check(); });

  py::class_<sched::RadixTrie>(m, "RadixTrie")
      .def(py::init<uint32_t>())
      .def("find",
           [](sched::RadixTrie& t, const std::vector<uint32_t>& key) {
             std::vector<uint32_t> blocks;
             int node = t.find(key, blocks);
             return py::make_tuple(node, blocks);
           })
      .def("insert", &sched::RadixTrie::insert)
      .def("incref", &sched::RadixTrie::incref)
      .def("decref", &sched::RadixTrie::decref)
      .def("evict", &sched::RadixTrie::evict)
      .def("cached_blocks", &sched::RadixTrie::cached_blocks)
      .def("live_nodes", &sched::RadixTrie::live_nodes)
      .def("check", &sched::RadixTrie::check);

  py::class_<sched::ResponseStream, std::shared_ptr<sched::ResponseStream>>(m, "ResponseStream")
      .def("pop",
           [](sched::ResponseStream& s, int timeout_ms) -> py::object {
             sched::StreamEvent ev;
             bool ok;
             {
               py::gil_scoped_release r;
               ok = s.pop(ev, timeout_ms);
             }
             if (!ok) return py::none();
             return event_to_dict(ev);
           })
      .def("close", &sched::ResponseStream::close);

  // Queue with its running map, for the batch-builder tests
  struct QueueBox {
    sched::Queue q;
    std::unordered_map<uint64_t, sched::Entry> running;
    std::vector<std::shared_ptr<sched::ResponseStream>> streams;
    explicit QueueBox(const sched::QueueConfig& c) : q(c) {}
  };
  py::class_<QueueBox>(m, "Queue")
      .def(py::init([](uint32_t block_size, bool prefix_caching, bool support_chunking, uint32_t max_batch_total_tokens,
                       uint32_t speculate, bool requires_padding) {
             sched::QueueConfig c;
             c.block_size = block_size;
             c.prefix_caching = prefix_caching;
             c.support_chunking = support_chunking;
             c.max_batch_total_tokens = max_batch_total_tokens;
             c.speculate = speculate;
             c.requires_padding = requires_padding;
             return new QueueBox(c);
           }),
           py::arg("block_size") = 16, py::arg("prefix_caching") = true, py::arg("support_chunking") = true,
           py::arg("max_batch_total_tokens") = 16384, py::arg("speculate") = 0, py::arg("requires_padding") = false)
      .def("append",
           [](QueueBox& b, uint32_t input_length, uint32_t max_new_tokens, std::vector<uint32_t> ids, bool details) {
             sched::Entry e;
             e.request = make_request(input_length, max_new_tokens, std::move(ids), details);
             e.stream = std::make_shared<sched::ResponseStream>();
             b.streams.push_back(e.stream);
             return b.q.append(std::move(e));
           },
           py::arg("input_length"), py::arg("max_new_tokens"), py::arg("ids") = std::vector<uint32_t>{},
           py::arg("decoder_input_details") = false)
      .def("drop_client", [](QueueBox& b, size_t i) { b.streams.at(i)->close(); })
      .def("size", [](QueueBox& b) { return b.q.size(); })
      .def("next_batch",
           [](QueueBox& b, std::optional<size_t> min_size, std::optional<size_t> max_size, uint32_t prefill_budget,
              uint32_t token_budget) -> py::object {
             auto nb = b.q.next_batch(min_size, max_size, prefill_budget, token_budget, b.running);
             if (!nb) return py::none();
             py::list reqs;
             for (auto& r : nb->batch.requests) {
               py::dict d;
               d["id"] = r.id;
               d["blocks"] = r.blocks;
               d["slots"] = r.slots.size();
               d["cache_len"] = r.cache_len;
               d["chunk_len"] = r.chunk_len ? py::cast(*r.chunk_len) : py::none();
               d["prefill_logprobs"] = r.prefill_logprobs;
               reqs.append(d);
             }
             py::dict out;
             out["id"] = nb->batch.id;
             out["size"] = nb->batch.size;
             out["max_tokens"] = nb->batch.max_tokens;
             out["requests"] = reqs;
             out["encoded"] = py::bytes(pb::encode_prefill_request(nb->batch, nullptr));
             return out;
           },
           py::arg("min_size") = std::nullopt, py::arg("max_size") = std::nullopt, py::arg("prefill_token_budget") = 4096,
           py::arg("token_budget") = 16384)
      .def("finish",
           [](QueueBox& b, uint64_t id, bool prefill_done) {
             auto it = b.running.find(id);
             if (it == b.running.end()) return false;
             it->second.prefill_done = prefill_done;
             b.q.release(it->second);
             b.running.erase(it);
             return true;
           },
           py::arg("id"), py::arg("prefill_done") = true)
      .def("free_blocks", [](QueueBox& b) { return b.q.allocator() ? b.q.allocator()->free_blocks() : 0; });

  py::class_<sched::Backend, std::shared_ptr<sched::Backend>>(m, "Backend")
      .def(py::init([](py::object shard, uint32_t block_size, bool support_chunking, uint32_t max_batch_prefill_tokens,
                       uint32_t max_batch_total_tokens, std::optional<size_t> max_batch_size) {
             sched::QueueConfig qc;
             qc.block_size = block_size;
             qc.support_chunking = support_chunking;
             qc.max_batch_total_tokens = max_batch_total_tokens;
             sched::BackendConfig bc;
             bc.max_batch_prefill_tokens = max_batch_prefill_tokens;
             bc.max_batch_total_tokens = max_batch_total_tokens;
             bc.max_batch_size = max_batch_size;
             return std::make_shared<sched::Backend>(std::make_shared<PyShard>(std::move(shard)), qc, bc, nullptr);
           }),
           py::arg("shard"), py::arg("block_size") = 16, py::arg("support_chunking") = true,
           py::arg("max_batch_prefill_tokens") = 4096, py::arg("max_batch_total_tokens") = 16384,
           py::arg("max_batch_size") = std::nullopt)
      .def("schedule",
           [](sched::Backend& b, uint32_t input_length, uint32_t max_new_tokens, std::vector<uint32_t> ids) {
             return b.schedule(make_request(input_length, max_new_tokens, std::move(ids), false));
           },
           py::arg("input_length"), py::arg("max_new_tokens"), py::arg("ids") = std::vector<uint32_t>{})
      .def("step_once",
           [](sched::Backend& b) {
             py::gil_scoped_release r;
             return b.step_once();
           })
      .def("queue_size", &sched::Backend::queue_size);

  // ---- request validation / chat conversion with fake text services -------------------------
  struct RouterBox {
    std::shared_ptr<sched::Backend> backend;
    std::unique_ptr<api::Router> router;
  };
  py::class_<RouterBox>(m, "Router")
      .def(py::init([](uint32_t max_input_tokens, uint32_t max_total_tokens, py::object chat_template_fn) {
             auto box = new RouterBox();
             api::TextServices t;
             t.encode = [](const std::string& text, bool, uint32_t truncate) {
               std::vector<uint32_t> ids;   // one token per whitespace-separated word
               bool in_word = false;
               for (char c : text) {
                 if (c == ' ' || c == '\n') in_word = false;
                 else if (!in_word) { in_word = true; ids.push_back(static_cast<uint32_t>(ids.size())); }
               }
               if (truncate && ids.size() > truncate) ids.erase(ids.begin(), ids.end() - truncate);
               return ids;
             };
             t.encode_with_offsets = [](const std::string&, bool) { return json::Value::array(); };
             t.chat_template = [chat_template_fn](const json::Value& messages, const json::Value& tools,
                                                  const std::string& tool_prompt) {
               py::gil_scoped_acquire g;
               return chat_template_fn(messages.dump(), tools.dump(), tool_prompt).cast<std::string>();
             };
             t.compile_grammar = [](const std::string& type, const json::Value& value) {
               return std::make_pair(type + ":" + value.dump(), 2u);
             };
             api::RouterConfig rc;
             rc.max_input_tokens = max_input_tokens;
             rc.max_total_tokens = max_total_tokens;
             box->router = std::make_unique<api::Router>(nullptr, t, rc, nullptr);
             return box;
           }),
           py::arg("max_input_tokens") = 100, py::arg("max_total_tokens") = 200,
           py::arg("chat_template") = py::cpp_function([](std::string m, std::string, std::string) { return m; }))
      .def("validate",
           [](RouterBox& b, const std::string& inputs, const std::string& params_json) {
             try {
               api::GenerateParams p = b.router->validate(inputs, json::Value::parse(params_json));
               py::dict d;
               d["input_length"] = p.valid.input_length;
               d["max_new_tokens"] = p.valid.stopping.max_new_tokens;
               d["max_total_new_tokens"] = p.max_total_new_tokens;
               d["temperature"] = p.valid.parameters.temperature;
               d["top_k"] = p.valid.parameters.top_k;
               d["top_p"] = p.valid.parameters.top_p;
               d["do_sample"] = p.valid.parameters.do_sample;
               d["seed"] = p.valid.parameters.seed;
               d["repetition_penalty"] = p.valid.parameters.repetition_penalty;
               d["grammar"] = p.valid.parameters.grammar;
               d["grammar_type"] = p.valid.parameters.grammar_type;
               d["stop"] = p.valid.stopping.stop_sequences;
               d["best_of"] = p.best_of ? py::cast(*p.best_of) : py::none();
               d["truncate"] = p.valid.truncate;
               d["adapter_id"] = p.valid.adapter_id ? py::cast(*p.valid.adapter_id) : py::none();
               d["add_special_tokens"] = p.valid.add_special_tokens;
               return py::object(d);
             } catch (const api::ApiError& e) {
               throw py::value_error(std::string(e.what()));
             }
           })
      .def("chat_to_generate", [](RouterBox& b, const std::string& chat_json) {
        try {
          std::string inputs;
          bool tools = false;
          json::Value params = b.router->chat_to_generate(json::Value::parse(chat_json), inputs, tools);
          return py::make_tuple(inputs, params.dump(), tools);
        } catch (const api::ApiError& e) {
          throw py::value_error(std::string(e.what()));
        }
      });

  m.def("tools_to_grammar_schema", [](const std::string& tools, const std::string& choice) {
    try {
      return api::tools_to_grammar_schema(json::Value::parse(tools), json::Value::parse(choice)).dump();
    } catch (const api::ApiError& e) {
      throw py::value_error(std::string(e.what()));
    }
  });
  m.def("json_roundtrip", [](const std::string& s) { return json::Value::parse(s).dump(); });
  m.def("decode_step_response", [](const std::string& raw) {
    pb::StepResponse r = pb::StepResponse::decode(raw);
    py::list gens;
    for (auto& g : r.generations) {
      py::dict d;
      d["request_id"] = g.request_id;
      d["ids"] = g.tokens.ids;
      d["logprobs"] = g.tokens.logprobs;
      d["texts"] = g.tokens.texts;
      d["is_special"] = g.tokens.is_special;
      d["finished"] = g.generated_text.has_value();
      if (g.generated_text) {
        d["text"] = g.generated_text->text;
        d["finish_reason"] = g.generated_text->finish_reason;
        d["seed"] = g.generated_text->seed ? py::cast(*g.generated_text->seed) : py::none();
      }
      d["n_top"] = g.top_tokens.size();
      d["prefill_ids"] = g.prefill_tokens ? py::cast(g.prefill_tokens->ids) : py::none();
      gens.append(d);
    }
    py::dict out;
    out["generations"] = gens;
    out["batch_id"] = r.batch ? py::cast(r.batch->id) : py::none();
    out["batch_request_ids"] = r.batch ? py::cast(r.batch->request_ids) : py::none();
    out["forward_ns"] = r.forward_ns;
    out["total_ns"] = r.total_ns;
    return out;
  });
  m.def("encode_warmup_request", [](uint32_t n_requests, uint32_t input_len) {
    pb::Batch b;
    for (uint32_t i = 0; i < n_requests; ++i) {
      pb::Request r;
      r.id = i;
      r.inputs = "hello";
      r.truncate = input_len;
      r.parameters.temperature = 0.5f;
      r.parameters.top_k = 3;
      r.parameters.seed = 1234567890123ull;
      r.stopping_parameters.max_new_tokens = 7;
      r.stopping_parameters.stop_sequences = {"a", "bc"};
      r.blocks = {1, 2, 300};
      r.slots = {16, 17};
      r.cache_len = 5;
      r.chunk_len = 9;
      r.adapter_id = "ad";
      pb::InputChunk c;
      c.text = "hello";
      r.input_chunks.push_back(c);
      b.requests.push_back(r);
    }
    b.id = 77;
    b.size = n_requests;
    b.max_tokens = 99;
    b.max_blocks = 3;
    return py::bytes(pb::encode_warmup_request(b, 11, 22, std::nullopt));
  });
}
