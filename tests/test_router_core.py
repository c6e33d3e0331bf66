"""Unit tests of the C++ router core through its pybind11 test module: block allocator and radix
trie (deterministic cases + randomized invariants), batch builder budgets, the batching loop against a
scripted shard, protobuf codec against the Python protobuf runtime, request validation, tool grammar."""
import json
import random

import pytest


@pytest.fixture(scope="session")
def rt():
    from tgi_b200.router.build import build

    build()
    from tgi_b200.router import _router_test

    return _router_test


# ---------------------------------------------------------------------------------------------
# allocator + radix trie
# ---------------------------------------------------------------------------------------------
def test_allocator_reserves_block_zero_and_frees(rt):
    a = rt.BlockAllocator(8, 2, False)
    assert a.free_blocks() == 7
    x = a.allocate(5, None)
    assert len(x.blocks) == 3 and 0 not in x.blocks
    assert len(x.slots) == 6 and x.slots[0] == x.blocks[0] * 2
    assert a.allocate(10, None) is None
    a.free(x.blocks, x.allocation_id)
    assert a.free_blocks() == 7


def test_prefix_sharing_and_duplicate_free(rt):
    a = rt.BlockAllocator(32, 2, True)
    p = [1, 2, 3, 4, 5, 6]
    x = a.allocate(8, p)
    assert x.prefix_len == 0
    y = a.allocate(8, p)            # nothing cached yet: second request allocates its own blocks
    assert y.prefix_len == 0
    a.free(x.blocks, x.allocation_id)   # x's prompt blocks enter the trie
    assert a.cached_blocks() == 3
    free_before = a.free_blocks()
    a.free(y.blocks, y.allocation_id)   # y's prompt blocks duplicate x's: all of y's blocks come back
    assert a.free_blocks() == free_before + len(y.blocks)
    z = a.allocate(8, p + [9, 9])
    assert z.prefix_len == 6 and z.blocks[:3] == x.blocks[:3]
    assert a.check()
    a.free(z.blocks, z.allocation_id)
    assert a.check()


def test_eviction_lru_and_pinning(rt):
    a = rt.BlockAllocator(9, 2, True)      # 8 usable blocks
    x = a.allocate(4, [1, 2, 3, 4])
    a.free(x.blocks, x.allocation_id)      # 2 blocks cached
    y = a.allocate(4, [5, 6, 7, 8])
    a.free(y.blocks, y.allocation_id)      # 4 cached, 4 free
    pinned = a.allocate(4, [1, 2, 3, 4])   # pins the first entry
    assert pinned.prefix_len == 4          # raw prefix; the batch builder keeps one token to compute
    # ask for more than is free: the unpinned entry must be evicted, the pinned one must survive
    big = a.allocate(12, None)
    assert big is not None and len(big.blocks) == 6
    assert a.cached_blocks() == 2
    assert a.allocate(2, None) is None
    a.free(big.blocks, big.allocation_id)
    a.free(pinned.blocks, pinned.allocation_id)
    assert a.check()


def test_radix_split_and_partial_match(rt):
    t = rt.RadixTrie(2)
    assert t.insert([1, 2, 3, 4, 5, 6], [10, 11, 12]) == 0
    node, blocks = t.find([1, 2, 3, 4, 9, 9])
    assert blocks == [10, 11]
    assert t.insert([1, 2, 3, 4, 7, 8], [20, 21, 22]) == 4     # first two blocks already present
    assert t.cached_blocks() == 4 and t.live_nodes() == 4      # root + shared + two tails
    node, blocks = t.find([1, 2, 3, 4, 7, 8, 1])
    assert blocks == [10, 11, 22]
    assert t.check()
    freed = t.evict(1)
    assert len(freed) == 1 and t.check()


def test_randomized_allocator_invariants(rt):
    rng = random.Random(0)
    bs, nblocks = 4, 200
    a = rt.BlockAllocator(nblocks, bs, True)
    live = []
    vocab = 6
    for step in range(3000):
        if live and (rng.random() < 0.45 or len(live) > 30):
            al = live.pop(rng.randrange(len(live)))
            a.free(al.blocks, al.allocation_id)
        else:
            n = rng.randint(1, 40)
            prompt = [rng.randrange(vocab) for _ in range(n)]
            tokens = n + rng.randint(1, 20)
            al = a.allocate(tokens, prompt)
            if al is not None:
                assert len(al.blocks) == (tokens + bs - 1) // bs
                assert al.prefix_len % bs == 0 and al.prefix_len <= n + bs
                assert len(set(al.blocks)) == len(al.blocks) and 0 not in al.blocks
                live.append(al)
        if step % 100 == 0:
            assert a.check()
            # no block is owned twice: free + cached + privately held blocks add up
            held = sum(len(x.blocks) - x.prefix_len // bs for x in live)
            assert a.free_blocks() + a.cached_blocks() + held == nblocks - 1
    for al in live:
        a.free(al.blocks, al.allocation_id)
    assert a.check()
    assert a.free_blocks() + a.cached_blocks() == nblocks - 1
    # nothing is live: no pin may survive, so every block but the reserved one can be had again
    everything = a.allocate((nblocks - 1) * bs, None)
    assert everything is not None and len(everything.blocks) == nblocks - 1
    assert a.cached_blocks() == 0
    a.free(everything.blocks, everything.allocation_id)
    assert a.check()


def test_split_of_a_pinned_edge_releases_both_halves(rt):
    a = rt.BlockAllocator(17, 2, True)          # 16 usable blocks
    x = a.allocate(4, [1, 2, 3, 4])
    a.free(x.blocks, x.allocation_id)           # edge [1,2,3,4] cached
    b = a.allocate(4, [1, 2, 3, 4])             # pins that edge
    assert b.prefix_len == 4
    c = a.allocate(4, [1, 2, 9, 9])             # shares one block
    assert c.prefix_len == 2
    a.free(c.blocks, c.allocation_id)           # inserting [1,2,9,9] splits the pinned edge
    assert a.check()
    a.free(b.blocks, b.allocation_id)
    assert a.check()
    full = a.allocate(32, None)                 # all 16 blocks must be evictable again
    assert full is not None and len(full.blocks) == 16
    a.free(full.blocks, full.allocation_id)
    assert a.allocate(30, None) is not None


def test_free_with_uncomputed_prompt_caches_nothing(rt):
    a = rt.BlockAllocator(17, 2, True)
    x = a.allocate(6, [1, 2, 3, 4, 5, 6])
    a.free(x.blocks, x.allocation_id, 0)        # never ran: its blocks hold no KV
    assert a.cached_blocks() == 0 and a.free_blocks() == 16
    y = a.allocate(6, [1, 2, 3, 4, 5, 6])
    assert y.prefix_len == 0
    a.free(y.blocks, y.allocation_id, 4)        # partial prefill: two of three blocks computed
    assert a.cached_blocks() == 2
    z = a.allocate(6, [1, 2, 3, 4, 5, 6])
    assert z.prefix_len == 4
    a.free(z.blocks, z.allocation_id)
    assert a.check()


# ---------------------------------------------------------------------------------------------
# batch builder
# ---------------------------------------------------------------------------------------------
def test_next_batch_budgets_and_chunking(rt):
    q = rt.Queue(block_size=16, prefix_caching=False, support_chunking=True, max_batch_total_tokens=4096)
    assert q.next_batch() is None
    for _ in range(3):
        q.append(100, 10)
    b = q.next_batch(prefill_token_budget=250, token_budget=4096)
    # budget rounds up to 256: two whole prompts (200) + 56 tokens of the third
    assert b["size"] == 3
    assert [r["chunk_len"] for r in b["requests"]] == [None, None, 56]
    assert q.size() == 0
    # tokens = input + max_new - 1 -> blocks
    assert all(len(r["blocks"]) == (100 + 10 - 1 + 15) // 16 for r in b["requests"])


def test_next_batch_without_chunking_and_sizes(rt):
    q = rt.Queue(block_size=16, prefix_caching=False, support_chunking=False, max_batch_total_tokens=4096)
    for _ in range(4):
        q.append(100, 10)
    assert q.next_batch(min_size=5) is None
    b = q.next_batch(prefill_token_budget=250)
    assert b["size"] == 2 and q.size() == 2
    b2 = q.next_batch(max_size=1)
    assert b2["size"] == 1 and b2["id"] == b["id"] + 1


def test_next_batch_backs_off_without_blocks_and_skips_dropped(rt):
    q = rt.Queue(block_size=16, prefix_caching=False, support_chunking=True, max_batch_total_tokens=160)   # 10 blocks
    q.append(64, 17)     # needs 5 blocks
    q.append(64, 17)     # needs 5 blocks -> only 9 usable (block 0 reserved)
    q.append(8, 2)
    q.drop_client(0)
    b = q.next_batch()
    assert b["size"] == 2 and [r["id"] for r in b["requests"]] == [1, 2]
    q.append(64, 17)
    assert q.next_batch() is None          # no blocks left
    assert q.finish(1)
    assert q.next_batch()["size"] == 1


def test_next_batch_prefix_cache_and_full_hit(rt):
    q = rt.Queue(block_size=4, prefix_caching=True, support_chunking=True, max_batch_total_tokens=400)
    ids = list(range(8))
    q.append(8, 4, ids)
    b = q.next_batch()
    assert b["requests"][0]["cache_len"] == 0
    q.finish(b["requests"][0]["id"])
    q.append(8, 4, ids)                      # whole prompt cached: one token must still be computed
    q.append(8, 4, ids, True)                # prompt logprobs requested: no prefix re-use
    b = q.next_batch()
    assert [r["cache_len"] for r in b["requests"]] == [7, 0]
    assert b["requests"][1]["prefill_logprobs"] is True


def test_pushed_back_request_finds_no_cache_entry_of_itself(rt):
    # over the prefill budget without chunking: the second request goes back to the queue and must come
    # back with cache_len 0 (its blocks were never written)
    q = rt.Queue(block_size=4, prefix_caching=True, support_chunking=False, max_batch_total_tokens=400)
    q.append(16, 4, list(range(100, 116)))
    q.append(16, 4, list(range(200, 216)))
    b = q.next_batch(prefill_token_budget=16)
    assert [(r["id"], r["cache_len"]) for r in b["requests"]] == [(0, 0)]
    b2 = q.next_batch(prefill_token_budget=16)
    assert [(r["id"], r["cache_len"]) for r in b2["requests"]] == [(1, 0)]
    # same with chunking when the earlier prompt fills the budget exactly
    q = rt.Queue(block_size=4, prefix_caching=True, support_chunking=True, max_batch_total_tokens=400)
    q.append(16, 4, list(range(100, 116)))
    q.append(16, 4, list(range(200, 216)))
    b = q.next_batch(prefill_token_budget=16)
    assert len(b["requests"]) == 1
    b2 = q.next_batch(prefill_token_budget=16)
    assert [(r["id"], r["cache_len"]) for r in b2["requests"]] == [(1, 0)]
    # a request released after a failed prefill leaves nothing behind either
    assert q.finish(1, False)
    q.append(16, 4, list(range(200, 216)))
    b3 = q.next_batch(prefill_token_budget=16)
    assert b3["requests"][0]["cache_len"] == 0


# ---------------------------------------------------------------------------------------------
# protobuf codec
# ---------------------------------------------------------------------------------------------
def test_codec_matches_python_protobuf(rt):
    from tgi_b200.proto import generate_v3 as pb

    raw = rt.encode_warmup_request(2, 33)
    w = pb.WarmupRequest.FromString(raw)
    assert w.max_input_tokens == 11 and w.max_prefill_tokens == 22 and not w.HasField("max_total_tokens")
    assert w.batch.id == 77 and w.batch.size == 2 and w.batch.max_blocks == 3
    r = w.batch.requests[1]
    assert r.id == 1 and r.inputs == "hello" and r.truncate == 33 and list(r.blocks) == [1, 2, 300]
    assert list(r.slots) == [16, 17] and r.cache_len == 5 and r.chunk_len == 9 and r.adapter_id == "ad"
    assert abs(r.parameters.temperature - 0.5) < 1e-7 and r.parameters.top_k == 3
    assert r.parameters.seed == 1234567890123 and list(r.stopping_parameters.stop_sequences) == ["a", "bc"]
    assert r.input_chunks.chunks[0].text == "hello" and r.add_special_tokens

    g = pb.Generation(request_id=5, tokens=pb.Tokens(ids=[7, 8], logprobs=[-0.5, -1.5], texts=["a", "é"], is_special=[False, True]))
    g.prefill_tokens.CopyFrom(pb.Tokens(ids=[1], logprobs=[float("nan")], texts=["p"], is_special=[False]))
    g.generated_text.CopyFrom(pb.GeneratedText(text="aé", generated_tokens=2, finish_reason=1, seed=42))
    g.top_tokens.append(pb.Tokens(ids=[9], logprobs=[-2.0], texts=["z"], is_special=[False]))
    resp = pb.DecodeResponse(generations=[g], forward_ns=10, decode_ns=20, total_ns=30)
    resp.batch.CopyFrom(pb.CachedBatch(id=3, request_ids=[5, 6], size=2, max_tokens=64, current_tokens=2))
    d = rt.decode_step_response(resp.SerializeToString())
    gen = d["generations"][0]
    assert gen["request_id"] == 5 and gen["ids"] == [7, 8] and gen["texts"] == ["a", "é"]
    assert gen["logprobs"] == [-0.5, -1.5] and gen["is_special"] == [False, True]
    assert gen["finished"] and gen["text"] == "aé" and gen["finish_reason"] == 1 and gen["seed"] == 42
    assert gen["n_top"] == 1 and gen["prefill_ids"] == [1]
    assert d["batch_id"] == 3 and d["batch_request_ids"] == [5, 6] and d["total_ns"] == 30


def test_json_roundtrip(rt):
    s = '{"a":[1,2.5,-3,true,null,"x\\n\\u00e9\\ud83d\\ude00"],"b":{"c":18446744073709551615}}'
    out = json.loads(rt.json_roundtrip(s))
    assert out == json.loads(s)
    with pytest.raises(Exception):
        rt.json_roundtrip('{"a":1,}')


# ---------------------------------------------------------------------------------------------
# batching loop against a scripted shard
# ---------------------------------------------------------------------------------------------
class FakeShard:
    """Generates `max_new_tokens` tokens per request, one per step, like a real shard would."""

    def __init__(self, fail_decode_at=None):
        from tgi_b200.proto import generate_v3 as pb

        self.pb = pb
        self.batches = {}
        self.calls = []
        self.fail_decode_at = fail_decode_at
        self.decodes = 0

    def _step(self, batch_id, reqs):
        pb = self.pb
        gens, alive = [], []
        for r in reqs:
            r["done"] += 1
            g = pb.Generation(request_id=r["id"], tokens=pb.Tokens(ids=[r["done"]], logprobs=[-1.0], texts=["t"], is_special=[False]))
            if r["done"] >= r["max_new"]:
                g.generated_text.CopyFrom(pb.GeneratedText(text="t" * r["done"], generated_tokens=r["done"], finish_reason=0))
            else:
                alive.append(r)
            gens.append(g)
        resp = pb.PrefillResponse(generations=gens, total_ns=1)
        if alive:
            self.batches[batch_id] = reqs
            resp.batch.CopyFrom(pb.CachedBatch(id=batch_id, request_ids=[r["id"] for r in reqs], size=len(reqs),
                                               max_tokens=sum(r["max_new"] + 4 for r in reqs), current_tokens=len(reqs)))
        else:
            self.batches.pop(batch_id, None)
        return resp.SerializeToString()

    def prefill(self, raw):
        req = self.pb.PrefillRequest.FromString(raw)
        self.calls.append(("prefill", len(req.batch.requests), req.HasField("cached_batch")))
        reqs = [{"id": r.id, "max_new": r.stopping_parameters.max_new_tokens, "done": 0} for r in req.batch.requests]
        old = self.batches.pop(req.cached_batch.id, []) if req.HasField("cached_batch") else []
        out_id = req.cached_batch.id if req.HasField("cached_batch") else req.batch.id
        # requests of the cached batch decode one step in the same forward
        return self._step(out_id, old + reqs)

    def decode(self, raw):
        req = self.pb.DecodeRequest.FromString(raw)
        self.decodes += 1
        if self.fail_decode_at is not None and self.decodes == self.fail_decode_at:
            raise RuntimeError("shard exploded")
        self.calls.append(("decode", len(req.batches)))
        reqs = []
        for b in req.batches:
            reqs += self.batches.pop(b.id)
        return self._step(req.batches[0].id, reqs)

    def filter_batch(self, raw):
        req = self.pb.FilterBatchRequest.FromString(raw)
        self.calls.append(("filter", list(req.request_ids)))
        keep = [r for r in self.batches[req.batch_id] if r["id"] in set(req.request_ids)]
        self.batches[req.batch_id] = keep
        cb = self.pb.CachedBatch(id=req.batch_id, request_ids=[r["id"] for r in keep], size=len(keep),
                                 max_tokens=sum(r["max_new"] + 4 for r in keep), current_tokens=len(keep))
        return self.pb.FilterBatchResponse(batch=cb).SerializeToString()

    def clear_cache(self, batch_id):
        self.calls.append(("clear", batch_id))
        if batch_id is None:
            self.batches.clear()
        else:
            self.batches.pop(batch_id, None)

    def health(self):
        pass


def drain(stream):
    out = []
    while True:
        ev = stream.pop(0)
        if ev is None:
            return out
        out.append(ev)


def test_continuous_batching_loop(rt):
    shard = FakeShard()
    be = rt.Backend(shard, block_size=16, max_batch_prefill_tokens=64, max_batch_total_tokens=1024)
    s1 = be.schedule(10, 3)
    s2 = be.schedule(10, 5)
    assert be.step_once()            # prefill of both
    s3 = be.schedule(10, 2)          # joins while the batch is running
    for _ in range(12):
        if not be.step_once():
            break
    e1, e2, e3 = drain(s1), drain(s2), drain(s3)
    assert [e["kind"] for e in e1] == ["token", "token", "end"] and e1[-1]["generated_tokens"] == 3
    assert len(e2) == 5 and e2[-1]["kind"] == "end"
    assert len(e3) == 2 and e3[-1]["generated_text"] == "tt"
    kinds = [c[0] for c in shard.calls]
    assert kinds[0] == "prefill" and ("prefill", 1, True) in shard.calls     # chunked merge into the running batch
    assert any(c[0] == "filter" for c in shard.calls)                        # finished requests are filtered out
    assert not shard.batches


def test_shard_failure_fails_the_batch_and_recovers(rt):
    shard = FakeShard(fail_decode_at=1)
    be = rt.Backend(shard, block_size=16)
    s1 = be.schedule(10, 4)
    be.step_once()
    be.step_once()                   # decode raises
    ev = drain(s1)
    assert ev[-1]["kind"] == "error" and "exploded" in ev[-1]["error"]
    assert any(c[0] == "clear" for c in shard.calls)
    s2 = be.schedule(10, 2)          # the scheduler keeps serving afterwards
    for _ in range(5):
        be.step_once()
    assert drain(s2)[-1]["kind"] == "end"


def test_client_disconnect_filters_request(rt):
    shard = FakeShard()
    be = rt.Backend(shard, block_size=16)
    s1 = be.schedule(10, 50)
    s2 = be.schedule(10, 3)
    be.step_once()
    s1.close()
    for _ in range(6):
        be.step_once()
    assert drain(s2)[-1]["kind"] == "end"
    assert ("filter", [1]) in shard.calls or any(c[0] == "clear" for c in shard.calls)
    assert not shard.batches


# ---------------------------------------------------------------------------------------------
# validation and chat conversion
# ---------------------------------------------------------------------------------------------
def test_validation_rules(rt):
    r = rt.Router(max_input_tokens=10, max_total_tokens=20)
    ok = r.validate("a b c", json.dumps({"max_new_tokens": 5, "temperature": 0.5, "top_k": 4, "stop": ["x"], "seed": 7}))
    assert ok["input_length"] == 3 and ok["max_new_tokens"] == 5 and ok["seed"] == 7 and ok["stop"] == ["x"]
    assert abs(ok["temperature"] - 0.5) < 1e-6 and ok["top_k"] == 4
    dflt = r.validate("a b c", "{}")
    assert dflt["max_new_tokens"] == 17 and dflt["max_total_new_tokens"] == 17      # the context that is left
    assert r.validate("a b c", "{}")["seed"] != dflt["seed"]                        # random seed per request
    for bad in ({"temperature": 0}, {"top_p": 1.0}, {"top_p": 0}, {"top_k": 0}, {"typical_p": 1.5},
                {"repetition_penalty": 0}, {"frequency_penalty": 3}, {"max_new_tokens": 0}, {"max_new_tokens": 18},
                {"best_of": 3}, {"best_of": 2}, {"best_of": 2, "do_sample": True, "seed": 1},
                {"stop": ["a", "b", "c", "d", "e"]}, {"top_n_tokens": 6}, {"truncate": 11}, {"truncate": 0}):
        with pytest.raises(ValueError):
            r.validate("a b c", json.dumps(bad))
    with pytest.raises(ValueError):
        r.validate("", "{}")
    with pytest.raises(ValueError):
        r.validate(" ".join("w" * 11), "{}")
    assert r.validate(" ".join("w" * 11), json.dumps({"truncate": 4, "max_new_tokens": 2}))["input_length"] == 4
    g = r.validate("a", json.dumps({"grammar": {"type": "regex", "value": "a+"}, "max_new_tokens": 1}))
    assert g["grammar"] == 'regex:"a+"' and g["grammar_type"] == 2


def test_chat_conversion(rt):
    seen = {}

    def template(messages, tools, tool_prompt):
        seen["messages"], seen["tools"] = json.loads(messages), json.loads(tools)
        return "PROMPT"

    r = rt.Router(max_input_tokens=10, max_total_tokens=20, chat_template=template)
    inputs, params, tools = r.chat_to_generate(json.dumps({
        "model": "tgi", "messages": [{"role": "user", "content": "hi"}], "temperature": 0, "presence_penalty": 0.5,
        "max_tokens": 7, "stop": "END", "seed": 3, "top_logprobs": 2}))
    p = json.loads(params)
    assert inputs == "PROMPT" and not tools
    assert p["do_sample"] is False and "temperature" not in p and p["repetition_penalty"] == 2.5
    assert p["max_new_tokens"] == 7 and p["stop"] == ["END"] and p["seed"] == 3 and p["top_n_tokens"] == 2
    assert p["add_special_tokens"] is False and "adapter_id" not in p
    _, params, _ = r.chat_to_generate(json.dumps({"model": "my-lora", "messages": [{"role": "user", "content": "x"}]}))
    assert json.loads(params)["adapter_id"] == "my-lora"
    tool = {"type": "function", "function": {"name": "get_weather", "description": "w",
                                             "parameters": {"type": "object", "properties": {"city": {"type": "string"}},
                                                            "required": ["city"]}}}
    _, params, tools = r.chat_to_generate(json.dumps({"messages": [{"role": "user", "content": "x"}], "tools": [tool]}))
    assert tools and json.loads(params)["grammar"]["type"] == "json"
    assert seen["tools"][0]["function"]["name"] == "get_weather"
    with pytest.raises(ValueError):
        r.chat_to_generate(json.dumps({"messages": []}))


def test_tool_grammar_schema(rt):
    tool = {"type": "function", "function": {"name": "f", "parameters": {"properties": {"a": {"type": "integer"}},
                                                                          "required": ["a"]}}}
    s = json.loads(rt.tools_to_grammar_schema(json.dumps([tool]), '"auto"'))
    assert set(s["$functions"]) == {"f", "no_tool"}
    assert s["$functions"]["f"]["properties"]["_name"] == {"type": "string", "const": "f"}
    assert s["$functions"]["f"]["required"] == ["_name", "a"]
    assert {"$ref": "#/$functions/no_tool"} in s["properties"]["function"]["anyOf"]
    s = json.loads(rt.tools_to_grammar_schema(json.dumps([tool]), '"required"'))
    assert set(s["$functions"]) == {"f"}
    s = json.loads(rt.tools_to_grammar_schema(json.dumps([tool]), json.dumps({"type": "function", "function": {"name": "f"}})))
    assert set(s["$functions"]) == {"f"}
    with pytest.raises(ValueError):
        rt.tools_to_grammar_schema(json.dumps([tool]), json.dumps({"type": "function", "function": {"name": "g"}}))


def test_image_token_counts_match_the_runners(rt):
    """The router reserves exactly the rows the runners produce for an image (Qwen2-VL: dynamic resolution)."""
    import json

    from tgi_b200.models.qwen2_vl import smart_resize

    vis = {"patch_size": 14, "spatial_merge_size": 2, "min_pixels": 56 * 56, "max_pixels": 28 * 28 * 1280}
    cfg = {"model_type": "qwen2_vl", "vision_config": vis, "vision_start_token_id": 1, "vision_end_token_id": 2}
    for w, h in [(1, 1), (52, 40), (640, 480), (1920, 1080), (4000, 3000), (30, 3000), (999, 1001)]:
        rh, rw = smart_resize(h, w, 28, vis["min_pixels"], vis["max_pixels"])
        assert rt.tokens_per_image(json.dumps(cfg), w, h) == (rh // 28) * (rw // 28) + 2, (w, h)
    # images at most 20 pixels wide are doubled before the resize (shard and router alike)
    rh, rw = smart_resize(800, 40, 28, vis["min_pixels"], vis["max_pixels"])
    assert rt.tokens_per_image(json.dumps(cfg), 20, 400) == (rh // 28) * (rw // 28) + 2
    cfg25 = dict(cfg, model_type="qwen2_5_vl")
    assert rt.tokens_per_image(json.dumps(cfg25), 640, 480) == rt.tokens_per_image(json.dumps(cfg), 640, 480)
    assert rt.tokens_per_image(json.dumps({"model_type": "idefics2", "vision_config": {},
                                           "perceiver_config": {"resampler_n_latents": 64}}), 10, 10) == 64
    assert rt.tokens_per_image(json.dumps({"model_type": "idefics3", "scale_factor": 2,
                                           "vision_config": {"image_size": 364, "patch_size": 14}}), 10, 10) == 169
    # Idefics3 image splitting: the router's count equals the shard's layout for every image size
    from tgi_b200.models.idefics3 import expansion_length, tile_grid

    for tile, longest, nl, nlnl in [(364, 1456, 1, 1), (384, 1536, 1, 2), (28, 112, 1, 2), (364, 364, 1, 1)]:
        seq = (tile // 14 // 2) ** 2 if tile >= 28 else 1
        cfg3 = {"model_type": "idefics3", "scale_factor": 2, "vision_config": {"image_size": tile, "patch_size": 14},
                "_idefics3": {"tile": tile, "longest_edge": longest, "split": True, "nl": nl, "nlnl": nlnl}}
        for w, h in [(1, 1), (52, 40), (40, 52), (640, 480), (480, 640), (1920, 1080), (4000, 3000), (30, 3000), (999, 1001),
                     (1456, 1456), (333, 777), (5000, 17), (364, 365)]:
            _, _, rows, cols = tile_grid(h, w, longest, tile)
            assert rt.tokens_per_image(json.dumps(cfg3), w, h) == expansion_length(rows, cols, seq, nl, nlnl), (tile, w, h)
    unsplit = {"model_type": "idefics3", "scale_factor": 2, "vision_config": {"image_size": 364, "patch_size": 14},
               "_idefics3": {"tile": 364, "longest_edge": 1456, "split": False, "nl": 1, "nlnl": 1}}
    assert rt.tokens_per_image(json.dumps(unsplit), 2000, 1000) == 169 + 3
    assert rt.tokens_per_image(json.dumps({"model_type": "gemma3", "mm_tokens_per_image": 256, "boi_token_index": 1,
                                           "eoi_token_index": 2, "vision_config": {}}), 10, 10) == 258
    assert rt.tokens_per_image(json.dumps({"model_type": "mllama", "vision_config": {"image_size": 560}}), 900, 400) == 1
    assert rt.tokens_per_image(json.dumps({"model_type": "llama"}), 10, 10) == 0


def test_traceparent_parsing(rt):
    ok, tid, sid, sampled = rt.parse_traceparent("00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01")
    assert ok and tid == "4bf92f3577b34da6a3ce929d0e0e4736" and sid == "00f067aa0ba902b7" and sampled
    assert rt.parse_traceparent("00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-00")[3] is False
    for bad in ["", "garbage", "ff-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01",
                "00-00000000000000000000000000000000-00f067aa0ba902b7-01",
                "00-4bf92f3577b34da6a3ce929d0e0e4736-0000000000000000-01",
                "00-4BF92F3577B34DA6A3CE929D0E0E4736-00f067aa0ba902b7-01",
                "00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01-extra"]:
        assert rt.parse_traceparent(bad)[0] is False, bad


def test_llava_next_row_counts_match_the_runner(rt):
    import json

    from tgi_b200.models.llava_next import anyres_rows

    pins = [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]]
    cfg = {"model_type": "llava_next", "image_grid_pinpoints": pins, "vision_config": {"image_size": 336, "patch_size": 14}}
    for w, h in [(640, 480), (480, 640), (1920, 1080), (100, 1000), (1000, 100), (336, 336), (50, 37), (2000, 1999)]:
        assert rt.tokens_per_image(json.dumps(cfg), w, h) == anyres_rows((h, w), pins, 336, 24), (w, h)
    plain = {"model_type": "llava_next", "vision_config": {"image_size": 336, "patch_size": 14}}
    assert rt.tokens_per_image(json.dumps(plain), 640, 480) == 576


def test_llava_next_row_counts_random_sizes(rt):
    import json
    import random

    from tgi_b200.models.llava_next import anyres_rows

    pins = [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]]
    cfg = json.dumps({"model_type": "llava_next", "image_grid_pinpoints": pins,
                      "vision_config": {"image_size": 336, "patch_size": 14}})
    rng = random.Random(1)
    for _ in range(500):
        w, h = rng.randint(8, 3000), rng.randint(8, 3000)
        assert rt.tokens_per_image(cfg, w, h) == anyres_rows((h, w), pins, 336, 24), (w, h)


def test_qwen2_vl_row_counts_random_sizes(rt):
    import json
    import random

    from tgi_b200.models.qwen2_vl import smart_resize

    vis = {"patch_size": 14, "spatial_merge_size": 2, "min_pixels": 56 * 56, "max_pixels": 28 * 28 * 1280}
    cfg = json.dumps({"model_type": "qwen2_vl", "vision_config": vis})
    rng = random.Random(2)
    for _ in range(500):
        w, h = rng.randint(4, 5000), rng.randint(4, 5000)
        if max(w, h) / min(w, h) > 200:
            continue
        k = 2 if w <= 20 else 1           # narrow images are doubled before the resize (shard and router)
        rh, rw = smart_resize(k * h, k * w, 28, vis["min_pixels"], vis["max_pixels"])
        assert rt.tokens_per_image(cfg, w, h) == (rh // 28) * (rw // 28), (w, h)
