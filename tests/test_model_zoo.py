"""Model families on CPU against transformers: a tiny random checkpoint of every architecture is saved
by transformers, loaded by the generic paged-KV decoder, and the prefill logits must agree."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.decoder import ForwardMeta  # noqa: E402

COMMON = dict(vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=256)


def _cfg(name):
    T = transformers
    if name == "llama":
        return T.LlamaConfig(**COMMON, intermediate_size=128, num_key_value_heads=2)
    if name == "mistral":
        return T.MistralConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, sliding_window=None)
    if name == "qwen2":
        return T.Qwen2Config(**COMMON, intermediate_size=128, num_key_value_heads=2)
    if name == "qwen3":
        return T.Qwen3Config(**COMMON, intermediate_size=128, num_key_value_heads=2, head_dim=16)
    if name == "gemma":
        return T.GemmaConfig(**COMMON, intermediate_size=128, num_key_value_heads=1, head_dim=16)
    if name == "gemma2":
        return T.Gemma2Config(**COMMON, intermediate_size=128, num_key_value_heads=2, head_dim=16, sliding_window=64,
                              query_pre_attn_scalar=16)
    if name == "phi3":
        return T.Phi3Config(**COMMON, intermediate_size=128, num_key_value_heads=2, pad_token_id=0)
    if name == "phi":
        return T.PhiConfig(**COMMON, intermediate_size=128, partial_rotary_factor=0.5)
    if name == "gpt2":
        return T.GPT2Config(vocab_size=320, n_embd=64, n_layer=2, n_head=4, n_positions=256)
    if name == "gptj":
        return T.GPTJConfig(vocab_size=320, n_embd=64, n_layer=2, n_head=4, n_positions=256, rotary_dim=8)
    if name == "gpt_neox":
        return T.GPTNeoXConfig(**COMMON, intermediate_size=128, rotary_pct=0.5)
    if name == "falcon":
        return T.FalconConfig(vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                              new_decoder_architecture=False, multi_query=True, parallel_attn=True, bias=False, alibi=False)
    if name == "starcoder2":
        return T.Starcoder2Config(**COMMON, intermediate_size=128, num_key_value_heads=2, sliding_window=None)
    if name == "cohere":
        return T.CohereConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, use_qk_norm=False)
    if name == "granite":
        return T.GraniteConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, embedding_multiplier=2.0,
                               residual_multiplier=0.5, attention_multiplier=0.2, logits_scaling=3.0)
    if name == "mixtral":
        return T.MixtralConfig(**COMMON, intermediate_size=96, num_key_value_heads=2, num_local_experts=4,
                               num_experts_per_tok=2, sliding_window=None)
    if name == "qwen2_moe":
        return T.Qwen2MoeConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, num_experts=4, num_experts_per_tok=2,
                                moe_intermediate_size=48, shared_expert_intermediate_size=64, decoder_sparse_step=1,
                                norm_topk_prob=False)
    if name == "qwen3_moe":
        return T.Qwen3MoeConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, head_dim=16, num_experts=4,
                                num_experts_per_tok=2, moe_intermediate_size=48, decoder_sparse_step=1, norm_topk_prob=True)
    if name == "gpt_bigcode":
        return T.GPTBigCodeConfig(vocab_size=320, n_embd=64, n_layer=2, n_head=4, n_positions=256, multi_query=True)
    if name == "phimoe":
        return T.PhimoeConfig(**COMMON, intermediate_size=96, num_key_value_heads=2, num_local_experts=4,
                              num_experts_per_tok=2, sliding_window=None)
    if name == "dbrx":
        return T.DbrxConfig(d_model=64, n_heads=4, n_layers=2, max_seq_len=256, vocab_size=320,
                            attn_config={"kv_n_heads": 2, "clip_qkv": 8.0, "rope_theta": 10000.0},
                            ffn_config={"hidden_size": 64, "ffn_hidden_size": 64, "moe_num_experts": 4, "moe_top_k": 2})  # router width quirk of this transformers version
    if name == "gemma3_text":
        return T.Gemma3TextConfig(**COMMON, intermediate_size=128, num_key_value_heads=2, head_dim=16, sliding_window=64,
                                  query_pre_attn_scalar=16)
    if name == "falcon_new":
        return T.FalconConfig(vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_kv_heads=2,
                              new_decoder_architecture=True, parallel_attn=True, bias=False, alibi=False)
    if name == "deepseek_v3":
        return T.DeepseekV3Config(vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=48,
                                  num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1,
                                  n_routed_experts=8, routed_scaling_factor=2.5, kv_lora_rank=32, q_lora_rank=24,
                                  qk_rope_head_dim=16, v_head_dim=24, qk_nope_head_dim=32, n_group=2, topk_group=1,
                                  num_experts_per_tok=2, first_k_dense_replace=1, norm_topk_prob=True,
                                  max_position_embeddings=256)
    if name == "deepseek_v2":
        return T.DeepseekV2Config(vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=48,
                                  num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, n_shared_experts=2,
                                  n_routed_experts=8, routed_scaling_factor=1.0, kv_lora_rank=32, q_lora_rank=None,
                                  qk_rope_head_dim=16, v_head_dim=24, qk_nope_head_dim=32, n_group=2, topk_group=1,
                                  num_experts_per_tok=2, first_k_dense_replace=1, norm_topk_prob=False,
                                  topk_method="greedy", max_position_embeddings=256)   # the grouped V2 path of this transformers version raises
    raise KeyError(name)


NAMES = ["llama", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "phi3", "phi", "gpt2", "gptj", "gpt_neox", "falcon",
         "starcoder2", "cohere", "granite", "mixtral", "qwen2_moe", "qwen3_moe", "gpt_bigcode", "phimoe", "gemma3_text",
         "falcon_new", "deepseek_v2", "deepseek_v3"]
# DBRX is left out: the expert matmul of this transformers version multiplies by the untransposed weight
# (it only runs at all when ffn_hidden_size == d_model), so it is no oracle; the engine follows the layout of the
# released checkpoints.


@pytest.mark.parametrize("name", NAMES)
def test_prefill_logits_match_transformers(tmp_path, name):
    torch.manual_seed(0)
    cfg = _cfg(name)
    hf = transformers.AutoModelForCausalLM.from_config(cfg).eval().float()
    # random norm weights / biases so that mistakes in their handling show up
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_(torch.randn_like(p) * 0.1 + (1.0 if "norm" in n or "ln" in n else 0.0))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    ids = torch.tensor([[5, 17, 100, 42, 7, 9, 250, 31, 64, 3, 77, 12]])
    with torch.no_grad():
        want = hf(ids).logits[0].float()
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    model.init_kv_cache(4)
    T = ids.shape[1]
    meta = ForwardMeta(input_ids=ids[0].to(torch.int32), positions=torch.arange(T, dtype=torch.int32),
                       slots=torch.arange(16, 16 + T, dtype=torch.int32), block_tables=torch.tensor([[1, 2]], dtype=torch.int32),
                       cu_seqlens_q=torch.tensor([0, T], dtype=torch.int32), kv_lens=torch.tensor([T], dtype=torch.int32),
                       max_q=T, max_kv=T)
    got = model.forward(meta).float()
    err = (got - want).abs().max().item()
    assert err < 2e-3 * max(1.0, want.abs().max().item()), f"{name}: logits differ by {err}"


def test_legacy_santacoder_layout(tmp_path):
    """The first SantaCoder checkpoints: a ``gpt2`` config with ``attention_head_type: multiquery``, q and the shared
    k/v projection stored separately, every linear weight in GPT-2's transposed layout.  Built here from a tiny
    multi-query GPTBigCode model (the same network in its later layout), which is also the oracle."""
    import json

    from safetensors.torch import save_file

    torch.manual_seed(0)
    cfg = transformers.GPTBigCodeConfig(vocab_size=320, n_embd=64, n_layer=2, n_head=4, n_positions=256, multi_query=True,
                                        activation_function="gelu_pytorch_tanh")
    hf = transformers.GPTBigCodeForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_(torch.randn_like(p) * 0.1 + (1.0 if "ln" in n else 0.0))
    H, D = 64, 16
    legacy = {}
    for name, t in hf.state_dict().items():
        if name == "lm_head.weight":
            continue                                  # tied to the embedding
        if ".attn.c_attn." in name:
            q, kv = t[:H], t[H:H + 2 * D]
            if name.endswith("weight"):
                q, kv = q.t(), kv.t()
            legacy[name.replace("c_attn", "q_attn")] = q.contiguous()
            legacy[name.replace("c_attn", "kv_attn")] = kv.contiguous()
        elif name.endswith("weight") and any(k in name for k in (".attn.c_proj.", ".mlp.c_fc.", ".mlp.c_proj.")):
            legacy[name] = t.t().contiguous()
        else:
            legacy[name] = t.contiguous()
    save_file(legacy, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(dict(
        model_type="gpt2", architectures=["GPT2LMHeadCustomModel"], attention_head_type="multiquery", vocab_size=320,
        n_embd=64, n_layer=2, n_head=4, n_positions=256, activation_function="gelu_pytorch_tanh",
        layer_norm_epsilon=cfg.layer_norm_epsilon)))
    ids = torch.tensor([[5, 17, 100, 42, 7, 9, 250, 31, 64, 3, 77, 12]])
    with torch.no_grad():
        want = hf(ids).logits[0].float()
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert model.model.dims.total_kv_heads == 1
    model.init_kv_cache(4)
    T = ids.shape[1]
    meta = ForwardMeta(input_ids=ids[0].to(torch.int32), positions=torch.arange(T, dtype=torch.int32),
                       slots=torch.arange(16, 16 + T, dtype=torch.int32), block_tables=torch.tensor([[1, 2]], dtype=torch.int32),
                       cu_seqlens_q=torch.tensor([0, T], dtype=torch.int32), kv_lens=torch.tensor([T], dtype=torch.int32),
                       max_q=T, max_kv=T)
    got = model.forward(meta).float()
    err = (got - want).abs().max().item()
    assert err < 2e-3 * max(1.0, want.abs().max().item()), f"logits differ by {err}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["llama", "gemma2", "qwen3", "gpt2", "falcon", "phi", "mixtral", "deepseek_v3", "starcoder2"])
def test_prefill_logits_on_gpu_kernels(tmp_path, name):
    """The same comparison through the sm_100a kernels (bf16 weights): head dims 16..256, softcap, sliding
    window, partial and interleaved rotary, q/k norms, learned positions, MoE, latent attention."""
    torch.manual_seed(0)
    cfg = _cfg(name)
    hf = transformers.AutoModelForCausalLM.from_config(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.copy_(torch.randn_like(p) * 0.1 + (1.0 if "norm" in n or "ln" in n else 0.0))
            p.copy_(p.to(torch.bfloat16).float())           # both sides see bf16-representable weights
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    ids = torch.tensor([[5, 17, 100, 42, 7, 9, 250, 31, 64, 3, 77, 12, 200, 150, 99, 21, 8, 44]])
    with torch.no_grad():
        want = hf(ids).logits[0].float()
    dev = torch.device("cuda", 0)
    model = get_model(str(tmp_path), dtype="bfloat16", device=dev)
    model.init_kv_cache(4)
    T = ids.shape[1]
    i32 = dict(dtype=torch.int32, device=dev)
    meta = ForwardMeta(input_ids=ids[0].to(**i32), positions=torch.arange(T, **i32), slots=torch.arange(16, 16 + T, **i32),
                       block_tables=torch.tensor([[1, 2]], **i32), cu_seqlens_q=torch.tensor([0, T], **i32),
                       kv_lens=torch.tensor([T], **i32), max_q=T, max_kv=T)
    got = model.forward(meta).float().cpu()
    from tgi_b200.ops import cuda as K

    assert K.check_status(dev) == 0
    err = (got - want).abs().max().item()
    assert err < 0.06 * max(1.0, want.abs().max().item()), f"{name}: logits differ by {err}"
