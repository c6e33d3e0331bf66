"""Local `paged_attention` kernel module for the reference (hub: kernels-community/paged-attention,
built from vllm's csrc/attention and csrc/cache_kernels): the same ops from the installed vllm wheel.
Only reached with ATTENTION=paged; the flashinfer and flashdecoding modes store KV with index_put."""
from vllm import _custom_ops as _ops


def reshape_and_cache(key, value, key_cache, value_cache, slots, kv_cache_dtype, k_scale, v_scale):
    _ops.reshape_and_cache(key, value, key_cache, value_cache, slots, kv_cache_dtype, k_scale, v_scale)


def paged_attention_v1(out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens, block_size,
                       max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale):
    _ops.paged_attention_v1(out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
                            block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale)


def paged_attention_v2(out, exp_sum, max_logits, tmp_out, query, key_cache, value_cache, num_kv_heads, scale,
                       block_tables, seq_lens, block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale):
    _ops.paged_attention_v2(out, exp_sum, max_logits, tmp_out, query, key_cache, value_cache, num_kv_heads, scale,
                            block_tables, seq_lens, block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale,
                            v_scale)
