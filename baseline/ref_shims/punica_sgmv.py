"""Import stand-in for the multi-LoRA SGMV/BGMV kernels (hub: kernels-community/punica-sgmv): the
benchmark serves no adapter, so only the names and the two limits the reference reads at import
have to exist."""
MIN_SGMV_RANK = 8
MIN_RANK_CUSTOM = 16
MAX_RANK_CUSTOM = 128
SGMV_BLOCK_SIZE = 16
BGMV_MAX_RANK = 64


def _absent(name):
    def f(*a, **k):
        raise NotImplementedError(f"punica_sgmv.{name}: multi-LoRA kernels are not installed")

    return f


for _n in ("lora_a_sgmv_cutlass", "lora_b_sgmv_cutlass", "add_lora_a_bgmv", "add_lora_b_bgmv", "get_tmp_tensors",
           "get_tmp_tensor_for_size", "get_tmp_expand_size", "orient_for_rank", "has_sgmv", "use_cutlass_shrink",
           "pad_rank", "segmented_matmul"):
    globals()[_n] = _absent(_n)
