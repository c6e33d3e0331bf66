"""Import stand-in: the reference uses `init_empty_weights` only as a context that skips parameter
allocation while it builds norm modules (`layers/layernorm.py:11-34`); the meta device does the same."""
import contextlib

import torch


@contextlib.contextmanager
def init_empty_weights(include_buffers: bool = False):
    with torch.device("meta"):
        yield
