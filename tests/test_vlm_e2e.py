"""Vision-language request through the whole CPU stack: the C++ router splits the markdown image out
of `inputs`, decodes the data URI, accounts for the placeholder tokens and sends an image chunk; the
shard's vision-language runner encodes it.  Also the image helpers of the router in isolation."""
import base64
import io
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _png(seed, size=(40, 52)):
    from PIL import Image

    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 255, size=(size[0], size[1], 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"content-type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=120) as r:
            return r.status, dict(r.headers), r.read().decode()
    except urllib.error.HTTPError as e:
        return e.code, dict(e.headers), e.read().decode()


@pytest.fixture(scope="module")
def vlm_stack(tmp_path_factory):
    from tests.test_vlm import _hub_names
    from tgi_b200.router.build import build
    from tgi_b200.utils.weights import save_safetensors

    torch.manual_seed(0)
    vis = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                        image_size=28, patch_size=14)
    txt = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=300, max_position_embeddings=512,
                                   tie_word_embeddings=False)
    cfg = transformers.LlavaConfig(vision_config=vis, text_config=txt, image_token_index=299, vision_feature_layer=-2,
                                   vision_feature_select_strategy="default")
    hf = transformers.LlavaForConditionalGeneration(cfg).eval()
    d = tmp_path_factory.mktemp("llava_e2e")
    save_safetensors(_hub_names(hf.state_dict()), d / "model.safetensors", {"format": "pt"})
    c = cfg.to_dict()
    c["model_type"] = "llava_next"
    (d / "config.json").write_text(json.dumps(c))
    router_bin = build()
    uds = str(d / "shard")
    env = dict(os.environ, PYTHONPATH=ROOT, TGI_B200_CPU_KV_BLOCKS="256")
    shard = subprocess.Popen([sys.executable, "-m", "tgi_b200.server.cli", "serve", str(d), "--uds-path", uds,
                              "--dtype", "float32"], env=env, cwd=ROOT)
    port = _free_port()
    router = subprocess.Popen([str(router_bin), "--master-shard-uds-path", uds, "--tokenizer-name", str(d),
                               "--port", str(port), "--hostname", "127.0.0.1", "--max-input-tokens", "64",
                               "--max-total-tokens", "128", "--max-batch-prefill-tokens", "128", "--repo-root", ROOT],
                              env=env, cwd=ROOT)
    try:
        deadline = time.time() + 180
        while time.time() < deadline:
            if shard.poll() is not None or router.poll() is not None:
                raise RuntimeError("a process of the stack exited during start-up")
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.3)
        else:
            raise RuntimeError("router did not come up")
        yield port
    finally:
        for p in (router, shard):
            p.send_signal(signal.SIGTERM)
        for p in (router, shard):
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()


def test_image_request_end_to_end(vlm_stack):
    port = vlm_stack
    uri1 = "data:image/png;base64," + base64.b64encode(_png(1)).decode()
    uri2 = "data:image/png;base64," + base64.b64encode(_png(2)).decode()
    body = {"inputs": f"ab![]({uri1})cde", "parameters": {"max_new_tokens": 6, "details": True}}
    st, headers, out = _post(port, "/generate", body)
    assert st == 200, out
    # 2 + 3 text tokens (byte tokenizer, one special token) + 4 placeholder tokens of the 28x28 / patch-14 tower
    assert int(headers["x-prompt-tokens"]) in (9, 10)
    first = json.loads(out)
    st, _, again = _post(port, "/generate", body)            # second time: served through the prefix cache
    assert st == 200 and json.loads(again)["generated_text"] == first["generated_text"]
    st, _, other = _post(port, "/generate", {"inputs": f"ab![]({uri2})cde", "parameters": {"max_new_tokens": 6}})
    assert st == 200
    st, _, txt = _post(port, "/generate", {"inputs": "no image here", "parameters": {"max_new_tokens": 3}})
    assert st == 200
    st, _, bad = _post(port, "/generate", {"inputs": "x![](data:image/png;base64,AAAA)y", "parameters": {"max_new_tokens": 3}})
    assert st == 422 and "image" in bad
    st, _, bad2 = _post(port, "/generate", {"inputs": "x![](https://example.com/a.png)y", "parameters": {"max_new_tokens": 3}})
    assert st == 422 and "https" in bad2


import contextlib


@contextlib.contextmanager
def _serve(model_dir, max_input=200):
    """Shard + router for the model in ``model_dir``; yields the router's port."""
    from tgi_b200.router.build import build

    router_bin = build()
    uds = str(model_dir / "shard")
    env = dict(os.environ, PYTHONPATH=ROOT, TGI_B200_CPU_KV_BLOCKS="256")
    shard = subprocess.Popen([sys.executable, "-m", "tgi_b200.server.cli", "serve", str(model_dir), "--uds-path", uds,
                              "--dtype", "float32"], env=env, cwd=ROOT)
    port = _free_port()
    router = subprocess.Popen([str(router_bin), "--master-shard-uds-path", uds, "--tokenizer-name", str(model_dir),
                               "--port", str(port), "--hostname", "127.0.0.1", "--max-input-tokens", str(max_input),
                               "--max-total-tokens", str(max_input + 56), "--max-batch-prefill-tokens", str(max_input + 56),
                               "--repo-root", ROOT], env=env, cwd=ROOT)
    try:
        deadline = time.time() + 180
        while time.time() < deadline:
            assert shard.poll() is None and router.poll() is None, "a process of the stack exited during start-up"
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.3)
        else:
            raise RuntimeError("router did not come up")
        yield port
    finally:
        for p in (router, shard):
            p.send_signal(signal.SIGTERM)
        for p in (router, shard):
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()


def test_idefics3_split_image_end_to_end(tmp_path):
    """Router and shard agree on the prompt length of a split image: the router counts the tiles, the marker tokens
    and the newlines from the image's size, the shard builds that layout (x-prompt-tokens is the router's count; the
    shard would run out of the blocks the router allotted if it needed more)."""
    from tests.test_vlm_idefics import TXT, VIS, _marker_tokenizer
    from tgi_b200.models.idefics3 import expansion_length, tile_grid

    torch.manual_seed(0)
    ids_of = _marker_tokenizer(tmp_path)
    cfg = transformers.Idefics3Config(vision_config=VIS, text_config=dict(TXT, model_type="llama"),
                                      image_token_id=ids_of["<image>"], scale_factor=2)
    transformers.Idefics3ForConditionalGeneration(cfg).eval().save_pretrained(str(tmp_path), safe_serialization=True)
    c = json.loads((tmp_path / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp_path / "config.json").write_text(json.dumps(c))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps(
        {"size": {"longest_edge": 84}, "max_image_size": {"longest_edge": 28}, "do_image_splitting": True}))
    with _serve(tmp_path) as port:
        for size in [(40, 52), (30, 90), (28, 28)]:                      # (height, width)
            uri = "data:image/png;base64," + base64.b64encode(_png(3, size)).decode()
            st, headers, out = _post(port, "/generate", {"inputs": f"ab![]({uri})cde",
                                                         "parameters": {"max_new_tokens": 4, "details": True}})
            assert st == 200, out
            _, _, rows, cols = tile_grid(size[0], size[1], 84, 28)
            want = 5 + expansion_length(rows, cols, 4, 1, 2)             # character tokenizer: "\n" 1 token, "\n\n" 2
            assert int(headers["x-prompt-tokens"]) == want, (size, rows, cols, headers["x-prompt-tokens"], want)
            assert json.loads(out)["details"]["generated_tokens"] == 4


def test_idefics2_markers_and_adjacent_images_end_to_end(tmp_path):
    """Idefics2 with image splitting: five views per image between markers, and two images in a row share one marker;
    the router's prompt length is the shard's."""
    from tests.test_vlm_idefics import TXT, VIS, _marker_tokenizer

    torch.manual_seed(0)
    ids_of = _marker_tokenizer(tmp_path)
    cfg = transformers.Idefics2Config(
        vision_config=VIS, text_config=dict(TXT, model_type="mistral", sliding_window=None),
        image_token_id=ids_of["<image>"],
        perceiver_config=dict(resampler_n_latents=4, resampler_depth=2, resampler_n_heads=2, resampler_head_dim=16,
                              num_key_value_heads=1, hidden_act="silu", hidden_size=64, rms_norm_eps=1e-6))
    transformers.Idefics2ForConditionalGeneration(cfg).eval().save_pretrained(str(tmp_path), safe_serialization=True)
    c = json.loads((tmp_path / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp_path / "config.json").write_text(json.dumps(c))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"do_image_splitting": True}))
    with _serve(tmp_path) as port:
        uri1 = "data:image/png;base64," + base64.b64encode(_png(1)).decode()
        uri2 = "data:image/png;base64," + base64.b64encode(_png(2)).decode()
        one = 5 * (4 + 1) + 1
        st, headers, out = _post(port, "/generate", {"inputs": f"ab![]({uri1})c", "parameters": {"max_new_tokens": 3}})
        assert st == 200 and int(headers["x-prompt-tokens"]) == 3 + one, (out, dict(headers))
        st, headers, out = _post(port, "/generate", {"inputs": f"ab![]({uri1})![]({uri2})c",
                                                     "parameters": {"max_new_tokens": 3}})
        assert st == 200 and int(headers["x-prompt-tokens"]) == 3 + 2 * one - 1, (out, dict(headers))
