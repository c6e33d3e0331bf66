"""Launcher on CPU: spawns a shard and the router, serves requests, shuts down cleanly on SIGTERM,
and tears the deployment down (non-zero exit) when a shard process dies: failure detection on the host."""
import json
import os
import signal
import socket
import subprocess
import time
import urllib.request

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _start(tmp_path, extra=()):
    from tgi_b200.router.build import HERE, build
    from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint

    build()
    d = tmp_path / "model"
    write_llama_checkpoint(d, llama_config(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=128, vocab=300, max_pos=512))
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, TGI_B200_CPU_KV_BLOCKS="256", CUDA_VISIBLE_DEVICES="")
    cmd = [str(HERE / "tgi-b200-launcher"), "--model-id", str(d), "--num-shard", "1", "--port", str(port),
           "--hostname", "127.0.0.1", "--shard-uds-path", str(tmp_path / "shard"), "--dtype", "float32",
           "--max-input-tokens", "64", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "128",
           "--master-port", str(_free_port()), *extra]
    log = open(tmp_path / "launcher.log", "w")
    proc = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    deadline = time.time() + 180
    while time.time() < deadline and proc.poll() is None:
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5) as r:
                if r.status == 200:
                    return proc, port, log
        except Exception:
            time.sleep(0.5)
    try:
        os.killpg(proc.pid, signal.SIGKILL)
    except ProcessLookupError:
        pass
    raise AssertionError("launcher did not come up:\n" + open(tmp_path / "launcher.log").read()[-4000:])


def _children(pid):
    out = subprocess.run(["ps", "-o", "pid=,args=", "--ppid", str(pid)], capture_output=True, text=True).stdout
    return [(int(l.split(None, 1)[0]), l.split(None, 1)[1]) for l in out.strip().splitlines() if l.strip()]


def test_launcher_serves_and_stops_cleanly(tmp_path):
    proc, port, log = _start(tmp_path)
    try:
        req = urllib.request.Request(f"http://127.0.0.1:{port}/generate",
                                     data=json.dumps({"inputs": "hello", "parameters": {"max_new_tokens": 4}}).encode(),
                                     headers={"content-type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            assert r.status == 200 and "generated_text" in json.loads(r.read().decode())
        os.kill(proc.pid, signal.SIGTERM)
        assert proc.wait(timeout=60) == 0
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()


def test_launcher_downloads_first_reemits_shard_logs_and_serves_metrics_on_its_own_port(tmp_path):
    prom = _free_port()
    proc, port, log = _start(tmp_path, extra=("--json-output", "--prometheus-port", str(prom),
                                              "--cors-allow-origin", "https://a.example", "--usage-stats", "off"))
    try:
        with urllib.request.urlopen(f"http://127.0.0.1:{prom}/metrics", timeout=10) as r:
            assert r.status == 200 and "tgi_queue_size" in r.read().decode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/info", headers={"origin": "https://a.example"})
        with urllib.request.urlopen(req, timeout=10) as r:
            assert r.headers.get("access-control-allow-origin") == "https://a.example"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/info", headers={"origin": "https://b.example"})
        with urllib.request.urlopen(req, timeout=10) as r:
            assert r.headers.get("access-control-allow-origin") is None
        os.kill(proc.pid, signal.SIGTERM)
        assert proc.wait(timeout=60) == 0
        records = []
        for line in open(tmp_path / "launcher.log").read().splitlines():
            if line.startswith("{"):
                records.append(json.loads(line))
        targets = [r["target"] for r in records]
        # the weight check ran (and finished) before the shard was started
        msgs = [r["message"] for r in records if r["target"] == "launcher"]
        assert any("download" in m.lower() for m in msgs)
        first_shard = next(i for i, r in enumerate(records) if r["target"] == "launcher" and "Starting shard-0" in r["message"])
        done = next(i for i, r in enumerate(records) if r["target"] == "launcher" and "Successfully downloaded" in r["message"])
        assert done < first_shard
        # the shard's own JSON records come back under its name, at their level
        shard_records = [r for r in records if r["target"] == "shard-0"]
        assert shard_records and all(r["level"] in ("DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL") for r in shard_records)
        assert any("Server started" in r["message"] for r in shard_records)
        assert "router" in targets
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()


def test_launcher_exits_when_a_shard_dies(tmp_path):
    proc, port, log = _start(tmp_path)
    try:
        shard = [pid for pid, args in _children(proc.pid) if "tgi_b200.server.cli" in args]
        assert shard, _children(proc.pid)
        os.kill(shard[0], signal.SIGKILL)          # the failure is injected on the host: the shard process vanishes
        rc = proc.wait(timeout=60)
        assert rc != 0
        assert "shard" in open(tmp_path / "launcher.log").read().lower()
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()
