"""Open-loop load generator for the HTTP API: Poisson arrivals, streamed responses, latency percentiles.

Plays the role of the reference's ``load_tests/`` scripts.  Requests arrive at ``--rate`` per second
(exponential gaps, independent of completions), each asks for ``--output-len`` tokens with
``/generate_stream`` and ``ignore_eos``-like behaviour obtained by a large ``max_new_tokens`` budget on a
random prompt; for every request the time to first token, the inter-token gaps and the end-to-end time
are recorded.  Prints one JSON document per arrival rate:

    python -m tgi_b200.client.load_test --url http://127.0.0.1:3000 --rates 1,4,16 --requests 256 \
        --prompt-len 128:2048 --output-len 256
    python -m tgi_b200.client.load_test --url http://127.0.0.1:3000 --concurrency 1,8,32 --requests 64   # closed loop
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import string
import time
from typing import Dict, List, Tuple


def percentile(v: List[float], p: float) -> float:
    if not v:
        return float("nan")
    s = sorted(v)
    pos = p * (len(s) - 1)
    i = int(pos)
    frac = pos - i
    return s[i] * (1 - frac) + s[min(i + 1, len(s) - 1)] * frac


def summarize(v: List[float]) -> Dict[str, float]:
    return {"avg": sum(v) / len(v) if v else float("nan"), "p50": percentile(v, 0.5), "p90": percentile(v, 0.9),
            "p99": percentile(v, 0.99), "max": max(v) if v else float("nan")}


def random_prompt(rng: random.Random, n_chars: int) -> str:
    words = []
    size = 0
    while size < n_chars:
        w = "".join(rng.choice(string.ascii_lowercase) for _ in range(rng.randint(2, 9)))
        words.append(w)
        size += len(w) + 1
    return " ".join(words)[:n_chars]


async def one_request(session, url: str, prompt: str, max_new_tokens: int) -> Tuple[float, List[float], float, int, bool]:
    body = {"inputs": prompt, "parameters": {"max_new_tokens": max_new_tokens, "details": False}}
    t0 = time.perf_counter()
    stamps: List[float] = []
    ok = True
    try:
        async with session.post(url + "/generate_stream", json=body) as resp:
            if resp.status != 200:
                return float("nan"), [], time.perf_counter() - t0, 0, False
            async for raw in resp.content:
                line = raw.decode("utf-8", "replace").strip()
                if line.startswith("data:") and '"token"' in line:
                    stamps.append(time.perf_counter())
    except Exception:  # noqa: BLE001 - a failed request is counted, not fatal for the run
        ok = False
    end = time.perf_counter()
    if not stamps:
        return float("nan"), [], end - t0, 0, False
    gaps = [b - a for a, b in zip(stamps, stamps[1:])]
    return stamps[0] - t0, gaps, end - t0, len(stamps), ok


async def run_rate(url: str, rate: float, n_requests: int, prompt_chars: Tuple[int, int], output_len: int,
                   seed: int, max_connections: int) -> Dict:
    import aiohttp

    rng = random.Random(seed)
    conn = aiohttp.TCPConnector(limit=max_connections)
    timeout = aiohttp.ClientTimeout(total=None)
    async with aiohttp.ClientSession(connector=conn, timeout=timeout) as session:
        tasks = []
        start = time.perf_counter()
        for _ in range(n_requests):
            prompt = random_prompt(rng, rng.randint(*prompt_chars))
            tasks.append(asyncio.create_task(one_request(session, url, prompt, output_len)))
            await asyncio.sleep(rng.expovariate(rate))
        results = await asyncio.gather(*tasks)
        wall = time.perf_counter() - start
    ttft = [r[0] for r in results if r[4]]
    gaps = [g for r in results if r[4] for g in r[1]]
    e2e = [r[2] for r in results if r[4]]
    tokens = sum(r[3] for r in results)
    return {"rate_req_s": rate, "requests": n_requests, "failed": sum(1 for r in results if not r[4]),
            "wall_s": round(wall, 3), "output_tok_s": round(tokens / wall, 2),
            "ttft_ms": {k: round(v * 1e3, 2) for k, v in summarize(ttft).items()},
            "itl_ms": {k: round(v * 1e3, 2) for k, v in summarize(gaps).items()},
            "e2e_s": {k: round(v, 3) for k, v in summarize(e2e).items()}}


async def run_closed_loop(url: str, concurrency: int, n_requests: int, prompt_chars: Tuple[int, int], output_len: int,
                          seed: int) -> Dict:
    """``concurrency`` virtual users, each sending its next request as soon as the previous one finished (the
    constant-VU scenario of the reference's k6 scripts, ``load_tests/common.js``)."""
    import aiohttp

    rng = random.Random(seed)
    prompts = [random_prompt(rng, rng.randint(*prompt_chars)) for _ in range(n_requests)]
    results = []
    cursor = 0

    async def user(session):
        nonlocal cursor
        while cursor < len(prompts):
            i = cursor
            cursor += 1
            results.append(await one_request(session, url, prompts[i], output_len))

    conn = aiohttp.TCPConnector(limit=concurrency + 8)
    async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=None)) as session:
        start = time.perf_counter()
        await asyncio.gather(*[user(session) for _ in range(concurrency)])
        wall = time.perf_counter() - start
    ok = [r for r in results if r[4]]
    return {"concurrency": concurrency, "requests": n_requests, "failed": len(results) - len(ok),
            "wall_s": round(wall, 3), "output_tok_s": round(sum(r[3] for r in results) / wall, 2),
            "ttft_ms": {k: round(v * 1e3, 2) for k, v in summarize([r[0] for r in ok]).items()},
            "itl_ms": {k: round(v * 1e3, 2) for k, v in summarize([g for r in ok for g in r[1]]).items()},
            "e2e_s": {k: round(v, 3) for k, v in summarize([r[2] for r in ok]).items()}}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:3000")
    ap.add_argument("--rates", default="1,2,4,8,16,32,64", help="arrival rates to sweep, requests per second")
    ap.add_argument("--concurrency", default="", help="closed loop instead: numbers of concurrent users to sweep, e.g. 1,8,32")
    ap.add_argument("--requests", type=int, default=1024)
    ap.add_argument("--prompt-len", default="128:2048", help="min:max prompt length in characters")
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-connections", type=int, default=1024)
    args = ap.parse_args(argv)
    lo, _, hi = args.prompt_len.partition(":")
    chars = (int(lo), int(hi or lo))
    out = []
    for users in [int(x) for x in args.concurrency.split(",") if x]:
        res = asyncio.run(run_closed_loop(args.url.rstrip("/"), users, args.requests, chars, args.output_len, args.seed))
        print(json.dumps(res), flush=True)
        out.append(res)
    if args.concurrency:
        return out
    for rate in [float(x) for x in args.rates.split(",") if x]:
        res = asyncio.run(run_rate(args.url.rstrip("/"), rate, args.requests, chars, args.output_len, args.seed,
                                   args.max_connections))
        print(json.dumps(res), flush=True)
        out.append(res)
    return out


if __name__ == "__main__":
    main()
