"""Serving benchmark over HTTP: aggregate tokens per second, time to first token and inter-token
latency of a running server at 1, 2, 4, 8 ... concurrent clients.

    python -m benchmarks.serving_concurrency --url http://127.0.0.1:8080 --clients 1,2,4,8 \\
        --prompt-tokens 512 --max-tokens 128 [--api-key K] [--rounds 2]

Every client streams one chat completion per round (``ignore_eos`` so that all of them emit
``max_tokens`` tokens); the clients of a level start together. Per level one JSON line:
aggregate tok/s (the server's completion-token counts, or content events when it sends none, / wall time of the level), mean and p95 TTFT, p50 and p95
inter-token latency. This is the measurement behind the reference's batched-serving table
(docs/CONTINUOUS_BATCHING.md:240-245 there): the same numbers for this server.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import statistics
import time


def _pct(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    s = sorted(xs)
    return s[min(len(s) - 1, int(round(q * (len(s) - 1))))]


async def _one(http, url: str, prompt: str, max_tokens: int) -> dict:
    """One streamed chat completion read off the wire: a time stamp per content event (an event may
    carry no text when the new bytes do not end a character) and the server's own token count."""
    body = dict(messages=[{"role": "user", "content": prompt}], max_tokens=max_tokens, temperature=0, ignore_eos=True,
                stream=True, stream_options={"include_usage": True})
    t0 = time.perf_counter()
    stamps, usage = [], None
    async with http.post(url + "/v1/chat/completions", json=body) as r:
        if r.status >= 400:
            raise RuntimeError(f"HTTP {r.status}: {(await r.text())[:300]}")
        async for raw in r.content:
            line = raw.decode().strip()
            if not line.startswith("data:") or line[5:].strip() == "[DONE]":
                continue
            ev = json.loads(line[5:])
            if ev.get("usage"):
                usage = ev["usage"].get("completion_tokens")
            if any("delta" in ch and ch.get("finish_reason") is None for ch in ev.get("choices") or []):
                stamps.append(time.perf_counter())
    tokens = usage if usage is not None else len(stamps)
    return dict(tokens=tokens, ttft=(stamps[0] - t0) if stamps else None, itl=[b - a for a, b in zip(stamps, stamps[1:])])


async def run_level(url: str, api_key: str | None, clients: int, prompt: str, max_tokens: int, rounds: int) -> dict:
    import aiohttp

    res, wall = [], 0.0
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    async with aiohttp.ClientSession(headers=headers, timeout=aiohttp.ClientTimeout(total=None)) as http:
        for r in range(rounds):
            t0 = time.perf_counter()
            # a different head per client and round keeps the prompt cache from answering the prefill
            got = await asyncio.gather(*(_one(http, url, f"[{r}:{i}] {prompt}", max_tokens) for i in range(clients)))
            wall += time.perf_counter() - t0
            res += got
    tokens = sum(g["tokens"] for g in res)
    ttft = [g["ttft"] for g in res if g["ttft"] is not None]
    itl = [x for g in res for x in g["itl"]]
    return dict(clients=clients, requests=len(res), output_tokens=tokens, wall_s=round(wall, 3),
                tok_per_s=round(tokens / wall, 2) if wall > 0 else None,
                ttft_mean_ms=round(1e3 * statistics.fmean(ttft), 2) if ttft else None,
                ttft_p95_ms=round(1e3 * _pct(ttft, 0.95), 2) if ttft else None,
                itl_p50_ms=round(1e3 * _pct(itl, 0.5), 3) if itl else None,
                itl_p95_ms=round(1e3 * _pct(itl, 0.95), 3) if itl else None)


def main(argv=None) -> list[dict]:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--url", required=True)
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--clients", default="1,2,4,8")
    ap.add_argument("--prompt-tokens", type=int, default=512, help="approximate prompt length (words of filler text)")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--rounds", type=int, default=2)
    a = ap.parse_args(argv)
    prompt = " ".join(f"w{i % 97}" for i in range(max(1, a.prompt_tokens)))
    out = []
    for n in (int(x) for x in a.clients.split(",") if x):
        row = asyncio.run(run_level(a.url, a.api_key, n, prompt, a.max_tokens, a.rounds))
        print(json.dumps(row), flush=True)
        out.append(row)
    return out


if __name__ == "__main__":
    main()
