"""Serving benchmark client: open-loop (Poisson) or closed-loop load against the OpenAI-compatible endpoint, with
client-side TTFT / TPOT / end-to-end latency percentiles and output tokens per second.

    python -m plow_b200.serve.bench_api --url http://127.0.0.1:8000 --model NAME --rate 4 --num-prompts 64 \
        --input-len 32768:131072 --output-len 1024 --shared-prefix 0.25:16384

Prompts are random token ids sent through /v1/completions (token-id prompts, streaming).  ``--shared-prefix F:N`` makes
a fraction F of the prompts start with the same N tokens (exercises the prefix cache).  ``--rate 0`` sends with a fixed
concurrency instead (closed loop).  Reference: tools/bench-api/{bench.py,corpus.py}, scripts/bench/serving_comparison.py."""
from __future__ import annotations

import argparse
import asyncio
import json
import time

import numpy as np


def _pct(a, q):
    return round(float(np.percentile(a, q)), 2) if len(a) else None


def make_prompts(n, vocab, in_lo, in_hi, shared_frac, shared_len, seed=0):
    rng = np.random.default_rng(seed)
    prefix = rng.integers(3, vocab, size=shared_len).tolist() if shared_len else []
    out = []
    for i in range(n):
        ln = int(rng.integers(in_lo, in_hi + 1))
        if prefix and rng.random() < shared_frac and ln > shared_len:
            out.append(prefix + rng.integers(3, vocab, size=ln - shared_len).tolist())
        else:
            out.append(rng.integers(3, vocab, size=ln).tolist())
    return out


async def _one(session, url, model, prompt, max_tokens, api_key, rec):
    hdr = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    body = dict(model=model, prompt=prompt, max_tokens=max_tokens, stream=True, temperature=0, ignore_eos=True)
    t0 = time.perf_counter()
    first = last = None
    n = 0
    try:
        async with session.post(url + "/v1/completions", json=body, headers=hdr) as resp:
            if resp.status != 200:
                rec.append(dict(ok=False, status=resp.status))
                return
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                payload = line[5:].strip()
                if payload == "[DONE]":
                    break
                ev = json.loads(payload)
                if "error" in ev:
                    rec.append(dict(ok=False, status=500))
                    return
                ch = ev["choices"][0] if ev.get("choices") else None
                if ch is not None and ch.get("finish_reason") is None:
                    now = time.perf_counter()
                    first = first or now
                    last = now
                    n += 1
    except Exception as e:                                   # connection errors count as failures, the run goes on
        rec.append(dict(ok=False, status=str(type(e).__name__)))
        return
    t1 = time.perf_counter()
    rec.append(dict(ok=True, ttft_ms=(first - t0) * 1e3 if first else None, n_out=n, e2e_ms=(t1 - t0) * 1e3,
                    tpot_ms=((last - first) * 1e3 / (n - 1)) if n > 1 else None, prompt_tokens=len(prompt)))


async def run(url, model, prompts, max_tokens, rate=0.0, concurrency=8, api_key=None, seed=0) -> dict:
    import aiohttp
    rec = []
    rng = np.random.default_rng(seed)
    t_start = time.perf_counter()
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
        if rate > 0:                                         # open loop: exponential inter-arrival times
            tasks = []
            for p in prompts:
                tasks.append(asyncio.create_task(_one(session, url, model, p, max_tokens, api_key, rec)))
                await asyncio.sleep(float(rng.exponential(1.0 / rate)))
            await asyncio.gather(*tasks)
        else:
            sem = asyncio.Semaphore(concurrency)

            async def guarded(p):
                async with sem:
                    await _one(session, url, model, p, max_tokens, api_key, rec)
            await asyncio.gather(*(guarded(p) for p in prompts))
    wall = time.perf_counter() - t_start
    ok = [r for r in rec if r["ok"]]
    ttft = [r["ttft_ms"] for r in ok if r["ttft_ms"] is not None]
    tpot = [r["tpot_ms"] for r in ok if r["tpot_ms"] is not None]
    e2e = [r["e2e_ms"] for r in ok]
    n_out = sum(r["n_out"] for r in ok)
    return dict(requests=len(rec), failed=len(rec) - len(ok), wall_s=round(wall, 3), rate_rps=rate, concurrency=(None if rate > 0 else concurrency),
                output_tok_s=round(n_out / wall, 1), total_tok_s=round((n_out + sum(r["prompt_tokens"] for r in ok)) / wall, 1),
                ttft_ms=dict(p50=_pct(ttft, 50), p99=_pct(ttft, 99)), tpot_ms=dict(p50=_pct(tpot, 50), p99=_pct(tpot, 99)),
                e2e_ms=dict(p50=_pct(e2e, 50), p99=_pct(e2e, 99)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--num-prompts", type=int, default=32)
    ap.add_argument("--input-len", default="128", help="N or LO:HI (uniform)")
    ap.add_argument("--output-len", type=int, default=64)
    ap.add_argument("--rate", type=float, default=0.0, help="Poisson arrival rate in req/s; 0 = closed loop")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--shared-prefix", default="", help="FRACTION:TOKENS")
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--api-key")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    lo, _, hi = a.input_len.partition(":")
    frac, _, plen = a.shared_prefix.partition(":")
    prompts = make_prompts(a.num_prompts, a.vocab, int(lo), int(hi or lo), float(frac or 0), int(plen or 0), a.seed)
    print(json.dumps(asyncio.run(run(a.url, a.model, prompts, a.output_len, a.rate, a.concurrency, a.api_key, a.seed))))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
