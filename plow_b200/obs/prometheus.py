"""Prometheus text exposition with vLLM-compatible ``vllm:*`` families plus ``plowrt_*``
(reference: crates/plowrt/src/obs/serving.rs, docs/arch/18-serving-metrics.md:52-80)."""
from __future__ import annotations

_BUCKETS_MS = [1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000]


def _hist(name, values_ms, labels):
    out = [f"# TYPE {name} histogram"]
    acc = 0
    vs = sorted(values_ms)
    j = 0
    for b in _BUCKETS_MS:
        while j < len(vs) and vs[j] <= b:
            j += 1
        acc = j
        out.append(f'{name}_bucket{{{labels},le="{b / 1000.0}"}} {acc}')
    out.append(f'{name}_bucket{{{labels},le="+Inf"}} {len(vs)}')
    out.append(f"{name}_sum{{{labels}}} {sum(vs) / 1000.0}")
    out.append(f"{name}_count{{{labels}}} {len(vs)}")
    return out


def render(model: str, mux) -> str:
    m = mux.metrics
    with m.lock:
        c = dict(m.c)
        ttft, tpot, e2e, qt = list(m.ttft), list(m.tpot), list(m.e2e), list(m.queue_time)
    lab = f'model_name="{model}"'
    lines = [
        "# TYPE vllm:num_requests_running gauge", f"vllm:num_requests_running{{{lab}}} {len(mux.live)}",
        "# TYPE vllm:num_requests_waiting gauge", f"vllm:num_requests_waiting{{{lab}}} {len(mux.waiting) + mux.ingress.qsize()}",
        "# TYPE vllm:gpu_cache_usage_perc gauge",
        f"vllm:gpu_cache_usage_perc{{{lab}}} {1.0 - mux.engine.pool.available() / max(1, mux.engine.pool.n_pages)}",
        "# TYPE vllm:prompt_tokens_total counter", f"vllm:prompt_tokens_total{{{lab}}} {c['prompt_tokens']}",
        "# TYPE vllm:generation_tokens_total counter", f"vllm:generation_tokens_total{{{lab}}} {c['generation_tokens']}",
        "# TYPE vllm:request_success_total counter", f"vllm:request_success_total{{{lab}}} {c['requests_finished']}",
        "# TYPE vllm:num_preemptions_total counter", f"vllm:num_preemptions_total{{{lab}}} {c['preemptions']}",
        "# TYPE vllm:prefix_cache_hits_total counter", f"vllm:prefix_cache_hits_total{{{lab}}} {mux.engine.pool.stats['hits']}",
        "# TYPE vllm:prefix_cache_queries_total counter",
        f"vllm:prefix_cache_queries_total{{{lab}}} {mux.engine.pool.stats['hits'] + mux.engine.pool.stats['misses']}",
        "# TYPE plowrt_ticks_total counter", f"plowrt_ticks_total{{{lab}}} {c['ticks']}",
        "# TYPE plowrt_requests_shed_total counter", f"plowrt_requests_shed_total{{{lab}}} {c['requests_shed']}",
        "# TYPE plowrt_engine_health gauge", f'plowrt_engine_health{{{lab},state="{mux.engine.health}"}} 1',
    ]
    lines += _hist("vllm:time_to_first_token_seconds", ttft, lab)
    lines += _hist("vllm:time_per_output_token_seconds", tpot, lab)
    lines += _hist("vllm:e2e_request_latency_seconds", e2e, lab)
    lines += _hist("vllm:request_queue_time_seconds", qt, lab)
    return "\n".join(lines) + "\n"
