"""Prometheus text exposition: the ``llamacpp:*`` families llama-server clients scrape, then
``mlxcel_*`` engine gauges (reference: src/server/routes/metrics.rs:15-120)."""
from __future__ import annotations


def render_metrics(state) -> str:
    w = state.worker
    c, e = w.counters, w.view()
    bm = e.bm.stats()
    lines = []

    def m(name, kind, help_, value):
        lines.append(f"# HELP {name} {help_}")
        lines.append(f"# TYPE {name} {kind}")
        lines.append(f"{name} {value}")

    m("llamacpp:prompt_tokens_total", "counter", "Number of prompt tokens processed.", c["prompt_tokens"])
    m("llamacpp:tokens_predicted_total", "counter", "Number of generation tokens processed.", c["generated_tokens"])
    m("llamacpp:prompt_seconds_total", "counter", "Prompt process time", round(c["prompt_seconds"], 6))
    m("llamacpp:tokens_predicted_seconds_total", "counter", "Predict process time", round(c["decode_seconds"], 6))
    m("llamacpp:prompt_tokens_seconds", "gauge", "Average prompt throughput in tokens/s.",
      round(c["prompt_tokens"] / c["prompt_seconds"], 3) if c["prompt_seconds"] else 0)
    m("llamacpp:predicted_tokens_seconds", "gauge", "Average generation throughput in tokens/s.",
      round(c["generated_tokens"] / c["decode_seconds"], 3) if c["decode_seconds"] else 0)
    m("llamacpp:requests_processing", "gauge", "Number of requests processing.", len(e.running))
    m("llamacpp:requests_deferred", "gauge", "Number of requests deferred.", len(e.waiting))
    m("llamacpp:n_decode_total", "counter", "Total number of decode steps.", e.stats["steps"])
    m("llamacpp:prompt_tokens_cached_total", "counter", "Prompt tokens served from the prefix cache.",
      e.stats["prefix_hit_tokens"])
    m("mlxcel_model_sleeping", "gauge", "1 while the idle model is unloaded.", int(getattr(w, "sleeping", False)))
    m("mlxcel_requests_total", "counter", "Requests admitted.", c["requests"])
    m("mlxcel_request_errors_total", "counter", "Requests that ended in an error.", c["errors"])
    m("mlxcel_requests_cancelled_total", "counter", "Requests cancelled by the client.", c["cancelled"])
    m("mlxcel_kv_blocks_total", "gauge", "KV pool size in blocks.", bm["num_blocks"])
    m("mlxcel_kv_blocks_free", "gauge", "Free KV blocks.", bm["free"])
    m("mlxcel_kv_blocks_cached", "gauge", "Unreferenced blocks kept for prefix reuse.", bm["cached"])
    m("mlxcel_prompt_cache_hit_blocks_total", "counter", "Prefix blocks adopted.", bm["prefix_hits"])
    m("mlxcel_prompt_cache_evictions_total", "counter", "Cached blocks evicted.", bm["evictions"])
    m("mlxcel_preemptions_total", "counter", "Rows preempted under block pressure.", e.stats["preemptions"])
    m("mlxcel_cuda_graph_replays_total", "counter", "Decode steps served by CUDA graph replay.", e.stats["graph_replays"])
    m("mlxcel_batch_decode_tokens_total", "counter", "Tokens produced by decode rows.", e.stats["decode_tokens"])
    m("mlxcel_batch_prefill_tokens_total", "counter", "Prompt tokens run through prefill.", e.stats["prefill_tokens"])
    m("mlxcel_spec_decode_rounds_total", "counter", "Speculative verify rounds.", e.stats.get("spec_rounds", 0))
    m("mlxcel_spec_decode_drafted_total", "counter", "Draft tokens proposed.", e.stats.get("spec_drafted", 0))
    m("mlxcel_spec_decode_accepted_total", "counter", "Draft tokens accepted.", e.stats.get("spec_accepted", 0))
    m("mlxcel_thinking_forced_total", "counter", "End-of-thinking tokens forced by a thinking budget.",
      e.stats.get("thinking_forced", 0))
    m("mlxcel_step_hangs_total", "counter", "Engine steps that exceeded the hang timeout.", c.get("hangs", 0))
    rs = getattr(getattr(state, "responses", None), "stats", None)
    if rs:
        m("mlxcel_responses_store_entries", "gauge", "Stored Responses API objects.", len(state.responses))
        m("mlxcel_responses_store_expired_total", "counter", "Stored responses dropped by TTL.", rs["expired"])
    hist = getattr(state, "hist", None)
    if hist:
        lines += hist["ttft"].render("mlxcel_request_ttft_seconds", "Time to first token per request.")
        lines += hist["decode_tps"].render("mlxcel_request_decode_tokens_per_second", "Decode throughput per request.")
    return "\n".join(lines) + "\n"
