"""Classic against speculative decoding on one engine configuration: tokens per second of the same
greedy requests without a drafter and with one (prompt lookup, a draft model directory, an MTP or
block-drafter directory), the acceptance rate, and a check that both runs emitted the same tokens.

    python -m benchmarks.speculative_compare -m <model dir | preset:name> [--draft-model DIR | --prompt-lookup]
        [--draft-max 4] [--requests 4] [--prompt-tokens 256] [--max-tokens 128] [--device cuda]

One JSON line. On a GPU the timed region is bracketed by ``torch.cuda.synchronize``; the first run of
each arm is a warm-up. (The reference's counterpart: scripts/bench_speculative*.sh and the MTP tables
of docs/CONTINUOUS_BATCHING.md.)
"""
from __future__ import annotations

import argparse
import json
import time


def _run(llm, prompts, sp, sync) -> tuple[list[list[int]], float]:
    llm.generate(prompt_token_ids=prompts[:1], sampling_params=sp)          # warm-up (graphs, caches)
    sync()
    t0 = time.perf_counter()
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=sp)
    sync()
    return [o.output for o in outs], time.perf_counter() - t0


def main(argv=None) -> dict:
    import torch

    from mlxcel_b200 import cli
    from mlxcel_b200.engine import SamplingParams

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    cli._add_model_args(ap)
    ap.add_argument("--requests", type=int, default=4)
    ap.add_argument("--prompt-tokens", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=128)
    a = ap.parse_args(argv)
    if not (a.draft_model or a.prompt_lookup):
        raise SystemExit("give --draft-model DIR or --prompt-lookup")
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    sync = torch.cuda.synchronize if dev.startswith("cuda") else (lambda: None)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=0.0, ignore_eos=True)
    res = {}
    draft, lookup = a.draft_model, a.prompt_lookup
    for arm in ("classic", "speculative"):
        a.draft_model, a.prompt_lookup = (draft, lookup) if arm == "speculative" else (None, False)
        llm = cli.load_llm(a)
        if arm == "classic":
            vocab = llm.cfg.vocab_size
            prompts = torch.randint(0, vocab, (a.requests, a.prompt_tokens), generator=g).tolist()
        outs, secs = _run(llm, prompts, sp, sync)
        st = llm.engine.stats
        res[arm] = dict(outs=outs, tok_s=round(sum(len(o) for o in outs) / secs, 2), seconds=round(secs, 3),
                        drafted=st.get("spec_drafted", 0), accepted=st.get("spec_accepted", 0), rounds=st.get("spec_rounds", 0))
        del llm
    c, s = res["classic"], res["speculative"]
    row = dict(model=a.model, drafter=draft or "prompt-lookup", requests=a.requests, prompt_tokens=a.prompt_tokens,
               max_tokens=a.max_tokens, classic_tok_s=c["tok_s"], speculative_tok_s=s["tok_s"],
               speedup=round(s["tok_s"] / c["tok_s"], 3) if c["tok_s"] else None,
               acceptance=round(s["accepted"] / s["drafted"], 4) if s["drafted"] else None, verify_rounds=s["rounds"],
               same_tokens=c["outs"] == s["outs"])
    print(json.dumps(row), flush=True)
    return row


if __name__ == "__main__":
    main()
