"""``mlxcel`` command line (python -m mlxcel_b200.cli ...).

Subcommands follow the reference's CLI (src/main.rs:97-378): ``generate``, ``run`` (chat REPL),
``serve``, ``inspect`` (memory estimate), ``arch``, ``list``, ``tokenize``, ``embed``, ``bench``,
``tune``, ``random-init`` (writes a random checkpoint of a preset architecture) and ``split-mtp``.
Flag names keep llama-server compatibility where one exists (``-m``, ``-c``, ``-n``, ``--parallel``,
``--temp``, ``--top-k``, ``--top-p``, ``--min-p``, ``--seed``, ``--host``, ``--port``, ``--api-key``,
``--kv-bits``, ``--prefill-chunk-size``, ``--tp``, ``--pp``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _add_model_args(p):
    p.add_argument("-m", "--model", required=True, help="checkpoint directory or preset:<name>")
    p.add_argument("--device", default=None)
    p.add_argument("-c", "--ctx-size", type=int, default=8192)
    p.add_argument("--parallel", "-np", type=int, default=4, help="concurrent sequences (slots)")
    p.add_argument("--max-batch-tokens", type=int, default=8192)
    p.add_argument("--prefill-chunk-size", type=int, default=2048)
    p.add_argument("--kv-bits", type=int, default=0, choices=[0, 4, 8, 16])
    p.add_argument("--kv-cache-blocks", type=int, default=0)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--max-kv-size", type=int, default=0,
                   help="KV window bound of one sequence in tokens (0 = the context size): a sequence that reaches it "
                        "ends with finish reason 'length', or keeps going under --context-shift")
    p.add_argument("--context-shift", dest="context_shift", action="store_true", default=False,
                   help="at the KV bound drop the oldest blocks behind the first --keep tokens and go on generating")
    p.add_argument("--no-context-shift", dest="context_shift", action="store_false")
    p.add_argument("--mla-latent-cache", dest="mla_latent_cache", action="store_true", default=False,
                   help="multi-head latent attention models: cache one [latent | rotary key] entry per token "
                        "(absorbed attention) instead of per-head keys and values")
    p.add_argument("--keep", type=int, default=0, help="tokens at the start of a sequence that context shifting never drops")
    p.add_argument("--no-prompt-cache", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--no-warmup", action="store_true", help="serve: skip the one-token request made before listening")
    p.add_argument("--dequantize", action="store_true", help="dequantize quantized checkpoints at load")
    p.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (launch with torch.distributed.run)")
    p.add_argument("--pp", type=int, default=1, help="pipeline stages; world size = tp * pp")
    p.add_argument("--ep-mode", choices=["replicated", "a2a"], default="replicated",
                   help="mixture-of-experts models on several processes: 'replicated' shards experts under --tp (tokens on "
                        "every rank, all-reduce combine); 'a2a' makes every process a server of its own requests (port + "
                        "rank) whose MoE layers exchange rows with the others (put `front` before them)")
    p.add_argument("--pp-layers", default=None, help="comma-separated layer counts per stage (default: equal split)")
    p.add_argument("--pp-micro-batches", type=int, default=2, help="micro-batches a step is cut into")
    p.add_argument("--draft-model", default=None)
    p.add_argument("--draft-max", type=int, default=4)
    p.add_argument("--prompt-lookup", action="store_true")
    p.add_argument("--rope-freq-base", type=float, default=None, help="RoPE base frequency (overrides the checkpoint)")
    p.add_argument("--rope-scaling", choices=["none", "linear", "yarn"], default=None)
    p.add_argument("--rope-scale", type=float, default=None, help="context scaling factor of --rope-scaling")
    p.add_argument("--yarn-orig-ctx", type=int, default=None, help="original context length of the YaRN scaling")
    p.add_argument("--override-kv", action="append", default=None, metavar="KEY=JSON",
                   help="replace a config.json key before the model is built (repeatable)")
    _add_compat_args(p)


_COMPAT_NOOPS = [("-ngl", "--n-gpu-layers", "--gpu-layers"), ("-t", "--threads"), ("-tb", "--threads-batch"),
                 ("-to", "--timeout"), ("--cache-reuse",), ("--defrag-thold",), ("-sm", "--split-mode"), ("-mg", "--main-gpu"),
                 ("--numa",), ("--poll",), ("--threads-http",)]
_COMPAT_NOOP_SWITCHES = [("--mlock",), ("--no-mmap",), ("-fa", "--flash-attn"), ("-cb", "--cont-batching"),
                         ("-nocb", "--no-cont-batching"), ("--jinja",), ("--metrics",), ("--slots",),
                         ("--no-slots",), ("--no-webui",), ("--no-kv-offload",),
                         ("--embeddings", "--embedding"), ("--reranking", "--rerank"), ("--props",), ("--log-disable",)]


def _add_compat_args(p):
    """llama-server spellings (reference src/cli/*_compat.rs, compat/llama-server manifest). Flags with a
    counterpart here are mapped onto it by :func:`_apply_compat`; flags about CPU threads, mmap, GPU layer
    offload and the like have no meaning on this runtime and are accepted so that existing launch scripts
    keep working (a note on stderr names the ones that were given)."""
    g = p.add_argument_group("llama-server compatible spellings")
    g.add_argument("-md", "--model-draft", dest="compat_model_draft", default=None, help="same as --draft-model")
    g.add_argument("--draft", "--draft-n", dest="compat_draft_n", type=int, default=None, help="same as --draft-max")
    g.add_argument("-b", "--batch-size", dest="compat_batch", type=int, default=None, help="same as --max-batch-tokens")
    g.add_argument("-ub", "--ubatch-size", dest="compat_ubatch", type=int, default=None,
                   help="same as --prefill-chunk-size")
    g.add_argument("-ctk", "--cache-type-k", dest="compat_ctk", default=None, help="f16 | bf16 | q8_0: q8_0 means --kv-bits 8")
    g.add_argument("-ctv", "--cache-type-v", dest="compat_ctv", default=None, help="f16 | bf16 | q8_0: q8_0 means --kv-bits 8")
    g.add_argument("--no-cache-prompt", dest="compat_no_cache_prompt", action="store_true", help="same as --no-prompt-cache")
    g.add_argument("--lookup-ngram-min", dest="compat_lookup", type=int, default=None, help="turns --prompt-lookup on")
    for names in _COMPAT_NOOPS:
        g.add_argument(*names, dest="compat_noop_" + names[-1].strip("-").replace("-", "_"), default=None, help="accepted, no effect")
    for names in _COMPAT_NOOP_SWITCHES:
        g.add_argument(*names, dest="compat_noop_" + names[-1].strip("-").replace("-", "_"), action="store_const", const=True,
                       default=None, help="accepted, no effect")


def _apply_compat(a) -> list[str]:
    """Fold the llama-server spellings into the native options; returns the no-effect flags that were given."""
    if getattr(a, "compat_model_draft", None) and not getattr(a, "draft_model", None):
        a.draft_model = a.compat_model_draft
    if getattr(a, "compat_draft_n", None) is not None:
        a.draft_max = a.compat_draft_n
    if getattr(a, "compat_batch", None) is not None:
        a.max_batch_tokens = a.compat_batch
    if getattr(a, "compat_ubatch", None) is not None:
        a.prefill_chunk_size = a.compat_ubatch
    types = [t for t in (getattr(a, "compat_ctk", None), getattr(a, "compat_ctv", None)) if t]
    for t in types:
        if t.lower() not in ("f16", "bf16", "f32", "q8_0", "int8", "fp8", "q4_0", "q4_1"):
            raise SystemExit(f"cache type {t!r} is not supported (f16, bf16, q8_0, q4_0)")
    if any(t.lower() in ("q8_0", "int8", "fp8") for t in types) and not getattr(a, "kv_bits", 0):
        a.kv_bits = 8
    if any(t.lower() in ("q4_0", "q4_1") for t in types) and not getattr(a, "kv_bits", 0):
        a.kv_bits = 4
    if getattr(a, "compat_no_cache_prompt", False):
        a.no_prompt_cache = True
    if getattr(a, "compat_lookup", None) is not None:
        a.prompt_lookup = True
    return sorted("--" + k[len("compat_noop_"):].replace("_", "-") for k, v in vars(a).items()
                  if k.startswith("compat_noop_") and v is not None)


# llama-server's environment spellings (reference docs/environment-variables.md:36-60): value of the
# variable -> default of the option; precedence stays command line > environment > built-in default.
LLAMA_ARG_ENV = {
    "LLAMA_ARG_MODEL": ("model", str), "LLAMA_ARG_CTX_SIZE": ("ctx_size", int), "LLAMA_ARG_N_PARALLEL": ("parallel", int),
    "LLAMA_ARG_BATCH": ("max_batch_tokens", int), "LLAMA_ARG_UBATCH": ("prefill_chunk_size", int),
    "LLAMA_ARG_HOST": ("host", str), "LLAMA_ARG_PORT": ("port", int), "LLAMA_ARG_ALIAS": ("alias", str),
    "LLAMA_ARG_N_PREDICT": ("max_tokens", int), "LLAMA_ARG_MODEL_DRAFT": ("draft_model", str),
    "LLAMA_ARG_DRAFT_MAX": ("draft_max", int), "LLAMA_ARG_CHAT_TEMPLATE_FILE": ("chat_template_file", str),
    "LLAMA_ARG_THINK_BUDGET": ("reasoning_budget", int), "LLAMA_ARG_REASONING_BUDGET": ("reasoning_budget", int),
    "LLAMA_ARG_SLOT_SAVE_PATH": ("slot_save_path", str), "LLAMA_ARG_API_KEY_FILE": ("api_key_file", str),
    "LLAMA_ARG_NO_WARMUP": ("no_warmup", "flag"), "LLAMA_ARG_TEMP": ("temperature", float),
    "LLAMA_ARG_TOP_K": ("top_k", int), "LLAMA_ARG_TOP_P": ("top_p", float), "LLAMA_ARG_SEED": ("seed", int),
}


def _apply_env_aliases(subparsers) -> None:
    """Every sub-command that has the option takes the variable's value as that option's default
    (and ``-m`` stops being required when LLAMA_ARG_MODEL names the model)."""
    for name, (dest, kind) in LLAMA_ARG_ENV.items():
        raw = os.environ.get(name)
        if raw is None or raw == "":
            continue
        try:
            val = (raw.lower() not in ("0", "false", "no", "off")) if kind == "flag" else kind(raw)
        except ValueError:
            raise SystemExit(f"{name}={raw!r}: expected {kind.__name__}")
        for parser in subparsers.choices.values():
            for act in parser._actions:
                if act.dest == dest:
                    act.default = val
                    if dest == "model":
                        act.required = False
    key = os.environ.get("LLAMA_ARG_API_KEY") or os.environ.get("LLAMA_API_KEY")
    if key:
        for parser in subparsers.choices.values():
            for act in parser._actions:
                if act.dest == "api_key" and not act.default:
                    act.default = [key]


def _add_sampling_args(p):
    p.add_argument("-n", "--n-predict", "--max-tokens", dest="max_tokens", type=int, default=256)
    p.add_argument("--temp", "--temperature", dest="temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--typical-p", type=float, default=1.0)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("--repeat-last-n", type=int, default=64)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--frequency-penalty", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--ignore-eos", action="store_true")


def _sampling(a):
    from .engine import SamplingParams
    return SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                          min_p=a.min_p, typical_p=a.typical_p, repetition_penalty=a.repeat_penalty,
                          repetition_context_size=a.repeat_last_n, presence_penalty=a.presence_penalty,
                          frequency_penalty=a.frequency_penalty, seed=a.seed, ignore_eos=a.ignore_eos)


def load_llm(a):
    import torch

    if getattr(a, "debug_trace", None):
        from .utils.tracing import TRACER
        TRACER.enable(path=a.debug_trace)

    from .engine import EngineConfig
    from .llm import LLM

    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    # several processes (torch.distributed.run): pick this rank's GPU and join the job
    from .parallel.control import init_distributed
    world = int(os.environ.get("WORLD_SIZE", "1"))
    tp, pp = max(1, int(getattr(a, "tp", 1))), max(1, int(getattr(a, "pp", 1)))
    if tp * pp > 1 and world != tp * pp:
        raise SystemExit(f"--tp {tp} --pp {pp} needs {tp * pp} processes: launch with "
                         f"`python -m torch.distributed.run --nproc-per-node {tp * pp} -m mlxcel_b200.cli ...`")
    a._control_group = None
    dp_ep = getattr(a, "ep_mode", "replicated") == "a2a"
    if dp_ep and world > 1:
        # data-parallel attention + expert-parallel MoE: every rank is a server of its own (own listener,
        # own requests), the ranks only share the routed experts
        dev, _ = init_distributed(dev)
        return _load_dp_ep(a, dev, ecfg_args=None)
    if world > 1 and tp * pp == 1:
        raise SystemExit(f"{world} processes were launched but neither --tp nor --pp was given")
    if world > 1:
        dev, a._control_group = init_distributed(dev)
    ecfg = EngineConfig(max_batch=a.parallel, max_num_batched_tokens=a.max_batch_tokens,
                        prefill_chunk_alone=a.prefill_chunk_size, prefill_chunk_contended=min(512, a.prefill_chunk_size),
                        block_size=a.block_size, kv_bits=a.kv_bits or 16, num_blocks=a.kv_cache_blocks,
                        prefix_cache=not a.no_prompt_cache, max_model_len=a.ctx_size,
                        max_kv_size=getattr(a, "max_kv_size", 0), context_shift=getattr(a, "context_shift", False),
                        mla_latent_cache=getattr(a, "mla_latent_cache", False),
                        n_keep=getattr(a, "keep", 0) or 0,
                        cuda_graphs=not a.no_cuda_graphs and dev != "cpu")
    comm = None
    if pp > 1:
        return _load_pipeline(a, dev, ecfg, tp, pp)
    if tp > 1:
        import torch.distributed as dist

        from .parallel.tp import TPComm
        on_gpu = str(dev).startswith("cuda")
        comm = TPComm(dist.group.WORLD, torch.device(dev), backend="fused" if on_gpu else "nccl")
    if a.model.startswith("preset:"):
        dtype = torch.bfloat16 if dev != "cpu" else torch.float32
        llm = LLM.from_preset(a.model.split(":", 1)[1], device=dev, engine_config=ecfg, comm=comm, dtype=dtype)
        from .tokenizer import ByteTokenizer
        llm.tokenizer = ByteTokenizer(llm.cfg.vocab_size)
    else:
        llm = LLM.from_pretrained(a.model, device=dev, engine_config=ecfg, comm=comm, dequantize=a.dequantize,
                                  surgery=getattr(a, "surgery", None), config_overrides=config_overrides(a))
    attach_drafter(llm, a, dev)
    if llm.engine.drafter is not None:
        from .speculative import SpecPolicy
        eng = llm.engine
        key = f"{a.model}|{type(eng.drafter).__name__}|K{eng.spec_k}|{dev}"
        eng.spec_policy = SpecPolicy(key=key)
    return llm


def _load_dp_ep(a, dev, ecfg_args=None):
    """One rank of ``serve --ep-mode a2a`` under ``torch.distributed.run``: a complete engine for this
    rank's own requests whose MoE layers exchange rows with the other ranks (parallel/dp_ep.py)."""
    import torch
    import torch.distributed as dist

    from .config import ModelConfig, preset
    from .engine import EngineConfig
    from .llm import LLM
    from .loading.checkpoint import _to_device, load_full_weights
    from .loading.shard import shard_weights
    from .parallel.dp_ep import DpEpComm
    rank, world = dist.get_rank(), dist.get_world_size()
    is_preset = a.model.startswith("preset:")
    cfg = preset(a.model.split(":", 1)[1]) if is_preset else ModelConfig.from_path(a.model, config_overrides(a))
    if not cfg.is_moe:
        raise SystemExit("--ep-mode a2a needs a mixture-of-experts model")
    ecfg = EngineConfig(max_batch=a.parallel, max_num_batched_tokens=a.max_batch_tokens,
                        prefill_chunk_alone=a.prefill_chunk_size, prefill_chunk_contended=min(512, a.prefill_chunk_size),
                        block_size=a.block_size, kv_bits=a.kv_bits or 16, num_blocks=a.kv_cache_blocks,
                        prefix_cache=not a.no_prompt_cache, max_model_len=a.ctx_size, cuda_graphs=False)
    comm = DpEpComm(dist.group.WORLD, dev, hidden=cfg.hidden_size, top_k=cfg.num_experts_per_tok,
                    num_experts=cfg.num_experts, max_tokens=a.max_batch_tokens)
    if is_preset:
        from .models.weights import random_weights
        from .tokenizer import ByteTokenizer
        dtype = torch.bfloat16 if str(dev) != "cpu" else torch.float32
        full = random_weights(cfg, seed=0, dtype=dtype)          # the same weights on every rank, then sharded
        w = _to_device(shard_weights(cfg, full, 0, 1, ep=world, ep_rank=rank, vocab_parallel=False), dev)
        llm = LLM(cfg, w, ecfg, comm=comm, tokenizer=ByteTokenizer(cfg.vocab_size))
    else:
        from .tokenizer import load_tokenizer
        full = load_full_weights(a.model, cfg, dequantize=a.dequantize, surgery=getattr(a, "surgery", None))
        w = _to_device(shard_weights(cfg, full, 0, 1, ep=world, ep_rank=rank, vocab_parallel=False), dev)
        llm = LLM(cfg, w, ecfg, comm=comm, tokenizer=load_tokenizer(a.model))
    a.port = a.port + rank                      # one listener per rank; `front` balances over them
    return llm


def _load_pipeline(a, dev, ecfg, tp: int, pp: int):
    """``--pp P`` (optionally with ``--tp T``): rank = stage * T + tp_rank; every stage holds a contiguous
    layer range (``--pp-layers`` or an equal split), tensor-parallel inside the stage over its own
    process group, activations between stages over send / recv (reference
    src/distributed/pipeline/runtime.rs:100-199, partition*.rs)."""
    import torch
    import torch.distributed as dist

    from .config import ModelConfig, preset
    from .llm import LLM
    from .loading.shard import partition_layers
    from .models.weights import random_weights
    from .parallel.pp import PipelineContext, PipelineModel
    from .parallel.tp import TPComm

    rank = dist.get_rank()
    stage, tp_rank = rank // tp, rank % tp
    tp_group = None
    for st in range(pp):                              # every rank creates every group, in the same order
        grp = dist.new_group(list(range(st * tp, (st + 1) * tp)))
        if st == stage:
            tp_group = grp
    on_gpu = str(dev).startswith("cuda")
    comm = TPComm(tp_group, torch.device(dev), backend="fused" if on_gpu else "nccl") if tp > 1 else None
    is_preset = a.model.startswith("preset:")
    cfg = preset(a.model.split(":", 1)[1]) if is_preset else ModelConfig.from_path(a.model, config_overrides(a))
    if getattr(a, "pp_layers", None):
        counts = [int(x) for x in str(a.pp_layers).split(",")]
        if len(counts) != pp or sum(counts) != cfg.num_hidden_layers or min(counts) < 1:
            raise SystemExit(f"--pp-layers {a.pp_layers}: expected {pp} positive counts summing to {cfg.num_hidden_layers}")
        ranges, lo = [], 0
        for c in counts:
            ranges.append(range(lo, lo + c))
            lo += c
    else:
        ranges = partition_layers(cfg.num_hidden_layers, pp)
    if is_preset:
        dtype = torch.bfloat16 if on_gpu else torch.float32
        w = random_weights(cfg, seed=0, dtype=dtype, device=dev, tp_rank=tp_rank, tp_size=tp, ep_rank=tp_rank,
                           ep_size=tp, layers=ranges[stage], vocab_parallel=tp > 1 and cfg.vocab_size % tp == 0)
        from .tokenizer import ByteTokenizer
        tok = ByteTokenizer(cfg.vocab_size)
    else:
        from .loading.checkpoint import load_model_weights
        from .tokenizer import load_tokenizer
        w = load_model_weights(a.model, cfg, device=dev, comm=comm, dequantize=a.dequantize, layers=ranges[stage],
                               surgery=getattr(a, "surgery", None), dtype=torch.bfloat16 if on_gpu else torch.float32)
        tok = load_tokenizer(a.model)
    ctx = PipelineContext(dist.group.WORLD, stage, pp, tp_size=tp, tp_rank=tp_rank)
    model = PipelineModel(cfg, w, ctx, comm=comm, num_micro=max(1, int(getattr(a, "pp_micro_batches", 2))),
                          layer_range=ranges[stage], kv_bits=ecfg.kv_bits)
    if getattr(a, "draft_model", None) or getattr(a, "prompt_lookup", False):
        raise SystemExit("speculative decoding is not available with --pp (the drafter needs the last stage's state)")
    return LLM(cfg, w, ecfg, comm=comm, tokenizer=tok, model=model)


def config_overrides(a) -> dict | None:
    """``--rope-freq-base``, ``--rope-scaling`` / ``--rope-scale`` / ``--yarn-orig-ctx`` and ``--override-kv`` as
    config.json replacements (reference src/cli/rope.rs)."""
    ov: dict = {}
    if getattr(a, "rope_freq_base", None):
        ov["rope_theta"] = float(a.rope_freq_base)
    kind = getattr(a, "rope_scaling", None)
    if kind == "none":
        ov["rope_scaling"] = None
    elif kind or getattr(a, "rope_scale", None):
        sc = dict(rope_type=kind or "linear", factor=float(getattr(a, "rope_scale", None) or 1.0))
        if getattr(a, "yarn_orig_ctx", None):
            sc["original_max_position_embeddings"] = int(a.yarn_orig_ctx)
        ov["rope_scaling"] = sc
    for item in getattr(a, "override_kv", None) or []:
        k, sep, v = item.partition("=")
        if not sep:
            raise SystemExit(f"--override-kv {item!r}: expected KEY=JSON")
        try:
            ov[k] = json.loads(v)
        except ValueError:
            ov[k] = v
    return ov or None


def attach_drafter(llm, a, dev) -> None:
    """``--draft-model`` (a smaller model of the same vocabulary, or a drafter directory written by
    ``split-mtp``) and ``--prompt-lookup`` put a speculative drafter on the engine; ``--draft-max`` is the
    number of draft tokens per verify round (reference src/commands/generate.rs draft routing)."""
    import os

    import torch

    draft, lookup = getattr(a, "draft_model", None), getattr(a, "prompt_lookup", False)
    if not draft and not lookup:
        return
    eng = llm.engine
    if getattr(eng.model, "recurrent", False):
        raise SystemExit("speculative decoding needs a KV-cache model (recurrent state cannot be rolled back)")
    eng.spec_k = max(1, int(getattr(a, "draft_max", 4))) + 1
    if not draft:
        from .speculative import PromptLookupDrafter
        nmin = getattr(a, "compat_lookup", None)
        eng.drafter = PromptLookupDrafter(min_ngram=max(1, int(nmin))) if nmin else PromptLookupDrafter()
        if nmin and eng.drafter.max_ngram < eng.drafter.min_ngram:
            eng.drafter.max_ngram = eng.drafter.min_ngram
        return
    from .loading.split_mtp import MARKER
    dtype = eng.model.w.final_norm.dtype
    nb = max(256, eng.ecfg.max_batch * ((eng.ecfg.max_model_len + eng.ecfg.block_size - 1) // eng.ecfg.block_size))
    if os.path.exists(os.path.join(draft, MARKER)):
        from .loading.split_mtp import load_mtp_weights
        from .speculative import MTPDrafter
        dcfg, w, _ = load_mtp_weights(draft, dtype=dtype, device=dev)
        if dcfg.hidden_size != llm.cfg.hidden_size or dcfg.vocab_size != llm.cfg.vocab_size:
            raise SystemExit(f"{draft}: the MTP drafter was split from a different model")
        eng.drafter = MTPDrafter(eng.model, dcfg, w, num_blocks=nb, block_size=eng.ecfg.block_size)
        return
    from .speculative.dflash import is_dflash_dir
    if is_dflash_dir(draft):
        # a block drafter that conditions on the target's hidden states (one forward per block)
        from .speculative.dflash import DFlashDrafter, load_dflash
        dcfg, w, info = load_dflash(draft, dtype=dtype, device=dev)
        if dcfg.hidden_size != llm.cfg.hidden_size or dcfg.vocab_size != llm.cfg.vocab_size:
            raise SystemExit(f"{draft}: the block drafter was trained for a different target")
        if not hasattr(eng.model, "capture_layers") or max(info["target_layers"]) >= llm.cfg.num_hidden_layers:
            raise SystemExit(f"{draft}: the block drafter needs the decoder executor's hidden states of layers {info['target_layers']}")
        block = min(info["block"], eng.spec_k_max)
        eng.drafter = DFlashDrafter(eng.model, dcfg, w, info["target_layers"], info["mask_token_id"], num_blocks=nb,
                                    block=block, block_size=eng.ecfg.block_size)
        eng.spec_k = block
        return
    from .config import ModelConfig
    from .loading.checkpoint import load_model_weights
    from .models.decoder import DecoderModel
    from .speculative import DraftModelDrafter
    dcfg = ModelConfig.from_path(draft)
    if dcfg.vocab_size != llm.cfg.vocab_size:
        raise SystemExit(f"{draft}: vocabulary size {dcfg.vocab_size} differs from the target's {llm.cfg.vocab_size}")
    dw = load_model_weights(draft, dcfg, device=dev, dtype=dtype if dev == "cpu" else torch.bfloat16)
    eng.drafter = DraftModelDrafter(DecoderModel(dcfg, dw), dcfg, num_blocks=nb, block_size=eng.ecfg.block_size,
                                    max_model_len=eng.ecfg.max_model_len)


def _generate_diffusion(a, llm, tk, prompt: str) -> None:
    """``generate --diffusion``: block-unmasking decoding of a masked-diffusion checkpoint (engine/diffusion.py)."""
    from .engine.diffusion import DiffusionGenerator, DiffusionOptions
    mask_id = a.mask_token_id
    if mask_id is None:
        mask_id = (getattr(tk, "special", None) or {}).get("<|mask|>", llm.cfg.extra.get("mask_token_id"))
    if mask_id is None:
        raise SystemExit("--diffusion needs --mask-token-id (the tokenizer names no <|mask|> token)")
    if a.chat:
        from .server.chat_template import render_chat
        prompt = render_chat([{"role": "user", "content": prompt}], getattr(tk, "chat_template", None))
    ids = tk.encode(prompt, add_special_tokens=not a.chat)
    sp = _sampling(a)
    gen = DiffusionGenerator(llm.model, llm.cfg, mask_id, max_len=min(a.ctx_size, len(ids) + sp.max_tokens + 2 * a.block_length))
    t0 = time.perf_counter()

    def show(block):
        sys.stdout.write(tk.decode(block))
        sys.stdout.flush()
    out = gen.generate(ids, DiffusionOptions(max_new_tokens=sp.max_tokens, block_length=a.block_length, steps=a.diffusion_steps,
                                             threshold=a.diffusion_threshold, min_threshold=a.diffusion_threshold,
                                             temperature=sp.temperature, eos_token_ids=[i for i in tk.eos_ids() if i is not None],
                                             seed=sp.seed or 0), on_block=show)
    dt = time.perf_counter() - t0
    print(f"\n[{len(out)} tokens in {gen.stats['blocks']} blocks, {gen.stats['forwards']} forward passes, "
          f"{len(out) / max(dt, 1e-9):.1f} tok/s]", file=sys.stderr)


def cmd_generate(a):
    llm = load_llm(a)
    tk = llm.tokenizer
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    if getattr(a, "diffusion", False):
        return _generate_diffusion(a, llm, tk, prompt)
    mm = {}
    if getattr(a, "audio", None):
        front = getattr(llm, "vision", None)
        if getattr(front, "modality", None) != "audio":
            raise SystemExit("--audio needs a speech-language checkpoint (voxtral, qwen2_audio)")
        if getattr(a, "image", None):
            raise SystemExit("--audio and --image do not combine")
        if prompt.count(front.placeholder_text) == 0:
            prompt = front.placeholder_text * len(a.audio) + "\n" + prompt
    if getattr(a, "image", None):
        vision = getattr(llm, "vision", None)
        if vision is None or getattr(vision, "modality", "image") != "image":
            raise SystemExit("--image needs a vision-language checkpoint")
        if prompt.count(vision.placeholder_text) == 0:       # images first, then the text (the usual layout)
            prompt = vision.placeholder_text * len(a.image) + "\n" + prompt
    if a.chat:
        from .server.chat_template import render_chat
        prompt = render_chat([{"role": "user", "content": prompt}], getattr(tk, "chat_template", None))
    ids = tk.encode(prompt, add_special_tokens=not a.chat)
    if getattr(a, "image", None):
        from .multimodal import load_image
        ids, mm = llm.vision.prepare(ids, [load_image(x) for x in a.image])
    if getattr(a, "audio", None):
        from pathlib import Path as _P

        from .audio.wav import decode_audio
        ids, mm = llm.vision.prepare(ids, [decode_audio(_P(x).read_bytes(), 16000) for x in a.audio])
    sp = _sampling(a)
    sp.stop_token_ids = [i for i in tk.eos_ids() if i is not None]
    from .tokenizer import IncrementalDetokenizer
    det = IncrementalDetokenizer(tk, ids)
    t0 = time.perf_counter()

    lead = int(os.environ.get("RANK", "0")) == 0      # several ranks run the same request in lockstep; one prints

    def on_token(seq, tok):
        piece = det.push(tok)
        if lead:
            sys.stdout.write(piece)
            sys.stdout.flush()

    mask_fn = None
    grammar = open(a.grammar_file).read() if getattr(a, "grammar_file", None) else getattr(a, "grammar", None)
    schema = open(a.json_schema_file).read() if getattr(a, "json_schema_file", None) else getattr(a, "json_schema", None)
    if grammar or schema or getattr(a, "regex", None):   # reference src/cli/grammar.rs: --grammar / --json-schema
        from .server.structured import constraint_from_request
        try:
            con = constraint_from_request(tk, grammar=grammar, json_schema=json.loads(schema) if schema else None,
                                          regex=getattr(a, "regex", None))
        except ValueError as ex:
            raise SystemExit(f"structured output: {ex}")
        mask_fn = con.mask
    sid = llm.engine.add_request(ids, sp, on_token=on_token, mask_fn=mask_fn, **mm)
    while llm.engine.has_work():
        llm.engine.step()
    s = llm.engine.seqs[sid]
    if not lead:
        _leave_distributed()
        return
    sys.stdout.write(det.flush() + "\n")
    dt = time.perf_counter() - t0
    ttft = (s.first_token_time - s.arrival) if s.first_token_time else 0.0
    n = len(s.output)
    print(f"[prompt {len(ids)} tok, {len(ids) / max(ttft, 1e-9):.1f} tok/s | generated {n} tok, "
          f"{max(n - 1, 0) / max(dt - ttft, 1e-9):.1f} tok/s | finish: {s.finish_reason.value}]", file=sys.stderr)
    st = llm.engine.stats
    if llm.engine.drafter is not None:
        print(f"[speculative: {st['spec_rounds']} verify rounds, {st['spec_accepted']} of {st['spec_drafted']} drafts "
              f"accepted]", file=sys.stderr)
    _leave_distributed()


def _leave_distributed() -> None:
    """End of a multi-process command: meet the other ranks once more, then leave without tearing
    the communicator down under live symmetric-memory mappings (seen to block for minutes)."""
    if int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


REPL_HELP = """Available commands:
  /bye, /exit    Exit the chat.
  /clear         Reset the conversation (clears all prior turns).
  /system TEXT   Replace the system prompt (clears the conversation).
  /stats         Engine counters of this session.
  /?, /help      Show this help.
  \"\"\" ... \"\"\"    Wrap multiline input as one message."""


def repl_turns(lines, system: str | None = None):
    """The chat REPL's input grammar as a generator over input lines: yields ``("send", messages)`` for
    every user message (the caller appends the assistant reply to ``messages``), ``("print", text)`` for
    command output, and stops on /bye, /exit, an empty line or end of input. Slash commands and the
    triple-quote multiline fence follow the reference's REPL (src/commands/chat.rs:449-500)."""
    msgs = [{"role": "system", "content": system}] if system else []
    it = iter(lines)
    for line in it:
        text = line.rstrip("\n")
        if text.strip().startswith('"""'):
            body = [text.strip()[3:]]
            while not body[-1].rstrip().endswith('"""'):
                nxt = next(it, None)
                if nxt is None:
                    break
                body.append(nxt.rstrip("\n"))
            text = "\n".join(body).rstrip()
            text = text[:-3] if text.endswith('"""') else text
            text = text.strip()
            if not text:
                continue
        elif not text.strip():
            return
        elif text.startswith("/"):
            cmd, _, rest = text.strip().partition(" ")
            if cmd in ("/bye", "/exit"):
                return
            if cmd == "/clear":
                del msgs[1 if msgs and msgs[0]["role"] == "system" else 0:]
                yield "print", "Conversation cleared."
            elif cmd == "/system":
                msgs[:] = [{"role": "system", "content": rest.strip()}] if rest.strip() else []
                yield "print", "System prompt set; conversation cleared."
            elif cmd == "/stats":
                yield "stats", None
            elif cmd in ("/?", "/help"):
                yield "print", REPL_HELP
            else:
                yield "print", f"Unknown command: {cmd}. Type /? for the list of commands."
            continue
        msgs.append({"role": "user", "content": text.strip()})
        yield "send", msgs


def cmd_run(a):
    llm = load_llm(a)
    tk = llm.tokenizer
    from .server.chat_template import render_chat
    from .tokenizer import IncrementalDetokenizer
    print("chat REPL: empty line or /bye to quit, /? for commands", file=sys.stderr)

    def lines():
        while True:
            try:
                yield input("> ")
            except EOFError:
                return

    for kind, payload in repl_turns(lines(), a.system):
        if kind == "print":
            print(payload)
            continue
        if kind == "stats":
            st = llm.engine.stats
            print(", ".join(f"{k}={st[k]}" for k in sorted(st) if isinstance(st[k], (int, float)) and st[k]))
            continue
        msgs = payload
        ids = tk.encode(render_chat(msgs, getattr(tk, "chat_template", None)))
        sp = _sampling(a)
        sp.stop_token_ids = [i for i in tk.eos_ids() if i is not None]
        det = IncrementalDetokenizer(tk, ids)
        parts = []

        def on_token(seq, tok):
            t = det.push(tok)
            parts.append(t)
            sys.stdout.write(t)
            sys.stdout.flush()

        llm.engine.add_request(ids, sp, on_token=on_token)
        while llm.engine.has_work():
            llm.engine.step()
        tail = det.flush()
        parts.append(tail)
        print(tail)
        msgs.append({"role": "assistant", "content": "".join(parts)})


def _encoder_checkpoint(path: str) -> bool:
    cj = os.path.join(path, "config.json")
    return os.path.exists(cj) and json.load(open(cj)).get("model_type") in ("bert", "modernbert", "deberta-v2")


def cmd_embed(a):
    """Offline counterpart of ``/v1/embeddings``: one vector per ``-p`` input, and the cosine matrix when
    there are several (reference src/main.rs:251, ``mlxcel embed``)."""
    import torch

    texts = list(a.prompt or [])
    if not texts:
        raise SystemExit("embed: give at least one -p/--prompt")
    if a.instruction:
        texts = [f"Instruct: {a.instruction}\nQuery: {t}" for t in texts]
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if _encoder_checkpoint(a.model):
        from .models.encoder import load_encoder
        from .tokenizer import load_tokenizer
        enc, tok = load_encoder(a.model, device=dev), load_tokenizer(a.model)
        vecs = [enc.embed(tok.encode(t, add_special_tokens=True) or [0], a.pooling or enc.default_pooling, False)
                for t in texts]
        if a.embd_normalize == "auto":
            a.embd_normalize = "l2" if enc.default_normalize else "none"
    else:
        from types import SimpleNamespace

        from .server.embeddings import embed_texts
        llm = load_llm(a)
        state = SimpleNamespace(worker=SimpleNamespace(engine=llm.engine), tokenizer=llm.tokenizer)
        vecs = [torch.tensor(v) for v in embed_texts(state, texts, a.pooling or "last")[0]]
    vecs = torch.stack([v.float().cpu() for v in vecs])
    if a.dimensions:
        vecs = vecs[:, : a.dimensions]
    if a.embd_normalize in ("l2", "auto"):
        vecs = vecs / vecs.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    unit = vecs / vecs.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    sim = (unit @ unit.T).tolist() if len(texts) > 1 else None
    if a.json:
        print(json.dumps(dict(embeddings=vecs.tolist(), cosine=sim)))
        return
    for t, v in zip(texts, vecs.tolist()):
        head = ", ".join(f"{x:+.4f}" for x in v[:8])
        print(f"{t!r}: dim={len(v)} [{head}{', ...' if len(v) > 8 else ''}]")
    if sim:
        print("cosine similarity:")
        for row in sim:
            print("  " + " ".join(f"{x:6.3f}" for x in row))


def _load_encoder_and_tokenizer(a):
    import torch

    from .models.encoder import load_encoder
    from .tokenizer import load_tokenizer
    if not _encoder_checkpoint(a.model):
        raise SystemExit(f"{a.model}: not an encoder checkpoint (bert, modernbert)")
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    return load_encoder(a.model, device=dev), load_tokenizer(a.model)


def cmd_rerank(a):
    """Offline counterpart of ``/v1/rerank`` (reference src/main.rs:281, ``mlxcel rerank``)."""
    if _encoder_checkpoint(a.model):
        from .server.embeddings import rerank_scores
        enc, tok = _load_encoder_and_tokenizer(a)
        scores = rerank_scores(enc, tok, a.query, a.document)
    else:                                          # a decoder LM: the generative yes/no reranker
        from argparse import Namespace

        from .engine.scoring import generative_rerank
        ap = argparse.ArgumentParser()
        _add_model_args(ap)
        full = ap.parse_args(["-m", a.model] + (["--device", a.device] if a.device else []))
        llm = load_llm(Namespace(**vars(full)))
        scores = generative_rerank(llm.model, llm.cfg, llm.tokenizer, a.query, a.document, a.instruction,
                                   llm.engine.ecfg.block_size, llm.engine.ecfg.max_model_len - 1)
    order = sorted(range(len(scores)), key=lambda i: -scores[i])
    if a.json:
        print(json.dumps(dict(results=[dict(index=i, relevance_score=scores[i]) for i in order])))
        return
    for rank, i in enumerate(order, 1):
        print(f"{rank:2d}. [{i}] {scores[i]:.4f}  {a.document[i][:80]}")


def cmd_tag(a):
    """Entity spans and a redacted copy from a token-classification checkpoint (reference
    src/main.rs:298, ``mlxcel tag``)."""
    from .server.embeddings import tag_text
    enc, tok = _load_encoder_and_tokenizer(a)
    keep = {k.strip() for k in (a.keep or "").split(",") if k.strip()}
    res = tag_text(enc, tok, a.text, keep, a.replacement, a.argmax)
    if a.json:
        print(json.dumps(res))
        return
    for sp in res["spans"]:
        print(f"{sp['entity']:<16} {sp['score']:.3f}  {sp['text']!r}")
    print(res["redacted"])


def cmd_list(a):
    """Models of the local store (reference src/main.rs:161, ``mlxcel list``)."""
    from . import store
    models = store.list_models(a.models_dir, a.sort)
    if a.json:
        print(json.dumps(store.as_json(models)))
    elif a.quiet:
        for m in models:
            print(m.repo_id)
    elif not models:
        print(f"no models under {store.store_root(a.models_dir)}")
    else:
        print(store.format_table(models, a.verbose))


def cmd_rm(a):
    """Remove one model of the local store (reference src/main.rs:328, ``mlxcel rm``)."""
    from . import store
    target = store.model_path(a.repo_id, a.models_dir)
    if not a.yes:
        if input(f"remove {target}? [y/N] ").strip().lower() not in ("y", "yes"):
            print("kept")
            return
    try:
        freed = store.remove_model(a.repo_id, a.models_dir)
    except (FileNotFoundError, ValueError) as ex:
        raise SystemExit(str(ex))
    print(f"removed {a.repo_id} ({store.human_size(freed)} freed)")


def cmd_download(a):
    """Bring a repository into the local store, reusing a HuggingFace cache copy (reference
    src/main.rs:199, ``mlxcel download``)."""
    from . import store
    try:
        print(store.download_model(a.repo_id, a.models_dir, a.local_dir))
    except (RuntimeError, ValueError) as ex:
        raise SystemExit(str(ex))


def cmd_tune(a):
    """Profile the launch knobs of the hot kernels and cache the winners (reference src/main.rs:348,
    ``mlxcel tune``)."""
    from . import autotune as at
    names = a.op or list(at.OPS)
    bad = [n for n in names if n not in at.OPS]
    if bad:
        raise SystemExit(f"unknown op {bad[0]!r}; known: {', '.join(at.OPS)}")
    geo = at.Geometry()
    if a.model:
        from .config import ModelConfig, preset
        cfg = preset(a.model.split(":", 1)[1]) if a.model.startswith("preset:") else ModelConfig.from_path(a.model)
        geo = at.Geometry.from_config(cfg)
    if a.dry_run:
        rows = [r for n in names for r in at.OPS[n].matrix()]
        if a.json:
            print(json.dumps(dict(geometry=geo.key(), matrix=rows)))
        else:
            print(f"geometry {geo.key()}")
            for r in rows:
                print(f"  {r['op']:<26} {r['env']}={r['value']}{'  (default)' if r['default'] else ''}")
        return
    store = at.TacticStore(a.cache_file)
    results = at.tune(names, geo, store, log=None if a.json else print)
    if a.json:
        print(json.dumps([r.__dict__ for r in results]))
        return
    for r in results:
        print(f"{r.op}: {'kept default (' + r.skipped + ')' if r.skipped else f'{at.OPS[r.op].env}={r.value} ({r.us:.1f} us)'}")
    print(f"wrote {store.path}; set {at.SWITCH}=cache to use it")


def cmd_split_mtp(a):
    """Write the MTP layers of a raw checkpoint as a drafter checkpoint (reference src/main.rs:362,
    ``mlxcel split-mtp``)."""
    from .loading.split_mtp import split_mtp_dir
    try:
        res = split_mtp_dir(a.model, a.output, a.block_size, a.q_bits, a.q_group_size, a.force)
    except ValueError as ex:
        raise SystemExit(str(ex))
    print(json.dumps(res) if a.json else
          f"wrote {a.output}: {res['layers']} MTP layer(s) from model.layers.{res['source_layer']}, {res['tensors']} tensors, "
          f"{res['bytes'] / 1e6:.1f} MB, block size {res['block_size']}; pass it as --draft-model")


def cmd_perplexity(a):
    """Windowed perplexity of a text file (reference examples/perplexity.rs)."""
    from .engine.scoring import perplexity
    llm = load_llm(a)
    text = open(a.file, encoding="utf-8").read() if a.file else sys.stdin.read()
    ids = llm.tokenizer.encode(text, add_special_tokens=True)
    if len(ids) < 2:
        raise SystemExit("perplexity: the text has fewer than two tokens")
    window = min(a.window, a.ctx_size)
    res = perplexity(llm.model, llm.cfg, ids, window, a.stride, llm.engine.ecfg.block_size,
                     progress=None if a.json else (lambda d, t: print(f"\r{d}/{t} tokens", end="", file=sys.stderr)))
    if a.json:
        print(json.dumps(res))
    else:
        print(f"\nperplexity {res['perplexity']:.4f} over {res['tokens']} tokens (window {res['window']}, stride {res['stride']})")


def cmd_serve(a):
    import uvicorn

    from .server.app import ServerState, create_app
    from .server.worker import ModelWorker
    from .audio.transcribe import is_whisper_checkpoint as _is_whisper
    if not _encoder_checkpoint(a.model) and not _is_whisper(a.model):        # preflight: does model + KV pool + activations fit (src/commands/serve.rs)
        from .config import ModelConfig, preset
        from .utils.memory import estimate_memory
        cfg = (preset(a.model.split(":", 1)[1]) if a.model.startswith("preset:")
               else ModelConfig.from_path(a.model, config_overrides(a)))
        est = estimate_memory(cfg, ctx=a.ctx_size, parallel=a.parallel, kv_bits=a.kv_bits or 16, tp=a.tp,
                              max_batch_tokens=a.max_batch_tokens, block_size=a.block_size)
        if a.estimate_memory:
            print(json.dumps(est, indent=1))
            return
        if not est["fits_b200"] and not a.no_preflight:
            # the KV pool is paged and shared: what must fit is the weights plus ONE full-context sequence
            one = estimate_memory(cfg, ctx=a.ctx_size, parallel=1, kv_bits=a.kv_bits or 16, tp=a.tp,
                                  max_batch_tokens=a.max_batch_tokens, block_size=a.block_size)
            if not one["fits_b200"]:
                raise SystemExit(f"preflight: {one['total_gib']} GiB per GPU for the weights and one {a.ctx_size}-token "
                                 f"sequence does not fit; lower --ctx-size, raise --tp, quantize the KV cache "
                                 f"(--kv-bits 8), or pass --no-preflight")
            print(f"preflight: {a.parallel} sequences of {a.ctx_size} tokens would need {est['total_gib']} GiB; the paged KV "
                  f"pool takes what is free, long requests will queue", file=sys.stderr)
    from .audio.transcribe import is_whisper_checkpoint
    if is_whisper_checkpoint(a.model):          # speech-to-text checkpoints get the audio routes
        import torch

        from .audio.transcribe import Transcriber
        from .server.audio import create_audio_app
        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        tr = Transcriber.from_pretrained(a.model, torch.bfloat16 if dev != "cpu" else torch.float32, dev)
        app = create_audio_app(tr, a.alias or os.path.basename(a.model.rstrip("/")), set(a.api_key or []))
        uvicorn.run(app, host=a.host, port=a.port, log_level="info" if a.verbose else "warning")
        return
    if _encoder_checkpoint(a.model):            # encoder checkpoints get the embeddings-only server
        import torch

        from .models.encoder import load_encoder
        from .server.embeddings import create_embedding_app
        from .tokenizer import load_tokenizer
        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        enc = load_encoder(a.model, device=dev)
        app = create_embedding_app(enc, load_tokenizer(a.model), a.alias or os.path.basename(a.model.rstrip("/")),
                                   set(a.api_key or []))
        uvicorn.run(app, host=a.host, port=a.port, log_level="info" if a.verbose else "warning")
        return
    llm = load_llm(a)
    control = None
    if getattr(a, "_control_group", None) is not None:
        # several processes serve the model together: rank 0 listens, schedules and broadcasts a step
        # descriptor per engine step; the other ranks run the executor loop (parallel/control.py)
        from .parallel.control import ControlPlane
        control = ControlPlane(a._control_group)
    budget = a.reasoning_budget if a.reasoning_budget is not None else os.environ.get(
        "LLAMA_ARG_THINK_BUDGET", os.environ.get("LLAMA_ARG_REASONING_BUDGET"))
    sleep_idle = float(getattr(a, "sleep_idle_seconds", -1) or -1)
    if sleep_idle > 0 and (control is not None or getattr(a, "lora", None)):
        raise SystemExit("--sleep-idle-seconds works with one process and without --lora (both keep the weights referenced)")
    worker = ModelWorker(llm.engine, llm.tokenizer, a.alias or os.path.basename(a.model.rstrip("/")), control=control,
                         hang_timeout=float(a.decode_hang_timeout), failfast=True,
                         engine_factory=(lambda: load_llm(a).engine) if sleep_idle > 0 else None, sleep_idle=max(sleep_idle, 0.0))
    if control is not None and not control.is_leader:
        worker.follow()
        _leave_distributed()
        return
    if not a.no_warmup:
        _startup_warmup(worker, llm)
    keys = set(a.api_key or [])
    if a.api_key_file:
        keys |= {l.strip() for l in open(a.api_key_file) if l.strip()}
    state = ServerState(worker, llm.tokenizer, worker.model_id, api_keys=keys,
                        chat_template=open(a.chat_template_file).read() if a.chat_template_file else None)
    state.slot_save_path = a.slot_save_path
    worker.vision = getattr(llm, "vision", None)
    state.media_path, state.allow_remote_media = a.media_path, bool(a.allow_remote_media)
    state.default_thinking_budget = int(budget) if budget not in (None, "") else None
    state.cors_origins = list(a.cors_origin or ["*"])
    state.settings_enabled = bool(a.enable_settings)
    from .server.extras import LogControl
    verbosity = a.log_verbosity if a.log_verbosity is not None else (2 if a.verbose else 1)
    state.log = LogControl(dest=a.log_file, fmt=a.log_format, verbosity=verbosity, redact=not a.no_log_redact)
    from .lora import LoraManager
    from .models.weights import QuantizedTensor
    if sleep_idle <= 0 and not any(isinstance(lw.wqkv, QuantizedTensor) for lw in llm.model.w.layers):
        comm = llm.model.comm
        state.lora = LoraManager(llm.cfg, llm.model.w, comm.tp_rank, comm.tp_size)
        for spec in getattr(a, "lora", None) or []:
            path, _, sc = spec.partition("=")
            state.lora.add(path, float(sc) if sc else 1.0)
    listen = dict(uds=a.listen_unix) if a.listen_unix else dict(host=a.host, port=a.port)
    if sleep_idle > 0:
        del llm                     # the worker holds the only reference to the engine, so sleeping frees it
    try:
        uvicorn.run(create_app(state), log_level="info" if a.verbose else "warning",
                    ssl_certfile=a.ssl_cert_file, ssl_keyfile=a.ssl_key_file, **listen)
    finally:
        worker.shutdown()        # under a control plane this also broadcasts the stop to the other ranks
        if control is not None:
            _leave_distributed()


def _startup_warmup(worker, llm) -> None:
    """One short greedy request before the listener opens (the reference's start-up warm-up,
    src/server/startup.rs:2237): kernels are loaded, tensor maps and CUDA graphs for batch 1 exist and
    the first client does not pay for them. Skipped with --no-warmup."""
    import queue as _q

    from .engine import SamplingParams
    from .server.worker import GenRequest
    out: _q.Queue = _q.Queue()
    bos = [i for i in (getattr(llm.tokenizer, "bos_id", None),) if i is not None] or [0]
    worker.submit(GenRequest(prompt_ids=bos * 4, params=SamplingParams(max_tokens=2, ignore_eos=True), out=out,
                             request_id="warmup"))
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < 600:
        try:
            ev = out.get(timeout=1.0)
        except _q.Empty:
            continue
        if ev.kind in ("done", "error"):
            if ev.kind == "error":
                print(f"warm-up request failed: {ev.error}", file=sys.stderr)
            return


def cmd_router(a):
    """Router mode: a pool of models behind one listener (see server/router.py)."""
    import torch
    import uvicorn

    from .server.router import create_router_app
    keys = set(a.api_key or [])
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    app = create_router_app(a.models_dir, a.models_preset, a.models_max, device=dev, api_keys=keys,
                            default=a.default_model,
                            engine_defaults=dict(ctx_size=a.ctx_size, parallel=a.parallel))
    uvicorn.run(app, host=a.host, port=a.port, log_level="info" if a.verbose else "warning")


def cmd_transcribe(a):
    """Speech to text for WAV files with a Whisper checkpoint."""
    import torch

    from .audio import decode_audio
    from .audio.transcribe import Transcriber
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    tr = Transcriber.from_pretrained(a.model, torch.bfloat16 if dev != "cpu" else torch.float32, dev)
    for f in a.files:
        r = tr.transcribe(decode_audio(open(f, "rb").read()), language=a.language, task="translate" if a.translate else "transcribe")
        if a.json:
            print(json.dumps(dict(file=f, **{k: r[k] for k in ("text", "language", "duration")})))
        else:
            print(r["text"])


def cmd_depth(a):
    """Monocular depth for image files with a Depth Anything checkpoint: a 16-bit PNG per image (depth scaled to
    the full range; nearer is brighter for relative depth) and one JSON line with the value range."""
    import numpy as np
    import torch
    from PIL import Image

    from .models.depth_anything import DepthAnything
    from .multimodal import load_image
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    m = DepthAnything.from_pretrained(a.model, torch.bfloat16 if dev != "cpu" else torch.float32, dev)
    for f in a.files:
        d = m.estimate(load_image(f), short_side=a.short_side)
        lo, hi = float(d.min()), float(d.max())
        out = os.path.splitext(f)[0] + ".depth.png" if a.out_dir is None else os.path.join(a.out_dir, os.path.basename(f) + ".depth.png")
        Image.fromarray(((d - lo) / max(hi - lo, 1e-12) * 65535.0).astype(np.uint16)).save(out)
        print(json.dumps(dict(file=f, out=out, min=lo, max=hi, height=int(d.shape[0]), width=int(d.shape[1]), metric=m.metric)))


def cmd_front(a):
    """One listener in front of several servers (server/front.py): given URLs, or ``--dp N`` replicas
    that this process starts itself, one per GPU, and stops again when it exits."""
    import signal
    import subprocess
    import urllib.request

    import uvicorn

    from .server.front import create_front_app
    replicas, children = list(a.replica_url or []), []
    if a.dp:
        rest = [x for x in (a.serve_args or []) if x != "--"]
        if not rest:
            raise SystemExit("front --dp N needs the serve arguments after '--' (at least -m MODEL)")
        for i in range(a.dp):
            port = a.base_port + i
            env = dict(os.environ)
            if not a.no_pin_gpus:
                env["CUDA_VISIBLE_DEVICES"] = str(a.first_gpu + i)
            children.append(subprocess.Popen([sys.executable, "-m", "mlxcel_b200.cli", "serve", *rest,
                                              "--host", "127.0.0.1", "--port", str(port)], env=env))
            replicas.append(f"http://127.0.0.1:{port}")

    def stop_children(*_):
        for c in children:
            if c.poll() is None:
                c.terminate()
        for c in children:
            try:
                c.wait(timeout=30)
            except subprocess.TimeoutExpired:
                c.kill()

    try:
        if children:        # wait until every replica answers /health (loading a large checkpoint takes minutes)
            deadline = time.monotonic() + a.start_timeout
            pending = list(zip(children, replicas[-len(children):]))
            while pending and time.monotonic() < deadline:
                for c, u in list(pending):
                    if c.poll() is not None:
                        raise SystemExit(f"replica {u} exited with code {c.returncode} while starting")
                    try:
                        with urllib.request.urlopen(u + "/health", timeout=2) as r:
                            if r.status == 200:
                                pending.remove((c, u))
                    except OSError:
                        pass
                if pending:
                    time.sleep(0.5)
            if pending:
                raise SystemExit(f"replicas not ready after {a.start_timeout} s: {[u for _, u in pending]}")

            def on_term(*_):
                raise SystemExit(0)
            signal.signal(signal.SIGTERM, on_term)
        app = create_front_app(replicas=replicas, prefill=a.prefill_url, decode=a.decode_url, cooldown_s=a.cooldown)
        uvicorn.run(app, host=a.host, port=a.port, log_level="info" if a.verbose else "warning")
    finally:
        stop_children()


def cmd_inspect(a):
    from .config import ModelConfig, preset
    from .utils.memory import estimate_memory
    cfg = preset(a.model.split(":", 1)[1]) if a.model.startswith("preset:") else ModelConfig.from_path(a.model)
    est = estimate_memory(cfg, ctx=a.ctx_size, parallel=a.parallel, kv_bits=a.kv_bits or 16, tp=a.tp)
    print(json.dumps(est, indent=1))


_HYBRID = {"nemotron_h", "granitemoehybrid", "jamba", "qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe",
           "qwen3_5_moe_text", "falcon_h1", "lfm2", "lfm2_moe", "recurrent_gemma"}
_STATE_SPACE = {"mamba", "mamba2"}
_CHECKED_BY_READING = {"internlm3", "minicpm", "mimo", "yi", "kimi_k2", "deepseek"}       # no independent implementation at hand
_CHECKED_BY_LAYOUT = {"internlm2", "baichuan", "exaone", "telechat3"}                                 # round trip against the Llama form


def arch_catalog() -> dict:
    """What this build loads: every model family with its executor and how its layout was checked, the
    encoder families, quantization formats, KV precisions and parallel modes (reference src/main.rs:174,
    ``mlxcel arch``)."""
    from .config import FAMILIES
    fams = []
    for name in sorted(FAMILIES):
        ex = "hybrid" if name in _HYBRID else "state-space" if name in _STATE_SPACE else "decoder"
        how = ("reading" if name in _CHECKED_BY_READING else "layout round trip" if name in _CHECKED_BY_LAYOUT
               else "transformers logits")
        if name == "gemma3":                     # the wrapper's text_config is the gemma3_text model
            how = "transformers logits (as gemma3_text)"
        if name in ("qwen3_5", "qwen3_5_moe", "llama4", "qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe"):
            how = f"transformers logits (as {name}_text)"
        if name == "deepseek_v32":
            how = "transformers logits (as glm_moe_dsa)"
        if name == "dbrx":
            how = "a plain PyTorch statement of the model (the transformers implementation is not usable)"
        fams.append(dict(name=name, executor=ex, checked_against=how))
    return {"families": fams, "encoders": ["bert", "modernbert", "deberta-v2", "siglip text"],
            "vision_language": ["llava (clip / siglip tower)", "qwen2_vl", "qwen2_5_vl", "qwen3_vl (DeepStack)", "idefics3 / smolvlm (one tile per image)", "internvl (one tile per image)", "mistral3 (pixtral tower)", "glm4v", "glm4v_moe", "cohere2_vision (one tile per image)", "paddleocr_vl", "glm_ocr"], "speech": ["whisper"], "dense_prediction": ["depth_anything (dinov2 backbone)"], "speech_language": ["voxtral", "qwen2_audio (clips up to one 30 s chunk)"],
            "quantization": ["affine", "mxfp4", "mxfp8", "fp8 (widened at load)", "nvfp4 (expanded at load)",
                             "bitlinear ternary (expanded at load)"],
            "kv_bits": [16, 8, 4], "parallelism": ["tp", "ep (replicated tokens)", "dp attention + ep (all-to-all)", "pp", "tp x pp",
                                                   "dp replicas (front)", "prefill / decode disaggregation (front)"]}


def cmd_arch(a):
    cat = arch_catalog()
    if getattr(a, "json", False):
        print(json.dumps(cat, indent=1))
        return
    w = max(len(f["name"]) for f in cat["families"])
    print(f"{'FAMILY'.ljust(w)}  EXECUTOR     CHECKED AGAINST")
    for f in cat["families"]:
        print(f"{f['name'].ljust(w)}  {f['executor']:<11}  {f['checked_against']}")
    print(f"encoders: {', '.join(cat['encoders'])}")
    print(f"vision-language: {', '.join(cat['vision_language'])}; speech: {', '.join(cat['speech'])}")
    print(f"quantization: {', '.join(cat['quantization'])}; kv bits: {cat['kv_bits']}; parallelism: {', '.join(cat['parallelism'])}")


def cmd_tokenize(a):
    from .tokenizer import load_tokenizer
    print(json.dumps(load_tokenizer(a.model).encode(a.text)))


def cmd_random_init(a):
    import torch

    from .config import preset
    from .loading.checkpoint import save_checkpoint
    from .models.weights import random_weights
    from .ops import quant
    cfg = preset(a.preset)
    if cfg.model_type == "mamba2":
        from .models.mamba2 import mamba2_config_dict, random_mamba2_weights, save_mamba2_checkpoint
        save_mamba2_checkpoint(a.out, mamba2_config_dict(cfg), random_mamba2_weights(cfg, seed=a.seed))
        print("wrote", a.out)
        return
    if cfg.model_type == "nemotron_h":
        from .models.hybrid import hybrid_config_dict, random_hybrid_weights, save_hybrid_checkpoint
        save_hybrid_checkpoint(a.out, hybrid_config_dict(cfg), random_hybrid_weights(cfg, seed=a.seed), cfg)
        print("wrote", a.out)
        return
    w = random_weights(cfg, seed=a.seed, dtype=torch.bfloat16)
    qd = None
    if a.quantize:
        mode, bits, group = a.quantize, (8 if a.quantize == "mxfp8" else a.bits), (32 if a.quantize != "affine" else a.group_size)
        for lw in w.layers:
            for name in ("wqkv", "wo", "w_gate_up", "w_down", "experts_gate_up", "experts_down"):
                v = getattr(lw, name)
                if v is not None and v.shape[-1] % group == 0:   # other shapes stay dense
                    setattr(lw, name, quant.quantize(v, mode, bits, group))
        qd = dict(mode=mode, bits=bits, group_size=group)
    cd = {k: v for k, v in cfg.to_dict().items() if k not in ("quantization", "extra")}
    save_checkpoint(a.out, cd, w, quantization=qd)
    print("wrote", a.out)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="mlxcel")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("generate", help="one-shot generation")
    _add_model_args(p)
    _add_sampling_args(p)
    p.add_argument("-p", "--prompt", default=None)
    p.add_argument("--chat", action="store_true", help="wrap the prompt with the chat template")
    p.add_argument("--grammar", default=None, help="GBNF grammar constraining the output")
    p.add_argument("--grammar-file", default=None)
    p.add_argument("-j", "--json-schema", default=None, help="JSON schema constraining the output ('{}' for any object)")
    p.add_argument("-jf", "--json-schema-file", default=None)
    p.add_argument("--regex", default=None, help="regular expression constraining the output")
    p.add_argument("--diffusion", action="store_true",
                   help="block-unmasking decoding for masked-diffusion checkpoints (LLaDA-style) instead of next-token decoding")
    p.add_argument("--mask-token-id", type=int, default=None)
    p.add_argument("--block-length", type=int, default=32)
    p.add_argument("--diffusion-steps", type=int, default=32)
    p.add_argument("--diffusion-threshold", type=float, default=0.95)
    p.add_argument("--image", action="append", default=None, metavar="FILE",
                   help="image for a vision-language checkpoint (repeatable; one per placeholder, or placed before the prompt)")
    p.add_argument("--audio", action="append", default=None, metavar="FILE",
                   help="WAV clip for a speech-language checkpoint (repeatable; one per placeholder, or placed before the prompt)")
    p.set_defaults(fn=cmd_generate)
    p = sub.add_parser("run", help="interactive chat")
    _add_model_args(p)
    _add_sampling_args(p)
    p.add_argument("--system", default=None)
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("serve", help="HTTP server")
    _add_model_args(p)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--api-key", action="append")
    p.add_argument("--api-key-file", default=None)
    p.add_argument("--alias", "-a", default=None)
    p.add_argument("--chat-template-file", default=None)
    p.add_argument("--slot-save-path", default=None, help="directory for POST /slots/{id}?action=save|restore")
    p.add_argument("--lora", action="append", default=None, metavar="DIR[=SCALE]",
                   help="attach a LoRA adapter directory (repeatable); scales can be changed live via /lora-adapters")
    p.add_argument("--debug-trace", "--debug-pp-trace", dest="debug_trace", default=None, metavar="FILE",
                   help="write a Chrome trace of engine steps and pipeline stages (same as MLXCEL_B200_TRACE)")
    p.add_argument("--surgery", default=None, metavar="YAML", help="load-time weight edits (see loading/surgery.py)")
    p.add_argument("--estimate-memory", action="store_true",
                   help="print the memory estimate for this model and these options, then exit")
    p.add_argument("--no-preflight", action="store_true", help="start even when the estimate does not fit the GPU")
    p.add_argument("--reasoning-budget", type=int, default=None,
                   help="default thinking-token budget of requests that give none (-1 unlimited, 0 close at once)")
    p.add_argument("--decode-hang-timeout", type=float, default=0.0,
                   help="seconds after which a step that has not returned fails its requests (0 = off)")
    p.add_argument("--media-path", default=None, help="directory image paths in requests must lie in (default: any readable path)")
    p.add_argument("--allow-remote-media", action="store_true", help="fetch http(s) image URLs named by requests")
    p.add_argument("--sleep-idle-seconds", type=float, default=-1,
                   help="unload the model after this many seconds without a request; the next request loads it again (-1 = never)")
    p.add_argument("--ssl-cert-file", default=None)
    p.add_argument("--ssl-key-file", default=None)
    p.add_argument("--cors-origin", action="append", default=None, metavar="ORIGIN",
                   help="origin allowed by CORS (repeatable; default: any)")
    p.add_argument("--enable-settings", action="store_true", help="serve GET/POST /v1/settings (needs --api-key)")
    p.add_argument("--log-file", default=None, help="write the server log there instead of stderr")
    p.add_argument("--log-format", choices=["text", "json"], default="text")
    p.add_argument("-lv", "--log-verbosity", "--verbosity", dest="log_verbosity", type=int, default=None,
                   help="0 errors, 1 warnings, 2 requests, 3 debug")
    p.add_argument("--no-log-redact", action="store_true", help="log request bodies verbatim (default: shape only)")
    p.add_argument("--listen-unix", default=None, metavar="PATH", help="listen on a Unix domain socket instead of host:port")
    p.add_argument("-v", "--verbose", action="store_true")
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("router", help="HTTP server over a pool of models (loaded on demand, LRU eviction)")
    p.add_argument("--models-dir", default=None, help="every sub-directory with a config.json is a model")
    p.add_argument("--models-preset", default=None, metavar="INI", help="[name] sections: model = <path> + options")
    p.add_argument("--models-max", type=int, default=1, help="resident models")
    p.add_argument("--default-model", default=None)
    p.add_argument("--device", default=None)
    p.add_argument("-c", "--ctx-size", type=int, default=8192)
    p.add_argument("--parallel", "-np", type=int, default=4)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--api-key", action="append")
    p.add_argument("-v", "--verbose", action="store_true")
    p.set_defaults(fn=cmd_router)
    p = sub.add_parser("transcribe", help="speech to text for WAV files (Whisper checkpoints)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("files", nargs="+")
    p.add_argument("--language", default=None, help="spoken language (default: detected from the first 30 s)")
    p.add_argument("--translate", action="store_true", help="translate to English instead of transcribing")
    p.add_argument("--device", default=None)
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_transcribe)
    p = sub.add_parser("depth", help="monocular depth maps for image files (Depth Anything checkpoints)")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("files", nargs="+")
    p.add_argument("--short-side", type=int, default=518, help="the shorter image side is resized to this many pixels")
    p.add_argument("--out-dir", default=None, help="where the PNGs go (default: beside each image)")
    p.add_argument("--device", default=None)
    p.set_defaults(fn=cmd_depth)
    p = sub.add_parser("front", help="one listener in front of data-parallel replicas or prefill/decode servers")
    p.add_argument("--replica-url", action="append", default=None, metavar="URL", help="a running server of the model (repeatable)")
    p.add_argument("--prefill-url", action="append", default=None, metavar="URL", help="prefill-role server (disaggregated serving)")
    p.add_argument("--decode-url", action="append", default=None, metavar="URL", help="decode-role server (disaggregated serving)")
    p.add_argument("--dp", type=int, default=0, help="start this many replicas here, one per GPU; serve arguments follow '--'")
    p.add_argument("--first-gpu", type=int, default=0)
    p.add_argument("--no-pin-gpus", action="store_true", help="do not set CUDA_VISIBLE_DEVICES for the replicas (CPU replicas)")
    p.add_argument("--base-port", type=int, default=18080, help="replica i listens on 127.0.0.1:(base+i)")
    p.add_argument("--start-timeout", type=float, default=1800.0)
    p.add_argument("--cooldown", type=float, default=5.0, help="seconds a failed backend stays out of the rotation")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("-v", "--verbose", action="store_true")
    p.add_argument("serve_args", nargs=argparse.REMAINDER)
    p.set_defaults(fn=cmd_front)
    p = sub.add_parser("embed", help="embed texts and print the vectors")
    _add_model_args(p)
    p.add_argument("-p", "--prompt", action="append")
    p.add_argument("--instruction", default=None)
    p.add_argument("--pooling", choices=["mean", "cls", "last"], default=None)
    p.add_argument("--embd-normalize", choices=["auto", "l2", "none"], default="auto",
                   help="auto: what the checkpoint's modules.json declares (l2 when it says nothing)")
    p.add_argument("--dimensions", type=int, default=None)
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_embed)
    p = sub.add_parser("rerank", help="score documents against a query")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("--device", default=None)
    p.add_argument("-q", "--query", required=True)
    p.add_argument("-d", "--document", action="append", required=True)
    p.add_argument("--instruction", default=None, help="task instruction of a generative reranker")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_rerank)
    p = sub.add_parser("tag", help="tag and redact entities with a token-classification checkpoint")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("--device", default=None)
    p.add_argument("--keep", default=None, help="comma-separated entity names left in the redacted copy")
    p.add_argument("--replacement", default=None)
    p.add_argument("--argmax", action="store_true", help="per-token argmax instead of the BIO-constrained Viterbi path")
    p.add_argument("--json", action="store_true")
    p.add_argument("text")
    p.set_defaults(fn=cmd_tag)
    p = sub.add_parser("list", aliases=["ls"], help="models in the local store")
    p.add_argument("--models-dir", default=None)
    p.add_argument("--json", action="store_true")
    p.add_argument("-q", "--quiet", action="store_true")
    p.add_argument("-v", "--verbose", action="store_true")
    p.add_argument("--sort", choices=["name", "size", "modified"], default="name")
    p.set_defaults(fn=cmd_list)
    p = sub.add_parser("rm", help="remove a model from the local store")
    p.add_argument("repo_id")
    p.add_argument("--models-dir", default=None)
    p.add_argument("-y", "--yes", action="store_true")
    p.set_defaults(fn=cmd_rm)
    p = sub.add_parser("download", help="bring a repository into the local store (HuggingFace cache reuse; no network fetch)")
    p.add_argument("repo_id")
    p.add_argument("--models-dir", default=None)
    p.add_argument("--local-dir", default=None)
    p.set_defaults(fn=cmd_download)
    p = sub.add_parser("tune", help="profile kernel launch knobs and cache the winners")
    p.add_argument("--op", action="append", default=None)
    p.add_argument("-m", "--model", default=None, help="take the problem geometry from this checkpoint or preset")
    p.add_argument("--dry-run", action="store_true", help="print the candidate matrix, profile nothing")
    p.add_argument("--cache-file", default=None)
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_tune)
    p = sub.add_parser("split-mtp", help="extract the MTP layers of a raw checkpoint into a drafter checkpoint")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--block-size", type=int, default=None)
    p.add_argument("--q-bits", type=int, default=None)
    p.add_argument("--q-group-size", type=int, default=64)
    p.add_argument("--force", action="store_true")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_split_mtp)
    p = sub.add_parser("perplexity", help="windowed perplexity of a text file")
    _add_model_args(p)
    p.add_argument("-f", "--file", default=None, help="text file (stdin when absent)")
    p.add_argument("--window", type=int, default=2048)
    p.add_argument("--stride", type=int, default=None)
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_perplexity)
    p = sub.add_parser("inspect", help="memory estimate")
    _add_model_args(p)
    p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("arch", aliases=["supported"], help="supported architectures")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_arch)
    p = sub.add_parser("tokenize")
    p.add_argument("-m", "--model", required=True)
    p.add_argument("text")
    p.set_defaults(fn=cmd_tokenize)
    p = sub.add_parser("random-init", help="write a random checkpoint of a preset architecture")
    p.add_argument("preset")
    p.add_argument("out")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--quantize", choices=["affine", "mxfp4", "mxfp8"], default=None)
    p.add_argument("--bits", type=int, default=4)
    p.add_argument("--group-size", type=int, default=64)
    p.set_defaults(fn=cmd_random_init)
    _apply_env_aliases(sub)
    a = ap.parse_args(argv)
    ignored = _apply_compat(a)
    if ignored:
        print(f"accepted for llama-server compatibility, no effect on this runtime: {' '.join(ignored)}", file=sys.stderr)
    if isinstance(getattr(a, "model", None), str) and a.model:   # owner/name ids resolve through the local store
        from .store import resolve_model
        a.model = resolve_model(a.model)
    a.fn(a)


if __name__ == "__main__":
    main()
