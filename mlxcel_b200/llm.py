"""Public in-process API: :class:`LLM` wraps weights + executor + engine.

``LLM.generate`` is the call a user makes (the in-process analogue of the reference's
``mlxcel.LLM(model).generate(...)`` Python client, python/src/mlxcel/_client.py, and of its
``DirectEngine``, src/lib/mlxcel-core/src/engine/direct.rs:192-655).
"""
from __future__ import annotations

from pathlib import Path

import torch

from .config import ModelConfig, preset
from .engine import Engine, EngineConfig, SamplingParams, Sequence
from .models.decoder import DecoderModel
from .models.weights import ModelWeights, random_weights


class LLM:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, engine_config: EngineConfig | None = None,
                 comm=None, tokenizer=None, fold_norms: bool = False, model=None):
        """``fold_norms``: the weights belong to this object alone, so the executor may fold the
        RMSNorm weights into the projections in place (deferred RMSNorm, see DecoderModel).
        ``model``: an executor built by the caller (a pipeline stage) instead of the default one."""
        self.cfg = cfg
        if engine_config is not None:
            cfg.extra.setdefault("served_context", int(engine_config.max_model_len))
        if model is not None:
            self.model = model
        elif cfg.model_type in ("mamba", "mamba2", "nemotron_h", "granitemoehybrid", "jamba", "qwen3_next", "qwen3_5", "qwen3_5_text",
                                "qwen3_5_moe", "qwen3_5_moe_text", "falcon_h1", "lfm2", "lfm2_moe", "recurrent_gemma"):
            from .models.hybrid import HybridModel
            from .models.mamba1 import Mamba1Model
            from .models.mamba2 import Mamba2Model
            cls = {"mamba": Mamba1Model, "mamba2": Mamba2Model}.get(cfg.model_type, HybridModel)
            self.model = cls(cfg, weights, comm=comm,
                             max_seqs=2 * (engine_config.max_batch if engine_config else EngineConfig().max_batch))
        else:
            self.model = DecoderModel(cfg, weights, comm=comm,
                                      kv_bits=(engine_config.kv_bits if engine_config else 16),
                                      fold_norms=fold_norms)
        self.engine = Engine(self.model, cfg, engine_config)
        self.tokenizer = tokenizer

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_preset(name: str, *, device="cuda", seed: int = 0, engine_config: EngineConfig | None = None,
                    comm=None, dtype=torch.bfloat16, quantize: dict | None = None) -> "LLM":
        """``quantize``: ``dict(dense=(mode, bits, group), experts=(mode, bits, group), lm_head=bool)`` packs the
        random weights into MLX quantization formats layer by layer (see ops.quant.quantize_model_weights)."""
        cfg = preset(name)
        if cfg.model_type == "mamba2":
            from .models.mamba2 import random_mamba2_weights
            return LLM(cfg, random_mamba2_weights(cfg, seed=seed, dtype=dtype, device=device), engine_config, comm=comm)
        if cfg.model_type == "mamba":
            from .models.mamba1 import random_mamba1_weights
            return LLM(cfg, random_mamba1_weights(cfg, seed=seed, dtype=dtype, device=device), engine_config, comm=comm)
        if cfg.model_type == "nemotron_h":
            from .models.hybrid import random_hybrid_weights
            return LLM(cfg, random_hybrid_weights(cfg, seed=seed, dtype=dtype, device=device), engine_config, comm=comm)
        tp = comm.tp_size if comm is not None else 1
        rank = comm.tp_rank if comm is not None else 0
        hook = None
        if quantize:
            from types import SimpleNamespace

            from .ops import quant

            def hook(lw):
                quant.quantize_model_weights(SimpleNamespace(layers=[lw], lm_head=None, embed=None),
                                             dense=quantize.get("dense"), experts=quantize.get("experts"))
        w = random_weights(cfg, seed=seed, dtype=dtype, device=device, tp_rank=rank, tp_size=tp,
                           ep_rank=getattr(comm, "ep_rank", 0), ep_size=getattr(comm, "ep_size", 1),
                           vocab_parallel=tp > 1 and cfg.vocab_size % tp == 0, layer_hook=hook)
        if quantize and quantize.get("lm_head") and quantize.get("dense") and w.lm_head is not w.embed:
            from .ops import quant
            w.lm_head = quant.quantize_chunked(w.lm_head, *quantize["dense"])
        return LLM(cfg, w, engine_config, comm=comm, fold_norms=True)

    @staticmethod
    def from_pretrained(path: str | Path, *, device="cuda", engine_config: EngineConfig | None = None,
                        comm=None, dequantize: bool = False, surgery: str | None = None,
                        config_overrides: dict | None = None) -> "LLM":
        from .loading.checkpoint import load_model_weights
        from .tokenizer import load_tokenizer

        cfg = ModelConfig.from_path(path, config_overrides)
        if cfg.model_type == "mamba2":
            from .models.mamba2 import load_mamba2_weights
            return LLM(cfg, load_mamba2_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "mamba":
            from .models.mamba1 import load_mamba1_weights
            return LLM(cfg, load_mamba1_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "nemotron_h":
            from .models.hybrid import load_hybrid_weights
            return LLM(cfg, load_hybrid_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "falcon_h1":
            from .models.hybrid import load_falcon_h1_weights
            return LLM(cfg, load_falcon_h1_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type in ("lfm2", "lfm2_moe"):
            from .models.hybrid import load_lfm2_weights
            return LLM(cfg, load_lfm2_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "recurrent_gemma":
            from .models.hybrid import load_recurrent_gemma_weights
            return LLM(cfg, load_recurrent_gemma_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.extra.get("hybrid_layout") == "qwen3_next":
            from .models.hybrid import load_qwen3_next_weights
            return LLM(cfg, load_qwen3_next_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "jamba":
            from .models.hybrid import load_jamba_weights
            return LLM(cfg, load_jamba_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        if cfg.model_type == "granitemoehybrid":
            from .models.hybrid import load_granite_hybrid_weights
            return LLM(cfg, load_granite_hybrid_weights(path, cfg, device=device), engine_config, comm=comm,
                       tokenizer=load_tokenizer(path))
        w = load_model_weights(path, cfg, device=device, comm=comm, dequantize=dequantize, surgery=surgery)
        tok = load_tokenizer(path)
        llm = LLM(cfg, w, engine_config, comm=comm, tokenizer=tok, fold_norms=True)
        from .multimodal import VisionLanguage, is_vlm_checkpoint
        if is_vlm_checkpoint(path):
            llm.vision = VisionLanguage.from_checkpoint(path, dtype=w.final_norm.dtype, device=device)
        from .multimodal.audio_lm import AudioLanguage, is_audio_lm_checkpoint
        if is_audio_lm_checkpoint(path):
            # speech-language checkpoints use the same media front-end slot: prompts carry audio placeholders
            llm.vision = AudioLanguage.from_checkpoint(path, dtype=w.final_norm.dtype, device=device)
        return llm

    # ------------------------------------------------------------------ scoring
    def loglikelihoods(self, token_ids: list[int]):
        """``log p(token[t] | token[:t])`` for t >= 1 (fp32 CPU tensor), without generating."""
        from .engine.scoring import sequence_logprobs
        return sequence_logprobs(self.model, self.cfg, token_ids, self.engine.ecfg.block_size)

    # ------------------------------------------------------------------ generation
    def generate(self, prompts=None, sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 prompt_token_ids: list[list[int]] | None = None, images: list[list] | None = None) -> list[Sequence]:
        """``images[i]``: the images of prompt i (paths, data URLs, bytes or PIL images), one per image
        placeholder of that prompt, for vision-language checkpoints."""
        if prompt_token_ids is None:
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer; pass prompt_token_ids")
            if isinstance(prompts, str):
                prompts = [prompts]
            prompt_token_ids = [self.tokenizer.encode(p) for p in prompts]
        media = None
        if images is not None and any(images):
            vision = getattr(self, "vision", None)
            if vision is None:
                raise ValueError("this model takes no image input")
            from .multimodal import load_image
            media, prompt_token_ids = [], list(prompt_token_ids)
            for i, imgs in enumerate(images):
                if not imgs:
                    media.append(None)
                    continue
                prompt_token_ids[i], mm = vision.prepare(prompt_token_ids[i], [load_image(x) for x in imgs])
                media.append(mm)
        outs = self.engine.generate(prompt_token_ids, sampling_params, media=media)
        for s in outs:
            self.engine.release(s.seq_id)
        return outs

    def decode(self, token_ids: list[int]) -> str:
        return self.tokenizer.decode(token_ids) if self.tokenizer else " ".join(map(str, token_ids))
