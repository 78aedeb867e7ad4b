"""Split the multi-token-prediction (MTP) layers off a raw checkpoint into a drafter checkpoint.

Checkpoints of the DeepSeek-V3 / GLM-4.x line carry ``num_nextn_predict_layers`` extra decoder layers
after the last regular one (``model.layers.{num_hidden_layers + k}.*``): a full decoder layer plus
``enorm`` / ``hnorm`` (RMSNorm of the token embedding and of the target's hidden state), ``eh_proj``
([H, 2H], fuses the two) and ``shared_head.{norm, head}``. The target model ignores them; a drafter is
made of exactly these. Reference: src/commands/split_mtp.rs and the ``split_mtp_dir`` routine of the
mlxcel-surgery crate (output refused when it is the source, when it is non-empty without ``--force``,
when it holds foreign weights or symlinks; optional affine quantization of the projections, never of
the router, norms or selection bias).

The drafter directory written here is a self-contained checkpoint of the same family with
``num_hidden_layers = num_nextn_predict_layers``: the MTP layers renumbered from 0, the shared-head
norm as ``model.norm``, embedding and output head (the MTP layer's own copies when it has them, else
the target's), and the fusion tensors under ``model.mtp.{k}.{enorm, hnorm, eh_proj}``. The ordinary
checkpoint loader therefore reads the layers; :func:`load_mtp_weights` adds the fusion tensors.
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path

import torch

MARKER = "mtp_drafter.json"
_NEVER_QUANTIZED = re.compile(r"(norm|mlp\.gate\.weight$|e_score_correction_bias|\.bias$|embed_tokens)")


def _refuse_output(src: Path, out: Path, force: bool) -> None:
    if out.resolve() == src.resolve():
        raise ValueError("split-mtp: the output directory is the source checkpoint")
    if not out.exists():
        return
    if out.is_symlink() or not out.is_dir():
        raise ValueError(f"split-mtp: {out} is not a plain directory")
    entries = list(out.iterdir())
    if not entries:
        return
    if not force:
        raise ValueError(f"split-mtp: {out} is not empty (pass --force to overwrite a previous drafter)")
    ours = (out / MARKER).exists()
    for e in entries:
        if e.is_symlink():
            raise ValueError(f"split-mtp: {e} is a symlink; refusing to write through it")
        if e.suffix == ".safetensors" and not ours:
            raise ValueError(f"split-mtp: {out} holds weights that no earlier split wrote ({e.name})")


def split_mtp_dir(model: str | Path, output: str | Path, block_size: int | None = None, q_bits: int | None = None,
                  q_group_size: int = 64, force: bool = False) -> dict:
    """Write the drafter directory; returns a summary (layers, tensors, bytes, block size)."""
    from safetensors.torch import save_file

    from .checkpoint import TensorSource

    src_dir, out = Path(model), Path(output)
    if not (src_dir / "config.json").is_file():
        raise ValueError(f"split-mtp: {src_dir} has no config.json; pass the raw checkpoint directory")
    if q_bits is not None and q_bits not in (2, 3, 4, 5, 6, 8):
        raise ValueError("split-mtp: --q-bits must be one of 2, 3, 4, 5, 6, 8")
    if q_bits is None and q_group_size != 64:
        raise ValueError("split-mtp: --q-group-size is only read with --q-bits")
    _refuse_output(src_dir, out, force)
    raw = json.loads((src_dir / "config.json").read_text())
    text = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw
    L = int(text["num_hidden_layers"])
    n = int(text.get("num_nextn_predict_layers", 0) or 0)
    if n < 1:
        raise ValueError("split-mtp: config.json declares no MTP layers (num_nextn_predict_layers)")
    src = TensorSource(src_dir)
    pre = "model."
    names = [k for k in src.keys() if k.startswith(f"{pre}layers.")]
    have = sorted({int(k.split(".")[2]) for k in names})
    missing = [L + k for k in range(n) if L + k not in have]
    if missing:
        raise ValueError(f"split-mtp: the checkpoint no longer holds model.layers.{missing[0]}.* "
                         "(converted checkpoints often drop the MTP layers; use the raw one)")
    tensors: dict[str, torch.Tensor] = {}
    own_embed = own_head = False
    for k in range(n):
        lp = f"{pre}layers.{L + k}."
        for name in names:
            if not name.startswith(lp):
                continue
            rest = name[len(lp):]
            t = src.get(name)
            if rest.startswith(("enorm.", "hnorm.", "eh_proj.")):
                tensors[f"{pre}mtp.{k}.{rest}"] = t
            elif rest.startswith("shared_head.norm."):
                if k == 0:
                    tensors[f"{pre}norm.{rest.split('.', 2)[2]}"] = t
            elif rest.startswith("shared_head.head."):
                if k == 0:
                    tensors["lm_head." + rest.split(".", 2)[2]] = t
                    own_head = True
            elif rest.startswith("embed_tokens."):
                if k == 0:
                    tensors[f"{pre}embed_tokens.{rest.split('.', 1)[1]}"] = t
                    own_embed = True
            else:
                tensors[f"{pre}layers.{k}.{rest}"] = t
    for k in range(n):
        for need in ("enorm.weight", "hnorm.weight", "eh_proj.weight"):
            if f"{pre}mtp.{k}.{need}" not in tensors:
                raise ValueError(f"split-mtp: model.layers.{L + k}.{need} is missing")
    if not own_embed:                                  # shared with the target: copy, the drafter stands alone
        for kname in [k for k in src.keys() if k.startswith(f"{pre}embed_tokens.")]:
            tensors[kname] = src.get(kname)
    tied = bool(text.get("tie_word_embeddings", False))
    if not own_head and not tied:
        for kname in [k for k in src.keys() if k.startswith("lm_head.")]:
            tensors[kname] = src.get(kname)
    quantized = 0
    if q_bits is not None:
        from ..ops.quant import quantize_affine
        for name in list(tensors):
            t = tensors[name]
            if (not name.endswith(".weight") or t.dim() != 2 or _NEVER_QUANTIZED.search(name)
                    or t.shape[-1] % q_group_size or name[:-7] + ".scales" in tensors):
                continue
            qt = quantize_affine(t.to(torch.bfloat16), q_bits, q_group_size)
            base = name[:-7]
            tensors[name], tensors[base + ".scales"], tensors[base + ".biases"] = qt.packed, qt.scales, qt.biases
            quantized += 1
    cfg = json.loads(json.dumps(text))
    cfg.update(num_hidden_layers=n, num_nextn_predict_layers=0, first_k_dense_replace=0,
               mtp_block_size=int(block_size) if block_size else n + 1, mtp_source_layer=L, mtp_layers=n)
    if q_bits is not None:
        cfg["quantization"] = dict(group_size=q_group_size, bits=q_bits)
    elif not any(k.endswith(".scales") for k in tensors):
        cfg.pop("quantization", None)
    out.mkdir(parents=True, exist_ok=True)
    for old in out.glob("*.safetensors"):
        old.unlink()
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(out / "model.safetensors"), metadata={"format": "pt"})
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    for side in ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "generation_config.json",
                 "chat_template.jinja", "tokenizer.model"):
        f = src_dir / side
        if f.is_file():
            (out / side).write_bytes(f.read_bytes())
    summary = dict(source=str(src_dir), layers=n, source_layer=L, tensors=len(tensors), quantized=quantized,
                   bytes=os.path.getsize(out / "model.safetensors"), block_size=cfg["mtp_block_size"],
                   own_embeddings=own_embed, own_head=own_head)
    (out / MARKER).write_text(json.dumps(summary, indent=1))
    return summary


def load_mtp_weights(path: str | Path, dtype=torch.bfloat16, device="cpu", dequantize: bool = True):
    """Read a drafter directory written by :func:`split_mtp_dir`: ``(cfg, MTPWeights, ModelWeights)``.
    The model weights carry the drafter's embedding / head, for use when the target's are not shared."""
    from ..config import ModelConfig
    from ..speculative.mtp import MTPWeights
    from .checkpoint import TensorSource, _Getter, _to_device, load_full_weights

    cfg = ModelConfig.from_path(str(path))
    mw = _to_device(load_full_weights(path, cfg, dtype=dtype, dequantize=dequantize), device)
    g = _Getter(TensorSource(path), cfg, dtype, True)
    fc = g.mat("model.mtp.0.eh_proj")
    w = MTPWeights(enorm=g.vec("model.mtp.0.enorm.weight").to(device), hnorm=g.vec("model.mtp.0.hnorm.weight").to(device),
                   fc=fc.to(device), layer=mw.layers[0], final_norm=mw.final_norm)
    return cfg, w, mw
