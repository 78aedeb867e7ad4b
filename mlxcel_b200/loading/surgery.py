"""Load-time weight surgery: a YAML list of edits applied to checkpoint tensors by name.

Counterpart of the reference's ``mlxcel-surgery`` crate (src/lib/mlxcel-surgery/, hooked into loading
through ``WeightTransform``, src/lib/mlxcel-core/src/weights.rs:58). Operations:

    - op: scale        # tensor *= factor
      match: "model.layers.(3|4).mlp.down_proj.weight"
      factor: 0.5
    - op: add          # tensor += value (a number) or += other tensor (by name)
      match: "lm_head.weight"
      value: 0.01
    - op: prune        # zero entries with |x| below a threshold, or rows / columns by index
      match: ".*q_proj.weight"
      threshold: 1.0e-3
    - op: replace      # tensor = other tensor (same shape), or = constant
      match: "model.norm.weight"
      source: "model.layers.0.input_layernorm.weight"
    - op: interpolate  # tensor = (1 - t) * tensor + t * other
      match: "model.layers.1.(.*)"
      source: "model.layers.0.\\\\1"
      t: 0.25

``match`` is a full-match regular expression over checkpoint tensor names; ``source`` may use
back-references to the match. Edits run in file order on fp32 copies and are cast back.
"""
from __future__ import annotations

import re
from typing import Callable

import torch

Edit = dict


def load_edits(path: str) -> list[Edit]:
    import yaml

    with open(path) as f:
        doc = yaml.safe_load(f) or []
    edits = doc.get("edits", doc) if isinstance(doc, dict) else doc
    for e in edits:
        if e.get("op") not in ("scale", "add", "prune", "replace", "interpolate"):
            raise ValueError(f"unknown surgery op: {e.get('op')!r}")
        if "match" not in e:
            raise ValueError("every surgery edit needs a 'match' pattern")
    return list(edits)


def apply_edits(edits: list[Edit], name: str, tensor: torch.Tensor,
                lookup: Callable[[str], torch.Tensor | None]) -> torch.Tensor:
    """Returns the edited tensor for checkpoint entry ``name`` (``lookup`` fetches other entries)."""
    out = tensor
    for e in edits:
        m = re.fullmatch(e["match"], name)
        if m is None:
            continue
        x = out.float()
        src = None
        if "source" in e:
            src_name = m.expand(e["source"]) if "\\" in e["source"] else e["source"]
            src = lookup(src_name)
            if src is None:
                raise KeyError(f"surgery: source tensor {src_name!r} not found (edit on {name!r})")
            if tuple(src.shape) != tuple(x.shape):
                raise ValueError(f"surgery: {src_name!r} {tuple(src.shape)} does not match {name!r} {tuple(x.shape)}")
            src = src.float()
        op = e["op"]
        if op == "scale":
            x = x * float(e["factor"])
        elif op == "add":
            x = x + (src if src is not None else float(e.get("value", 0.0)))
        elif op == "prune":
            if "threshold" in e:
                x = torch.where(x.abs() < float(e["threshold"]), torch.zeros_like(x), x)
            for r in e.get("rows", []):
                x[int(r)] = 0
            for c in e.get("cols", []):
                x[..., int(c)] = 0
        elif op == "replace":
            x = src.clone() if src is not None else torch.full_like(x, float(e.get("value", 0.0)))
        elif op == "interpolate":
            t = float(e.get("t", 0.5))
            x = (1.0 - t) * x + t * src
        out = x.to(tensor.dtype)
    return out
