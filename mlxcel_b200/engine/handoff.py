"""KV handoff between engines: a prefill-role engine computes a prompt's KV blocks and ships them, a
decode-role engine ingests them and continues as if it had prefilled the prompt itself.

Reference: the disaggregated role workers and ``scheduler/handoff.rs:58-624`` (KV extract / ingest,
``src/server/model_worker.rs:1000`` role loop). Here a handoff is one binary blob: a JSON header
(model geometry, block size, dtype names, token ids, tensor table) followed by the raw bytes of every
layer's K / V (and 8-bit metadata) block tensors. ``export_prefix`` prefills on the source engine and
snapshots the full blocks; ``import_prefix`` restores them into freshly reserved blocks of the
destination pool and registers them in its prefix index, so the next request with that prompt starts
from the cache. Geometry mismatches (layers, heads, head size, block size, KV bits) are refused.
"""
from __future__ import annotations

import json
import struct

import numpy as np
import torch

from ..cache.prompt_cache import Snapshot, adopt_snapshot, snapshot_sequence
from .params import SamplingParams

_MAGIC = b"MXKV1\0\0\0"
_DT = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "uint8": torch.uint8,
       "int8": torch.int8}


def _geometry(engine) -> dict:
    p = engine.pool
    return dict(layers=len(p.layers), kv_heads=p.Hkv, head_dim=p.D, block_size=engine.ecfg.block_size,
                kv_bits=engine.ecfg.kv_bits)


def export_prefix(engine, tokens: list[int]) -> bytes:
    """Prefill ``tokens`` on this engine and return the blob of its full KV blocks."""
    if getattr(engine, "recurrent", False):
        raise ValueError("KV handoff covers attention models; recurrent state is not in the block pool")
    # two tokens, so that the sequence is still alive (and owns its blocks) when the prefill has finished
    sid = engine.add_request(list(tokens), SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
    bs = engine.ecfg.block_size
    want = (len(tokens) // bs) * bs
    snap = None
    while engine.has_work() and snap is None:
        engine.step()
        s = engine.seqs.get(sid)
        if s is not None and s.num_computed >= want and engine.bm.has_seq(sid):
            snap = snapshot_sequence(engine, s)
    engine.abort(sid)
    while engine.has_work():
        engine.step()
    engine.release(sid)
    if snap is None or not snap.tokens:
        raise ValueError("the prompt is shorter than one KV block: nothing to hand off")
    table, payload, off = [], [], 0
    for li, layer in enumerate(snap.blocks):
        for name, t in layer.items():
            raw = t.contiguous().view(torch.uint8).numpy().tobytes()
            table.append(dict(layer=li, name=name, dtype=str(t.dtype).replace("torch.", ""), shape=list(t.shape),
                              offset=off, nbytes=len(raw)))
            payload.append(raw)
            off += len(raw)
    head = json.dumps(dict(geometry=_geometry(engine), tokens=snap.tokens, tensors=table)).encode()
    return _MAGIC + struct.pack("<Q", len(head)) + head + b"".join(payload)


def parse_blob(blob: bytes) -> tuple[dict, Snapshot]:
    if blob[:8] != _MAGIC:
        raise ValueError("not a KV handoff blob")
    (n,) = struct.unpack("<Q", blob[8:16])
    head = json.loads(blob[16:16 + n])
    base = 16 + n
    layers: list[dict] = [dict() for _ in range(head["geometry"]["layers"])]
    for e in head["tensors"]:
        raw = np.frombuffer(blob, dtype=np.uint8, count=e["nbytes"], offset=base + e["offset"]).copy()
        layers[e["layer"]][e["name"]] = torch.from_numpy(raw).view(_DT[e["dtype"]]).view(*e["shape"])
    return head, Snapshot(tokens=list(head["tokens"]), blocks=layers, nbytes=len(blob) - base)


def import_prefix(engine, blob: bytes) -> int:
    """Ingest a blob: its blocks go into the pool and the prefix index. Returns the tokens now cached."""
    head, snap = parse_blob(blob)
    if head["geometry"] != _geometry(engine):
        raise ValueError(f"KV geometry mismatch: blob {head['geometry']} vs engine {_geometry(engine)}")
    sid = engine.add_request(list(snap.tokens) + [0], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    seq = engine.seqs[sid]
    got = adopt_snapshot(engine, seq, snap, len(snap.tokens))
    engine.abort(sid)                      # the carrier request never runs; its blocks stay in the prefix cache
    engine.release(sid)
    return got
