"""A plain-PyTorch executor for the comparison arm of ``bench.py`` (``--impl torch``).

``install()`` replaces the kernel-library entry points of ``mlxcel_b200.ops`` that the Llama-style
decoder uses with library calls: ``torch.nn.functional.linear`` (cuBLAS), ``rms_norm``,
``scaled_dot_product_attention`` (flash / cuDNN back ends) over K/V gathered from the same paged
pool through the block tables, ``torch.argmax``; tensor parallelism then runs the ``nccl`` back end
of ``parallel/tp.py`` (GEMM followed by a NCCL all-reduce / all-gather). The engine, scheduler,
block manager, CUDA-graph capture of decode steps and the workload are the ones the product arm
uses, so the two arms differ only in who executes the tensor math. None of this library's CUDA
kernels run on this path. It is the "NCCL + cuBLAS PyTorch baseline" that stands in for the
reference's own multi-GPU build, which does not exist (its tensor parallelism is a one-process
simulation, src/distributed/tensor_parallel/llama_runtime.rs:64-68).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

CALLS = 0     # library calls issued (the counterpart of the product arm's kernel-launch counter)


def _count(n: int = 1) -> None:
    global CALLS
    CALLS += n


def linear(x, w, bias=None, residual=None, out=None, out_fp32=False, **_):
    y = F.linear(x, w, bias)
    _count()
    if residual is not None:
        y = y + residual
        _count()
    if out_fp32:
        y = y.float()
    if out is not None and out.data_ptr() != y.data_ptr():
        out.copy_(y)
        _count()
        return out
    return y


def glu_linear(x, w, inter, act="silu", bias=None, alpha=1.702, limit=7.0, out=None, **_):
    y = F.linear(x, w, bias)
    g, u = y[:, :inter], y[:, inter:]
    if act == "silu":
        r = F.silu(g) * u
    elif act == "gelu_tanh":
        r = F.gelu(g, approximate="tanh") * u
    else:     # clipped SwiGLU (gpt-oss)
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
        r = g * torch.sigmoid(alpha * g) * (u + 1)
    _count(3)
    if out is not None:
        out.copy_(r)
        return out
    return r


def add_rmsnorm(x, residual, weight, eps, w_bias=0.0):
    h = x if residual is None else x + residual
    w = weight if w_bias == 0.0 else (weight.float() + w_bias).to(weight.dtype)
    y = F.rms_norm(h, (h.shape[-1],), w, eps)
    _count(2 if residual is not None else 1)
    return y, h


def rmsnorm(x, weight, eps, w_bias=0.0):
    return add_rmsnorm(x, None, weight, eps, w_bias)[0]


def embedding(ids, table, scale=1.0):
    _count()
    e = F.embedding(ids.long(), table)
    return e if scale == 1.0 else (e.float() * scale).to(e.dtype)


def argmax(logits, out=None):
    _count()
    t = torch.argmax(logits, dim=-1).to(torch.int32)
    if out is not None:
        out.copy_(t)
        return out
    return t


def rope_append(qkv, positions, slot_mapping, inv_freq, kv, *, Hq, Hkv, D, rot_dim, traditional=False, mscale=1.0,
                q_norm_w=None, k_norm_w=None, norm_eps=1e-6):
    T = qkv.shape[0]
    x = qkv.view(T, Hq + 2 * Hkv, D)
    qk = x[:, :Hq + Hkv]
    if q_norm_w is not None:
        qn = F.rms_norm(x[:, :Hq], (D,), q_norm_w, norm_eps)
        kn = F.rms_norm(x[:, Hq:Hq + Hkv], (D,), k_norm_w, norm_eps)
        qk = torch.cat([qn, kn], dim=1)
    if rot_dim:
        ang = positions.float()[:, None] * inv_freq[None, :].float()          # [T, rot/2]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        r = qk[..., :rot_dim].float()
        if traditional:
            a, b = r[..., 0::2], r[..., 1::2]
            rot = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
        else:
            a, b = r[..., : rot_dim // 2], r[..., rot_dim // 2:]
            rot = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
        qk = torch.cat([(rot * mscale).to(qkv.dtype), qk[..., rot_dim:]], dim=-1)
    x[:, :Hq + Hkv] = qk
    k, v = x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]
    bs = kv.block_size
    valid = slot_mapping >= 0
    # padding rows (slot -1) rewrite the pool's last slot with what it already holds, so the op has
    # static shapes (CUDA-graph capture); the engine hands out blocks from the front of the pool
    last = kv.k.shape[0] * bs - 1
    slot = torch.where(valid, slot_mapping, torch.full_like(slot_mapping, last)).long()
    blk, off = slot // bs, slot % bs
    cur_k, cur_v = kv.k[blk, :, off, :], kv.v[blk, :, off, :]
    m = valid[:, None, None]
    kv.k[blk, :, off, :] = torch.where(m, k.to(kv.k.dtype), cur_k)
    kv.v[blk, :, off, :] = torch.where(m, v.to(kv.v.dtype), cur_v)
    _count(12)


def _gather(pool, tables):
    """[B, MB] block ids -> [B, Hkv, MB * block, D] keys or values of the paged pool."""
    g = pool[tables.long()]                                   # [B, MB, Hkv, bs, D]
    B, MB, H, bs, D = g.shape
    return g.permute(0, 2, 1, 3, 4).reshape(B, H, MB * bs, D)


def paged_decode(q, kv, block_tables, context_lens, *, Hq, Hkv, D, scale, window=0, sinks=None, softcap=0.0,
                 num_splits=0, max_len=0, out=None):
    assert sinks is None and softcap == 0.0, "the comparison executor covers plain causal attention"
    B = q.shape[0]
    kk, vv = _gather(kv.k, block_tables), _gather(kv.v, block_tables)
    L = kk.shape[2]
    pos = torch.arange(L, device=q.device)[None, :]
    mask = pos < context_lens[:, None]
    if window > 0:
        mask = mask & (pos >= (context_lens[:, None] - window))
    o = F.scaled_dot_product_attention(q.reshape(B, Hq, 1, D), kk, vv, attn_mask=mask[:, None, None, :], scale=scale,
                                       enable_gqa=True)
    o = o.reshape(B, Hq * D)
    _count(5)
    if out is not None:
        out.copy_(o)
        return out
    return o


def paged_prefill(q, kv, block_tables, cu_q, context_lens, *, Hq, Hkv, D, scale, max_q_len, window=0, sinks=None,
                  softcap=0.0, out=None):
    assert sinks is None and softcap == 0.0 and window == 0
    T = q.shape[0]
    o = out if out is not None else torch.empty(T, Hq * D, dtype=q.dtype, device=q.device)
    cu, ctx = cu_q.tolist(), context_lens.tolist()
    S = len(ctx)
    bs = kv.block_size
    if S and all(cu[i + 1] - cu[i] == max_q_len and ctx[i] == max_q_len for i in range(S)):
        # every piece is a whole prompt of the same length: one batched causal call
        nb = (max_q_len + bs - 1) // bs
        kk = _gather(kv.k, block_tables[:, :nb])[:, :, :max_q_len]
        vv = _gather(kv.v, block_tables[:, :nb])[:, :, :max_q_len]
        qq = q.reshape(S, max_q_len, Hq, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale, enable_gqa=True)
        o.copy_(a.transpose(1, 2).reshape(T, Hq * D))
        _count(4)
        return o
    for i in range(S):
        lq, c = cu[i + 1] - cu[i], ctx[i]
        nb = (c + bs - 1) // bs
        kk = _gather(kv.k, block_tables[i:i + 1, :nb])[:, :, :c]
        vv = _gather(kv.v, block_tables[i:i + 1, :nb])[:, :, :c]
        qq = q[cu[i]:cu[i + 1]].reshape(1, lq, Hq, D).transpose(1, 2)
        if lq == c:
            a = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale, enable_gqa=True)
        else:
            qi = torch.arange(c - lq, c, device=q.device)[:, None]
            mask = torch.arange(c, device=q.device)[None, :] <= qi
            a = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=scale, enable_gqa=True)
        o[cu[i]:cu[i + 1]] = a.transpose(1, 2).reshape(lq, Hq * D)
        _count(4)
    return o


def install() -> None:
    """Route the decoder's ops to the functions above (process-wide)."""
    import os

    os.environ["MLXCEL_B200_FOLD_NORMS"] = "0"      # the deferred-RMSNorm epilogues belong to the library's GEMM
    from mlxcel_b200 import ops

    for name in ("linear", "glu_linear", "add_rmsnorm", "rmsnorm", "embedding", "argmax", "rope_append",
                 "paged_decode", "paged_prefill"):
        setattr(ops, name, globals()[name])
