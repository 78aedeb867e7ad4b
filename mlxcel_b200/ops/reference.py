"""Plain PyTorch (fp32 math) statements of every op in the kernel library.

These are the numerical oracles of the CUDA kernels and the execution path on CPU
(configuration 1 of the benchmark set runs on them). They favour clarity over speed.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU, EPI_GEGLU, EPI_CLIPPED_SWIGLU = range(6)


def glu_act(kind: int, g: torch.Tensor, u: torch.Tensor, alpha: float = 1.702,
            limit: float = 7.0) -> torch.Tensor:
    if kind == EPI_SWIGLU:
        return F.silu(g) * u
    if kind == EPI_GEGLU:
        return F.gelu(g, approximate="tanh") * u
    if kind == EPI_CLIPPED_SWIGLU:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
        return g * torch.sigmoid(alpha * g) * (u + 1.0)
    raise ValueError(kind)


def linear(x, w, bias=None, residual=None, out_dtype=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def glu_linear(x, w, inter: int, kind: int, bias=None, alpha=1.702, limit=7.0, glu_offset=None):
    off = inter if glu_offset is None else glu_offset
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    g, u = y[..., :inter], y[..., off:off + inter]
    return glu_act(kind, g, u, alpha, limit).to(x.dtype)


def add_rmsnorm(x, residual, weight, eps: float, w_bias: float = 0.0):
    """Returns (normed, new_residual). The residual stream is rounded to x.dtype first."""
    h = x.float() if residual is None else x.float() + residual.float()
    h = h.to(x.dtype)
    hf = h.float()
    var = hf.pow(2).mean(-1, keepdim=True)
    y = hf * torch.rsqrt(var + eps) * (weight.float() + w_bias)
    return y.to(x.dtype), h


def rope_inv_freq(head_dim_rot: int, theta: float, scaling: dict | None,
                  max_pos: int = 0) -> tuple[torch.Tensor, float]:
    """Per-pair inverse frequencies (fp32) and the q/k magnitude scale (YaRN mscale).

    Implements plain, linear, llama3, yarn, longrope (Phi-3) and dynamic-NTK scaling the way the reference builds its
    frequency tables (src/models/rope_utils.rs:343-400,608; src/models/gpt_oss.rs:269-305).
    """
    half = head_dim_rot // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim_rot))
    mscale = 1.0
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            inv = inv / factor
        elif kind == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv
            low_wl, high_wl = orig / low, orig / high
            smooth = (orig / wavelen - low) / (high - low)
            scaled = torch.where(wavelen > low_wl, inv / factor, inv)
            mid = (1 - smooth) * inv / factor + smooth * inv
            is_mid = (wavelen <= low_wl) & (wavelen >= high_wl)
            inv = torch.where(is_mid, mid, scaled)
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast = float(scaling.get("beta_fast", 32.0))
            beta_slow = float(scaling.get("beta_slow", 1.0))
            truncate = bool(scaling.get("truncate", True))

            def corr_dim(n_rot):
                return head_dim_rot * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

            lo, hi = corr_dim(beta_fast), corr_dim(beta_slow)
            if truncate:
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, head_dim_rot - 1)
            if hi == lo:
                hi = lo + 0.001
            ramp = ((torch.arange(half, dtype=torch.float64) - lo) / (hi - lo)).clamp(0, 1)
            extrap_w = 1.0 - ramp
            inv = inv / factor * (1 - extrap_w) + inv * extrap_w
            ms, mad = scaling.get("mscale"), scaling.get("mscale_all_dim")

            def yarn_ms(m):
                return 0.1 * float(m) * math.log(factor) + 1.0 if factor > 1 else 1.0
            if scaling.get("attention_factor") is not None:
                mscale = float(scaling["attention_factor"])
            elif ms and mad:
                mscale = yarn_ms(ms) / yarn_ms(mad)        # both given: only their ratio scales q and k
            else:
                mscale = yarn_ms(1.0)
        elif kind in ("longrope", "su"):
            # Phi-3 long context: per-pair divisors, the long set once the served context exceeds the
            # original training length (the short set otherwise), and a magnitude scale
            # sqrt(1 + ln(factor) / ln(original)) on the rotated q / k
            orig = float(scaling.get("original_max_position_embeddings") or 4096)
            total = float(scaling.get("max_position_embeddings") or max_pos or orig)
            use_long = (max_pos or total) > orig
            ext = torch.tensor(scaling["long_factor" if use_long else "short_factor"], dtype=torch.float64)
            inv = inv / ext[:half]
            f = float(scaling.get("factor") or total / orig)
            if scaling.get("attention_factor") is not None:
                mscale = float(scaling["attention_factor"])
            elif f > 1.0:
                mscale = math.sqrt(1.0 + math.log(f) / math.log(orig))
        elif kind == "dynamic":
            # dynamic NTK: the base grows with the served context beyond the original length
            orig = float(scaling.get("original_max_position_embeddings") or max_pos or 0)
            if max_pos and orig and max_pos > orig and head_dim_rot > 2:
                base = theta * ((factor * max_pos / orig) - (factor - 1)) ** (head_dim_rot / (head_dim_rot - 2))
                inv = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim_rot))
        elif kind in ("default", None):
            pass
        else:
            raise ValueError(f"unsupported rope scaling {kind}")
    return inv.to(torch.float32), float(mscale)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rot_dim: int,
               traditional: bool, mscale: float = 1.0) -> torch.Tensor:
    """x: [T, H, D] (any float dtype) → rotated fp32 tensor."""
    xf = x.float()
    half = rot_dim // 2
    if half == 0:                                   # a layer without positional encoding
        return xf * mscale
    ang = positions.float()[:, None] * inv_freq.float()[None, :half]  # [T, half]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = xf.clone()
    if traditional:
        a, b = xf[..., 0:rot_dim:2], xf[..., 1:rot_dim:2]
        out[..., 0:rot_dim:2] = a * cos - b * sin
        out[..., 1:rot_dim:2] = b * cos + a * sin
    else:
        a, b = xf[..., :half], xf[..., half:rot_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rot_dim] = b * cos + a * sin
    return out * mscale


def apply_mrope(x: torch.Tensor, positions3: torch.Tensor, inv_freq: torch.Tensor, sections, mscale: float = 1.0,
                interleaved: bool = False, rot_dim: int | None = None, traditional: bool = False) -> torch.Tensor:
    """Multimodal rotary embedding (Qwen2-VL): ``positions3`` [3, T] holds temporal / height / width
    positions; frequency i of the rotated width's half takes the position of the section it falls in
    (``sections`` = frequencies per component, e.g. [16, 24, 24]; further sections cycle T H W again).
    ``interleaved`` (Qwen3-VL, Qwen3.5): the components alternate T H W T H W ... over the first
    3 * sections[1] (height) and 3 * sections[2] (width) frequencies and the rest are temporal, instead
    of contiguous chunks. ``rot_dim`` rotates only the head's first columns (GLM-4V: half of each head);
    ``traditional`` pairs columns (2i, 2i + 1) instead of (i, i + rot_dim / 2). x: [T, H, D] → fp32."""
    xf = x.float()
    rd = int(rot_dim or xf.shape[-1])
    half = rd // 2
    if interleaved:
        which = torch.zeros(half, dtype=torch.long, device=xf.device)
        for comp, offset in ((1, 1), (2, 2)):
            which[offset:int(sections[comp]) * 3:3] = comp
    else:
        which = torch.repeat_interleave(torch.arange(len(sections), device=xf.device) % 3,
                                        torch.tensor(list(sections), device=xf.device))[:half]  # [half] -> 0/1/2
    pos = positions3.float().to(xf.device)[which]                   # [half, T]
    ang = pos.t() * inv_freq.float()[None, :half]                   # [T, half]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if traditional:
        a, b = xf[..., 0:rd:2], xf[..., 1:rd:2]
        rot = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    else:
        a, b = xf[..., :half], xf[..., half:rd]
        rot = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    rot = rot * mscale
    return rot if rd == xf.shape[-1] else torch.cat([rot, xf[..., rd:]], dim=-1)


def head_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def quantize_kv8(x: torch.Tensor):
    """[..., D] float → (uint8 [..., D], meta bf16 [..., D/64, 2]) affine per group of 64."""
    D = x.shape[-1]
    g = x.float().reshape(*x.shape[:-1], D // 64, 64)
    mn, mx = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = ((mx - mn) / 255.0).to(torch.bfloat16).float()
    bias = mn.to(torch.bfloat16).float()
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.round((g - bias) / scale).clamp(0, 255).to(torch.uint8)
    meta = torch.cat([scale, bias], dim=-1).to(torch.bfloat16)
    return q.reshape(x.shape), meta


def quantize_kv4(x: torch.Tensor):
    """[..., D] float → (uint8 [..., D/2] with two 4-bit codes per byte, even element in the low
    nibble; meta bf16 [..., D/64, 2]) affine per group of 64 with 16 levels."""
    D = x.shape[-1]
    g = x.float().reshape(*x.shape[:-1], D // 64, 64)
    mn, mx = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = ((mx - mn) / 15.0).to(torch.bfloat16).float()
    bias = mn.to(torch.bfloat16).float()
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.round((g - bias) / scale).clamp(0, 15).to(torch.uint8).reshape(*x.shape[:-1], D // 2, 2)
    packed = q[..., 0] | (q[..., 1] << 4)
    meta = torch.cat([scale, bias], dim=-1).to(torch.bfloat16)
    return packed, meta


def dequantize_kv4(packed: torch.Tensor, meta: torch.Tensor) -> torch.Tensor:
    q = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return dequantize_kv8(q, meta)


def dequantize_kv8(q: torch.Tensor, meta: torch.Tensor) -> torch.Tensor:
    D = q.shape[-1]
    g = q.float().reshape(*q.shape[:-1], D // 64, 64)
    m = meta.float()
    return (g * m[..., 0:1] + m[..., 1:2]).reshape(q.shape)


def rope_append(qkv, positions, slot_mapping, inv_freq, kv, *, Hq, Hkv, D, rot_dim, traditional,
                mscale=1.0, q_norm_w=None, k_norm_w=None, norm_eps=1e-6):
    """In place: rotates q inside ``qkv``; writes rotated k and v into the paged pool ``kv``."""
    T = qkv.shape[0]
    x = qkv.view(T, Hq + 2 * Hkv, D)
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]
    if q_norm_w is not None:
        q = head_rmsnorm(q, q_norm_w, norm_eps)
    if k_norm_w is not None:
        k = head_rmsnorm(k, k_norm_w, norm_eps)
    qr = apply_rope(q, positions, inv_freq, rot_dim, traditional, mscale)
    kr = apply_rope(k, positions, inv_freq, rot_dim, traditional, mscale)
    x[:, :Hq] = qr.to(qkv.dtype)
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    blk, off = slots // kv.block_size, slots % kv.block_size
    kw, vw = kr[valid], v[valid].float()
    if kv.kv_bits == 16:
        kv.k[blk, :, off] = kw.to(kv.k.dtype)
        kv.v[blk, :, off] = vw.to(kv.v.dtype)
    else:
        qz = quantize_kv4 if kv.kv_bits == 4 else quantize_kv8
        kq, km = qz(kw)
        vq, vm = qz(vw)
        kv.k[blk, :, off] = kq
        kv.v[blk, :, off] = vq
        kv.k_meta[blk, :, off] = km
        kv.v_meta[blk, :, off] = vm


def _gather_kv(kv, table: torch.Tensor, n: int):
    """Dense fp32 K, V [Hkv, n, D] of one sequence from its block table."""
    nb = (n + kv.block_size - 1) // kv.block_size
    idx = table[:nb].long()
    if kv.kv_bits == 16:
        k = kv.k[idx].float()
        v = kv.v[idx].float()
    else:
        dq = dequantize_kv4 if kv.kv_bits == 4 else dequantize_kv8
        k = dq(kv.k[idx], kv.k_meta[idx])
        v = dq(kv.v[idx], kv.v_meta[idx])
    # [nb, Hkv, bs, D] -> [Hkv, nb*bs, D]
    k = k.permute(1, 0, 2, 3).reshape(k.shape[1], -1, k.shape[-1])[:, :n]
    v = v.permute(1, 0, 2, 3).reshape(v.shape[1], -1, v.shape[-1])[:, :n]
    return k, v


def paged_attention(q, kv, block_tables, context_lens, cu_q, *, Hq, Hkv, D, scale, window=0,
                    sinks=None, softcap=0.0):
    """General paged attention. q: [T, Hq*D] (rows may be strided views); sequence s owns rows
    [cu_q[s], cu_q[s+1]) = the last q_len tokens of its context_lens[s] tokens. Returns [T, Hq*D]."""
    T = q.shape[0]
    out = torch.zeros(T, Hq * D, dtype=q.dtype, device=q.device)
    G = Hq // Hkv
    cu = cu_q.tolist()
    lens = context_lens.tolist()
    for s in range(len(lens)):
        q0, q1 = cu[s], cu[s + 1]
        ql, n = q1 - q0, lens[s]
        if ql == 0:
            continue
        k, v = _gather_kv(kv, block_tables[s], n)              # [Hkv, n, D]
        qs = q[q0:q1].float().reshape(ql, Hkv, G, D).permute(1, 2, 0, 3)  # [Hkv, G, ql, D]
        sc = torch.einsum("hgqd,hkd->hgqk", qs, k) * scale
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        qpos = torch.arange(n - ql, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        vis = kpos <= qpos
        if window > 0:
            vis = vis & (kpos > qpos - window)
        sc = sc.masked_fill(~vis[None, None], float("-inf"))
        if sinks is not None:
            sk = sinks.float().reshape(Hkv, G, 1, 1).expand(Hkv, G, ql, 1)
            full = torch.cat([sc, sk], dim=-1)
            p = torch.softmax(full, dim=-1)[..., :-1]
        else:
            p = torch.softmax(sc, dim=-1)
        o = torch.einsum("hgqk,hkd->hgqd", p, v)               # [Hkv, G, ql, D]
        out[q0:q1] = o.permute(2, 0, 1, 3).reshape(ql, Hq * D).to(q.dtype)
    return out


def embedding(ids, table, scale: float = 1.0):
    ok = (ids >= 0) & (ids < table.shape[0])
    out = table[ids.clamp(0, table.shape[0] - 1).long()]
    out = torch.where(ok[:, None], out, torch.zeros_like(out))
    if scale != 1.0:
        out = (out.float() * scale).to(table.dtype)
    return out


def argmax(logits):
    l = torch.nan_to_num(logits.float(), nan=float("-inf"))
    return l.argmax(-1).to(torch.int32)


# ----------------------------------------------------------------------------- sampling
def philox4x32_10(counter, key):
    """Vectorised Philox-4x32-10 over int64-held uint32 lanes. counter: [N,4], key: [2]."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    c = [counter[:, i].clone().to(torch.int64) & mask for i in range(4)]
    k0, k1 = int(key[0]) & mask, int(key[1]) & mask

    def mulhilo(a: int, b: torch.Tensor):
        # 32x32 -> 64 without overflowing int64: split b into 16-bit halves
        b_lo, b_hi = b & 0xFFFF, b >> 16
        p0 = a * b_lo                     # < 2^48
        p1 = a * b_hi                     # < 2^48
        lo = (p0 + ((p1 & 0xFFFF) << 16)) & mask
        carry = (p0 + ((p1 & 0xFFFF) << 16)) >> 32
        hi = ((p1 >> 16) + carry) & mask
        return hi, lo

    for _ in range(10):
        hi0, lo0 = mulhilo(M0, c[0])
        hi1, lo1 = mulhilo(M1, c[2])
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return torch.stack(c, dim=1)


def gumbel_noise(V: int, seed: int, step: int, device="cpu") -> torch.Tensor:
    ng = (V + 3) // 4
    ctr = torch.zeros(ng, 4, dtype=torch.int64)
    ctr[:, 0] = torch.arange(ng)
    ctr[:, 2] = step & 0xFFFFFFFF
    ctr[:, 3] = (step >> 32) & 0xFFFFFFFF
    r = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)).reshape(-1)[:V]
    u = ((r >> 8).to(torch.float32) + 0.5) * (1.0 / 16777216.0)
    return (-torch.log(-torch.log(u))).to(device)


def filter_mask(logits_row: torch.Tensor, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """Kept-token mask of the top-k → top-p → min-p chain on the untempered distribution."""
    l = torch.nan_to_num(logits_row.float(), nan=float("-inf"))
    V = l.numel()
    keep = torch.ones(V, dtype=torch.bool, device=l.device)
    m = l.max()
    e = torch.exp(l - m)
    if 0 < top_k < V:
        kth = torch.topk(l, top_k).values[-1]
        keep &= l >= kth
    if top_p < 1.0:
        mass = (e * keep).sum()
        order = torch.argsort(l, descending=True, stable=True)
        es = (e * keep)[order]
        ls = l[order]
        cum = torch.cumsum(es.double(), 0)
        # smallest threshold value whose ">= value" set reaches top_p * mass
        reach = cum >= top_p * mass.double() - 1e-12
        first = int(torch.nonzero(reach)[0]) if reach.any() else V - 1
        thr = ls[first]
        keep &= l >= thr
    if min_p > 0.0:
        keep &= l >= m + math.log(min_p)
    keep[l.argmax()] = True
    return keep


def typical_mask(l: torch.Tensor, keep: torch.Tensor, typical_p: float) -> torch.Tensor:
    """Locally typical filter on the kept distribution: rank by |(-log p) - H|, keep the smallest
    set whose mass reaches ``typical_p`` (the most likely token always stays)."""
    lk = torch.where(keep & (l > float("-inf")), l, torch.full_like(l, float("-inf")))
    logp = torch.log_softmax(lk.double(), 0)
    p = logp.exp()
    ent = -(p * torch.where(p > 0, logp, torch.zeros_like(logp))).sum()
    dev = torch.where(p > 0, (-logp - ent).abs(), torch.full_like(logp, float("inf")))
    order = torch.argsort(dev, stable=True)
    cum = torch.cumsum(p[order], 0)
    last = int((cum < typical_p).sum())
    out = torch.zeros_like(keep)
    out[order[: last + 1]] = True
    # tokens tied with the cut belong to the set as well (the kernel cuts by value, not by rank)
    out |= (dev <= dev[order[min(last, dev.numel() - 1)]]) & (p > 0)
    out[l.argmax()] = True
    return out & keep


def sigma_mask(l: torch.Tensor, n_sigma: float) -> torch.Tensor:
    fin = l[torch.isfinite(l)]
    if fin.numel() < 2:
        return torch.ones_like(l, dtype=torch.bool)
    return l >= l.max() - n_sigma * fin.std()


def sample(logits, temperature, top_k, top_p, min_p, seeds, steps, typical_p=None, top_n_sigma=None):
    """Row-wise sampler with the same Philox/Gumbel stream as the CUDA kernel."""
    B, V = logits.shape
    toks = torch.zeros(B, dtype=torch.int32)
    lps = torch.zeros(B, dtype=torch.float32)
    for b in range(B):
        l = torch.nan_to_num(logits[b].float().cpu(), nan=float("-inf"))
        logz = torch.logsumexp(l, 0)
        T = float(temperature[b])
        k = int(top_k[b])
        if not T > 0 or k == 1:
            t = int(l.argmax())
        else:
            keep = filter_mask(l, k, float(top_p[b]), float(min_p[b]))
            if top_n_sigma is not None and float(top_n_sigma[b]) > 0:
                keep &= sigma_mask(l, float(top_n_sigma[b]))
                keep[l.argmax()] = True
            if typical_p is not None and float(typical_p[b]) < 1.0:
                keep = typical_mask(l, keep, float(typical_p[b]))
            g = gumbel_noise(V, int(seeds[b]), int(steps[b]))
            score = torch.where(keep & (l > float("-inf")), l / T + g, torch.full_like(l, float("-inf")))
            t = int(score.argmax())
        toks[b] = t
        lps[b] = l[t] - logz
    return toks.to(logits.device), lps.to(logits.device)


def apply_penalties(logits, history, rep, freq, pres):
    out = logits.float().clone()
    B, V = out.shape
    for b in range(B):
        h = history[b]
        h = h[(h >= 0) & (h < V)].long()
        if h.numel() == 0:
            continue
        uniq, cnt = torch.unique(h, return_counts=True)
        l = out[b, uniq]
        r = float(rep[b])
        if r != 1.0:
            l = torch.where(l > 0, l / r, l * r)
        l = l - float(freq[b]) * cnt.float() - float(pres[b])
        out[b, uniq] = l
    return out.to(logits.dtype)


def spec_verify(logits, draft):
    """logits [B, K, V], draft [B, K-1] → (target [B,K], accept_len [B], next_token [B])."""
    target = argmax(logits.reshape(-1, logits.shape[-1])).reshape(logits.shape[0], logits.shape[1])
    B, K = target.shape
    acc = torch.zeros(B, dtype=torch.int32, device=logits.device)
    nxt = torch.zeros(B, dtype=torch.int32, device=logits.device)
    for b in range(B):
        a = 0
        while a < K - 1 and int(draft[b, a]) == int(target[b, a]):
            a += 1
        acc[b] = a
        nxt[b] = target[b, a]
    return target, acc, nxt
