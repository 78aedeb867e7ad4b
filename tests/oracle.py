"""Independent PyTorch-CPU f32 statement of the Llama-3 math (HF-transformers semantics):
RMSNorm eps → separate q/k/v projections → half-split RoPE → GQA SDPA with dense KV → o_proj →
SwiGLU → tied LM head, greedy argmax. It shares no code with mlxcel_b200's executor: dense
KV tensors, whole-sequence recompute per step."""
import math

import torch


def oracle_greedy(cfg, w, prompt, n_new):
    """cfg: ModelConfig, w: ModelWeights (full, unsharded, float32). Returns n_new greedy tokens."""
    H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    G = Hq // Hkv
    half = D // 2
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float32) * 2 / D))

    def rms(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g

    def rope(x, pos):  # x [T, h, D]
        ang = pos[:, None].float() * inv[None]
        c, s = ang.cos()[:, None], ang.sin()[:, None]
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    toks = list(prompt)
    out = []
    for _ in range(n_new):
        ids = torch.tensor(toks)
        T = len(toks)
        pos = torch.arange(T)
        h = w.embed.float()[ids]
        for lw in w.layers:
            x = rms(h, lw.ln1.float())
            qkv = x @ lw.wqkv.float().t()
            q = qkv[:, : Hq * D].view(T, Hq, D)
            k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
            v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
            q, k = rope(q, pos), rope(k, pos)
            k = k.repeat_interleave(G, dim=1)
            v = v.repeat_interleave(G, dim=1)
            sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
            mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
            sc = sc.masked_fill(~mask, float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(T, Hq * D)
            h = h + a @ lw.wo.float().t()
            x = rms(h, lw.ln2.float())
            gu = x @ lw.w_gate_up.float().t()
            I = gu.shape[1] // 2
            h = h + (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]) @ lw.w_down.float().t()
        x = rms(h[-1:], w.final_norm.float())
        logits = x @ w.lm_head.float().t()
        t = int(logits.argmax())
        out.append(t)
        toks.append(t)
    return out
