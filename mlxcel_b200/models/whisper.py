"""Whisper speech-to-text: audio encoder + autoregressive text decoder with cross-attention.

Encoder: two 1-D convolutions (kernel 3; the second with stride 2) with GELU over the log-mel
frames, fixed sinusoidal positions, pre-LayerNorm transformer blocks, final LayerNorm: 3000 mel
frames (30 s) become 1500 states. Decoder: token + learned position embeddings, pre-LayerNorm blocks
of causal self-attention, cross-attention over the encoder states and a GELU MLP; the output
projection is the transposed token embedding. Greedy decoding keeps a preallocated self-attention
KV cache per layer and computes the cross-attention keys / values once per chunk
(reference: src/audio/encoder.rs, src/audio/attention.rs, src/models/whisper*.rs).

The convolutions run as GEMMs over unfolded frames and every projection goes through
``ops.linear`` (the tcgen05 GEMM on a GPU); the attention products use PyTorch's
``scaled_dot_product_attention`` (1500 x 1500 per chunk in the encoder, at most 448 query rows in
the decoder).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops


@dataclass
class WhisperConfig:
    d_model: int = 384
    n_mels: int = 80
    enc_layers: int = 4
    enc_heads: int = 6
    dec_layers: int = 4
    dec_heads: int = 6
    enc_ffn: int = 1536
    dec_ffn: int = 1536
    vocab_size: int = 51865
    max_source_positions: int = 1500
    max_target_positions: int = 448
    act: str = "gelu"
    decoder_start_token_id: int = 50258
    eos_token_id: int = 50257

    @staticmethod
    def from_dict(r: dict) -> "WhisperConfig":
        return WhisperConfig(
            d_model=int(r["d_model"]), n_mels=int(r.get("num_mel_bins", 80)), enc_layers=int(r["encoder_layers"]),
            enc_heads=int(r["encoder_attention_heads"]), dec_layers=int(r["decoder_layers"]),
            dec_heads=int(r["decoder_attention_heads"]), enc_ffn=int(r["encoder_ffn_dim"]), dec_ffn=int(r["decoder_ffn_dim"]),
            vocab_size=int(r["vocab_size"]), max_source_positions=int(r.get("max_source_positions", 1500)),
            max_target_positions=int(r.get("max_target_positions", 448)),
            act={"gelu": "gelu", "gelu_new": "gelu_tanh"}.get(r.get("activation_function", "gelu"), "gelu"),
            decoder_start_token_id=int(r.get("decoder_start_token_id", 50258)), eos_token_id=int(r.get("eos_token_id", 50257)))


class _Attn:
    """Projection weights of one attention (q / v / out with bias, k without)."""

    def __init__(self, t, p):
        self.wq, self.bq = t(p + "q_proj.weight"), t(p + "q_proj.bias")
        self.wk = t(p + "k_proj.weight")
        self.wv, self.bv = t(p + "v_proj.weight"), t(p + "v_proj.bias")
        self.wo, self.bo = t(p + "out_proj.weight"), t(p + "out_proj.bias")
        # self-attention projects q, k, v of the same rows in one GEMM
        self.wqkv = torch.cat([self.wq, self.wk, self.wv]).contiguous()
        self.bqkv = torch.cat([self.bq, torch.zeros_like(self.bq), self.bv]).contiguous()
        self.wkv = torch.cat([self.wk, self.wv]).contiguous()
        self.bkv = torch.cat([torch.zeros_like(self.bv), self.bv]).contiguous()


class WhisperModel:
    def __init__(self, cfg: WhisperConfig, tensors: dict, dtype=torch.bfloat16, device="cpu", *, encoder_only: bool = False,
                 prefix: str | None = None):
        """``encoder_only`` builds the audio encoder alone (speech-language models keep a Whisper encoder
        in front of a projector and a text decoder); ``prefix`` names where its tensors live."""
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        pre = prefix if prefix is not None else ("model." if any(k.startswith("model.") for k in tensors) else "")

        def t(n):
            return tensors[pre + n].to(dtype).to(self.device).contiguous()

        def ln(p):
            return t(p + ".weight"), t(p + ".bias")

        e = "" if encoder_only else "encoder."
        # conv weights [out, in, 3] -> GEMM weights over frames unfolded as (tap, channel)
        self.c1w = t(e + "conv1.weight").permute(0, 2, 1).reshape(cfg.d_model, -1).contiguous()
        self.c1b = t(e + "conv1.bias")
        self.c2w = t(e + "conv2.weight").permute(0, 2, 1).reshape(cfg.d_model, -1).contiguous()
        self.c2b = t(e + "conv2.bias")
        self.enc_pos = t(e + "embed_positions.weight")
        self.enc = [dict(attn=_Attn(t, f"{e}layers.{i}.self_attn."), ln1=ln(f"{e}layers.{i}.self_attn_layer_norm"),
                         w1=t(f"{e}layers.{i}.fc1.weight"), b1=t(f"{e}layers.{i}.fc1.bias"),
                         w2=t(f"{e}layers.{i}.fc2.weight"), b2=t(f"{e}layers.{i}.fc2.bias"),
                         ln2=ln(f"{e}layers.{i}.final_layer_norm")) for i in range(cfg.enc_layers)]
        self.enc_ln = ln(e + "layer_norm")
        if encoder_only:
            return
        d = "decoder."
        self.tok = t(d + "embed_tokens.weight")
        self.dec_pos = t(d + "embed_positions.weight")
        self.dec = [dict(attn=_Attn(t, f"{d}layers.{i}.self_attn."), ln1=ln(f"{d}layers.{i}.self_attn_layer_norm"),
                         cross=_Attn(t, f"{d}layers.{i}.encoder_attn."), lnx=ln(f"{d}layers.{i}.encoder_attn_layer_norm"),
                         w1=t(f"{d}layers.{i}.fc1.weight"), b1=t(f"{d}layers.{i}.fc1.bias"),
                         w2=t(f"{d}layers.{i}.fc2.weight"), b2=t(f"{d}layers.{i}.fc2.bias"),
                         ln2=ln(f"{d}layers.{i}.final_layer_norm")) for i in range(cfg.dec_layers)]
        self.dec_ln = ln(d + "layer_norm")
        head = tensors["proj_out.weight"].to(dtype).to(self.device) if "proj_out.weight" in tensors else self.tok
        # the GEMM writes rows of 16-byte multiples: pad the vocabulary to a multiple of 8, cut the logits back
        self.head = F.pad(head, (0, 0, 0, (-head.shape[0]) % 8)).contiguous()

    @staticmethod
    def from_pretrained(path: str | Path, dtype=torch.bfloat16, device="cpu") -> "WhisperModel":
        from ..loading.checkpoint import TensorSource
        path = Path(path)
        cfg = WhisperConfig.from_dict(json.loads((path / "config.json").read_text()))
        src = TensorSource(path)
        tensors = {k: src.get(k) for k in src.keys()}
        m = WhisperModel(cfg, tensors, dtype, device)
        g = path / "generation_config.json"
        m.generation = json.loads(g.read_text()) if g.exists() else {}
        return m

    # ------------------------------------------------------------------ encoder
    def _conv(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, stride: int) -> torch.Tensor:
        """[B, T, C] → [B, T / stride, d_model]: kernel-3 convolution with padding 1 as one GEMM."""
        B, T, C = x.shape
        xp = F.pad(x, (0, 0, 1, 1))
        cols = xp.unfold(1, 3, stride)                            # [B, T/stride, C, 3]
        cols = cols.permute(0, 1, 3, 2).reshape(B * cols.shape[1], 3 * C).contiguous()
        y = rops.activation(ops.linear(cols, w, bias=b), "gelu")
        return y.view(B, -1, w.shape[0])

    def _mha(self, q, k, v, heads: int, causal: bool = False, key_len: int | None = None) -> torch.Tensor:
        """q [B, Tq, d], k / v [B, Tk, d] → [B * Tq, d]. ``key_len`` hides the keys from that index on
        (the zero-padded tail of a clip shorter than its chunk)."""
        B, Tq, d = q.shape
        D = d // heads
        sp = lambda z: z.reshape(B, -1, heads, D).transpose(1, 2)    # noqa: E731
        mask = None
        if key_len is not None and key_len < k.shape[1]:
            mask = (torch.arange(k.shape[1], device=q.device) < key_len).view(1, 1, 1, -1)
        o = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), attn_mask=mask, is_causal=causal and Tq > 1)
        return o.transpose(1, 2).reshape(B * Tq, d).contiguous()

    @torch.no_grad()
    def encode(self, mel: torch.Tensor, key_len: int | None = None, final_norm: bool = True) -> torch.Tensor:
        """[B, n_mels, frames] → [B, frames / 2, d_model]."""
        c = self.cfg
        x = mel.to(self.device, self.dtype).transpose(1, 2).contiguous()
        x = self._conv(self._conv(x, self.c1w, self.c1b, 1), self.c2w, self.c2b, 2)
        B, T, d = x.shape
        h = (x.float() + self.enc_pos[:T].float()).to(self.dtype).reshape(B * T, d).contiguous()
        for L in self.enc:
            a = L["attn"]
            y = rops.layernorm(h, *L["ln1"], 1e-5)
            qkv = ops.linear(y, a.wqkv, bias=a.bqkv).view(B, T, 3, d)
            o = self._mha(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], c.enc_heads, key_len=key_len)
            h = ops.linear(o, a.wo, bias=a.bo, residual=h)
            y = rops.layernorm(h, *L["ln2"], 1e-5)
            h = ops.linear(rops.activation(ops.linear(y, L["w1"], bias=L["b1"]), c.act), L["w2"], bias=L["b2"], residual=h)
        return (rops.layernorm(h, *self.enc_ln, 1e-5) if final_norm else h).view(B, T, d)

    # ------------------------------------------------------------------ decoder
    def _cross_kv(self, enc: torch.Tensor):
        B, S, d = enc.shape
        flat = enc.reshape(B * S, d).contiguous()
        out = []
        for L in self.dec:
            kv = ops.linear(flat, L["cross"].wkv, bias=L["cross"].bkv).view(B, S, 2, d)
            out.append((kv[:, :, 0].contiguous(), kv[:, :, 1].contiguous()))
        return out

    def _decode_rows(self, tokens: torch.Tensor, start: int, cache, cross) -> torch.Tensor:
        """Run ``tokens`` [B, T] at positions start .. start+T; appends to the self-attention cache.
        Returns the logits of every row [B, T, vocab] (fp32)."""
        c = self.cfg
        B, T = tokens.shape
        d = c.d_model
        h = (self.tok[tokens].float() + self.dec_pos[start:start + T].float()).to(self.dtype).reshape(B * T, d).contiguous()
        for li, L in enumerate(self.dec):
            a, x = L["attn"], L["cross"]
            y = rops.layernorm(h, *L["ln1"], 1e-5)
            qkv = ops.linear(y, a.wqkv, bias=a.bqkv).view(B, T, 3, d)
            kc, vc = cache[li]
            kc[:, start:start + T] = qkv[:, :, 1]
            vc[:, start:start + T] = qkv[:, :, 2]
            if T > 1:       # prompt rows: causal inside the block, everything before it visible
                D = d // c.dec_heads
                sp = lambda z: z.reshape(B, -1, c.dec_heads, D).transpose(1, 2)    # noqa: E731
                mask = torch.ones(T, start + T, dtype=torch.bool, device=h.device).tril(diagonal=start)
                o = F.scaled_dot_product_attention(sp(qkv[:, :, 0]), sp(kc[:, :start + T]), sp(vc[:, :start + T]), attn_mask=mask)
                o = o.transpose(1, 2).reshape(B * T, d).contiguous()
            else:
                o = self._mha(qkv[:, :, 0], kc[:, :start + 1], vc[:, :start + 1], c.dec_heads)
            h = ops.linear(o, a.wo, bias=a.bo, residual=h)
            y = rops.layernorm(h, *L["lnx"], 1e-5)
            q = ops.linear(y, x.wq, bias=x.bq).view(B, T, d)
            o = self._mha(q, cross[li][0], cross[li][1], c.dec_heads)
            h = ops.linear(o, x.wo, bias=x.bo, residual=h)
            y = rops.layernorm(h, *L["ln2"], 1e-5)
            h = ops.linear(rops.activation(ops.linear(y, L["w1"], bias=L["b1"]), c.act), L["w2"], bias=L["b2"], residual=h)
        h = rops.layernorm(h, *self.dec_ln, 1e-5)
        logits = ops.linear(h, self.head, out_fp32=True) if h.is_cuda else h.float() @ self.head.float().t()
        return logits[:, : c.vocab_size].reshape(B, T, c.vocab_size)

    @torch.no_grad()
    def generate(self, mel: torch.Tensor, prompt: list[int], max_new_tokens: int = 224, suppress: list[int] | None = None,
                 begin_suppress: list[int] | None = None, eos: int | None = None) -> list[list[int]]:
        """Greedy decoding of every chunk of ``mel`` [B, n_mels, frames] after the forced ``prompt``
        (start-of-transcript, language, task, timestamp mode). ``suppress``: ids never produced;
        ``begin_suppress``: ids not allowed as the first generated token."""
        c = self.cfg
        eos = c.eos_token_id if eos is None else eos
        enc = self.encode(mel)
        B = enc.shape[0]
        cross = self._cross_kv(enc)
        Tmax = c.max_target_positions
        cache = [(torch.zeros(B, Tmax, c.d_model, dtype=self.dtype, device=self.device),
                  torch.zeros(B, Tmax, c.d_model, dtype=self.dtype, device=self.device)) for _ in self.dec]
        toks = torch.tensor([prompt] * B, dtype=torch.long, device=self.device)
        logits = self._decode_rows(toks, 0, cache, cross)[:, -1]
        out = [[] for _ in range(B)]
        done = [False] * B
        pos = len(prompt)
        sup = torch.tensor(sorted(set(suppress or [])), dtype=torch.long, device=self.device)
        bsup = torch.tensor(sorted(set(begin_suppress or [])), dtype=torch.long, device=self.device)
        for step in range(min(max_new_tokens, Tmax - len(prompt))):
            if sup.numel():
                logits[:, sup] = float("-inf")
            if step == 0 and bsup.numel():
                logits[:, bsup] = float("-inf")
            nxt = logits.argmax(-1)
            for b, tkn in enumerate(nxt.tolist()):
                if not done[b]:
                    if tkn == eos:
                        done[b] = True
                    else:
                        out[b].append(tkn)
            if all(done):
                break
            logits = self._decode_rows(nxt[:, None], pos, cache, cross)[:, -1]
            pos += 1
        return out
