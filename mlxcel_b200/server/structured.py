"""Structured output: JSON schema / regex / Lark / GBNF constraints as per-step token masks.

The matcher is llguidance (the library the reference uses, src/server/structured.rs:15-35). A
constraint owns one matcher per request; the engine asks for a boolean mask over the vocabulary
before sampling (``mask_fn``) and reports the sampled token afterwards (``consume``) — the same
two hooks the reference's scheduler has (batch/scheduler/run_loop.rs:80-118). GBNF grammars are
lowered to Lark first (src/server/gbnf/*).
"""
from __future__ import annotations

import json
import re

import torch


def gbnf_to_lark(gbnf: str) -> str:
    """llama.cpp GBNF → Lark (llguidance dialect). Handles rule definitions, alternation,
    grouping, repetition operators, character classes and string literals; ``root`` becomes
    ``start``."""
    out = []
    rules = re.split(r"\n(?=[A-Za-z_][\w\-]*\s*::=)", gbnf.strip())
    for r in rules:
        r = re.sub(r"#.*", "", r).strip()
        if not r:
            continue
        name, body = r.split("::=", 1)
        name = name.strip().replace("-", "_")
        name = "start" if name == "root" else name.lower()
        body = " ".join(body.split())
        body = re.sub(r"\b([A-Za-z_][\w\-]*)\b(?=(?:[^\"]*\"[^\"]*\")*[^\"]*$)",
                      lambda m: ("start" if m.group(1) == "root" else m.group(1).replace("-", "_").lower()), body)
        body = re.sub(r"(\[[^\]]*\])", lambda m: "/" + m.group(1) + "/", body)
        out.append(f"{name}: {body}")
    return "\n".join(out)


class Constraint:
    def __init__(self, tokenizer, *, json_schema=None, regex: str | None = None, lark: str | None = None,
                 gbnf: str | None = None, json_object: bool = False):
        import llguidance
        import llguidance.hf

        # what rebuilds this constraint elsewhere (follower ranks of a multi-process engine)
        self.spec = dict(json_schema=json_schema, regex=regex, lark=lark, gbnf=gbnf, json_object=json_object)
        tk = getattr(tokenizer, "tk", None)
        if tk is None:
            raise ValueError("structured output needs an HF tokenizer")
        self.ll_tok = llguidance.hf.from_tokenizer(_as_transformers(tokenizer))
        if json_schema is not None:
            g = llguidance.LLMatcher.grammar_from_json_schema(
                json_schema if isinstance(json_schema, str) else json.dumps(json_schema))
        elif json_object:
            g = llguidance.LLMatcher.grammar_from_json_schema('{"type": "object"}')
        elif regex is not None:
            g = llguidance.LLMatcher.grammar_from_regex(regex)
        elif gbnf is not None:
            g = llguidance.LLMatcher.grammar_from_lark(gbnf_to_lark(gbnf))
        elif lark is not None:
            g = llguidance.LLMatcher.grammar_from_lark(lark)
        else:
            raise ValueError("no constraint given")
        self.matcher = llguidance.LLMatcher(self.ll_tok, g)
        err = self.matcher.get_error()
        if err:
            raise ValueError(f"invalid grammar: {err}")
        self.vocab = self.ll_tok.vocab_size
        self._consumed = 0
        self._eos = [i for i in (tokenizer.eos_ids() if hasattr(tokenizer, "eos_ids") else [])
                     if i is not None and 0 <= i < self.vocab]

    def mask(self, seq) -> torch.Tensor | None:
        """Boolean allow-mask [V] for the next token of ``seq`` (consumes tokens sampled since)."""
        import llguidance.torch as llt

        while self._consumed < len(seq.output):
            self.matcher.consume_token(seq.output[self._consumed])
            self._consumed += 1
        if self.matcher.is_stopped():
            # the grammar is complete: only an end-of-sequence token may follow, so the request ends
            # here instead of running on unconstrained
            if not self._eos:
                return None
            m = torch.zeros(self.vocab, dtype=torch.bool)
            m[self._eos] = True
            return m
        bits = llt.allocate_token_bitmask(1, self.vocab)
        llt.fill_next_token_bitmask(self.matcher, bits, 0)
        words = bits[0].to(torch.int64) & 0xFFFFFFFF
        idx = torch.arange(32, dtype=torch.int64)
        m = ((words[:, None] >> idx[None, :]) & 1).bool().reshape(-1)[: self.vocab]
        return m

    def finished(self) -> bool:
        return self.matcher.is_stopped()


def _as_transformers(tokenizer):
    from transformers import PreTrainedTokenizerFast

    return PreTrainedTokenizerFast(tokenizer_object=tokenizer.tk)


def constraint_from_request(tokenizer, response_format: dict | None = None, grammar: str | None = None,
                            json_schema=None, regex: str | None = None) -> Constraint | None:
    """OpenAI ``response_format`` / llama-server ``grammar`` + ``json_schema`` → Constraint."""
    if grammar:
        return Constraint(tokenizer, gbnf=grammar)
    if json_schema is not None:
        return Constraint(tokenizer, json_schema=json_schema)
    if regex:
        return Constraint(tokenizer, regex=regex)
    if response_format:
        t = response_format.get("type")
        if t == "json_object":
            return Constraint(tokenizer, json_object=True)
        if t == "json_schema":
            js = response_format.get("json_schema", {})
            return Constraint(tokenizer, json_schema=js.get("schema", js))
    return None
