"""Per-request sampling parameters and finish bookkeeping.

Field set follows the reference's ``SamplingConfig`` (src/lib/mlxcel-core/src/generate.rs:1236-1653)
and the OpenAI / llama-server request fields it accepts (src/server/types/request.rs:725-1070).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum


class FinishReason(str, Enum):
    STOP = "stop"                # EOS or stop token
    STOP_SEQUENCE = "stop_sequence"
    LENGTH = "length"
    REPETITION_LOOP = "repetition_loop"
    CANCELLED = "cancelled"
    ERROR = "error"


class SeqStatus(str, Enum):
    QUEUED = "queued"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    FINISHED = "finished"
    PREEMPTED = "preempted"


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    typical_p: float = 1.0
    top_n_sigma: float = 0.0
    repetition_penalty: float = 1.0
    repetition_context_size: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_sequence_breakers: list[int] = field(default_factory=list)
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    mirostat: int = 0
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    dynatemp_range: float = 0.0
    dynatemp_exponent: float = 1.0
    seed: int | None = None
    stop_token_ids: list[int] = field(default_factory=list)
    stop: list[str] = field(default_factory=list)
    ignore_eos: bool = False
    logprobs: bool = False
    top_logprobs: int = 0
    logit_bias: dict[int, float] = field(default_factory=dict)
    min_tokens: int = 0
    # loop detection (src/lib/mlxcel-core/src/loop_detection.rs): stop when a pattern of
    # min..max tokens repeats at least `min_count` times at the tail
    loop_max_pattern: int = 0
    loop_min_pattern: int = 4
    loop_min_count: int = 8
    # Thinking-token budget (src/server/thinking_budget.rs): None or -1 = unbounded, 0 = the first
    # reasoning token is replaced by the end-of-thinking token, N > 0 = at most N tokens inside the
    # block (the opening token is not counted), after which the next token is forced to be the
    # end-of-thinking token. The ids come from the tokenizer (filled in by the front end).
    thinking_budget: int | None = None
    think_start_id: int | None = None
    think_end_id: int | None = None
    priority: int = 0

    @property
    def greedy(self) -> bool:
        """Greedy ⇔ top_k == 1 or (temperature == 0 and no dynamic temperature)
        (src/lib/mlxcel-core/src/generate.rs:1539-1543)."""
        return self.top_k == 1 or (self.temperature <= 0.0 and self.dynatemp_range <= 0.0)

    @property
    def thinking_cap(self) -> int | None:
        """Effective cap of the reasoning block, or None when nothing has to be enforced."""
        b = self.thinking_budget
        if b is None or int(b) < 0 or self.think_end_id is None:
            return None
        return int(b)

    @property
    def needs_history(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or
                self.presence_penalty != 0.0 or self.dry_multiplier > 0.0)

    @property
    def fused_eligible(self) -> bool:
        """Rows whose chain is bias/penalties → top-k/top-p/min-p/top-n-sigma → typical-p →
        temperature draw go through the fused CUDA sampler; the rest take the extended chain."""
        return (self.xtc_probability <= 0.0 and
                self.mirostat == 0 and self.dynatemp_range <= 0.0 and self.dry_multiplier <= 0.0 and
                not self.logit_bias and self.top_logprobs == 0)
