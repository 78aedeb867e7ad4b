"""Speculative decoding: drafters (prompt lookup, draft model, MTP head) behind one interface.

A drafter proposes up to K-1 tokens per decoding row; ``Engine._spec_step`` verifies them with
one target forward and keeps the longest prefix that equals the target's greedy tokens
(lossless for greedy decoding: output is token-identical to plain decoding).
"""
from .prompt_lookup import PromptLookupDrafter  # noqa: F401
from .draft_model import DraftModelDrafter  # noqa: F401
from .mtp import MTPDrafter, MTPWeights, random_mtp_weights  # noqa: F401
from .policy import SpecPolicy, exactness_probe  # noqa: F401
from .dflash import DFlashDrafter, DFlashWeights, random_dflash_weights  # noqa: F401


class Drafter:
    needs_hidden = False

    def propose(self, engine, seqs, max_draft: int) -> list[list[int]]:
        raise NotImplementedError

    def on_forward(self, engine, decode, pieces, hidden) -> None:
        pass

    def on_verify(self, engine, accepted_info, hidden) -> None:
        pass

    def release(self, seq_id: int) -> None:
        pass
