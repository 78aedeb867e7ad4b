"""Host-side prompt cache: KV snapshots that outlive the GPU block pool.

The block manager's chained-hash prefix index reuses KV that is still resident in the pool
(automatic prefix caching). This store is the second tier the reference keeps beside it
(src/server/prompt_cache/store.rs, trie.rs, key.rs, policy.rs): detached copies of a sequence's KV
blocks in host memory, keyed by (model, adapter, template signature, session) and looked up by
longest token prefix through a radix trie, with an LRU + TTL + byte-budget policy. A hit is
restored into freshly reserved blocks and re-registered in the prefix index, so the request then
proceeds exactly like an in-pool prefix hit.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field

import numpy as np


@dataclass
class Snapshot:
    tokens: list[int]                 # tokens covered (a whole number of blocks)
    blocks: list[dict]                # per layer: {"k": tensor, "v": tensor, ...} on the host
    nbytes: int
    created: float = field(default_factory=time.time)
    hits: int = 0


class _TrieNode:
    __slots__ = ("children", "entry")

    def __init__(self):
        self.children: dict[tuple, "_TrieNode"] = {}
        self.entry: str | None = None


class PromptCacheStore:
    def __init__(self, block_size: int = 16, max_bytes: int = 2 << 30, ttl_s: float = 3600.0):
        self.block_size, self.max_bytes, self.ttl_s = block_size, max_bytes, ttl_s
        self.entries: "OrderedDict[str, tuple[tuple, Snapshot]]" = OrderedDict()
        self.roots: dict[tuple, _TrieNode] = {}
        self.bytes = 0
        self.stats = dict(lookups=0, hits=0, hit_tokens=0, stores=0, evictions=0, rejects=0)
        self._n = 0

    # ------------------------------------------------------------------ keys
    @staticmethod
    def scope(model: str, adapter: str = "", template_sig: str = "", session: str = "") -> tuple:
        return (model, adapter, template_sig, session)

    def _chunks(self, tokens: list[int]):
        bs = self.block_size
        for i in range(0, len(tokens) - len(tokens) % bs, bs):
            yield tuple(tokens[i:i + bs])

    # ------------------------------------------------------------------ store / lookup
    def put(self, scope: tuple, snap: Snapshot) -> bool:
        if snap.nbytes > self.max_bytes or not snap.tokens:
            self.stats["rejects"] += 1
            return False
        self._expire()
        while self.bytes + snap.nbytes > self.max_bytes and self.entries:
            self._evict_lru()
        node = self.roots.setdefault(scope, _TrieNode())
        for ch in self._chunks(snap.tokens):
            node = node.children.setdefault(ch, _TrieNode())
        if node.entry is not None and node.entry in self.entries:
            self._drop(node.entry)
        self._n += 1
        eid = f"e{self._n}"
        node.entry = eid
        self.entries[eid] = (scope, snap)
        self.bytes += snap.nbytes
        self.stats["stores"] += 1
        return True

    def lookup(self, scope: tuple, tokens: list[int]) -> tuple[Snapshot | None, int]:
        """Longest stored prefix of ``tokens`` (whole blocks, leaving at least one token to compute).
        Returns (snapshot, usable token count)."""
        self.stats["lookups"] += 1
        self._expire()
        node = self.roots.get(scope)
        if node is None:
            return None, 0
        best, depth, n = None, 0, 0
        usable = (len(tokens) - 1) // self.block_size
        for ch in self._chunks(tokens[: usable * self.block_size]):
            node = node.children.get(ch)
            if node is None:
                break
            n += 1
            # any entry at or below this node covers these n blocks
            e = self._any_entry(node)
            if e is not None:
                best, depth = e, n
        if best is None:
            return None, 0
        scope_, snap = self.entries[best]
        self.entries.move_to_end(best)
        snap.hits += 1
        self.stats["hits"] += 1
        self.stats["hit_tokens"] += depth * self.block_size
        return snap, depth * self.block_size

    def _any_entry(self, node: _TrieNode) -> str | None:
        stack = [node]
        while stack:
            nd = stack.pop()
            if nd.entry is not None and nd.entry in self.entries:
                return nd.entry
            stack.extend(nd.children.values())
        return None

    # ------------------------------------------------------------------ policy
    def _drop(self, eid: str) -> None:
        scope, snap = self.entries.pop(eid)
        self.bytes -= snap.nbytes

    def _evict_lru(self) -> None:
        eid = next(iter(self.entries))
        self._drop(eid)
        self.stats["evictions"] += 1

    def _expire(self) -> None:
        now = time.time()
        for eid in [e for e, (_, s) in self.entries.items() if now - s.created > self.ttl_s]:
            self._drop(eid)
            self.stats["evictions"] += 1

    def reset(self) -> int:
        n = len(self.entries)
        self.entries.clear()
        self.roots.clear()
        self.bytes = 0
        return n


# ----------------------------------------------------------------------------- engine glue
def snapshot_sequence(engine, seq) -> Snapshot | None:
    """Detach the computed full blocks of a sequence into host memory."""
    bs = engine.ecfg.block_size
    n_full = seq.num_computed // bs
    if n_full == 0 or not engine.bm.has_seq(seq.seq_id):
        return None
    ids = engine.bm.seq_blocks(seq.seq_id)[:n_full]
    data = engine.pool.extract_blocks(ids)
    nbytes = sum(t.numel() * t.element_size() for layer in data for t in layer.values())
    return Snapshot(tokens=seq.tokens[: n_full * bs], blocks=data, nbytes=nbytes)


def adopt_snapshot(engine, seq, snap: Snapshot, n_tokens: int) -> int:
    """Restore the first ``n_tokens`` of a snapshot into fresh blocks of a not-yet-started sequence
    and register them in the prefix index. Returns the number of tokens adopted."""
    bs = engine.ecfg.block_size
    n_blocks = n_tokens // bs
    if n_blocks == 0:
        return 0
    if not engine.bm.has_seq(seq.seq_id):
        engine.bm.create(seq.seq_id, 0)
    have = engine.bm.seq_len(seq.seq_id)
    if have >= n_blocks * bs:
        return have
    if not engine.bm.reserve(seq.seq_id, n_blocks * bs):
        return 0
    ids = engine.bm.seq_blocks(seq.seq_id)[:n_blocks]
    first = have // bs
    data = [{k: v[first:n_blocks] for k, v in layer.items()} for layer in snap.blocks]
    engine.pool.restore_blocks(ids[first:], data)
    toks = np.asarray(snap.tokens[: n_blocks * bs], dtype=np.int32)
    engine.bm.commit(seq.seq_id, toks, n_blocks * bs)
    seq.num_computed = seq.num_cached = n_blocks * bs
    return n_blocks * bs
