"""Host prompt-cache tier: snapshot → evict from the pool → restore; tokens must not change."""
import torch

from mlxcel_b200.cache.prompt_cache import PromptCacheStore, adopt_snapshot, snapshot_sequence
from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams, Sequence
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights


def test_store_policy():
    st = PromptCacheStore(block_size=4, max_bytes=100)
    from mlxcel_b200.cache.prompt_cache import Snapshot
    sc = st.scope("m")
    assert st.put(sc, Snapshot(list(range(8)), [], 60))
    assert st.put(sc, Snapshot(list(range(100, 112)), [], 60))      # evicts the first (LRU)
    assert st.stats["evictions"] == 1 and st.bytes == 60
    snap, n = st.lookup(sc, list(range(100, 112)) + [7])
    assert snap is not None and n == 12
    snap, n = st.lookup(sc, list(range(100, 108)) + [9, 9, 9, 9, 9])  # shares two blocks
    assert n == 8
    assert st.lookup(st.scope("other"), list(range(100, 113)))[0] is None
    assert not st.put(sc, Snapshot([1] * 4, [], 1000))


def test_snapshot_restore_roundtrip():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=2, dtype=torch.float32, std=0.05)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=32,
                                                         max_model_len=256, cuda_graphs=False))
    prompt = list(range(50))
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    sid = eng.add_request(prompt, sp)
    snap = None
    while eng.has_work():
        eng.step()
        s = eng.seqs[sid]
        if snap is None and s.num_computed >= 48 and eng.bm.has_seq(sid):
            snap = snapshot_sequence(eng, s)
    want = eng.seqs[sid].output
    assert snap is not None and len(snap.tokens) == 48
    store = PromptCacheStore(block_size=16)
    store.put(store.scope("tiny"), snap)
    eng.bm.reset_prefix_cache()                      # the pool forgets everything
    hit, n = store.lookup(store.scope("tiny"), prompt)
    assert n == 48
    sid2 = eng.add_request(prompt, sp)
    s2 = eng.seqs[sid2]
    assert adopt_snapshot(eng, s2, hit, n) == 48
    while eng.has_work():
        eng.step()
    assert s2.output == want and s2.num_cached == 48 and eng.stats["prefill_tokens"] < 2 * 50


def test_kv_handoff_between_engines():
    """Disaggregated roles: engine A prefills and exports a prompt's KV blocks, engine B imports the
    blob and generates from the cache with the same result as a local run."""
    from mlxcel_b200.engine.handoff import export_prefix, import_prefix, parse_blob

    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=2, dtype=torch.float32, std=0.05)

    def engine():
        return Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=32,
                                                              max_model_len=256, cuda_graphs=False))

    prompt = list(range(3, 60))
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a, b = engine(), engine()
    want = a.generate([prompt], sp)[0].output
    a.bm.reset_prefix_cache()
    blob = export_prefix(a, prompt)
    head, snap = parse_blob(blob)
    assert len(snap.tokens) == 48 and head["geometry"]["layers"] == cfg.num_hidden_layers
    assert import_prefix(b, blob) == 48
    out = b.generate([prompt], sp)[0]
    assert out.output == want and out.num_cached == 48
    other = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=32,
                                                           max_model_len=256, cuda_graphs=False, block_size=32))
    import pytest
    with pytest.raises(ValueError):
        import_prefix(other, blob)
