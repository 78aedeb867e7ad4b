"""Engine policies on the CPU path: thinking-token budget, speculative rounds alternating with
classic work, and requests that exceed what the KV pool can hold."""
import pytest
import torch

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, FinishReason, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.speculative import DraftModelDrafter


def _engine(**kw):
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=4, dtype=torch.float32, std=0.05)
    base = dict(max_batch=4, max_num_batched_tokens=128, num_blocks=96, max_model_len=384, cuda_graphs=False)
    base.update(kw)
    return cfg, w, Engine(DecoderModel(cfg, w), cfg, EngineConfig(**base))


START, END = 1000, 1001    # stand-ins for <think> / </think> (the random model never needs to emit them)


def _prompt(cfg, n=12, seed=2):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 900, (n,), generator=g).tolist()


@pytest.mark.parametrize("budget", [0, 5])
def test_thinking_budget_forces_the_end_token(budget):
    """The prompt opens the reasoning block; after ``budget`` tokens inside it the next token is the
    end-of-thinking token, and sampling resumes normally afterwards (thinking_budget.rs value rules)."""
    cfg, w, eng = _engine()
    free = eng.generate([_prompt(cfg) + [START]], SamplingParams(max_tokens=12, ignore_eos=True))[0].output
    assert END not in free
    cfg, w, eng = _engine()
    sp = SamplingParams(max_tokens=12, ignore_eos=True, thinking_budget=budget, think_start_id=START, think_end_id=END)
    s = eng.generate([_prompt(cfg) + [START]], sp)[0]
    assert s.output[:budget] == free[:budget]            # untouched up to the cap
    assert s.output[budget] == END and s.think_forced == 1
    assert s.output.count(END) == 1 and len(s.output) == 12
    assert eng.stats["thinking_forced"] == 1


def test_thinking_budget_unbounded_and_outside_block():
    cfg, w, eng = _engine()
    base = eng.generate([_prompt(cfg)], SamplingParams(max_tokens=10, ignore_eos=True))[0].output
    for b in (None, -1):
        cfg, w, eng = _engine()
        sp = SamplingParams(max_tokens=10, ignore_eos=True, thinking_budget=b, think_start_id=START, think_end_id=END)
        assert eng.generate([_prompt(cfg) + [START]], sp)[0].think_forced == 0
    # a budget without an open block changes nothing
    cfg, w, eng = _engine()
    sp = SamplingParams(max_tokens=10, ignore_eos=True, thinking_budget=2, think_start_id=START, think_end_id=END)
    assert eng.generate([_prompt(cfg)], sp)[0].output == base


def test_prompt_larger_than_the_pool_is_refused_and_long_rows_end_by_length():
    cfg, w, eng = _engine(num_blocks=4, max_model_len=384)
    with pytest.raises(ValueError, match="KV blocks"):
        eng.add_request(list(range(100)), SamplingParams(max_tokens=4))
    # fits at first, then outgrows the pool while decoding: ends with LENGTH instead of spinning
    cfg, w, eng = _engine(num_blocks=4, max_model_len=384)
    s = eng.generate([_prompt(cfg, 20)], SamplingParams(max_tokens=200, ignore_eos=True))[0]
    assert s.finish_reason == FinishReason.LENGTH and 0 < len(s.output) < 200
    assert not eng.has_work()


def test_speculative_rounds_alternate_with_admission():
    """With requests still queued the tick policy never grants two verify rounds in a row
    (tick_policy.rs:284-356); greedy output is unchanged."""
    cfg, w, eng = _engine(max_batch=2)
    prompts = [_prompt(cfg, n, seed=n) for n in (9, 14, 11, 17)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    want = [s.output for s in eng.generate(prompts, sp)]
    cfg, w, eng = _engine(max_batch=2)
    eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    actions = []
    orig = eng._spec_step

    def spy(decode):
        actions.append(("spec", len(eng.waiting)))
        return orig(decode)
    eng._spec_step = spy
    ids = [eng.add_request(p, sp) for p in prompts]
    prev_spec_while_waiting = False
    while eng.has_work():
        n0 = len(actions)
        waiting_before = len(eng.waiting)
        eng.step()
        was_spec = len(actions) > n0
        if was_spec and waiting_before > 0:
            assert not prev_spec_while_waiting, "two speculative rounds in a row while requests wait"
        prev_spec_while_waiting = was_spec and waiting_before > 0
    got = [eng.seqs[i].output for i in ids]
    assert got == want and eng.stats["spec_rounds"] > 0
    assert all(eng.seqs[i].draft_n >= eng.seqs[i].draft_n_accepted > 0 for i in ids)


def test_sliding_window_layers_release_blocks_behind_the_window():
    """gpt-oss style alternating layers: the windowed layers live in their own pool and give back
    every block that fell out of the window; tokens are identical to keeping everything."""
    cfg = preset("tiny-gpt-oss")            # sliding_window 32 on every other layer, sinks, MoE
    w = random_weights(cfg, seed=5, dtype=torch.float32, std=0.05)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 47, 90)]
    sp = SamplingParams(max_tokens=40, ignore_eos=True)

    def run(release):
        eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=128, num_blocks=96,
                                                             max_model_len=384, cuda_graphs=False, prefill_chunk_alone=64,
                                                             prefill_chunk_contended=32, window_release=release))
        peak = [0]
        ids = [eng.add_request(p, sp) for p in prompts]
        while eng.has_work():
            eng.step()
            if eng.bm_win is not None:
                st = eng.bm_win.stats()
                peak[0] = max(peak[0], st["num_blocks"] - st["free"])
        return [eng.seqs[i].output for i in ids], eng, peak[0]

    keep, eng0, _ = run(False)
    rel, eng1, peak = run(True)
    assert eng0.bm_win is None and eng1.bm_win is not None
    assert rel == keep
    st = eng1.bm_win.stats()
    assert st["front_released"] > 0 and st["free"] == st["num_blocks"]        # everything returned at the end
    # the three sequences end at 190 / 87 / 130 tokens = 27 blocks of 16; the window pool never held
    # more than window + chunk per prefilling row plus the window per decoding row
    assert peak <= 3 * ((32 + 64) // 16 + 3) and peak < 27, peak
    assert eng1.pool_win.num_blocks <= eng1.pool.num_blocks
    assert len(eng1.pool.layers) + len(eng1.pool_win.layers) == cfg.num_hidden_layers


def test_adaptive_speculation_policy_profiles_then_decides(tmp_path):
    from mlxcel_b200.speculative import SpecPolicy
    t = [0.0]
    pol = SpecPolicy(key="m|d|K4|cpu", profile_requests=2, classic_probes=2, cache_dir=str(tmp_path), clock=lambda: t[0])
    assert pol.state.mode == "profiling" and pol.allow()
    for _ in range(4):
        pol.record_spec(10.0, 12)            # 1.2 tok/ms
    assert not pol.allow()                   # a classic probe step is due after 4 rounds
    pol.record_classic(10.0, 8)              # 0.8 tok/ms
    assert pol.allow()
    pol.on_request_finished()
    assert pol.state.mode == "profiling"
    pol.on_request_finished()
    assert pol.state.mode == "enabled" and "tok/ms" in pol.state.verdict_reason
    # the verdict is persisted per key and picked up by the next process
    again = SpecPolicy(key="m|d|K4|cpu", cache_dir=str(tmp_path))
    assert again.state.mode == "enabled" and "persisted" in again.state.verdict_reason
    other = SpecPolicy(key="other", cache_dir=str(tmp_path))
    assert other.state.mode == "profiling"
    # a drafter that does not pay is switched off; forcing and resetting work
    slow = SpecPolicy(key="slow", profile_requests=1, cache_dir=str(tmp_path))
    slow.record_spec(10.0, 4)
    slow.record_classic(10.0, 8)
    slow.on_request_finished()
    assert slow.state.mode == "disabled" and not slow.allow()
    slow.force("on")
    assert slow.allow()
    slow.force("reset")
    assert slow.state.mode == "profiling" and not slow.path.exists()
    with pytest.raises(ValueError):
        slow.force("sideways")


def test_exactness_probe_and_policy_on_the_engine(tmp_path):
    """Block verification equals chain decoding on the fp32 CPU path, so the probe passes; with the
    policy attached the engine profiles, decides, and greedy output stays the same."""
    from mlxcel_b200.speculative import SpecPolicy, exactness_probe
    cfg, w, eng = _engine()
    assert exactness_probe(eng, _prompt(cfg, 10), k=4, tokens=10) is True
    assert eng.drafter is None and not eng.has_work()
    prompts = [_prompt(cfg, n, seed=n) for n in (9, 14, 11)]
    sp = SamplingParams(max_tokens=40, ignore_eos=True)
    want = [s.output for s in eng.generate(prompts, sp)]
    cfg, w, eng = _engine()
    eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    eng.spec_policy = SpecPolicy(key="t", profile_requests=2, classic_probes=1, cache_dir=str(tmp_path))
    got = [s.output for s in eng.generate(prompts, sp)]
    assert got == want
    st = eng.spec_policy.state
    assert st.spec_rounds > 0 and st.classic_steps >= 1 and st.mode in ("enabled", "disabled")
    eng.spec_policy.state.exact = False           # a failed probe keeps speculation off
    assert not eng.spec_policy.allow()


def test_sampler_match_acceptance_reproduces_classic_sampling():
    """Sampled rows in a verify round draw every position with their own seed and step counter, so the
    text equals what the same seeds give without a drafter, and the drafts still save steps."""
    cfg, w, eng = _engine()
    prompts = [_prompt(cfg, n, seed=n) for n in (9, 14, 11)]
    sps = [SamplingParams(max_tokens=24, ignore_eos=True, temperature=0.7, top_k=20, top_p=0.9, seed=11 + i) for i in range(2)]
    sps.append(SamplingParams(max_tokens=24, ignore_eos=True))         # a greedy row in the same rounds
    want = [s.output for s in eng.generate(prompts, sps)]
    assert want[0] != want[1]
    cfg, w, eng = _engine()
    eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    got = [s.output for s in eng.generate(prompts, sps)]
    assert got == want
    assert eng.stats["spec_sampled_rounds"] > 0 and eng.stats["spec_accepted"] > 0
    # penalties over the history keep a row out of verify rounds
    cfg, w, eng = _engine()
    eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    eng.generate(prompts[:1], SamplingParams(max_tokens=8, ignore_eos=True, temperature=0.7, repetition_penalty=1.3, seed=3))
    assert eng.stats["spec_rounds"] == 0


def test_context_shift_generates_past_the_window_and_bounds_the_cache():
    """--max-kv-size with context shifting: a sequence keeps generating past max_model_len, its live KV
    never exceeds the bound, the first n_keep tokens' blocks stay, every block returns to the pool at the
    end, tokens before the first shift equal those of an engine without the bound, and a sequence
    decodes the same alone as beside another one. Without context shifting the bound ends the
    sequence with finish reason "length"."""
    import torch

    from mlxcel_b200.config import preset
    from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
    from mlxcel_b200.models.decoder import DecoderModel
    from mlxcel_b200.models.weights import random_weights

    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=11, dtype=torch.float32, std=0.05)
    g = torch.Generator().manual_seed(5)
    p1 = torch.randint(0, cfg.vocab_size, (21,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab_size, (9,), generator=g).tolist()

    def eng(**kw):
        base = dict(max_batch=4, max_num_batched_tokens=64, num_blocks=40, block_size=8, max_model_len=64,
                    cuda_graphs=False, prefix_cache=False)
        base.update(kw)
        return Engine(DecoderModel(cfg, w), cfg, EngineConfig(**base))

    sp = SamplingParams(max_tokens=150, temperature=0.0, ignore_eos=True)
    plain = eng(max_model_len=256, num_blocks=80).generate([p1], SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))[0].output
    e = eng(max_kv_size=48, context_shift=True, n_keep=6)
    free0 = e.bm.num_free
    outs = e.generate([p1], sp)
    o = outs[0]
    assert len(o.output) == 150 and o.finish_reason == "length"            # ended by max_tokens, far past max_model_len
    assert o.output[:20] == plain                                          # nothing changes before the first shift
    assert e.stats["context_shifts"] >= 5 and e.stats["context_shift_tokens"] % 8 == 0
    assert e.bm.num_free == free0                                          # every block came back
    # batch invariance with shifting on
    e2 = eng(max_kv_size=48, context_shift=True, n_keep=6)
    both = e2.generate([p2, p1], sp)
    assert both[1].output == o.output
    # the live window stays under the bound (checked on the block manager while decoding)
    e3 = eng(max_kv_size=48, context_shift=True, n_keep=6)
    sid = e3.add_request(p1, sp)
    peak = 0
    while e3.has_work():
        e3.step()
        if e3.bm.has_seq(sid):
            live = e3.bm.seq_len(sid) - e3.bm.shifted(sid)
            peak = max(peak, live)
            assert e3.bm.seq_blocks(sid)[0] >= 0 and len(e3.bm.seq_blocks(sid)) <= 48 // 8 + 1
    assert 40 <= peak <= 48
    # no shifting: the bound is a stop
    e4 = eng(max_kv_size=48)
    o4 = e4.generate([p1], sp)[0]
    assert o4.finish_reason == "length" and len(p1) + len(o4.output) + 1 == 48
