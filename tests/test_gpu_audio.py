"""Whisper on a B200 (bf16, the package's GEMM / LayerNorm / activation kernels) against the fp32 CPU
path of the same checkpoint."""
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def test_whisper_gpu_matches_cpu():
    sys.path.insert(0, str(Path(__file__).parent))
    import test_audio_cpu as t
    from mlxcel_b200.audio import LogMel
    from mlxcel_b200.models.whisper import WhisperModel
    m, d = t._tiny_whisper()
    cpu = WhisperModel.from_pretrained(d, dtype=torch.float32)
    gpu = WhisperModel.from_pretrained(d, dtype=torch.bfloat16, device="cuda")
    fe = LogMel(80)
    mel = torch.stack([fe(t._tone(5.0, f=300.0, seed=1)), fe(t._tone(7.0, f=800.0, seed=2))])
    a, b = cpu.encode(mel), gpu.encode(mel).float().cpu()
    assert (a - b).abs().max().item() < 0.08 * max(a.abs().max().item(), 1.0)
    prompt = [t.SOT, t.EN, t.TRANSCRIBE, t.NOTS]
    want = cpu.generate(mel, prompt, 10, eos=t.EOS)
    got = gpu.generate(mel, prompt, 10, eos=t.EOS)
    agree = sum(x == y for w, g in zip(want, got) for x, y in zip(w, g)) / max(1, sum(len(w) for w in want))
    assert [g[0] for g in got] == [w[0] for w in want] and agree >= 0.5, (got, want)
