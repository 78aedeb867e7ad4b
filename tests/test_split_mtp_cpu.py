"""split-mtp: the MTP layer of a raw checkpoint becomes a self-contained one-layer drafter checkpoint."""
import json
import tempfile
from pathlib import Path

import pytest
import torch

transformers = pytest.importorskip("transformers")

from mlxcel_b200 import cli  # noqa: E402
from mlxcel_b200.loading.split_mtp import MARKER, load_mtp_weights, split_mtp_dir  # noqa: E402


@pytest.fixture(scope="module")
def raw_checkpoint():
    """A GLM-4.5 style checkpoint with 2 regular layers and 1 MTP layer: transformers writes 3 layers, the
    last one is declared as the MTP layer and given the fusion tensors."""
    from safetensors.torch import load_file, save_file
    from transformers import AutoConfig, AutoModelForCausalLM

    torch.manual_seed(0)
    hc = AutoConfig.for_model("glm4_moe", hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                              num_key_value_heads=2, vocab_size=300, max_position_embeddings=256, n_routed_experts=8,
                              num_experts_per_tok=2, moe_intermediate_size=48, n_shared_experts=1, n_group=2, topk_group=1,
                              first_k_dense_replace=1, routed_scaling_factor=1.5, head_dim=16, use_qk_norm=True,
                              pad_token_id=0, attention_bias=True)
    m = AutoModelForCausalLM.from_config(hc).float()
    d = Path(tempfile.mkdtemp(prefix="raw_mtp_"))
    m.save_pretrained(d, safe_serialization=True)
    t = {k: v.clone() for k, v in load_file(str(d / "model.safetensors")).items()}   # not views of the file rewritten below
    g = torch.Generator().manual_seed(1)
    t["model.layers.2.enorm.weight"] = torch.rand(64, generator=g) + 0.5
    t["model.layers.2.hnorm.weight"] = torch.rand(64, generator=g) + 0.5
    t["model.layers.2.eh_proj.weight"] = torch.randn(64, 128, generator=g) * 0.05
    t["model.layers.2.shared_head.norm.weight"] = torch.rand(64, generator=g) + 0.5
    save_file(t, str(d / "model.safetensors"), metadata={"format": "pt"})
    cfg = json.loads((d / "config.json").read_text())
    cfg.update(num_hidden_layers=2, num_nextn_predict_layers=1)
    (d / "config.json").write_text(json.dumps(cfg))
    return d, t


def test_split_writes_a_loadable_drafter(raw_checkpoint, tmp_path):
    src, t = raw_checkpoint
    out = tmp_path / "drafter"
    res = split_mtp_dir(src, out)
    assert res["layers"] == 1 and res["source_layer"] == 2 and res["block_size"] == 2 and not res["own_embeddings"]
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["num_hidden_layers"] == 1 and cfg["first_k_dense_replace"] == 0 and cfg["mtp_block_size"] == 2
    assert (out / MARKER).exists()
    mcfg, w, mw = load_mtp_weights(out, dtype=torch.float32)
    assert mcfg.num_hidden_layers == 1 and w.layer.router_w is not None          # the MTP layer is a MoE layer
    assert torch.equal(w.enorm, t["model.layers.2.enorm.weight"]) and torch.equal(w.fc, t["model.layers.2.eh_proj.weight"])
    assert torch.equal(w.final_norm, t["model.layers.2.shared_head.norm.weight"])
    assert torch.equal(w.layer.wo, t["model.layers.2.self_attn.o_proj.weight"])
    assert torch.equal(mw.embed, t["model.embed_tokens.weight"]) and torch.equal(mw.lm_head, t["lm_head.weight"])


def test_refusals_and_force(raw_checkpoint, tmp_path):
    src, _ = raw_checkpoint
    with pytest.raises(ValueError, match="source"):
        split_mtp_dir(src, src)
    out = tmp_path / "d"
    split_mtp_dir(src, out)
    with pytest.raises(ValueError, match="not empty"):
        split_mtp_dir(src, out)
    split_mtp_dir(src, out, force=True, block_size=3)                         # our own earlier output: allowed
    assert json.loads((out / "config.json").read_text())["mtp_block_size"] == 3
    foreign = tmp_path / "f"
    foreign.mkdir()
    (foreign / "other.safetensors").write_bytes(b"x")
    with pytest.raises(ValueError, match="no earlier split"):
        split_mtp_dir(src, foreign, force=True)
    with pytest.raises(ValueError, match="q-bits"):
        split_mtp_dir(src, tmp_path / "q", q_bits=7)
    nomtp = tmp_path / "nomtp"
    nomtp.mkdir()
    cfg = json.loads((src / "config.json").read_text())
    cfg["num_nextn_predict_layers"] = 0
    (nomtp / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="no MTP layers"):
        split_mtp_dir(nomtp, tmp_path / "o2")


def test_quantized_drafter_and_cli(raw_checkpoint, tmp_path, capsys):
    src, t = raw_checkpoint
    out = tmp_path / "q4"
    cli.main(["split-mtp", "-m", str(src), "-o", str(out), "--q-bits", "8", "--q-group-size", "32", "--json"])
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["quantized"] > 0
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["quantization"] == dict(group_size=32, bits=8)
    from safetensors.torch import load_file
    names = set(load_file(str(out / "model.safetensors")))
    assert "model.layers.0.self_attn.o_proj.scales" in names and "model.layers.0.mlp.gate.scales" not in names
    assert "model.norm.scales" not in names and "model.mtp.0.eh_proj.scales" in names
    _, w, _ = load_mtp_weights(out, dtype=torch.float32)
    ref = t["model.layers.2.eh_proj.weight"]
    assert (w.fc.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3


def _generate(capsys, *extra):
    cli.main(["generate", "--device", "cpu", "-n", "12", "--temp", "0", "--ignore-eos", "-p", "hello world, hello world, hello",
              *extra])
    cap = capsys.readouterr()
    return cap.out, cap.err


def test_drafter_flags_keep_greedy_output(raw_checkpoint, tmp_path, capsys):
    """``--draft-model <split-mtp dir>``, ``--draft-model <model dir>`` and ``--prompt-lookup`` are lossless
    under greedy decoding: same text as the plain run, and drafts were verified."""
    src, _ = raw_checkpoint
    out = tmp_path / "drafter"
    split_mtp_dir(src, out)
    plain, _ = _generate(capsys, "-m", str(src))
    for extra in (["--draft-model", str(out), "--draft-max", "2"], ["--draft-model", str(src)], ["--prompt-lookup"]):
        text, err = _generate(capsys, "-m", str(src), *extra)
        assert text == plain, extra
        rounds = int(err.split("[speculative: ")[1].split(" verify")[0])
        assert rounds > 0, extra
        if extra[-1] == str(src):                        # the target drafting for itself: every draft accepted
            acc, drafted = (int(x) for x in err.split("rounds, ")[1].split(" drafts")[0].split(" of "))
            assert acc == drafted > 0
