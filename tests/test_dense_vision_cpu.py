"""DINOv2 backbone and Depth Anything against transformers."""
import tempfile

import numpy as np
import pytest
import torch

from mlxcel_b200.models.depth_anything import DepthAnything, Dinov2Backbone


def _randomise(m):
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
            else:
                p.add_(torch.randn_like(p) * 0.1)


@pytest.mark.parametrize("swiglu", [False, True])
def test_dinov2_backbone_stages_match_transformers(swiglu):
    from transformers import Dinov2Backbone as HF
    from transformers import Dinov2Config
    torch.manual_seed(0)
    cfg = Dinov2Config(hidden_size=32, num_hidden_layers=4, num_attention_heads=4, mlp_ratio=2, image_size=28, patch_size=7,
                       use_swiglu_ffn=swiglu, out_features=["stage2", "stage4"], apply_layernorm=True, reshape_hidden_states=False)
    m = HF(cfg).eval()
    _randomise(m)
    ours = Dinov2Backbone(cfg.to_dict(), dict(m.state_dict()), dtype=torch.float32)
    for size in ((28, 28), (35, 21)):                     # the trained grid, then an interpolated one
        px = torch.randn(2, 3, *size)
        with torch.no_grad():
            want = m(px).feature_maps
        got = ours.forward(px)
        assert len(got) == 2
        for g, w in zip(got, want):
            torch.testing.assert_close(g, w, rtol=2e-4, atol=2e-4)
    assert ours.embed(torch.randn(1, 3, 28, 28)).shape == (1, 32)


@pytest.mark.parametrize("kind", ["relative", "metric"])
def test_depth_anything_matches_transformers(kind):
    from PIL import Image
    from transformers import DepthAnythingConfig, DepthAnythingForDepthEstimation, Dinov2Config
    torch.manual_seed(0)
    bc = Dinov2Config(hidden_size=32, num_hidden_layers=4, num_attention_heads=4, mlp_ratio=2, image_size=28, patch_size=7,
                      out_features=["stage1", "stage2", "stage3", "stage4"], apply_layernorm=True, reshape_hidden_states=False)
    cfg = DepthAnythingConfig(backbone_config=bc, patch_size=7, reassemble_hidden_size=32, neck_hidden_sizes=[8, 16, 24, 32],
                              fusion_hidden_size=16, head_hidden_size=8, depth_estimation_type=kind,
                              max_depth=20 if kind == "metric" else None)
    m = DepthAnythingForDepthEstimation(cfg).eval()
    _randomise(m)
    d = tempfile.mkdtemp(prefix="depth_anything_")
    m.save_pretrained(d, safe_serialization=True)
    ours = DepthAnything.from_pretrained(d, dtype=torch.float32)
    px = torch.randn(2, 3, 42, 28)
    with torch.no_grad():
        want = m(pixel_values=px).predicted_depth
    got = ours.predict(px)
    assert got.shape == want.shape == (2, 42, 28)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (40, 60, 3), dtype=np.uint8))
    depth = ours.estimate(img, short_side=28)
    assert depth.shape == (40, 60) and np.isfinite(depth).all()


def test_depth_command_writes_a_16_bit_png(tmp_path, capsys):
    import json

    from PIL import Image
    from transformers import DepthAnythingConfig, DepthAnythingForDepthEstimation, Dinov2Config

    from mlxcel_b200 import cli
    torch.manual_seed(0)
    bc = Dinov2Config(hidden_size=32, num_hidden_layers=4, num_attention_heads=4, mlp_ratio=2, image_size=28, patch_size=7,
                      out_features=["stage1", "stage2", "stage3", "stage4"], apply_layernorm=True, reshape_hidden_states=False)
    cfg = DepthAnythingConfig(backbone_config=bc, patch_size=7, reassemble_hidden_size=32, neck_hidden_sizes=[8, 16, 24, 32],
                              fusion_hidden_size=16, head_hidden_size=8)
    m = DepthAnythingForDepthEstimation(cfg).eval()
    _randomise(m)
    m.save_pretrained(tmp_path / "model", safe_serialization=True)
    img = tmp_path / "a.png"
    Image.fromarray(np.random.default_rng(1).integers(0, 255, (30, 44, 3), dtype=np.uint8)).save(img)
    cli.main(["depth", "-m", str(tmp_path / "model"), str(img), "--short-side", "28", "--device", "cpu"])
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    out = Image.open(rec["out"])
    assert out.size == (44, 30) and out.mode in ("I;16", "I") and rec["max"] >= rec["min"]
