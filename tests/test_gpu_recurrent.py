"""State-space / linear-attention / BitLinear / activation kernels vs their PyTorch references."""
import pytest
import torch

from mlxcel_b200.ops import recurrent as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, rtol=2e-2, atol=2e-2):
    err = (got.float() - want.float()).abs()
    bad = (err > atol + rtol * want.float().abs()).sum().item()
    assert bad == 0, f"{bad}/{err.numel()} mismatches, max err {err.max().item():.4g}"


def _bf(*s, sc=1.0):
    return (torch.randn(*s, device=DEV) * sc).to(torch.bfloat16)


def test_ssm_update():
    B, H, Dh, N, G = 3, 8, 64, 128, 2
    st = torch.randn(B, H, Dh, N, device=DEV)
    x, dt = _bf(B, H, Dh), _bf(B, H)
    A = -torch.rand(H, device=DEV) - 0.1
    Bm, C = _bf(B, G, N), _bf(B, G, N)
    D, db = torch.randn(H, device=DEV), torch.randn(H, device=DEV) * 0.1
    st2 = st.clone()
    y = R.ssm_update(st, x, dt, A, Bm, C, D, db)
    yr = R.ssm_update_ref(st2, x, dt, A, Bm, C, D, db)
    _close(y, yr, atol=0.1)
    _close(st, st2, rtol=1e-3, atol=1e-3)


def test_selective_scan():
    B, L, Di, N = 2, 37, 96, 16
    x, dt = _bf(B, L, Di), _bf(B, L, Di, sc=0.5)
    A = -torch.rand(Di, N, device=DEV) - 0.1
    Bm, C = _bf(B, L, N), _bf(B, L, N)
    D = torch.randn(Di, device=DEV)
    st = torch.randn(B, Di, N, device=DEV) * 0.1
    st2 = st.clone()
    y = R.selective_scan(x, dt, A, Bm, C, D, st)
    yr = R.selective_scan_ref(x, dt, A, Bm, C, D, st2)
    _close(y, yr, atol=0.1)
    _close(st, st2, rtol=2e-3, atol=2e-3)


def test_gated_delta_update():
    B, Hv, Dk, Dv = 2, 4, 128, 128
    S = torch.randn(B, Hv, Dk, Dv, device=DEV) * 0.1
    q = torch.nn.functional.normalize(torch.randn(B, Hv, Dk, device=DEV), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(B, Hv, Dk, device=DEV), dim=-1).to(torch.bfloat16)
    v = _bf(B, Hv, Dv)
    g = -torch.rand(B, Hv, device=DEV)
    beta = torch.rand(B, Hv, device=DEV)
    S2 = S.clone()
    o = R.gated_delta_update(S, q, k, v, g, beta, Dk ** -0.5)
    o_r = R.gated_delta_update_ref(S2, q, k, v, g, beta, Dk ** -0.5)
    _close(o, o_r, atol=3e-2)
    _close(S, S2, rtol=1e-3, atol=1e-3)


def test_bitlinear_and_activations():
    M, N, K = 5, 96, 256
    w = torch.randint(-1, 2, (N, K))
    x = _bf(M, K)
    got = R.bitlinear(x, R.pack_ternary(w).to(DEV), 0.37)
    want = (x.float() @ w.float().to(DEV).t()) * 0.37
    _close(got, want, atol=0.1)
    z = _bf(1000, sc=3.0)
    _close(R.gelu_tanh(z), torch.nn.functional.gelu(z.float(), approximate="tanh"))
    _close(R.xielu(z, 0.8, 0.8, 0.5, -1e-6), R.xielu_ref(z, 0.8, 0.8, 0.5, -1e-6), atol=5e-2)
    a, b, c, wt, bs = _bf(7, 640), _bf(7, 640), _bf(7, 640), _bf(640), _bf(640)
    y, s = R.add3_layernorm(a, b, c, wt, bs)
    yr, sr = R.add3_layernorm(a.cpu(), b.cpu(), c.cpu(), wt.cpu(), bs.cpu())
    assert torch.equal(s.cpu(), sr)
    _close(y.cpu(), yr, atol=5e-2)
