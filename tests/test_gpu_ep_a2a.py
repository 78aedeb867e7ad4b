"""Expert-parallel dispatch / combine kernels with the ranks emulated on one GPU: the instances share
peer tables over buffers of the same device and their stages run rank after rank in protocol order,
so every flag is set before a kernel looks at it (no kernel waits on another)."""
import pytest
import torch

from mlxcel_b200.ops import _lib, moe as moe_ops
from mlxcel_b200.parallel.ep_a2a import EpAllToAll

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("world,E,k,H,I,act,slack", [(4, 8, 2, 256, 128, "silu", 1), (2, 6, 3, 320, 192, "clipped_swiglu", 1),
                                                     (8, 32, 4, 2880, 256, "clipped_swiglu", 1),
                                                     (8, 32, 4, 512, 256, "clipped_swiglu", 32)])
def test_ep_dispatch_combine_emulated(world, E, k, H, I, act, slack):
    """``slack``: the receive area is that many times larger than any step fills (as in serving, where
    it is sized for the longest prefill step and a decode step uses a sliver of it)."""
    epr = E // world
    Ts = [5, 0, 64, 33, 1, 17, 40, 8][:world]
    Tmax = max(Ts) * slack
    cap = Tmax * k
    eps = EpAllToAll.emulated(world, torch.device(DEV), H, cap, epr, Tmax, k)
    g = torch.Generator().manual_seed(world + E)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16).to(DEV)  # noqa: E731
    wgu, wd = r(E, 2 * I, H, sc=0.05), r(E, H, I, sc=0.05)
    bias = act == "clipped_swiglu"
    bgu, bd = (r(E, 2 * I, sc=0.1), r(E, H, sc=0.1)) if bias else (None, None)
    for epoch in range(2):                              # the second pass reuses every buffer
        xs, idss, wtss, ress = [], [], [], []
        for rk in range(world):
            T = Ts[rk] if epoch == 0 else Ts[world - 1 - rk]
            x = r(T, H)
            if T:
                ids, wts = moe_ops.route(r(T, E), k, "topk_softmax", True)
            else:
                ids = torch.zeros(0, k, dtype=torch.int32, device=DEV)
                wts = torch.zeros(0, k, dtype=torch.float32, device=DEV)
            xs.append(x), idss.append(ids.contiguous()), wtss.append(wts.contiguous()), ress.append(r(T, H))
        for rk in range(world):
            eps[rk].dispatch(xs[rk], idss[rk])
        for rk in range(world):
            lo, hi = rk * epr, (rk + 1) * epr
            eps[rk].expert_stage(wgu[lo:hi].contiguous(), wd[lo:hi].contiguous(), I, act,
                                 None if bgu is None else bgu[lo:hi].contiguous(),
                                 None if bd is None else bd[lo:hi].contiguous())
        for rk in range(world):
            got = eps[rk].combine(wtss[rk], ress[rk])
            if xs[rk].shape[0] == 0:
                assert got.shape[0] == 0
                continue
            want = moe_ops.moe_ref(xs[rk], idss[rk], wtss[rk], wgu, wd, I, act, bgu, bd) + ress[rk].float()
            err = (got.float() - want).abs()
            bad = (err > 6e-2 + 3e-2 * want.abs()).sum().item()
            assert bad == 0, f"rank {rk} epoch {epoch}: {bad} mismatches, max err {err.max().item():.4g}"
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


def test_ep_dispatch_reports_overflow():
    """More rows for one destination than the receive area holds: the status word says so and the
    surplus rows are dropped (their route entry is -1), nothing is written out of bounds."""
    world, E, k, H = 2, 2, 1, 64
    eps = EpAllToAll.emulated(world, torch.device(DEV), H, 4, 1, 16, k)
    x = torch.randn(16, H, device=DEV).to(torch.bfloat16)
    ids = torch.zeros(16, 1, dtype=torch.int32, device=DEV)          # all 16 rows to rank 0, cap 4
    eps[0].dispatch(x, ids)
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 203
    assert (eps[0].route[:16] >= 0).sum().item() == 4
