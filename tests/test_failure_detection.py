"""Failure detection without faulting a GPU: host-injected failures on gloo ranks and a fake clock;
the device-side bounded wait is exercised by a flag that nothing sets (GPU test below)."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

from mlxcel_b200.parallel.health import ElasticPipelineState, FailureDetector, Heartbeat, PeerFailure

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_detector_threshold_with_fake_clock():
    store, t = FakeStore(), [0.0]
    hb1 = Heartbeat(store, 1, interval=5.0)
    det = FailureDetector(store, 0, 3, interval=5.0, threshold=3, clock=lambda: t[0])
    hb1.beat()
    assert det.poll() == set()
    t[0] = 14.0
    hb1.beat()                      # rank 1 keeps beating, rank 2 never did
    assert det.poll() == set()
    t[0] = 16.0
    assert det.poll() == {2}        # 16 s > 3 * 5 s without a beat from rank 2
    store.set("hb/2", "1")          # rank 2 comes back
    assert det.poll() == set()
    t[0] = 40.0
    with pytest.raises(PeerFailure) as e:
        det.raise_if_failed()
    assert e.value.ranks == [1, 2]


def test_elastic_state_machine():
    st = ElasticPipelineState(32, 4)
    assert [len(r) for r in st.partition] == [8, 8, 8, 8]
    st.begin(3)
    with pytest.raises(RuntimeError):
        st.begin(2)
    st.drained()
    assert sum(len(r) for r in st.partition) == 32 and len(st.partition) == 3
    st.loaded()
    st.resumed()
    assert st.state == "idle" and st.generation == 1


def test_rank_exit_is_detected_by_survivors(tmp_path):
    """Rank 1 leaves between steps (exits cleanly after its last collective); rank 0 learns of it on
    the host from the missing heartbeat before it would start another collective."""
    script = tmp_path / "hb.py"
    script.write_text(textwrap.dedent("""
        import os, sys, time, torch, torch.distributed as dist
        sys.path.insert(0, %r)
        from mlxcel_b200.parallel.health import Heartbeat, FailureDetector, PeerFailure
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        store = dist.TCPStore("127.0.0.1", int(os.environ["HB_PORT"]), world, rank == 0)
        hb = Heartbeat(store, rank, interval=0.1).start()
        det = FailureDetector(store, rank, world, interval=0.1, threshold=3)
        time.sleep(0.5)
        assert det.poll() == set()
        if rank == 1:
            hb.stop(); sys.exit(0)          # leaves between steps, nothing in flight
        deadline = time.time() + 10
        while time.time() < deadline and not det.poll():
            time.sleep(0.05)
        try:
            det.raise_if_failed()
            print("NOT_DETECTED")
        except PeerFailure as e:
            print("DETECTED", e.ranks)
    """ % ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", HB_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert "DETECTED [1]" in outs[0], outs


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    """A wait on a flag that nothing sets returns after its limit with an error status; the context
    stays usable and the next kernel runs."""
    import ctypes
    from mlxcel_b200 import ops
    from mlxcel_b200.ops import _lib
    lib = _lib.load()
    lib.mx_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p, ctypes.c_longlong,
                                  ctypes.c_void_p, ctypes.c_void_p]
    lib.mx_wait_probe.restype = ctypes.c_int
    dev = torch.device("cuda")
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    rc = lib.mx_wait_probe(flag.data_ptr(), 1, status.data_ptr(), 50_000_000, waited.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status) == 201 and 40_000_000 <= int(waited) < 1_000_000_000
    # a flag that IS set passes at once and leaves the status alone
    flag.fill_(1)
    status.zero_()
    lib.mx_wait_probe(flag.data_ptr(), 1, status.data_ptr(), 50_000_000, waited.data_ptr(),
                      torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert int(status) == 0 and int(waited) < 10_000_000
    x = torch.randn(8, 64, device=dev).to(torch.bfloat16)
    assert torch.isfinite(ops.linear(x, x).float()).all()
