"""Failure detection without a GPU fault: a wait that can never complete runs into its time limit, the kernel
returns, the host reads B200HT_ERR_TIMEOUT, and the context keeps working.  The host-side half (a rank that
never joins) runs as gloo ranks on the CPU."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_context_survives(pkg, lib):
    l = lib.load()
    assert l.b200ht_device_status(1) == 0
    rc = l.b200ht_selftest_wait_timeout(2000, torch.cuda.current_stream().cuda_stream)   # 2 ms limit
    assert rc == -8, lib.error_string(rc)
    assert l.b200ht_device_status(1) == -8          # the kernel left the code in the status word ...
    assert l.b200ht_device_status(0) == 0           # ... and clearing works
    # the context is still usable: run a real kernel afterwards
    x = torch.randn(8, 32768, device="cuda").bfloat16()
    y = pkg.hadamard_transform(pkg.hadamard_transform(x))
    assert (y.float() - x.float()).abs().max().item() < 0.2
    assert pkg.device_status() == 0


@pytest.mark.gpu
def test_row_sharded_gemv_gives_up_on_a_peer_that_never_sends(pkg, lib):
    """The one cross-GPU wait of the library, run out on one GPU: a row-sharded GEMV call whose "peer" is a slot array
    that nothing fills.  The kernel computes its own rows, waits a second for the other half, gives up with
    B200HT_ERR_TIMEOUT in the status word, and the context keeps working.  The second rank of the same exchange, run
    afterwards on the same GPU, finds the first rank's values waiting and completes the result."""
    import ctypes
    l = lib.load()
    assert l.b200ht_device_status(1) == 0
    M, N, B = 512, 1024, 4
    g = torch.Generator(device="cuda").manual_seed(11)
    W = (torch.randn(M, N, generator=g, device="cuda") / 32).bfloat16()
    X = torch.randn(N, B, generator=g, device="cuda").bfloat16()
    half = M // 2
    y_full = torch.full((M, B), 7.0, device="cuda")
    my_slots = torch.zeros(M * B, dtype=torch.int64, device="cuda")       # the peer would write here; nobody does
    peer_slots = torch.zeros(M * B, dtype=torch.int64, device="cuda")     # stands in for the peer's memory
    count = torch.zeros(2, dtype=torch.int32, device="cuda")
    peers = (ctypes.c_void_p * 1)(peer_slots.data_ptr())
    torch.cuda.synchronize()
    rc = l.b200ht_fused_gemv_peers(W.data_ptr(), X.data_ptr(), y_full.data_ptr(), half, N, B, lib.BF16, lib.F32,
                                   float(N ** -0.5), 0, M, 1, peers, my_slots.data_ptr(), count.data_ptr(), 1,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    assert l.b200ht_device_status(1) == -8
    # its own rows are there, the other half was never touched, and the values it sent carry the call's number
    ref = pkg.fused_ht_gemv(W[:half], X)
    assert torch.equal(y_full[:half], ref)
    assert bool((y_full[half:] == 7.0).all())
    sent = peer_slots[: half * B].view(torch.int32).view(-1, 2)          # (value bits, tag) per slot
    assert bool((sent[:, 1] == 1).all())
    assert torch.equal(sent[:, 0].contiguous().view(torch.float32).view(half, B), ref)
    assert bool((peer_slots[half * B:] == 0).all())
    assert int(count[0]) == 0 and int(count[1]) == 1          # scratch word back at zero, one call counted
    assert pkg.device_status() == 0
    # Now the other rank of that exchange, on the same GPU: its slot array is the one the first call filled, so it
    # finds the first half there at once, adds its own rows, and holds the complete result.
    y_full1 = torch.full((M, B), 7.0, device="cuda")
    count1 = torch.zeros(2, dtype=torch.int32, device="cuda")
    peers1 = (ctypes.c_void_p * 1)(my_slots.data_ptr())
    rc = l.b200ht_fused_gemv_peers(W[half:].data_ptr(), X.data_ptr(), y_full1.data_ptr(), M - half, N, B, lib.BF16,
                                   lib.F32, float(N ** -0.5), half, M, 1, peers1, peer_slots.data_ptr(),
                                   count1.data_ptr(), 1, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    assert l.b200ht_device_status(1) == 0
    full = pkg.fused_ht_gemv(W, X)
    assert float((y_full1 - full).norm() / full.norm()) < 1e-5
    assert torch.equal(y_full1[:half], ref)                   # the collected rows are the sender's values, bit for bit


def test_missing_rank_is_detected_by_the_survivor(tmp_path):
    """Two gloo ranks; rank 1 exits between steps (never joins the second gather).  Rank 0's collective ends with an
    error after the short process-group timeout instead of hanging."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import datetime, importlib, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
        rank = dist.get_rank()
        local = torch.full((3, 4), float(rank))
        full = pkg.gather_result(local, 6, "nm")          # step 1: both ranks present
        assert full.shape == (6, 4)
        if rank == 1:
            sys.exit(0)                                   # leaves between steps, nothing in flight
        try:
            pkg.gather_result(local, 6, "nm")             # step 2: the peer is gone
        except Exception as e:                            # noqa: BLE001
            print("survivor saw:", type(e).__name__, flush=True)
            open({str(tmp_path / "survivor.txt")!r}, "w").write(type(e).__name__)
            sys.exit(0)
        sys.exit(3)                                       # the collective returned although the peer never joined
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29633", str(script)],
        capture_output=True, text=True, env=env, timeout=300)
    # both workers must exit 0: rank 1 by leaving, rank 0 by catching the error of its collective (exit code 3 would
    # mean the collective returned, any other code that the worker crashed)
    assert r.returncode == 0, r.stdout + r.stderr
    assert (tmp_path / "survivor.txt").exists(), r.stdout + r.stderr
    assert "survivor saw:" in r.stdout + r.stderr, r.stdout + r.stderr
