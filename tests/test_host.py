"""CPU-only checks of the boundary: exported symbols, argument validation that
returns before any CUDA call, the wrapper's reference-compatible errors, and
the token partitioning (including a 2-rank gloo run)."""
import ctypes
import os
import re
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "b200ht.h").read_text()
    declared = set(re.findall(r"\b(b200ht_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/b200ht.h"
    l = lib.load()
    for name in declared:
        assert hasattr(l, name), f"{name} declared in the header but not exported"
    assert declared == set(lib.EXPORTS)
    assert l.b200ht_version() >= 100


def test_error_strings(lib):
    l = lib.load()
    assert l.b200ht_error_string(0) == b"success"
    for code in range(-8, 0):
        assert l.b200ht_error_string(code).startswith(b"b200ht:")


def test_c_abi_rejects_bad_arguments_before_touching_the_gpu(lib):
    l = lib.load()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    # size not a power of two / out of range
    assert l.b200ht_fwht(p16, p16, 1, 3, lib.BF16, 1.0, None) == -2
    assert l.b200ht_fwht(p16, p16, 1, 1 << 16, lib.BF16, 1.0, None) == -2
    assert l.b200ht_fwht(p16, p16, 1, 1, lib.BF16, 1.0, None) == -2
    # dtype
    assert l.b200ht_fwht(p16, p16, 1, 8, 7, 1.0, None) == -3
    # rows == 0 is a no-op
    assert l.b200ht_fwht(None, None, 0, 8, lib.BF16, 1.0, None) == 0
    # null / alignment / partial overlap
    assert l.b200ht_fwht(None, p16, 1, 8, lib.BF16, 1.0, None) == -1
    assert l.b200ht_fwht(p16 + 2, p16, 1, 8, lib.BF16, 1.0, None) == -4
    assert l.b200ht_fwht(p16, p16 + 16, 2, 8, lib.BF16, 1.0, None) == -6
    # fused entry points
    assert l.b200ht_fused_gemm(p16, p16, p16, 4, 4, 6, lib.F32, lib.F32, 0, 1.0, p16, 1 << 20, None) == -2
    assert l.b200ht_fused_gemm(p16, p16, p16, 4, 4, 8, lib.F16, lib.F32, 0, 1.0, p16, 1 << 20, None) == -3
    assert l.b200ht_fused_gemm(p16, p16, p16, 4, 4, 8, lib.F32, lib.F32, 0, 1.0, None, 0, None) == -5
    assert l.b200ht_fused_gemm(p16, p16, p16, 0, 4, 8, lib.F32, lib.F32, 0, 1.0, None, 0, None) == 0
    assert l.b200ht_fused_gemv(p16, p16, p16, 4, 12, 1, lib.F32, lib.F32, 1.0, None) == -2
    assert l.b200ht_fused_gemv(p16, p16, p16, 4, 16, 65537, lib.F32, lib.F32, 1.0, None) == -2
    assert l.b200ht_fused_gemv(p16, p16, p16, 4, 16, 1, lib.F16, lib.F32, 1.0, None) == -3
    assert l.b200ht_fused_gemm_workspace_bytes(128, 32, 256, lib.F32) == 32 * 256 * 4
    assert l.b200ht_fused_gemm_workspace_bytes(128, 32, 256, lib.BF16) == 32 * 256 * 2


def test_wrapper_keeps_the_reference_error_messages(pkg):
    # csrc/hadamard_transform.cpp:15-26
    with pytest.raises(RuntimeError, match="Only fp16 and bf16 supported currently"):
        pkg.hadamard_transform(torch.zeros(4, 8, dtype=torch.float32))
    with pytest.raises(RuntimeError, match="is_cuda"):
        pkg.hadamard_transform(torch.zeros(4, 8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        pkg.fused_ht_gemm(torch.zeros(4, 8), torch.zeros(4, 8))  # CPU tensors
    with pytest.raises(RuntimeError):
        pkg.fused_ht_gemv(torch.zeros(4, 8), torch.zeros(8, 2))


def test_no_cpu_fallback_in_product_sources():
    pkg_dir = ROOT / "6s894_project_2025_b200"
    for f in pkg_dir.rglob("*.py"):
        text = f.read_text()
        assert "oracle" not in text, f"{f} mentions the oracle: the product must not route through it"
    for f in pkg_dir.rglob("*.cu*"):
        assert "oracle" not in f.read_text()


@pytest.mark.parametrize("n,world", [(16384, 1), (16384, 2), (16384, 8), (10, 4), (3, 8)])
def test_token_ranges_tile_the_tokens(pkg, n, world):
    prev = 0
    for r in range(world):
        a, b = pkg.token_range(n, r, world)
        assert a == prev and b >= a
        prev = b
    assert prev == n
    sizes = [pkg.token_range(n, r, world) for r in range(world)]
    assert max(b - a for a, b in sizes) - min(b - a for a, b in sizes) <= 1


def test_two_rank_gloo_shard_and_gather(tmp_path):
    """World-size-2 run on CPU: shard tokens, fake the per-rank result with the
    oracle, gather in both layouts, compare with the unsharded result."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import numpy as np, torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        oracle = importlib.import_module("oracle.fwht_oracle")
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        inp = oracle.make_inputs("c5", K=64, M=24, N=10)
        X, W = inp["X"].float(), inp["W"].float()
        full = torch.from_numpy(oracle.fused_gemm_ref(X.numpy(), W.numpy())).float()   # (M, N)
        Xs = pkg.shard_tokens(X, rank, world)
        local = torch.from_numpy(oracle.fused_gemm_ref(Xs.numpy(), W.numpy())).float()  # (M, n_local)
        got_mn = pkg.gather_result(local, X.shape[0], "mn")
        got_nm = pkg.gather_result(local.t().contiguous(), X.shape[0], "nm")
        assert torch.equal(got_mn, full), "mn gather differs"
        assert torch.equal(got_nm, full.t()), "nm gather differs"
        # equal split path (all_gather_into_tensor)
        inp = oracle.make_inputs("c5", K=64, M=8, N=12)
        X, W = inp["X"].float(), inp["W"].float()
        full = torch.from_numpy(oracle.fused_gemm_ref(X.numpy(), W.numpy())).float()
        local = torch.from_numpy(oracle.fused_gemm_ref(pkg.shard_tokens(X, rank, world).numpy(), W.numpy())).float()
        assert torch.equal(pkg.gather_result(local.t().contiguous(), 12, "nm"), full.t())
        # uneven split (7 tokens over 2 ranks: 4 + 3)
        inp = oracle.make_inputs("c5", K=64, M=8, N=7)
        X, W = inp["X"].float(), inp["W"].float()
        full = torch.from_numpy(oracle.fused_gemm_ref(X.numpy(), W.numpy())).float()
        local = torch.from_numpy(oracle.fused_gemm_ref(pkg.shard_tokens(X, rank, world).numpy(), W.numpy())).float()
        assert torch.equal(pkg.gather_result(local, 7, "mn"), full)
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29617", str(script)],
        capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok") == 2


def test_two_rank_gloo_row_sharded_gemv(tmp_path):
    """World-size-2 run on CPU for the small-batch split: every rank keeps a block of rows of W, the per-rank result
    is faked with the oracle, one all-gather assembles Y; uneven and even row counts."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import numpy as np, torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        oracle = importlib.import_module("oracle.fwht_oracle")
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        for M, N, B in ((37, 64, 3), (16, 32, 4)):
            g = torch.Generator().manual_seed(9)
            W = torch.randn(M, N, generator=g); X = torch.randn(N, B, generator=g)
            full = torch.from_numpy(oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy())).float()
            Ws = pkg.shard_rows(W, rank, world)
            assert Ws.shape[0] == pkg.row_range(M, rank, world)[1] - pkg.row_range(M, rank, world)[0]
            local = torch.from_numpy(oracle.fused_gemv_ref(Ws.double().numpy(), X.double().numpy())).float()
            got = pkg.gather_rows(local, M)
            assert torch.equal(got, full), "row gather differs"
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29618", str(script)],
        capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok") == 2


def test_two_rank_gloo_peer_store_gemv_bookkeeping(tmp_path):
    """Host side of the peer-store row-sharded GEMV, two gloo ranks on the CPU with a stand-in for the CUDA side:
    the handle exchange gives every rank the other ranks' buffers (never its own as a peer), the slot array a rank
    sends into sits at the same offset in every buffer and is the one the peer reads for that call, results and
    slot arrays do not overlap, the number of the call grows by one per call and the two buffers alternate."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()

        class Fake:
            launches = []
            def allocate(self, nbytes): self.nbytes = nbytes; return torch.zeros(nbytes, dtype=torch.uint8)
            def address(self, buf): return 1000000 * (rank + 1)
            def export(self, buf): return ("handle-of", rank)
            def open(self, handle): assert handle[0] == "handle-of"; return 1000000 * (handle[1] + 1)
            def close(self, addr): pass
            def launch(self, op, X, batch, plan, scale): Fake.launches.append(plan)
            def view(self, buf, offset, shape, dtype):
                n = shape[0] * shape[1] * 4
                return buf[offset: offset + n].view(dtype).view(shape)

        M, N, B = 11, 256, 3                      # 11 rows over 2 ranks: 6 + 5
        a, b = pkg.row_range(M, rank, world)
        W = torch.zeros(b - a, N, dtype=torch.bfloat16)
        op = pkg.RowShardedGemv(W, M, 4, backend=Fake())
        other = 1 - rank
        assert op.peers == [other]
        for call in range(3):
            y = op(torch.zeros(N, B, dtype=torch.bfloat16))
            plan = Fake.launches[-1]
            assert y.shape == (M, B)
            assert plan["call"] == call + 1 and plan["parity"] == call % 2
            mine, peer = 1000000 * (rank + 1), 1000000 * (other + 1)
            par = call % 2
            assert plan["local_count"] == mine + 128 and plan["local_count"] % 8 == 0
            assert plan["y_full"] == mine + 256 + par * op.y_bytes
            slot_off = 256 + 2 * op.y_bytes + par * op.slot_bytes
            assert plan["my_slots"] == mine + slot_off and plan["peer_slots"] == [peer + slot_off]
            assert plan["my_slots"] % 8 == 0 and op.slot_bytes >= M * 4 * 8 and op.y_bytes >= M * 4 * 4
            # the two results and the two slot arrays tile the buffer behind the counter word
            assert slot_off + op.slot_bytes <= op.backend.nbytes and 256 + (par + 1) * op.y_bytes <= 256 + 2 * op.y_bytes
        try:
            op(torch.zeros(N, 5, dtype=torch.bfloat16))
            raise SystemExit("batch beyond max_batch was accepted")
        except RuntimeError:
            pass
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29619", str(script)],
        capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok") == 2
