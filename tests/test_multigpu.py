"""Token sharding on real GPUs (needs at least two; skipped otherwise): every rank runs the fused kernel on its
shard, the NCCL gather assembles C, and the result equals the unsharded call bit for bit."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.gpu
def test_two_gpu_token_shards_and_nccl_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        oracle = importlib.import_module("oracle.fwht_oracle")
        rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        inp = oracle.make_inputs("c5", K=2048, M=512, N=1024)
        X, W = inp["X"].cuda(), inp["W"].cuda()
        full = pkg.fused_ht_gemm(X, W, out_layout="nm", out_dtype=torch.bfloat16)
        local = pkg.fused_ht_gemm(pkg.shard_tokens(X, rank, world), W, out_layout="nm", out_dtype=torch.bfloat16)
        got = pkg.gather_result(local, X.shape[0], "nm")
        assert torch.equal(got, full), "sharded result differs"
        assert pkg.device_status() == 0
        dist.barrier(); dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29644", str(script)],
        capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.count("ok") == 2, r.stdout + r.stderr


@pytest.mark.gpu
def test_two_gpu_row_sharded_gemv(tmp_path):
    """Small-batch split: each GPU streams half of the rows of W, transforms the same X, and an NCCL all-gather of
    M x B values assembles Y; the result equals the single-GPU call up to fp32 summation order."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        oracle = importlib.import_module("oracle.fwht_oracle")
        rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        for B in (1, 4, 16):
            inp = oracle.make_inputs("c4", B=B)
            W, X = inp["W"].cuda(), inp["X"].cuda()
            full = pkg.fused_ht_gemv(W, X)
            local = pkg.fused_ht_gemv(pkg.shard_rows(W, rank, world).contiguous(), X)
            got = pkg.gather_rows(local, W.shape[0])
            # a shard has other rows per CTA than the full matrix, hence another split of K over the warps and
            # another order of the fp32 partial sums: equal up to fp32 rounding, not bit for bit
            err = float((got - full).norm() / full.norm())
            assert err < 1e-5, f"row-sharded result differs: {{err}}"
        assert pkg.device_status() == 0
        dist.barrier(); dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29645", str(script)],
        capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.count("ok") == 2, r.stdout + r.stderr


@pytest.mark.gpu
def test_row_sharded_gemv_on_one_rank(tmp_path):
    """The degenerate split: one rank holds all rows, there is no peer, and the call is the plain GEMV writing into
    the wrapper's result buffer (runs on any box)."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        torch.cuda.set_device(0)
        dist.init_process_group("gloo")
        g = torch.Generator().manual_seed(5)
        W = (torch.randn(1000, 2048, generator=g) / 45).bfloat16().cuda()
        op = pkg.RowShardedGemv(W, 1000, 8)
        for B in (8, 3, 8):
            X = torch.randn(2048, B, generator=g).bfloat16().cuda()
            assert torch.equal(op(X), pkg.fused_ht_gemv(W, X))
        op.close()
        assert pkg.device_status() == 0
        dist.destroy_process_group()
        print("ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29647", RANK="0", WORLD_SIZE="1")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_two_gpu_row_sharded_gemv_with_peer_stores(tmp_path):
    """The same split with the exchange inside the kernel: every GPU sends its rows of Y, tagged with the number of
    the call, into a slot array on the other GPU through peer-mapped pointers and collects the other's rows from its
    own.  Several calls back to back
    (the two result buffers alternate), ragged row split, both output types; compared with the single-GPU call."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import importlib, os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        pkg = importlib.import_module("6s894_project_2025_b200")
        rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        g = torch.Generator().manual_seed(9)
        for M, N, odt in ((4096, 4096, torch.float32), (4097, 1024, torch.bfloat16)):
            W = (torch.randn(M, N, generator=g) / N ** 0.5).bfloat16().cuda()
            op = pkg.RowShardedGemv(pkg.shard_rows(W, rank, world).contiguous(), M, 16, out_dtype=odt)
            for B in (1, 4, 16, 3):
                X = torch.randn(N, B, generator=g).bfloat16().cuda()
                got = op(X).clone()
                full = pkg.fused_ht_gemv(W, X, out_dtype=odt)
                err = float((got.float() - full.float()).norm() / full.float().norm())
                assert err < (1e-5 if odt == torch.float32 else 1e-2), f"peer-store result differs: {{err}}"
            # the same calls replayed from a CUDA graph (the kernel counts the calls itself): two calls per graph,
            # so the result buffers keep alternating; new X before every replay
            X = torch.randn(N, 4, generator=g).bfloat16().cuda()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    y0 = op(X)
                    y1 = op(X)
            for rep in range(3):
                X.copy_(torch.randn(N, 4, generator=g).bfloat16())
                graph.replay()
                torch.cuda.synchronize()
                full = pkg.fused_ht_gemv(W, X, out_dtype=odt).float()
                for y in (y0, y1):
                    err = float((y.float() - full).norm() / full.norm())
                    assert err < (1e-5 if odt == torch.float32 else 1e-2), f"graph replay {{rep}} differs: {{err}}"
            got = op(X).clone()      # and an ordinary call behind the replays
            assert float((got.float() - full).norm() / full.norm()) < (1e-5 if odt == torch.float32 else 1e-2)
            op.close()
        assert pkg.device_status() == 0
        dist.barrier(); dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29646", str(script)],
        capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.count("ok") == 2, r.stdout + r.stderr
