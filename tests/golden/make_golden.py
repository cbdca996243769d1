"""Generate the golden vectors in this directory from the reference itself.

Run once, in a container that has the reference checkout (no GPU needed):

    python tests/golden/make_golden.py /path/to/reference

The reference's only CPU-runnable statement of the transform is
``hadamard_ref`` in bench/bench.py:55-59 (``t @ (scipy.linalg.hadamard(n) *
sqrt(1/n))``).  That module imports ``cappa``, ``csrc`` and ``hada_core`` (a CLI
package and two CUDA extensions, none installable here) and builds its matrix
with ``device="cuda"`` (bench/bench.py:50-52).  This script therefore loads the
module with three empty stand-in modules and a ``torch`` proxy whose
``tensor`` drops the ``device`` argument; ``hadamard_ref`` itself runs
unmodified.  The outputs are stored with their inputs so the tests need neither
the reference nor this script.

Fixtures written (all inputs from ``torch.manual_seed(0)`` as in
bench/bench.py:255 and HadaCore/test.py:46):
  fwht_golden.npz   x_{n} (rows x n fp32 input), y32_{n} = hadamard_ref in fp32,
                    yb16_{n}/yf16_{n} = hadamard_ref applied to the bf16/fp16
                    cast, for n = 2 .. 4096
  fused_golden.npz  C = W @ hadamard_ref(X)^T for the K=64, B=8, M=32 case and
                    a 128 x 256 x 32 case (token-major X), fp32
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch


class _TorchProxy:
    """Forwards to torch; ``tensor`` ignores device= (no GPU in the container)."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def tensor(*a, **kw):
        kw.pop("device", None)
        return torch.tensor(*a, **kw)


def load_reference_bench(ref_root: Path):
    class _Anything(types.ModuleType):
        def __getattr__(self, name):  # cappa.command, cappa.Arg, ... -> inert callables
            def f(*a, **k):
                if len(a) == 1 and callable(a[0]) and not k:
                    return a[0]
                return None
            return f

    for name in ("cappa", "csrc", "hada_core"):
        sys.modules.setdefault(name, _Anything(name))
    spec = importlib.util.spec_from_file_location("_ref_bench", ref_root / "bench" / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.torch = _TorchProxy()
    return mod


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of Alan-Chen99/6s894_project_2025>")
    ref_root = Path(sys.argv[1])
    out_dir = Path(__file__).resolve().parent
    bench = load_reference_bench(ref_root)

    torch.manual_seed(0)
    fw = {}
    for logn in range(1, 13):
        n = 1 << logn
        rows = 5 if n <= 1024 else 3
        a = torch.randn((rows, n), dtype=torch.float32)
        t32 = a.clone()
        bench.hadamard_ref(t32)            # in place, bench/bench.py:55-59
        tb = a.clone().to(torch.bfloat16)
        bench.hadamard_ref(tb)
        th = a.clone().to(torch.float16)
        bench.hadamard_ref(th)
        fw[f"x_{n}"] = a.numpy()
        fw[f"y32_{n}"] = t32.numpy()
        fw[f"yb16_{n}"] = tb.float().numpy()
        fw[f"yf16_{n}"] = th.float().numpy()
    np.savez_compressed(out_dir / "fwht_golden.npz", **fw)

    fu = {}
    # K=64, B=8, M=32 (first self-test shape of fused_ht/fwht_gemv_fusion.cu:632)
    W = torch.randn(32, 64)
    X = torch.randn(64, 8)                 # K x B, b fastest
    Yt = X.t().contiguous().clone()        # B x K, one row per column
    bench.hadamard_ref(Yt)
    fu["c1_W"], fu["c1_X"] = W.numpy(), X.numpy()
    fu["c1_Y"] = (W @ Yt.t()).numpy()      # M x B
    # token-major fused GEMM, K=256, N=32 tokens, M=128
    Xg = torch.randn(32, 256)
    Wg = torch.randn(128, 256)
    Yg = Xg.clone()
    bench.hadamard_ref(Yg)
    fu["g_X"], fu["g_W"] = Xg.numpy(), Wg.numpy()
    fu["g_C"] = (Wg @ Yg.t()).numpy()      # M x N
    np.savez_compressed(out_dir / "fused_golden.npz", **fu)
    for f in ("fwht_golden.npz", "fused_golden.npz"):
        print(f, (out_dir / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
