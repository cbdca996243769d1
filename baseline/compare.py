#!/usr/bin/env python
"""Same-box GPU comparators: the reference's own kernels, rebuilt unmodified for sm_100, beside this library.

    python baseline/compare.py build --ref <checkout of Alan-Chen99/6s894_project_2025>
    python baseline/compare.py run [--json out.json] [--only fwht,gemv,gemm]
    python baseline/compare.py report --json out.json        # markdown tables of a run

``build`` compiles, from the sources where they lie in the checkout and into ``baseline/_ref/`` (git-ignored):

    ref_fht           csrc/main.cu + csrc/hada_handler.cu behind ref_fht_driver.cu        (case "Ours" of the reference's
                      bench/bench.py: its own tensor-core transform)
    ref_hadacore      HadaCore/hadamard_transform_cuda.cu behind the same driver          (case "HadaCore")
    fusion_pipelined  fused_ht/fusion_pipelined.cu, the program as it is                   (fp32, K=1024, 4096 x 4096)
    ref_gemv          fused_ht/fwht_gemv_fusion.cu's two kernels behind ref_gemv_driver.cu (fp32, W 4096 x 4096)

The reference ships these for sm_80/89/90 only (csrc/setup.py:5-12, HadaCore/setup.py:4-11); nothing of it is copied
into this repository, and nothing here is on the product path or an oracle.  ``run`` needs a B200: it executes
whichever of the binaries exist, times this library on the same shapes in the same process sequence, and prints one
JSON document whose ``results`` entries carry the fields of the reference's own payload (bench/bench.py:226-237
there: device, case, m, n, dtype, runs, per_iter_ms, total_ms) plus GB/s or TFLOP/s.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import re
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "_ref"
ARCH = ["-gencode", "arch=compute_100,code=sm_100"]
TORCH_DEFS = ["-D_GLIBCXX_USE_CXX11_ABI=1", "--expt-relaxed-constexpr", "-D__CUDA_NO_HALF_OPERATORS__",
              "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"]


def _torch_dir() -> Path:
    import torch

    return Path(torch.__file__).resolve().parent


def build(ref: Path) -> None:
    nvcc = os.environ.get("NVCC", "nvcc")
    OUT.mkdir(exist_ok=True)
    t = _torch_dir()
    inc = ["-I", str(t / "include"), "-I", str(t / "include/torch/csrc/api/include")]
    link = ["-L", str(t / "lib"), "-lc10", "-lc10_cuda", "-Xlinker", "-rpath", "-Xlinker", str(t / "lib")]
    jobs = {
        "fusion_pipelined": [nvcc, "-O3", *ARCH, "-o", str(OUT / "fusion_pipelined"), str(ref / "fused_ht/fusion_pipelined.cu")],
        "ref_gemv": [nvcc, "-O3", *ARCH, "-I", str(ref / "fused_ht"), "-o", str(OUT / "ref_gemv"),
                     str(HERE / "ref_gemv_driver.cu"), "-lcublas"],
        "ref_fht": [nvcc, "-O3", "-std=c++20", "-diag-suppress=3189", *ARCH, "-I", str(ref / "csrc"), *inc, *TORCH_DEFS,
                    "-o", str(OUT / "ref_fht"), str(HERE / "ref_fht_driver.cu"), str(ref / "csrc/main.cu"),
                    str(ref / "csrc/hada_handler.cu"), *link],
        # torch/extension.h (included by the reference file) needs the Python headers; several minutes of compile time
        "ref_hadacore": [nvcc, "-O3", "-std=c++17", *ARCH, *inc, "-I", sysconfig.get_paths()["include"], *TORCH_DEFS,
                         "-DUSE_HADACORE", "-o", str(OUT / "ref_hadacore"), str(HERE / "ref_fht_driver.cu"),
                         str(ref / "HadaCore/hadamard_transform_cuda.cu"), *link, "-ltorch_cpu", "-ltorch"],
    }
    for name, cmd in jobs.items():
        print("building", name, flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(f"  FAILED ({name}):\n" + (r.stdout + r.stderr)[-3000:])
        else:
            print("  ok")


_RESULT = re.compile(r"^RESULT (.*)$")


def _parse_results(text: str) -> list[dict]:
    out = []
    for line in text.splitlines():
        m = _RESULT.match(line.strip())
        if not m:
            continue
        d = {}
        for k, v in re.findall(r"(\w+)=((?:[^= ]| (?!\w+=))+)", m.group(1)):
            d[k] = v.strip()
        for k in ("m", "n", "runs", "batch"):
            if k in d:
                d[k] = int(d[k])
        for k in ("per_iter_ms", "total_ms", "max_rel_err"):
            if k in d:
                d[k] = float(d[k])
        out.append(d)
    return out


def _run_binary(name: str, *args: str) -> str | None:
    exe = OUT / name
    if not exe.exists():
        return None
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = str(_torch_dir() / "lib") + ":" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([str(exe), *args], capture_output=True, text=True, env=env, timeout=1800)
    if r.returncode != 0:
        print(f"{name} exited {r.returncode}:\n{(r.stdout + r.stderr)[-2000:]}", file=sys.stderr)
    return r.stdout


def _ours_fwht(torch, pkg, device_name):
    """This library on the two transform shapes of ref_fht_driver.cu (same rotation, same in-place calls)."""
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    res = []
    for shape in ("rot", "2p30"):
        for logn in range(8, 16):
            n = 1 << logn
            rows = 16384 if shape == "rot" else (1 << 30) // n
            nbytes = rows * n * 2
            nbuf = max(2, math.ceil((512 << 20) / nbytes)) if shape == "rot" else 1
            bufs = [torch.full((rows, n), 0.0115, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
            reps = 10

            def call(b):
                rc = lib.b200ht_fwht(b.data_ptr(), b.data_ptr(), rows, n, pkg._lib.BF16, float(n ** -0.5), st)
                assert rc == 0, pkg._lib.error_string(rc)

            for b in bufs:
                call(b)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                for b in bufs:
                    call(b)
            e1.record()
            torch.cuda.synchronize()
            total = e0.elapsed_time(e1)
            res.append({"device": device_name, "case": "b200ht", "shape": shape, "m": n, "n": rows, "dtype": "bfloat16",
                        "runs": reps * nbuf, "per_iter_ms": total / (reps * nbuf), "total_ms": total})
            del bufs
    return res


def _ours_gemv(torch, pkg, device_name):
    M = N = 4096
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(7)
    res = []
    for dt, code, name in ((torch.bfloat16, pkg._lib.BF16, "bfloat16"), (torch.float32, pkg._lib.F32, "float32")):
        Ws = [(torch.randn(M, N, generator=g, device="cuda") / 64).to(dt) for _ in range(16)]
        for B in (1, 4, 16):
            X = torch.randn(N, B, generator=g, device="cuda").to(dt)
            Y = torch.empty(M, B, dtype=torch.float32, device="cuda")

            def call(W):
                rc = lib.b200ht_fused_gemv(W.data_ptr(), X.data_ptr(), Y.data_ptr(), M, N, B, code, pkg._lib.F32, 1.0, st)
                assert rc == 0, pkg._lib.error_string(rc)

            for W in Ws[:3]:
                call(W)
            torch.cuda.synchronize()
            reps = 3 if dt == torch.float32 else 20
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                for W in Ws:
                    call(W)
            e1.record()
            torch.cuda.synchronize()
            total = e0.elapsed_time(e1)
            res.append({"device": device_name, "case": "b200ht_fused_gemv", "shape": "gemv", "m": M, "n": N, "batch": B,
                        "dtype": name, "runs": reps * 16, "per_iter_ms": total / (reps * 16), "total_ms": total})
        del Ws
    return res


def _ours_gemm(torch, pkg, device_name):
    """K=1024, 4096 tokens, M=4096 (the shape compiled into fusion_pipelined.cu:51-53), unscaled like the reference."""
    K, N, M = 1024, 4096, 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    res = []
    for name, dt, exact in (("float32 (FFMA, exact)", torch.float32, True), ("float32 (tensor cores, 3 x bf16)", torch.float32, False),
                            ("bfloat16", torch.bfloat16, False)):
        X = torch.rand(N, K, generator=g, device="cuda").to(dt)
        W = torch.rand(M, K, generator=g, device="cuda").to(dt)
        ws = torch.empty(pkg.fused_gemm_workspace_bytes(M, N, K, dt, exact=exact), dtype=torch.uint8, device="cuda")
        C = torch.empty(M, N, dtype=torch.float32, device="cuda")
        for _ in range(2):
            pkg.fused_ht_gemm(X, W, scale=1.0, out=C, workspace=ws, exact=exact)
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(8):   # the reference reports the minimum of 8 timed runs (fusion_pipelined.cu:631-655)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            pkg.fused_ht_gemm(X, W, scale=1.0, out=C, workspace=ws, exact=exact)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        res.append({"device": device_name, "case": "b200ht_fused_gemm", "shape": "gemm_k1024_4096x4096", "m": M, "n": N,
                    "dtype": name, "runs": 8, "per_iter_ms": best, "total_ms": best, "statistic": "min"})
    return res


def run(args) -> None:
    import torch

    sys.path.insert(0, str(ROOT))
    pkg = importlib.import_module("6s894_project_2025_b200")
    device_name = torch.cuda.get_device_name(0)
    only = set(args.only.split(",")) if args.only else {"fwht", "gemv", "gemm"}
    results, checks, raw = [], [], {}

    if "fwht" in only:
        for exe in ("ref_fht", "ref_hadacore"):
            text = _run_binary(exe)
            if text is None:
                raw[exe] = "not built"
                continue
            for r in _parse_results(text):
                r["device"] = device_name
                results.append(r)
            checks += [ln for ln in text.splitlines() if ln.startswith("CHECK")]
        results += _ours_fwht(torch, pkg, device_name)
        for r in results:
            if r.get("shape") in ("rot", "2p30"):
                r["gbs"] = r["m"] * r["n"] * 4 / (r["per_iter_ms"] * 1e-3) / 1e9
    if "gemv" in only:
        text = _run_binary("ref_gemv")
        if text is None:
            raw["ref_gemv"] = "not built"
        else:
            for r in _parse_results(text):
                r["device"] = device_name
                results.append(r)
        results += _ours_gemv(torch, pkg, device_name)
    if "gemm" in only:
        text = _run_binary("fusion_pipelined")
        if text is None:
            raw["fusion_pipelined"] = "not built"
        else:
            raw["fusion_pipelined"] = text[-1500:]
            for label, case in (("Baseline (Parallel HT + Unfused GEMM) min time", "reference unfused baseline"),
                                ("Pipelined (Parallel HT + Fused GEMM) min time", "fused_ht_gemm_pipelined")):
                m = re.search(re.escape(label) + r":\s*([0-9.]+) ms", text)
                if m:
                    results.append({"device": device_name, "case": case, "shape": "gemm_k1024_4096x4096", "m": 4096,
                                    "n": 4096, "dtype": "float32", "runs": 8, "per_iter_ms": float(m.group(1)),
                                    "total_ms": float(m.group(1)), "statistic": "min"})
        results += _ours_gemm(torch, pkg, device_name)
        for r in results:
            if r.get("shape") == "gemm_k1024_4096x4096":
                r["tflops"] = 2.0 * 4096 * 4096 * 1024 / (r["per_iter_ms"] * 1e-3) / 1e12
    payload = {"device": device_name, "cases": sorted({r["case"] for r in results}), "pytorch": torch.__version__,
               "results": results, "checks": checks, "notes": raw}
    text = json.dumps(payload, indent=1)
    if args.json:
        Path(args.json).write_text(text)
    print(text)


def report(args) -> None:
    """Markdown tables from the JSON that ``run`` wrote (what profiles/reference_kernels_on_b200.md holds)."""
    d = json.loads(Path(args.json).read_text())
    res = d["results"]
    print(f"Device: {d['device']}; PyTorch {d['pytorch']}.\n")
    for shape, title in (("rot", "(16384, n) bf16, in place on >= 512 MB of rotating buffers"),
                         ("2p30", "2^30 elements per n, bf16, in place (the reference's own benchmark shape)")):
        rows = [r for r in res if r.get("shape") == shape]
        if not rows:
            continue
        cases = ["Ours(reference csrc)", "HadaCore", "b200ht"]
        print(f"### Transform, {title}\n")
        print("| n | reference `csrc` GB/s (us) | `HadaCore` GB/s (us) | this library GB/s (us) | vs `csrc` | vs `HadaCore` |")
        print("|---:|---:|---:|---:|---:|---:|")
        for n in sorted({r["m"] for r in rows}):
            cell, val = {}, {}
            for c in cases:
                m = [r for r in rows if r["case"] == c and r["m"] == n]
                if m:
                    cell[c] = f"{m[0]['gbs']:.0f} ({m[0]['per_iter_ms'] * 1e3:.1f})"
                    val[c] = m[0]["gbs"]
                else:
                    cell[c] = "-"
            ratio = lambda c: f"{val['b200ht'] / val[c]:.2f}" if c in val and "b200ht" in val else "-"   # noqa: E731
            print(f"| {n} | {cell[cases[0]]} | {cell[cases[1]]} | {cell[cases[2]]} | {ratio(cases[0])} | {ratio(cases[1])} |")
        print()
    rows = [r for r in res if r.get("shape") == "gemv"]
    if rows:
        print("### Fused GEMV, W 4096 x 4096, 16 rotating copies of W (us per call)\n")
        print("| case | dtype | B = 1 | B = 4 | B = 16 |")
        print("|---|---|---:|---:|---:|")
        for case, dt in sorted({(r["case"], r["dtype"]) for r in rows}):
            t = {r["batch"]: r["per_iter_ms"] * 1e3 for r in rows if r["case"] == case and r["dtype"] == dt}
            print(f"| `{case}` | {dt} | " + " | ".join(f"{t[b]:.1f}" if b in t else "-" for b in (1, 4, 16)) + " |")
        print()
    rows = [r for r in res if r.get("shape") == "gemm_k1024_4096x4096"]
    if rows:
        print("### Fused W.H(X), K = 1024, 4096 tokens, M = 4096, unscaled, minimum of 8 runs\n")
        print("| case | dtype | ms | TFLOP/s |")
        print("|---|---|---:|---:|")
        for r in rows:
            print(f"| `{r['case']}` | {r['dtype']} | {r['per_iter_ms']:.3f} | {r['tflops']:.1f} |")
        print()
    if d.get("checks"):
        print("Reference transform outputs against a host butterfly (4 rows per n, inputs in [-2, 2]): max |err| "
              + ", ".join(sorted({c.split("max_abs_err=")[1] for c in d["checks"]})[:1]) + " ... "
              + max(c.split("max_abs_err=")[1] for c in d["checks"]) + " (their own tolerance is 5e-2).")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("--ref", required=True, type=Path, help="root of a checkout of the reference")
    r = sub.add_parser("run")
    r.add_argument("--json", default=None)
    r.add_argument("--only", default=None, help="comma-separated subset of fwht,gemv,gemm")
    rp = sub.add_parser("report")
    rp.add_argument("--json", required=True)
    args = ap.parse_args()
    if args.cmd == "build":
        build(args.ref)
    elif args.cmd == "report":
        report(args)
    else:
        run(args)


if __name__ == "__main__":
    main()
