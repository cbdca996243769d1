"""Build libb200ht.so (sm_100a) in-tree with nvcc.

    python -m 6s894_project_2025_b200.build      # not importable as a dotted name;
    python 6s894_project_2025_b200/build.py      # run the file instead

The library is written for B200 only: one ``-gencode arch=compute_100a,
code=sm_100a`` target, no PTX for other architectures, no fallback build.
Objects are rebuilt only when their source (or a header) changed.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
ROOT = HERE.parent
OUT = HERE / "libb200ht.so"
OBJ_DIR = HERE / "build"
STAMP = HERE / "libb200ht.so.sha"   # digest of the sources the library was built from

SOURCES = ["api.cu", "fwht.cu", "fwht_tcgen05.cu", "fused_gemm.cu", "gemm_tcgen05.cu", "fused_gemv.cu", "fused_gemv_tc.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
INCLUDE_FLAGS = ["-I", str(ROOT / "include")]   # not part of the digest: the checkout may sit at any path


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: libb200ht.so cannot be built (there is no fallback path)")
    return nvcc


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def source_digest() -> str:
    """Digest of everything libb200ht.so is built from (sources, headers, flags)."""
    return _digest([CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "b200ht.h"])


def is_current() -> bool:
    """True when libb200ht.so exists and was built from the sources as they are now."""
    return OUT.exists() and STAMP.exists() and STAMP.read_text().strip() == source_digest()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what changed and link.  Safe to call from several processes at once (one builds, the others wait)."""
    import fcntl

    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    with open(HERE / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current():
            return OUT
        headers = list(CSRC.glob("*.cuh")) + [ROOT / "include" / "b200ht.h"]
        jobs = []
        objs = []
        for src in SOURCES:
            s = CSRC / src
            o = OBJ_DIR / (s.stem + ".o")
            stamp = OBJ_DIR / (s.stem + ".sha")
            dig = _digest([s] + headers)
            objs.append(o)
            if force or not o.exists() or not stamp.exists() or stamp.read_text() != dig:
                cmd = [nvcc, *NVCC_FLAGS, *INCLUDE_FLAGS, "-c", str(s), "-o", str(o)]
                if verbose:
                    cmd.insert(1, "-Xptxas=-v")
                jobs.append((cmd, stamp, dig))

        def run(job):
            cmd, stamp, dig = job
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
            if verbose:
                sys.stderr.write(r.stderr)
            stamp.write_text(dig)

        if jobs:
            with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
                list(ex.map(run, jobs))
        cmd = [nvcc, "-shared", "-o", str(OUT), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        STAMP.write_text(source_digest())
    return OUT


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(p)
