"""Builds liblbk.so (the CUDA C-ABI library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "liblbk.so"
OBJ = PKG / "_build"  # object files (git-ignored)

SOURCES = ["lbk_api.cu", "lbk_gemv.cu", "lbk_quant.cu", "lbk_bf16.cu", "lbk_plan.cu", "lbk_sweep.cu", "lbk_gemm.cu", "lbk_noalloc.cu", "lbk_decoder.cu", "lbk_tp.cu", "lbk_model.cu", "lbk_convert.cu", "lbk_probe.cu", "lbk_attn_tc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; liblbk.so cannot be built")


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "lbk.h"]
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd, env):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout)
    return res.stdout


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu (one object each, side by side, only the ones whose source or any header
    changed) and link lemonade_burn_b200/liblbk.so. Returns the library path."""
    if not force and not is_stale():
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    OBJ.mkdir(exist_ok=True)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    nvcc = nvcc_path()
    headers = list(CSRC.glob("*.cuh")) + [ROOT / "include" / "lbk.h"]
    newest_header = max(h.stat().st_mtime for h in headers)
    jobs = []
    for s in SOURCES:
        src, obj = CSRC / s, OBJ / (Path(s).stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header):
            cmd = [nvcc, *NVCC_FLAGS, "-c", f"-I{ROOT / 'include'}", f"-I{CSRC}", "-o", str(obj), str(src)]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4) or 1) as pool:
        logs = list(pool.map(lambda c: _run(c, env), jobs))
    if verbose:
        print("\n".join(logs))
    _run([nvcc, "-shared", "-o", str(LIB)] + [str(OBJ / (Path(s).stem + ".o")) for s in SOURCES], env)
    return LIB


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
