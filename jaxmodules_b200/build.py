"""Builds libbma.so (the C-ABI library with every CUDA kernel) in-tree with nvcc for sm_100a.

    python -m jaxmodules_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects go to jaxmodules_b200/csrc/build/, the library
to jaxmodules_b200/libbma.so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libbma.so"

SOURCES = ["bma_api.cu", "mask_compile.cu", "mask_program.cu", "attn_simt.cu", "attn_fwd_sm100.cu", "attn_bwd_sm100.cu", "attn_bwd_dq_sm100.cu", "attn_bwd_dq_replay_sm100.cu", "bwd_slots.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    headers = list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h")) + [Path(__file__)]

    def compile_one(src: str):
        s, o = CSRC / src, OBJ / (src + ".o")
        if not force and not _stale(o, [s] + headers):
            return o, ""
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(s), "-o", str(o)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return o, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        results = list(ex.map(compile_one, SOURCES))
    objs = [str(o) for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart", "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    _build_jax_adapter(force)
    return LIB


def _build_jax_adapter(force: bool) -> None:
    """libbma_jax.so (the XLA-FFI handlers of csrc/bma_jax.cc) -- only where jax ships its FFI headers; skipped,
    silently, everywhere else (the torch/ctypes binding needs none of it)."""
    try:
        import jax
        inc = jax.ffi.include_dir()
    except Exception:
        return
    out, src = PKG / "libbma_jax.so", CSRC / "bma_jax.cc"
    if not force and not _stale(out, [src, LIB]):
        return
    cmd = [_nvcc(), "-shared", "-std=c++17", "-Xcompiler", "-fPIC", "-I", inc, str(src), "-o", str(out),
           "-L", str(PKG), "-lbma", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the jax adapter failed:\n{r.stdout}\n{r.stderr}")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
