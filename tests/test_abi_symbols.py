"""The C-ABI library loads, exports every function include/bma.h declares, and the ctypes
mirrors of its structs have the C compiler's layout.  No compute call is made."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

from jaxmodules_b200 import _native as nat

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "bma.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(bma_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 10
    lib = nat.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bma.h but not exported"
    assert set(names) == set(nat.SIGNATURES), "ctypes signature table and header disagree"
    assert lib.bma_version() >= 1000
    assert b"ok" == lib.bma_error_string(0)
    assert b"workspace" in lib.bma_error_string(nat.BMA_ERR_WORKSPACE)


def test_struct_layouts_match_the_c_compiler(tmp_path):
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "bma.h"\n'
        "int main(void){\n"
        'printf("%zu %zu %zu %zu\\n", sizeof(bma_mask_spec), sizeof(bma_block_lists), sizeof(bma_tensor), sizeof(bma_attn_args));\n'
        'printf("%zu %zu %zu\\n", offsetof(bma_mask_spec, seg_q), offsetof(bma_mask_spec, bitmap), offsetof(bma_block_lists, kv_num));\n'
        'printf("%zu %zu %zu %zu\\n", offsetof(bma_attn_args, q), offsetof(bma_attn_args, lse), offsetof(bma_attn_args, d_o), offsetof(bma_attn_args, dv));\n'
        "return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    got = [int(x) for x in out]
    want = [C.sizeof(nat.MaskSpec), C.sizeof(nat.BlockLists), C.sizeof(nat.Tensor), C.sizeof(nat.AttnArgs),
            nat.MaskSpec.seg_q.offset, nat.MaskSpec.bitmap.offset, nat.BlockLists.kv_num.offset,
            nat.AttnArgs.q.offset, nat.AttnArgs.lse.offset, nat.AttnArgs.d_o.offset, nat.AttnArgs.dv.offset]
    assert got == want


def test_argument_validation_without_a_device():
    """Rejected arguments return before any CUDA call, so this runs on a CPU-only host."""
    lib = nat.lib()
    assert lib.bma_attn_plan(None, None, None, None) == nat.BMA_ERR_ARG
    a = nat.AttnArgs()
    a.B, a.N, a.L, a.Hq, a.Hkv, a.d = 1, 8, 8, 3, 2, 16
    assert lib.bma_attn_plan(C.byref(a), None, None, None) == nat.BMA_ERR_ARG        # Hq % Hkv
    a.Hq, a.d = 2, 512
    assert lib.bma_attn_plan(C.byref(a), None, None, None) == nat.BMA_ERR_UNSUPPORTED  # head dim
    assert lib.bma_mask_compile(None, 1, 1, None, None, 0, None) == nat.BMA_ERR_ARG
    assert lib.bma_mask_compile_workspace_bytes(None, 1, 1, 1, 1) == 0


def test_jax_adapter_is_guarded():
    """The jax.ffi adapter is source only where jax is absent: importing it must fail with ImportError (not half-load),
    the package itself must import without it, and the build must skip it silently."""
    import importlib.util
    import jaxmodules_b200  # noqa: F401
    from jaxmodules_b200 import build
    assert (build.CSRC / "bma_jax.cc").exists()
    if importlib.util.find_spec("jax") is None:
        with pytest.raises(ImportError):
            importlib.import_module("jaxmodules_b200.jax_binding")
        build._build_jax_adapter(force=False)          # no jax: returns without building anything
        assert not (build.PKG / "libbma_jax.so").exists()
