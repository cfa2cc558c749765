"""CPU-only checks of the drop-in boundary: the library loads and exports what the header declares."""
import ctypes
import os
import re

import pytest

import infr_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "infr_cuda.h")).read()
    return sorted(set(re.findall(r"INFR_API\s+[\w\s\*]+?\b(infr_(?:cuda|gguf)_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _header_symbols() == sorted(infr_b200.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = infr_b200.load_library()
    for name in _header_symbols():
        assert hasattr(lib, name), name


def test_no_unexpected_exports():
    import subprocess

    out = subprocess.run(["nm", "-D", "--defined-only", infr_b200.LIB_PATH], capture_output=True, text=True).stdout
    syms = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    assert syms == set(_header_symbols())


def test_create_without_a_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(infr_b200.BackendError) as ei:
        infr_b200.CudaBackend(device=0)
    assert ei.value.code == infr_b200.E_CUDA
    assert "no CPU fallback" in str(ei.value)


def test_null_context_is_rejected_not_dereferenced():
    lib = infr_b200.load_library()
    assert lib.infr_cuda_sync(None) == infr_b200.E_INVALID
    assert lib.infr_cuda_launch_count(None) == 0
    lib.infr_cuda_destroy(None)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "infr_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"import\s+oracle|from\s+oracle|oracle/|cpu_oracle|libinfr_cpu_oracle", text), (dirpath, f)


def test_struct_sizes_match_the_header():
    # infr_op_desc: tag + 8 + 12 u32 + 4 f32 = 25 words; infr_tensor_decl: 2 u32 + u64
    assert ctypes.sizeof(infr_b200._OpDesc) == 100
    assert ctypes.sizeof(infr_b200._TensorDecl) == 16
    assert ctypes.sizeof(infr_b200._Opts) == 32
