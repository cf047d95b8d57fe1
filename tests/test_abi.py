"""CPU-only: the C-ABI library exists, loads, and exports exactly what include/flare_attn.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "flare_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"FLARE_API\s+[\w\s\*]+?\b(flare_\w+)\s*\(", text)


@pytest.fixture(scope="module")
def built():
    from flarellm_b200 import build
    return build.build()


def test_header_declares_what_python_binds(built):
    import flarellm_b200 as fb
    declared = header_functions()
    assert len(declared) == len(set(declared)) and len(declared) >= 30
    assert sorted(declared) == sorted(name for name, _, _ in fb.SYMBOLS)


def test_library_exports_every_declared_symbol(built):
    L = ctypes.CDLL(built)
    for name in header_functions():
        assert hasattr(L, name), f"libflare_attn.so does not export {name}"


def test_python_layer_loads_and_names_backend(built):
    import flarellm_b200 as fb
    L = fb.lib()
    assert L.flare_attn_backend_name() == b"cuda"          # ComputeBackend::name
    assert L.flare_attn_last_error(None) == b"null context"
    assert L.flare_attn_launch_count(None) == 0
    assert L.flare_kv_plane_bytes(None, 0) == 0


def test_no_cpu_fallback_without_a_device(built):
    """Without a CUDA device the engine refuses to come up (there is no CPU path)."""
    import flarellm_b200 as fb
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a CUDA device is present")
    with pytest.raises(fb.FlareError) as e:
        fb.Engine(0)
    assert e.value.status == fb.ERR_CUDA


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "flarellm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
