"""The range-checked build of the library (-DFLARE_DEBUG_BOUNDS) on small and edge shapes.

compute-sanitizer cannot be used where this library is developed, so the kernels that index shared memory by
hand-computed offsets (swizzled TMA tiles, ldmatrix rows, stage rings) have a build variant in which every such
offset, and every record written to global memory, is checked against the extent of its buffer; a violation
stores FLARE_ERR_BOUNDS in the context's status word instead of trapping.  This test runs the parity tests that
walk those kernels through their edge cases — ragged lengths, rings that are not a tile multiple, every split
count, wrapped rings, prompt lengths that are not a tile multiple — against that build: they must pass, which
also means no call reported FLARE_ERR_BOUNDS (a reported status fails the call that reads results).
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DBG = os.path.join(ROOT, "flarellm_b200", "libflare_attn_dbg.so")

SELECTION = [
    ("tests/test_gpu_decode.py", "q8_split_counts or ring_size_not_a_tile or q8_ring_wrap or speculative or two_items or bounded_wait"),
    ("tests/test_gpu_kivi.py", "tensor_core_path or wrapped_ring or ragged_batch"),
    ("tests/test_gpu_prefill.py", "tensor_core"),
]


@pytest.mark.parametrize("path,expr", SELECTION)
def test_edge_shapes_on_the_range_checked_build(path, expr):
    if not os.path.exists(DBG):
        pytest.skip("libflare_attn_dbg.so has not been built (python -m flarellm_b200.build --variant _dbg -DFLARE_DEBUG_BOUNDS)")
    env = dict(os.environ, FLARE_ATTN_LIB=DBG)
    r = subprocess.run([sys.executable, "-m", "pytest", path, "-m", "gpu", "-q", "-x", "-k", expr, "-p", "no:cacheprovider"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=1200)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "BOUNDS" not in r.stdout, tail
