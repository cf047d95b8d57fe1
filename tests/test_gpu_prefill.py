"""GPU parity: causal / sliding-window prefill attention against the oracle's loop of decode calls
(flare-core/src/model.rs:336-368)."""
import numpy as np
import pytest

from util import assert_close, normal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb():
    import flarellm_b200 as fb
    return fb


@pytest.fixture(scope="module")
def eng(fb):
    e = fb.Engine(0)
    yield e
    e.close()


def bf16_inputs(orc, seed, B, S, nh, nkv, hd, scale=0.5):
    """N(0,1)*scale rounded to bf16, so that the f32 -> bf16 conversion inside the engine is exact."""
    q = orc.bf16_round(normal(seed, (B, S, nh * hd), scale))
    k = orc.bf16_round(normal(seed + 1, (B, S, nkv * hd), scale))
    v = orc.bf16_round(normal(seed + 2, (B, S, nkv * hd), scale))
    return q, k, v


def check(orc, got, q, k, v, S, nh, nkv, hd, window=0, row_step=1, what=""):
    B = q.shape[0]
    got = np.asarray(got, dtype=np.float32).reshape(B, S, nh * hd)
    worst = 0.0
    for b in range(B):
        want = orc.prefill(q[b], k[b], v[b], S, nh, nkv, hd, window=window, row_start=(b * 7) % row_step, row_step=row_step, threads=8)
        rows = ~np.isnan(want[:, 0])
        worst = max(worst, assert_close(got[b][rows], want[rows], f"{what} seq {b}"))
    return worst


def test_reference_recipe_small_shapes_through_trait_hook(fb, orc):
    """flare-gpu/src/backend.rs:6165-6212 (seq 4, 2 heads, head_dim 8, |d| < 1e-4) and two more odd shapes."""
    be = fb.CudaBackend(0)
    for (S, nh, nkv, hd) in [(4, 2, 2, 8), (9, 4, 2, 16), (1, 2, 1, 4), (33, 3, 1, 3)]:
        q, k, v = normal(S, (S, nh * hd)), normal(S + 1, (S, nkv * hd)), normal(S + 2, (S, nkv * hd))
        got = be.prefill_attention_gpu(q, k, v, S, nh, nkv, hd)
        want = orc.prefill(q, k, v, S, nh, nkv, hd)
        assert np.max(np.abs(got.reshape(S, -1) - want)) < 1e-4


def test_generic_window(eng, fb, orc):
    S, nh, nkv, hd, W = 50, 4, 2, 16, 7
    q, k, v = normal(1, (1, S, nh * hd)), normal(2, (1, S, nkv * hd)), normal(3, (1, S, nkv * hd))
    got = eng.prefill(q, k, v, 1, S, nh, nkv, hd, window=W)
    check(orc, got, q, k, v, S, nh, nkv, hd, window=W, what="generic window")


def test_generic_path_with_more_rows_than_one_launch_holds(eng, fb, orc):
    """head_dim 32 takes the general path, where every prompt row is one grid.z entry: 8 x 8200 = 65600 rows are more
    than the 65535 a launch can hold, so the rows go out in two launches."""
    B, S, nh, nkv, hd, W = 8, 8200, 2, 1, 32, 64
    q, k, v = normal(61, (B, S, nh * hd)), normal(62, (B, S, nkv * hd)), normal(63, (B, S, nkv * hd))
    got = eng.prefill(q, k, v, B, S, nh, nkv, hd, window=W).reshape(B, S, nh * hd)
    for b in (0, B - 1):             # the last rows of the last sequence are the ones past the first launch
        want = orc.prefill(q[b], k[b], v[b], S, nh, nkv, hd, window=W, row_start=S - 1 - 7 * 1000, row_step=1000)
        rows = ~np.isnan(want[:, 0])
        assert rows.sum() == 8
        assert_close(got[b][rows], want[rows], f"general path, 65600 rows, seq {b}")


@pytest.mark.parametrize("B,S,nh,nkv,hd", [(1, 128, 2, 1, 128), (2, 300, 4, 2, 128), (1, 257, 4, 4, 64), (1, 640, 8, 2, 128)])
def test_tensor_core_causal(eng, fb, orc, B, S, nh, nkv, hd):
    q, k, v = bf16_inputs(orc, 10 + S, B, S, nh, nkv, hd)
    got = eng.prefill(q, k, v, B, S, nh, nkv, hd)
    check(orc, got, q, k, v, S, nh, nkv, hd, what=f"tc causal S={S} hd={hd}")


def test_tensor_core_window(eng, fb, orc):
    B, S, nh, nkv, hd, W = 1, 700, 4, 2, 128, 200
    q, k, v = bf16_inputs(orc, 31, B, S, nh, nkv, hd)
    got = eng.prefill(q, k, v, B, S, nh, nkv, hd, window=W)
    check(orc, got, q, k, v, S, nh, nkv, hd, window=W, what="tc window")


def test_tensor_core_bf16_in_out(eng, fb, orc):
    B, S, nh, nkv, hd = 2, 384, 4, 1, 128
    q, k, v = bf16_inputs(orc, 41, B, S, nh, nkv, hd)
    qb, kb, vb = (orc.f32_to_bf16(x) for x in (q, k, v))
    got = eng.prefill(qb, kb, vb, B, S, nh, nkv, hd, in_dtype=fb.DT_BF16, out_dtype=fb.DT_BF16)
    got32 = (got.astype(np.uint32) << 16).view(np.float32)
    # the output itself is rounded to bf16: one more 2^-9 relative step on top of the tolerance
    B_, want_all = q.shape[0], []
    for b in range(B):
        want = orc.prefill(q[b], k[b], v[b], S, nh, nkv, hd, threads=8)
        err = np.abs(got32[b].reshape(S, -1) - want)
        assert np.all(err <= 2e-3 + (1e-3 + 2.0 ** -8) * np.abs(want))


def test_llama8b_shape_prefill_spot_rows(eng, fb, orc):
    """32 q / 8 kv heads, head_dim 128, S = 2048 (one sequence); every 97th row is checked."""
    B, S, nh, nkv, hd = 1, 2048, 32, 8, 128
    q, k, v = bf16_inputs(orc, 51, B, S, nh, nkv, hd)
    got = eng.prefill(q, k, v, B, S, nh, nkv, hd)
    check(orc, got, q, k, v, S, nh, nkv, hd, row_step=97, what="llama-8b shape")
    # causality: output rows 0..999 do not depend on later tokens
    q2, k2, v2 = q.copy(), k.copy(), v.copy()
    k2[:, 1000:] = 0; v2[:, 1000:] = 7
    got2 = eng.prefill(q2, k2, v2, B, S, nh, nkv, hd)
    assert np.array_equal(got.reshape(S, -1)[:1000], got2.reshape(S, -1)[:1000])
