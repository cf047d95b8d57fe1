"""flare_decode_attn_noalloc — the decode entry point for callers that cannot allocate.

Some hosts of this library may not call cudaMalloc at the moment they need attention: a
server that handed every byte of GPU memory to its own pool when it started, a real-time
callback that must never block on the driver's allocator, a process whose policy freezes
allocation after initialisation.  For them the library keeps a fixed split-KV workspace
inside its own image.  This test drives that entry point through the C ABI with caller-owned
device buffers and checks it, twice in a row (the workspace keeps the previous call's
contents), against the ordinary entry point and the CPU oracle.

The file name sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import numpy as np
import pytest

from util import assert_close, normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype_name,hd,nh,nkv,B,ctx", [("KV_Q8_0", 64, 32, 8, 4, 4096), ("KV_F32", 128, 8, 2, 2, 1500)])
def test_noalloc_matches_regular_entry_point_twice(orc, dtype_name, hd, nh, nkv, B, ctx):
    import torch
    import flarellm_b200 as fb

    eng = fb.Engine(0)
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, getattr(fb, dtype_name))
    k, v = normal(301, (B, ctx, nkv * hd)), normal(302, (B, ctx, nkv * hd))
    for b in range(B):
        kv.append(0, b, k[b, :-1], v[b, :-1])
        kv.advance(b, ctx - 1)
        kv.write(0, b, ctx - 1, k[b, -1], v[b, -1])
    kd = np.stack([kv.export_dequant(0, b)[0] for b in range(B)])
    vd = np.stack([kv.export_dequant(0, b)[1] for b in range(B)])
    assert eng.L.flare_decode_attn_noalloc_scratch_bytes() == 8 << 20

    for call, (seed, attend) in enumerate([(311, None), (312, np.array([ctx - 7 * b for b in range(B)], np.int32))]):
        q = normal(seed, (B, 1, nh, hd), 0.4)
        q_dev = torch.from_numpy(q).cuda()
        out_dev = torch.full((B, 1, nh, hd), float("nan"), device="cuda")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()          # driver-level: sees any cudaMalloc in the process
        eng.decode_noalloc(kv, 0, nh, q_dev.data_ptr(), out_dev.data_ptr(), attend_len=attend)
        eng.sync()
        if call > 0:
            # The first call on a device is the set-up call: the driver may load the library's device
            # image then, and that image contains the 8 MiB workspace.  From the second call on,
            # free device memory must not move at all.
            assert torch.cuda.mem_get_info()[0] == free_before, "the no-allocation entry point allocated device memory"
        got = out_dev.cpu().numpy()
        regular = eng.decode(kv, 0, nh, q, attend_len=attend)
        # the ordinary entry point may take another kernel for this shape: compare within the output tolerance
        assert_close(got, regular, f"call {call}: no-alloc vs regular entry point")
        al = attend if attend is not None else np.full(B, ctx, np.int32)
        want = orc.gqa_decode_batched(q.reshape(B, 1, -1), kd, vd, al, nh, nkv, hd, threads=4)
        assert_close(got, want, f"call {call}: no-alloc vs oracle")
    kv.free()
    eng.close()


def test_noalloc_rejects_what_does_not_fit():
    import torch
    import flarellm_b200 as fb

    eng = fb.Engine(0)
    q = torch.zeros(1, device="cuda")
    # 2-bit caches and odd head sizes are not served by this entry point
    kv = eng.kv_alloc(1, 1, 256, 2, 64, fb.KV_KIVI_G32)
    with pytest.raises(fb.FlareError) as e:
        eng.decode_noalloc(kv, 0, 8, q.data_ptr(), q.data_ptr())
    assert e.value.status == fb.ERR_UNSUPPORTED
    kv.free()
    # more sequences than the built-in per-sequence records hold (256)
    B = 257
    kv = eng.kv_alloc(1, B, 8, 1, 64, fb.KV_F32)
    qd = torch.zeros(B * 64, device="cuda")
    od = torch.zeros(B * 64, device="cuda")
    with pytest.raises(fb.FlareError) as e:
        eng.decode_noalloc(kv, 0, 1, qd.data_ptr(), od.data_ptr())
    assert e.value.status == fb.ERR_INVALID_ARG and "no-allocation maximum" in str(e.value)
    kv.free()
    eng.close()


def test_noalloc_serves_the_largest_batch_it_accepts(orc):
    """256 sequences x 32 heads is the most rows the entry point takes.  The workspace guard (partials larger
    than the 8 MiB array are refused) cannot fire below that: the split count falls as the rows grow, and rows x
    splits x (head_dim + 2) floats stays under 5 MiB.  So the largest batch must simply run, and run right."""
    import torch
    import flarellm_b200 as fb

    nh, nkv, hd, B, ctx = 32, 8, 64, 256, 96
    eng = fb.Engine(0)
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, fb.KV_F32)
    k, v = normal(321, (B, ctx, nkv * hd)), normal(322, (B, ctx, nkv * hd))
    for b in range(B):
        kv.append(0, b, k[b], v[b])
    attend = (np.arange(B, dtype=np.int32) % ctx) + 1
    q = normal(323, (B, 1, nh, hd), 0.4)
    q_dev = torch.from_numpy(q).cuda()
    out_dev = torch.full((B, 1, nh, hd), float("nan"), device="cuda")
    eng.decode_noalloc(kv, 0, nh, q_dev.data_ptr(), out_dev.data_ptr(), attend_len=attend)
    eng.sync()
    want = orc.gqa_decode_batched(q.reshape(B, 1, -1), k, v, attend, nh, nkv, hd, threads=8)
    assert_close(out_dev.cpu().numpy(), want, "no-alloc at batch 256")
    kv.free()
    eng.close()
