"""Two GPUs, one process each (NCCL): a single sequence's Q8_0 cache split along the slot axis,
per-rank partial attention, all-gather of the (m, l, o) records, merge — against the oracle on the
whole sequence.  Skipped when fewer than two devices are visible."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, nh, nkv, hd, ret):
    import torch
    import torch.distributed as dist
    import flarellm_b200 as fb
    import oracle
    from flarellm_b200.splitkv import SplitKvDecoder, shard_slots
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    rng = np.random.default_rng(17)
    q = rng.standard_normal((1, 1, nh, hd), dtype=np.float32) * np.float32(0.3)
    k = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    v = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    lo, hi = shard_slots(total, world, rank)
    eng = fb.Engine(rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)
    kv = eng.kv_alloc(1, 1, max(hi - lo, 32), nkv, hd, fb.KV_Q8_0)
    kv.append(0, 0, k[lo:hi], v[lo:hi]); kv.advance(0, hi - lo)
    dec = SplitKvDecoder(eng, kv, nh, hi - lo)
    qd = torch.from_numpy(q).cuda()
    for _ in range(3):                      # repeated calls reuse the buffers
        out = dec.decode(0, qd)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(-1)
    kd, vd = oracle.dequant_q8_0(oracle.quantize_q8_0(k)), oracle.dequant_q8_0(oracle.quantize_q8_0(v))
    want = oracle.gqa_decode(q.reshape(-1), kd, vd, nh, nkv, hd, total)
    err = np.abs(got - want)
    ret[rank] = (float(err.max()), bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want))))
    dist.barrier()
    kv.free(); eng.close()
    dist.destroy_process_group()


def _worker_cabi(rank, world, port, total, nh, nkv, hd, direct, ret):
    """The same sequence through the library's own multi-GPU call (flare_decode_attn_splitkv_multi)."""
    import torch
    import torch.distributed as dist
    import flarellm_b200 as fb
    import oracle
    from flarellm_b200.splitkv import CAbiSplitDecoder, shard_slots
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    rng = np.random.default_rng(19)
    q = rng.standard_normal((1, 1, nh, hd), dtype=np.float32) * np.float32(0.3)
    k = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    v = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    lo, hi = shard_slots(total, world, rank)
    eng = fb.Engine(rank)
    kv = eng.kv_alloc(1, 1, max(hi - lo, 32), nkv, hd, fb.KV_Q8_0)
    kv.append(0, 0, k[lo:hi], v[lo:hi]); kv.advance(0, hi - lo)
    dec = CAbiSplitDecoder(eng, kv, nh, hi - lo, dist, direct=direct)
    qd = torch.from_numpy(q).cuda()
    for _ in range(5):                      # repeated calls alternate the halves of the record buffers
        out = dec.decode(0, qd)
    status = dec.status()
    got = out.cpu().numpy().reshape(-1)
    host = eng.decode_splitkv_multi(kv, 0, nh, q, hi - lo).reshape(-1)      # host buffers in and out
    kd, vd = oracle.dequant_q8_0(oracle.quantize_q8_0(k)), oracle.dequant_q8_0(oracle.quantize_q8_0(v))
    want = oracle.gqa_decode(q.reshape(-1), kd, vd, nh, nkv, hd, total)
    err = np.maximum(np.abs(got - want), np.abs(host - want))
    ret[rank] = (float(err.max()), bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want))) and status == "ok", dec.how, status)
    dec.close()
    kv.free(); eng.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("direct", [True, False])
@pytest.mark.parametrize("total,hd", [(6000, 128), (333, 64), (40, 64)])
def test_two_gpu_split_kv_through_the_c_abi(total, hd, direct):
    """Records exchanged by peer stores inside the merging kernel (direct) or by ncclAllGather inside the library;
    40 slots leave rank 1 with 8 slots only."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker_cabi, args=(world, port, total, 32, 8, hd, direct, ret), nprocs=world, join=True)
    assert len(ret) == world and all(r[1] for r in ret.values()), dict(ret)


def test_one_gpu_world_of_one_and_missing_peer(orc):
    """flare_decode_attn_splitkv_multi without a second rank is plain attention over the slots given; and the
    direct exchange's wait gives up (FLARE_ERR_TIMEOUT) when a peer never publishes, leaving the context usable."""
    import flarellm_b200 as fb
    nh, nkv, hd, n = 32, 8, 128, 5000
    eng = fb.Engine(0)
    kv = eng.kv_alloc(1, 1, n, nkv, hd, fb.KV_Q8_0)
    rng = np.random.default_rng(23)
    k = rng.standard_normal((n, nkv * hd), dtype=np.float32)
    v = rng.standard_normal((n, nkv * hd), dtype=np.float32)
    q = rng.standard_normal((1, 1, nh, hd), dtype=np.float32) * np.float32(0.3)
    kv.append(0, 0, k, v); kv.advance(0, n)
    kd, vd = orc.dequant_q8_0(orc.quantize_q8_0(k)), orc.dequant_q8_0(orc.quantize_q8_0(v))
    want = orc.gqa_decode(q.reshape(-1), kd, vd, nh, nkv, hd, n)
    got = eng.decode_splitkv_multi(kv, 0, nh, q, n)                  # no communicator at all
    assert np.all(np.abs(got.reshape(-1) - want) <= 2e-3 + 1e-3 * np.abs(want))
    eng.comm_init(None, 0, 1)
    got = eng.decode_splitkv_multi(kv, 0, nh, q, n)                  # a world of one
    assert np.all(np.abs(got.reshape(-1) - want) <= 2e-3 + 1e-3 * np.abs(want))
    part = eng.decode_splitkv_multi(kv, 0, nh, q, 3000)              # a prefix of the slots
    want_p = orc.gqa_decode(q.reshape(-1), kd, vd, nh, nkv, hd, 3000)
    assert np.all(np.abs(part.reshape(-1) - want_p) <= 2e-3 + 1e-3 * np.abs(want_p))
    assert eng.comm_selftest_missing_peer() == fb.ERR_TIMEOUT
    assert eng.comm_selftest_missing_peer() == fb.ERR_TIMEOUT        # the status word was cleared in between
    got = eng.decode_splitkv_multi(kv, 0, nh, q, n)
    assert np.all(np.abs(got.reshape(-1) - want) <= 2e-3 + 1e-3 * np.abs(want))
    eng.comm_destroy()
    kv.free(); eng.close()


@pytest.mark.parametrize("total,hd", [(6000, 128), (333, 64)])
def test_two_gpu_split_kv_matches_oracle(total, hd):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, total, 32, 8, hd, ret), nprocs=world, join=True)
    assert len(ret) == world and all(ok for _, ok in ret.values()), dict(ret)
