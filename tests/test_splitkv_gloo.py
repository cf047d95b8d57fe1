"""CPU, world_size 2 (gloo): the host-side split-KV plumbing — slot sharding, all-gather of the
per-rank (m, l, o) records, log-sum-exp merge — with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_slots_covers_range_on_tile_boundaries():
    from flarellm_b200.splitkv import shard_slots
    for total, world in [(131072, 8), (131072, 1), (4100, 4), (31, 4), (0, 2), (96, 5)]:
        cuts = [shard_slots(total, world, r) for r in range(world)]
        assert cuts[0][0] == 0 and cuts[-1][1] == total
        for (a, b), (c, d) in zip(cuts[:-1], cuts[1:]):
            assert b == c and a <= b
        assert all(a % 32 == 0 for a, _ in cuts)
    with pytest.raises(ValueError):
        shard_slots(10, 2, 2)


def _worker(rank, world, port, seed, total, nh, nkv, hd, ret):
    import torch
    import torch.distributed as dist
    import oracle
    from flarellm_b200.splitkv import SplitKvDecoder, shard_slots
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(seed)                       # every rank draws the same sequence
    q = rng.standard_normal(nh * hd, dtype=np.float32) * np.float32(0.3)
    k = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    v = rng.standard_normal((total, nkv * hd), dtype=np.float32)
    lo, hi = shard_slots(total, world, rank)
    k_local, v_local = k[lo:hi], v[lo:hi]                   # this rank only ever touches its shard

    def partial_fn(layer, q_t):
        rec = oracle.gqa_decode_partial(q_t.numpy(), k_local, v_local, nh, nkv, hd, 0, hi - lo)
        return torch.from_numpy(rec)

    def merge_fn(gathered):
        return torch.from_numpy(oracle.merge_partials(gathered.numpy(), nh, hd).reshape(nh, hd))

    dec = SplitKvDecoder(num_heads=nh, n_local=hi - lo, partial_fn=partial_fn, merge_fn=merge_fn)
    out = dec.decode(0, torch.from_numpy(q)).numpy().reshape(-1)
    want = oracle.gqa_decode(q, k, v, nh, nkv, hd, total)
    ret[rank] = float(np.max(np.abs(out - want)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [1000, 40])
def test_two_rank_split_equals_single_device(total):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, 5, total, 8, 2, 32, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert all(err < 2e-6 for err in ret.values()), dict(ret)


def _worker_absent(rank, world, port, ret):
    """Rank 1 never makes the call; rank 0's all-gather ends with an error after the group's short timeout."""
    import datetime
    import torch
    import torch.distributed as dist
    from flarellm_b200.splitkv import SplitKvDecoder
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    nh, hd = 4, 8
    dec = SplitKvDecoder(num_heads=nh, n_local=0, partial_fn=lambda layer, q: torch.zeros(nh, hd + 2),
                         merge_fn=lambda g: torch.zeros(nh, hd))
    dec.decode(0, torch.zeros(nh * hd))            # a first step with every rank present
    if rank == 1:
        ret[rank] = "left between steps"
        return                                      # leaves between steps: nothing of it is in flight
    try:
        dec.decode(0, torch.zeros(nh * hd))
        ret[rank] = "no error"
    except Exception as e:                          # the collective reports the missing rank; nothing hangs
        ret[rank] = "error: " + type(e).__name__


def test_a_rank_that_skips_the_call_gives_the_others_an_error_not_a_hang():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker_absent, args=(world, port, ret), nprocs=world, join=True)
    assert ret[1] == "left between steps"
    assert ret[0].startswith("error"), dict(ret)
