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
