"""Long-context decode of ONE sequence whose KV cache is split along the slot axis over the
ranks of a process group (one process per GPU).

The reference has no multi-device path; this is the block form of its online-softmax recurrence
(flare-core/src/model.rs:9945-9956): every rank attends its own slot range and produces, per
query head, ``[m, l, o[head_dim]]`` (running max, sum, unnormalised output); the records are
all-gathered (NCCL over NVLink on GPUs) and every rank merges them by log-sum-exp:

    m* = max_r m_r,   l = sum_r l_r e^(m_r - m*),   o = sum_r o_r e^(m_r - m*) / l

The only collective is that all-gather of ``num_heads * (head_dim + 2)`` floats per rank.

Two front ends:

* ``CAbiSplitDecoder`` — what a host of the library uses: ``flare_attn_comm_init`` +
  ``flare_decode_attn_splitkv_multi``; the exchange happens inside the library (records stored straight
  into the peers' buffers by the merging kernel, or ``ncclAllGather``), ``torch.distributed`` only carries
  the 128-byte communicator id to the other ranks.
* ``SplitKvDecoder`` — the same step spelled out on the host with ``torch.distributed`` (any backend),
  with pluggable partial / merge functions; the CPU tests run it over gloo with a CPU routine standing in
  for the kernels.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple


def shard_slots(total_slots: int, world: int, rank: int, granule: int = 32) -> Tuple[int, int]:
    """Even split of ``[0, total_slots)`` into ``world`` contiguous ranges whose boundaries are
    multiples of ``granule`` (the decode kernels' tile).  Returns ``(begin, end)`` for ``rank``;
    ranges may be empty when there are more ranks than granules."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    granules = (total_slots + granule - 1) // granule
    lo = (granules * rank) // world * granule
    hi = (granules * (rank + 1)) // world * granule
    return min(lo, total_slots), min(hi, total_slots)


class SplitKvDecoder:
    """Decode attention for one sequence sharded over ``group``.

    ``partial_fn(layer, q) -> tensor [rows, head_dim + 2]`` computes this rank's records and
    ``merge_fn(gathered [world, rows, head_dim + 2]) -> tensor [rows, head_dim]`` merges them; by
    default both are the engine's ``flare_decode_attn_partial`` / ``flare_merge_partials`` on the
    local cache shard (local slots ``0 .. n_local-1`` hold global slots ``begin .. end-1``).
    """

    def __init__(self, eng=None, kv_local=None, num_heads: int = 0, n_local: int = 0, group=None,
                 partial_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.eng, self.kv, self.num_heads, self.n_local = eng, kv_local, num_heads, n_local
        if eng is not None and partial_fn is None:
            # The collective is ordered against torch's current stream only, so the engine's kernels must run
            # on that stream too: otherwise the all-gather could read the records before they are written.
            import torch
            eng.set_stream(torch.cuda.current_stream(torch.device("cuda", eng.device)).cuda_stream)
        self.partial_fn = partial_fn or self._partial_engine
        self.merge_fn = merge_fn or self._merge_engine
        self._bufs = None

    # ---- engine-backed defaults (device tensors) --------------------------------------------
    def _buffers(self):
        import torch
        if self._bufs is None:
            rows, hd = self.kv.batch * self.num_heads, self.kv.head_dim
            dev = torch.device("cuda", self.eng.device)
            self._bufs = (torch.empty(rows, hd + 2, device=dev), torch.empty(self.world, rows, hd + 2, device=dev),
                          torch.empty(rows, hd, device=dev))
        return self._bufs

    def _partial_engine(self, layer, q):
        part, _, _ = self._buffers()
        self.eng.decode_partial(self.kv, layer, self.num_heads, q.data_ptr(), 0, self.n_local, out=part.data_ptr())
        return part

    def _merge_engine(self, gathered):
        _, _, out = self._buffers()
        rows, hd = out.shape
        self.eng.merge_partials(gathered.data_ptr(), self.world, rows, hd, out=out.data_ptr())
        return out

    # ---- the step ------------------------------------------------------------------------------
    def decode(self, layer, q):
        """One attention call: local records -> all-gather -> merge.  Returns ``[rows, head_dim]``."""
        import torch
        part = self.partial_fn(layer, q)
        if self.world == 1:
            return self.merge_fn(part.unsqueeze(0))
        if self._bufs is not None and part.is_cuda:
            gathered = self._bufs[1]
        else:
            gathered = torch.empty((self.world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
        if part.is_cuda:
            self.dist.all_gather_into_tensor(gathered, part.contiguous(), group=self.group)     # NCCL
        else:
            self.dist.all_gather(list(gathered.unbind(0)), part.contiguous(), group=self.group)  # gloo (CPU tests)
        return self.merge_fn(gathered)


class CAbiSplitDecoder:
    """Decode attention for one sequence sharded over the ranks of ``dist`` through the library's own
    multi-GPU entry points (include/flare_attn.h: flare_attn_comm_*, flare_decode_attn_splitkv_multi).

    ``kv_local`` holds this rank's slots ``0 .. n_local-1``.  ``direct=True`` asks for the exchange without
    a collective (peer stores); if the set-up is refused (no peer access between the GPUs) the NCCL
    all-gather inside the library is used and ``direct_error`` says why.
    """

    def __init__(self, eng, kv_local, num_heads: int, n_local: int, dist=None, direct: bool = True, wait_ms: int = 0):
        import torch
        self.torch, self.eng, self.kv, self.num_heads, self.n_local, self.dist = torch, eng, kv_local, num_heads, n_local, dist
        self.world = dist.get_world_size() if dist is not None else 1
        self.rank = dist.get_rank() if dist is not None else 0
        self.direct_error = None
        rows, hd = kv_local.batch * num_heads, kv_local.head_dim
        if self.world > 1:
            box = [type(eng).comm_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            eng.comm_init(box[0], self.rank, self.world)
            self.how = "ncclAllGather issued inside the library + merge kernel"
            if direct:
                # the set-up is collective: every rank must attempt it, and all must agree on the outcome
                try:
                    eng.comm_enable_direct(rows, hd)
                    ok = 1 if eng.comm_info()[2] else 0      # the library's own probe may have switched it off again
                    if not ok:
                        self.direct_error = eng.L.flare_attn_last_error(eng.h).decode()
                except Exception as e:      # FlareError: no peer access / IPC refused
                    self.direct_error, ok = str(e), 0
                flag = torch.tensor([ok], device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 1:
                    self.how = ("records stored into the peers' buffers by the merging kernel (peer stores, bounded wait, "
                                "no collective; probe %.1f us per exchange)" % eng.comm_probe_us())
                elif ok:
                    raise RuntimeError("direct exchange set up on this rank but not on every rank")
                else:
                    self.how += " (direct exchange not used: %s)" % self.direct_error
            if wait_ms:
                eng.comm_set_wait_ms(wait_ms)
        else:
            eng.comm_init(None, 0, 1)
            self.how = "one GPU: merge kernel only"
        dev = torch.device("cuda", eng.device)
        self.out = torch.empty(rows, hd, device=dev)
        self.part = torch.empty(rows, hd + 2, device=dev)

    def decode(self, layer, q):
        self.eng.decode_splitkv_multi(self.kv, layer, self.num_heads, q.data_ptr(), self.n_local, out=self.out.data_ptr())
        return self.out

    def partial_only(self, layer, q):
        """This rank's attention kernels alone (no exchange), for timing."""
        self.eng.decode_partial(self.kv, layer, self.num_heads, q.data_ptr(), 0, self.n_local, out=self.part.data_ptr())
        return self.part

    def status(self) -> str:
        """Waits for the queued calls; "ok", or the library's message (e.g. a rank that did not show up in time)."""
        try:
            self.eng.sync()
            return "ok"
        except Exception as e:
            return str(e)

    def close(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()             # nobody frees a buffer that a peer may still be writing
        self.eng.comm_destroy()


def make_split_decoder(eng, kv_local, num_heads, n_local, dist=None, direct=True):
    return CAbiSplitDecoder(eng, kv_local, num_heads, n_local, dist, direct)
