"""Long-context decode of ONE sequence whose KV cache is split along the slot axis over the
ranks of a process group (one process per GPU).

The reference has no multi-device path; this is the block form of its online-softmax recurrence
(flare-core/src/model.rs:9945-9956): every rank attends its own slot range and produces, per
query head, ``[m, l, o[head_dim]]`` (running max, sum, unnormalised output); the records are
all-gathered (NCCL over NVLink on GPUs) and every rank merges them by log-sum-exp:

    m* = max_r m_r,   l = sum_r l_r e^(m_r - m*),   o = sum_r o_r e^(m_r - m*) / l

The only collective is that all-gather of ``num_heads * (head_dim + 2)`` floats per rank.
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
