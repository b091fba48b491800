"""N-sharded (tensor-parallel) int8 weight-only linears: one process per GPU.

The quantized-matmul path shards along the output columns of each weight:
rank r of P holds ``w[:, r*N/P:(r+1)*N/P]`` and the matching per-channel
scales, computes ``y[:, shard]`` from the replicated activations with no
reduction across ranks, and one all-gather rebuilds the output.  The reference
has nothing to compare with here: its collectives are identity ops on a single
device (src/pjrt_plugin/ops/collective_ops.mm:34-84,118-146); the semantics
implemented are those of ``stablehlo.all_gather`` over one replica group.

``ncclAllGather`` (``torch.distributed.all_gather_into_tensor``) concatenates
whole rank buffers, so gathering row-major ``[M, N/P]`` shards yields
``[P, M, N/P]``; :func:`gathered_to_logical` describes that buffer as the
logical ``[M, N]`` result (a strided view, no copy), which is how a consumer
addresses it.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Columns ``[start, stop)`` of an N-wide weight held by ``rank`` of ``world`` ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % world:
        raise ValueError(f"N ({n}) must be divisible by the number of ranks ({world})")
    per = n // world
    return rank * per, (rank + 1) * per


def gathered_to_logical(gathered: torch.Tensor) -> torch.Tensor:
    """View the all-gathered ``[P, M, N/P]`` buffer as the logical ``[M, N]`` output (no copy)."""
    p, m, ns = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, p * ns) if not gathered.is_contiguous() else \
        gathered.as_strided((m, p, ns), (ns, m * ns, 1)).reshape(m, p * ns)


class ColumnShardedLinear:
    """One rank's shard of an int8 per-channel weight-only linear."""

    def __init__(self, w_shard: torch.Tensor, scale_shard: torch.Tensor, n_total: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        start, stop = shard_bounds(n_total, self.world, self.rank)
        if w_shard.shape[1] != stop - start or scale_shard.shape != (stop - start,):
            raise ValueError("shard shapes do not match this rank's column range")
        self.w, self.scale, self.n_total = w_shard, scale_shard, n_total
        self.columns = (start, stop)

    def local(self, x: torch.Tensor, out: torch.Tensor | None = None, matmul=None) -> torch.Tensor:
        """``x @ dequant(w_shard)`` -> ``[M, N/P]``.  ``matmul`` replaces the CUDA kernel in host-logic tests."""
        if matmul is None:
            from . import ops

            return ops.w8a16_perchannel(x, self.w, self.scale, out=out)
        y = matmul(x, self.w, self.scale)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def forward(self, x: torch.Tensor, matmul=None) -> torch.Tensor:
        """Local matmul followed by the all-gather; returns the ``[P, M, N/P]`` buffer."""
        y = self.local(x, matmul=matmul)
        if self.world == 1:
            return y.unsqueeze(0)
        gathered = torch.empty((self.world,) + tuple(y.shape), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(gathered.view(-1), y.contiguous().view(-1), group=self.group)
        return gathered
