"""Column-sharded mixed-precision linear for one box of 2/4/8 GPUs: each rank keeps the weight columns
[r*N/g, (r+1)*N/g) of the prepacked (K/16, N, 16) weight (dim 1), the activations are replicated, every rank computes
its [M, N/g] block and the blocks are all-gathered along N.

The reference has no multi-GPU path; this layer is new.  K is never split, so each output element sees the same
additions in the same order on any number of ranks: the sharded result is bitwise the single-GPU result.

Exchange step: `torch.distributed.all_gather_into_tensor` (NCCL over NVLink) delivers [g, M, N/g]; the [M, N] row-major
layout the next layer expects is then one strided copy.  With world size 1 there is no exchange and no copy.
"""

import torch
import torch.distributed as dist

from . import native


def shard_columns(b_prepacked, bias, rank, world):
    """The contiguous weight (and bias) shard of `rank`.  N must divide evenly."""
    n = b_prepacked.shape[1]
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by the number of ranks {world}")
    per = n // world
    b_local = b_prepacked[:, rank * per:(rank + 1) * per, :].contiguous()
    bias_local = bias[rank * per:(rank + 1) * per].contiguous() if bias is not None else None
    return b_local, bias_local


class ColumnShardedLinear:
    def __init__(self, b_prepacked, scale, bias, rank, world, device, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.n_total = b_prepacked.shape[1]
        self.k = b_prepacked.shape[0] * 16
        self.b_local, self.bias_local = shard_columns(b_prepacked.to(device), bias.to(device) if bias is not None else None, rank, world)
        self.n_local = self.b_local.shape[1]
        self.scale = scale.to(device=device, dtype=torch.float32)
        # the heuristic sees the full N so that a shard picks the variant (in particular the K split) of the whole
        self._variant_shape_n = self.n_total
        self.launches_per_call = 1

    def _variant(self, m, variant):
        if variant is not None:
            return variant
        if self.world == 1:
            return None
        v = native.choose_variant(m, self._variant_shape_n, self.k)
        return v

    def gemm_only(self, a, out_dtype, variant=None, out=None):
        if out is None:
            out = torch.empty((a.shape[0], self.n_local), dtype=out_dtype, device=a.device)
        native.scaled_mm_into(a, self.b_local, self.scale, self.bias_local, out, variant=self._variant(a.shape[0], variant))
        return out

    def __call__(self, a, out_dtype, variant=None):
        local = self.gemm_only(a, out_dtype, variant)
        if self.world == 1:
            return local
        m = a.shape[0]
        gathered = torch.empty((self.world * m, self.n_local), dtype=out_dtype, device=a.device)    # rank-major concatenation
        dist.all_gather_into_tensor(gathered, local, group=self.group)
        return gathered.view(self.world, m, self.n_local).permute(1, 0, 2).reshape(m, self.n_total)
