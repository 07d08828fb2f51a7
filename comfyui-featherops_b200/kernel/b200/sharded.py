"""Column-sharded mixed-precision linear for one box of 2/4/8 GPUs: each rank keeps the weight columns
[r*N/g, (r+1)*N/g) of the prepacked (K/16, N, 16) weight (dim 1), the activations are replicated, every rank computes
its [M, N/g] block and the blocks are all-gathered along N.

The reference has no multi-GPU path; this layer is new.  K is never split, so each output element sees the same
additions in the same order on any number of ranks: the sharded result is bitwise the single-GPU result.

Two exchange steps are provided:

  "all_gather"  `torch.distributed.all_gather_into_tensor` (NCCL over NVLink) delivers [g, M, N/g]; the [M, N] row-major
                layout the next layer expects is then one strided copy.  This is the baseline.
  "peer_store"  the exchange is fused into the GEMM: the output lives in symmetric memory (one [M, N] buffer per rank, every
                rank can address every peer's buffer), and the kernel's epilogue TMA-stores each finished block into its
                column range of ALL ranks' buffers while the tensor cores work on the next tile.  No separate collective, no
                relayout copy; a cross-rank barrier before (peers are done reading the previous output) and after (all
                stores have landed) brackets the launch.  Only stores cross NVLink; nothing loads from peer memory.

With world size 1 there is no exchange and no copy.
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
    def __init__(self, b_prepacked, scale, bias, rank, world, device, group=None, exchange="all_gather"):
        if exchange not in ("all_gather", "peer_store"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.rank, self.world, self.group = rank, world, group
        self.exchange = exchange
        self._symm = {}
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

    def _symmetric_output(self, m, out_dtype, device):
        """[m, N] output buffer in symmetric memory plus views of every rank's buffer (cached per (m, dtype))."""
        key = (m, out_dtype)
        entry = self._symm.get(key)
        if entry is None:
            import torch.distributed._symmetric_memory as symm_mem

            group = self.group if self.group is not None else dist.group.WORLD
            buf = symm_mem.empty((m, self.n_total), dtype=out_dtype, device=device)
            handle = symm_mem.rendezvous(buf, group.group_name)
            views = [buf if r == self.rank else handle.get_buffer(r, (m, self.n_total), out_dtype) for r in range(self.world)]
            entry = (buf, handle, views)
            self._symm[key] = entry
        return entry

    def _peer_store(self, a, out_dtype, variant):
        m = a.shape[0]
        buf, handle, views = self._symmetric_output(m, out_dtype, a.device)
        lo, hi = self.rank * self.n_local, (self.rank + 1) * self.n_local
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]      # own buffer first
        outputs = [views[r][:, lo:hi] for r in order]
        handle.barrier()                       # every rank has finished reading the previous contents of its buffer
        native.scaled_mm_multi_into(a, self.b_local, self.scale, self.bias_local, outputs, variant=variant)
        handle.barrier()                       # every rank's blocks have landed everywhere
        return buf

    def __call__(self, a, out_dtype, variant=None):
        if self.world > 1 and self.exchange == "peer_store":
            return self._peer_store(a, out_dtype, variant)
        local = self.gemm_only(a, out_dtype, variant)
        if self.world == 1:
            return local
        m = a.shape[0]
        gathered = torch.empty((self.world * m, self.n_local), dtype=out_dtype, device=a.device)    # rank-major concatenation
        dist.all_gather_into_tensor(gathered, local, group=self.group)
        return gathered.view(self.world, m, self.n_local).permute(1, 0, 2).reshape(m, self.n_total)
