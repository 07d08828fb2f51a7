"""Mixed-precision linears sharded over the 2/4/8 GPUs of one box, one process per GPU.

The reference has no multi-GPU path; everything here is new.  Two shardings of the prepacked (K/16, N, 16) weight:

ColumnShardedLinear   rank r keeps the weight columns [r*N/g, (r+1)*N/g) (dim 1).  The activations are replicated, every rank
                      computes its [M, N/g] block.  K is never split, so each output element sees the same additions in the
                      same order on any number of ranks: the result is bitwise the single-GPU result.  Exchanges:
    "peer_store"      fused into the GEMM.  The output is an [M, N] buffer in symmetric memory on every rank; the kernel's
                      epilogue TMA-stores each finished block into its column range of ALL ranks' buffers while the tensor
                      cores run the next tile (two staging buffers per epilogue group, so a block is staged while NVLink
                      still takes the previous one).  Outputs are double-buffered per (M, dtype), so ONE cross-rank barrier per call is enough, the one
                      after the launch ("all blocks have landed"): a rank reaches the barrier of call n only after its own
                      stream has run everything that read the output of call n-1, so once call n's barrier has passed, nobody
                      still reads the buffer that call n+1 overwrites.
    "copy_engine"     the GEMM writes its block into its own [M, N] symmetric buffer and copy engines push the block into
                      every peer's buffer on a second stream (`feather_copy_block`), followed by the cross-rank barrier on
                      that stream.  No SM waits for NVLink, so the transfer overlaps whatever the compute stream runs next:
                      with `defer=True` the call returns at once and the caller orders its reads with `wait_exchange()`
                      (independent linears in a row: the exchange of one runs under the GEMM of the next); without it
                      the compute stream waits for the exchange before it goes on.  From 4 GPUs on, where the exchange of
                      these shapes takes longer than the GEMM, this is the faster form when there is independent work to
                      overlap; the fused form is faster when the next operation needs the output at once.
    "all_gather"      `all_gather_into_tensor` (NCCL) of the [M, N/g] blocks, then a relayout copy to [M, N].  Baseline.
    "none"            no exchange: the call returns the local [M, N/g] block (first half of a tensor-parallel pair).

RowShardedLinear      rank r keeps the k16-planes [r*K/16g, (r+1)*K/16g) (dim 0, a contiguous slice) and multiplies its own
                      K/g activation columns: every rank holds a partial sum of the whole output.  The reduction is a
                      reduce-scatter fused into the GEMM (each finished block, rounded to the output dtype, is TMA-stored to
                      the rank that owns its token rows) followed by one small kernel that adds the g partials of the owned
                      rows in fp32 in rank order, rounds once, adds bias and residual, and writes the rows into every rank's
                      output (plain stores over NVLink: the all-gather).  K is split across ranks, so this is NOT bitwise
                      the single-GPU result: the partials are rounded to 16 bits before they are summed.  It is deterministic
                      (same bits on every rank, every run) and within the GEMM gate of the tests.

ReplicatedLinear      the whole weight on every rank (an e5m2 weight is small against the activations it multiplies); rank r
                      multiplies its own token rows and nothing is exchanged.  The launch takes the tile class of the launch
                      over all tokens, so a row has the same bits on any number of ranks.
RowGather             the all-gather that a token-sharded model needs where an operation reads every token (attention's keys and
                      values): every rank writes its rows into its own [T, C] symmetric buffer, copy engines push them into
                      the peers' buffers on the exchange stream, one cross-rank barrier there; `wait()` orders the reader.

Only stores ever cross NVLink; no load reads peer memory.  With world size 1 there is no exchange and no copy.
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


def shard_k_planes(b_prepacked, rank, world):
    """The k16-planes of `rank`: dim 0 of (K/16, N, 16), a contiguous slice.  K/16 must divide evenly."""
    kb = b_prepacked.shape[0]
    if kb % world != 0:
        raise ValueError(f"K={kb * 16} is not divisible by 16 x the number of ranks {world}")
    per = kb // world
    return b_prepacked[rank * per:(rank + 1) * per].contiguous()


class _SymmetricBuffers:
    """Double-buffered symmetric-memory tensors of one shape: entry p is (own tensor, handle, views of every rank's tensor)."""

    def __init__(self, shape, dtype, device, rank, world, group):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.entries = []
        for _ in range(2):
            buf = symm_mem.empty(shape, dtype=dtype, device=device)
            handle = symm_mem.rendezvous(buf, group.group_name)
            views = [buf if r == rank else handle.get_buffer(r, shape, dtype) for r in range(world)]
            self.entries.append((buf, handle, views))
        self.calls = 0

    def next(self):
        entry = self.entries[self.calls & 1]
        self.calls += 1
        return entry


_exchange_streams = {}


def exchange_stream(device):
    """The second stream of `device` that carries the copy-engine exchanges, one per device so that they run in call order."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    stream = _exchange_streams.get(index)
    if stream is None:
        stream = _exchange_streams[index] = torch.cuda.Stream(device)
    return stream


class ColumnShardedLinear:
    def __init__(self, b_prepacked, scale, bias, rank, world, device, group=None, exchange="all_gather"):
        if exchange not in ("all_gather", "peer_store", "copy_engine", "none"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.rank, self.world, self.group = rank, world, group
        self.exchange = exchange
        self._symm = {}
        self._exchange_done = {}
        self._last_done = None
        self.n_total = b_prepacked.shape[1]
        self.k = b_prepacked.shape[0] * 16
        self.b_local, self.bias_local = shard_columns(b_prepacked.to(device), bias.to(device) if bias is not None else None, rank, world)
        self.n_local = self.b_local.shape[1]
        self.scale = scale.to(device=device, dtype=torch.float32)
        # the heuristic sees the full N so that a shard picks the variant (in particular the K split) of the whole
        self._variant_shape_n = self.n_total
        self.launches_per_call = 1

    def with_exchange(self, exchange):
        """The same weight shard behind another exchange (buffers of its own)."""
        if exchange not in ("all_gather", "peer_store", "copy_engine", "none"):
            raise ValueError(f"unknown exchange {exchange!r}")
        other = object.__new__(ColumnShardedLinear)
        other.__dict__.update(self.__dict__)
        other.exchange, other._symm, other._exchange_done, other._last_done = exchange, {}, {}, None
        return other

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

    def bytes_out_per_call(self, m, itemsize=2):
        """Bytes this rank pushes to its peers per call of the fused exchange (its block, once per peer)."""
        return (self.world - 1) * m * self.n_local * itemsize

    def _peer_store(self, a, out_dtype, variant):
        m = a.shape[0]
        key = (m, out_dtype)
        bufs = self._symm.get(key)
        if bufs is None:
            bufs = self._symm[key] = _SymmetricBuffers((m, self.n_total), out_dtype, a.device, self.rank, self.world, self.group)
        buf, handle, views = bufs.next()
        lo, hi = self.rank * self.n_local, (self.rank + 1) * self.n_local
        # own buffer first, then the peers in a rotated order: at any moment the ranks' stores head for different GPUs
        order = [(self.rank + i) % self.world for i in range(self.world)]
        outputs = [views[r][:, lo:hi] for r in order]
        native.scaled_mm_multi_into(a, self.b_local, self.scale, self.bias_local, outputs, variant=variant)
        handle.barrier()                       # every rank's blocks have landed everywhere
        return buf

    def _copy_engine(self, a, out_dtype, variant, defer):
        m = a.shape[0]
        key = (m, out_dtype)
        bufs = self._symm.get(key)
        if bufs is None:
            bufs = self._symm[key] = _SymmetricBuffers((m, self.n_total), out_dtype, a.device, self.rank, self.world, self.group)
        parity = bufs.calls & 1
        buf, handle, views = bufs.next()
        lo, hi = self.rank * self.n_local, (self.rank + 1) * self.n_local
        compute = torch.cuda.current_stream(a.device)
        side = exchange_stream(a.device)
        # The copies that read this buffer two calls ago must be done before the GEMM overwrites the block.
        previous = self._exchange_done.get((key, parity))
        if previous is not None:
            compute.wait_event(previous)
        block = buf[:, lo:hi]
        native.scaled_mm_into(a, self.b_local, self.scale, self.bias_local, block, variant=self._variant(m, variant))
        ready = torch.cuda.Event()
        ready.record(compute)
        side.wait_event(ready)
        # A peer's buffer of this parity may be overwritten once that peer has run every reader of its previous contents.
        # The readers precede the peer's previous call of this linear on its compute stream; that call's barrier follows
        # its GEMM; and these copies follow this rank's side of that barrier on the exchange stream.
        for i in range(1, self.world):                 # rotated order: at any moment the ranks' copies head for different GPUs
            peer = (self.rank + i) % self.world
            native.copy_block_into(views[peer][:, lo:hi], block, stream=side)
        with torch.cuda.stream(side):
            handle.barrier()                           # every rank's blocks have landed everywhere
        done = torch.cuda.Event()
        done.record(side)
        self._exchange_done[(key, parity)] = done
        self._last_done = done
        if not defer:
            compute.wait_event(done)
        return buf

    def wait_exchange(self, stream=None):
        """Orders `stream` (default: the current one) after the exchange of the last deferred call."""
        if self._last_done is not None:
            (stream if stream is not None else torch.cuda.current_stream()).wait_event(self._last_done)

    def __call__(self, a, out_dtype, variant=None, defer=False):
        if self.exchange == "none":
            return self.gemm_only(a, out_dtype, variant)
        if self.world > 1 and self.exchange == "peer_store":
            return self._peer_store(a, out_dtype, variant)
        if self.world > 1 and self.exchange == "copy_engine":
            return self._copy_engine(a, out_dtype, variant, defer)
        local = self.gemm_only(a, out_dtype, variant)
        if self.world == 1:
            return local
        m = a.shape[0]
        gathered = torch.empty((self.world * m, self.n_local), dtype=out_dtype, device=a.device)    # rank-major concatenation
        dist.all_gather_into_tensor(gathered, local, group=self.group)
        return gathered.view(self.world, m, self.n_local).permute(1, 0, 2).reshape(m, self.n_total)


class RowShardedLinear:
    """y = x @ W (+ bias, + residual) with K sharded over the ranks: `a_local` holds this rank's K/g activation columns."""

    def __init__(self, b_prepacked, scale, bias, rank, world, device, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.n = b_prepacked.shape[1]
        self.k = b_prepacked.shape[0] * 16
        self.b_local = shard_k_planes(b_prepacked.to(device), rank, world)
        self.k_local = self.b_local.shape[0] * 16
        self.scale = scale.to(device=device, dtype=torch.float32)
        self.bias = bias.to(device) if bias is not None else None
        self._symm = {}
        self.launches_per_call = 1 if world == 1 else 2

    def bytes_out_per_call(self, m, itemsize=2):
        """Bytes this rank pushes to its peers per call: its partials of the rows it does not own, then its reduced rows."""
        rows = m // self.world
        return 2 * (self.world - 1) * rows * self.n * itemsize

    def __call__(self, a_local, out_dtype, residual=None, variant=None):
        m = a_local.shape[0]
        if self.world == 1:
            out = torch.empty((m, self.n), dtype=out_dtype, device=a_local.device)
            native.scaled_mm_into(a_local, self.b_local, self.scale, self.bias, out, variant=variant)
            if residual is not None:
                out += residual
            return out
        g = self.world
        if m % (32 * g) != 0:
            raise ValueError(f"the row-parallel linear needs a token count divisible by 32 x the number of ranks ({32 * g}), got {m}")
        rows = m // g
        key = (m, out_dtype)
        entry = self._symm.get(key)
        if entry is None:
            entry = self._symm[key] = (
                _SymmetricBuffers((g, rows, self.n), out_dtype, a_local.device, self.rank, g, self.group),    # partials, one slot per source rank
                _SymmetricBuffers((m, self.n), out_dtype, a_local.device, self.rank, g, self.group),          # reduced output
            )
        part, part_handle, part_views = entry[0].next()
        out, out_handle, out_views = entry[1].next()
        # 1. GEMM over this rank's K slice; each finished block goes to slot `rank` of the rank that owns its token rows
        native.scaled_mm_scatter_into(a_local, self.b_local, self.scale, [part_views[d][self.rank] for d in range(g)], rows, variant=variant)
        part_handle.barrier()                  # all g partials of my rows have landed
        # 2. add the partials of my rows (fp32, rank order), + bias, + residual; write the rows into every rank's output
        lo, hi = self.rank * rows, (self.rank + 1) * rows
        order = [(self.rank + i) % g for i in range(g)]
        native.reduce_partials_into(part, self.bias, residual[lo:hi] if residual is not None else None, [out_views[r][lo:hi] for r in order])
        out_handle.barrier()                   # every rank's rows have landed everywhere
        return out


class ReplicatedLinear:
    """y = x @ W (+ bias, + residual) on this rank's token rows, the whole weight on every rank: no exchange."""

    def __init__(self, b_prepacked, scale, bias, device):
        self.b = b_prepacked.to(device)
        self.n = self.b.shape[1]
        self.k = self.b.shape[0] * 16
        self.scale = scale.to(device=device, dtype=torch.float32)
        self.bias = bias.to(device) if bias is not None else None
        self.launches_per_call = 1

    def __call__(self, a_rows, out_dtype, total_rows=None, residual=None, variant=None, out=None):
        m = a_rows.shape[0]
        if out is None:
            out = torch.empty((m, self.n), dtype=out_dtype, device=a_rows.device)
        if variant is None and total_rows is not None and total_rows != m:
            # the tile class (and K split) of the launch over all tokens: every row then sees the additions of that launch
            variant = native.choose_variant(total_rows, self.n, self.k)
        native.scaled_mm_into(a_rows, self.b, self.scale, self.bias, out, variant=variant)
        if residual is not None:
            out += residual
        return out


class RowGather:
    """All-gather of token rows into a [total_rows, cols] buffer on every rank: `begin()` returns this rank's rows of the next
    buffer for the caller to fill on the compute stream, `push()` sends them to the peers (copy engines, exchange stream,
    then the cross-rank barrier), `wait()` makes the current stream wait and returns the full buffer.  Buffers are
    double-buffered: a rank's readers of buffer p precede its next begin() on the compute stream, that call's push follows
    on the exchange stream, and only after its barrier do the peers' copies of the call after it arrive."""

    def __init__(self, total_rows, cols, dtype, device, rank, world, group=None):
        if total_rows % world != 0:
            raise ValueError(f"{total_rows} token rows do not divide over {world} ranks")
        self.rank, self.world, self.device = rank, world, device
        self.rows = total_rows // world
        self.bufs = _SymmetricBuffers((total_rows, cols), dtype, device, rank, world, group) if world > 1 else None
        self.local = torch.empty((total_rows, cols), dtype=dtype, device=device) if world == 1 else None
        self._done = [None, None]
        self._cur = None

    def begin(self):
        if self.world == 1:
            return self.local
        parity = self.bufs.calls & 1
        if self._done[parity] is not None:         # the copies that read these rows two calls ago are done
            torch.cuda.current_stream(self.device).wait_event(self._done[parity])
        self._cur = (parity,) + self.bufs.next()
        lo = self.rank * self.rows
        return self._cur[1][lo:lo + self.rows]

    def push(self):
        if self.world == 1:
            return
        parity, buf, handle, views = self._cur
        lo = self.rank * self.rows
        compute, side = torch.cuda.current_stream(self.device), exchange_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(compute)
        side.wait_event(ready)
        mine = buf[lo:lo + self.rows]
        for i in range(1, self.world):
            peer = (self.rank + i) % self.world
            native.copy_block_into(views[peer][lo:lo + self.rows], mine, stream=side)
        with torch.cuda.stream(side):
            handle.barrier()
        done = torch.cuda.Event()
        done.record(side)
        self._done[parity] = done

    def wait(self):
        if self.world == 1:
            return self.local
        parity, buf, _, _ = self._cur
        torch.cuda.current_stream(self.device).wait_event(self._done[parity])
        return buf
