"""CPU stand-ins for the DiT harness's linears.  TEST INFRASTRUCTURE ONLY: the CUDA GEMM is replaced by the torch-CPU
restatement of the reference's kernel/naive.py (oracle/naive_torch.py), so the same forward code can run on CPU as the
checker of the CUDA forward and as gloo ranks that exercise the multi-rank control path."""

import torch

from oracle import naive_torch


class CpuOracleFactory:
    """Same interface as feather_b200.kernel.b200.dit.CudaLinearFactory, world size 1, every linear through the oracle."""

    def to_fp16(self, x):
        return x.to(torch.float16)

    @staticmethod
    def _linear(w, bias):
        q, s = naive_torch.quantize_prepack_cpu(w.to("cpu", torch.float32))
        b = bias.to("cpu", torch.bfloat16)

        def lin(a16, out_dtype, residual=None, variant=None, total_rows=None, out=None):
            y = naive_torch.scaled_mm_cpu(a16, q, s, b, out_dtype)
            y = y + residual if residual is not None else y
            if out is not None:
                out.copy_(y)
                return out
            return y

        lin.q, lin.s, lin.b = q, s, b
        return lin

    def column(self, w, bias, gather=True):
        return self._linear(w, bias)

    def row(self, w, bias):
        return self._linear(w, bias)

    def full(self, w, bias):
        return self._linear(w, bias)

    def row_gather(self, total_rows, cols, dtype):
        return CpuRowGather(total_rows, cols, dtype, 0, 1)

    def gather_rows(self, local_rows):
        return local_rows


class CpuRowGather:
    """Same interface as kernel.b200.sharded.RowGather; the exchange is a gloo all-gather at wait()."""

    def __init__(self, total_rows, cols, dtype, rank, world):
        self.rank, self.world, self.rows = rank, world, total_rows // world
        self.full = torch.empty((total_rows, cols), dtype=dtype)

    def begin(self):
        return self.full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def push(self):
        pass

    def wait(self):
        if self.world > 1:
            import torch.distributed as dist
            mine = self.full[self.rank * self.rows:(self.rank + 1) * self.rows].clone()
            dist.all_gather_into_tensor(self.full, mine)
        return self.full


class GlooShardedFactory:
    """CPU ranks over gloo: the real ColumnShardedLinear (NCCL-style all-gather exchange) with its local GEMM replaced by
    the oracle port, so the sharding and exchange logic of the harness runs without a GPU."""

    def __init__(self, rank, world, sharded_module):
        self.rank, self.world, self.sharded = rank, world, sharded_module

    def to_fp16(self, x):
        return x.to(torch.float16)

    def column(self, w, bias, gather=True):
        q, s = naive_torch.quantize_prepack_cpu(w.to(torch.float32))
        lin = self.sharded.ColumnShardedLinear(q, s.reshape(1), bias.to(torch.bfloat16), self.rank, self.world, torch.device("cpu"),
                                               exchange="all_gather" if gather else "none")
        lin.gemm_only = lambda x, dt, variant=None, out=None: naive_torch.scaled_mm_cpu(x, lin.b_local, lin.scale, lin.bias_local, dt)
        return lin

    def row(self, w, bias):
        raise NotImplementedError("the row-parallel linear exchanges through CUDA symmetric memory; it has no CPU stand-in")

    def full(self, w, bias):
        return CpuOracleFactory._linear(w, bias)

    def row_gather(self, total_rows, cols, dtype):
        return CpuRowGather(total_rows, cols, dtype, self.rank, self.world)

    def gather_rows(self, local_rows):
        import torch.distributed as dist
        out = torch.empty((self.world * local_rows.shape[0], local_rows.shape[1]), dtype=local_rows.dtype)
        dist.all_gather_into_tensor(out, local_rows.contiguous())
        return out
