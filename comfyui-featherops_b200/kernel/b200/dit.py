"""A random-init Wan-like diffusion-transformer forward whose every linear is the Feather mixed-precision linear
(fp16 activations @ prepacked fp8e5m2 weights, bf16 out), on 1, 2, 4 or 8 GPUs of one box.

This is the benchmark/test harness for the "4-block DiT forward" configuration: hidden 5120, 40 heads x 128, FFN 13824 with
tanh-GELU, RMSNorm, attention through torch's scaled_dot_product_attention, bf16 compute.  It is not a model of the reference
(which ships none); the linears do what the reference's `FeatherOps.Linear.forward` does for a bf16 input
(comfy_feather/ops.py:84-104: cast the activations to fp16, `scaled_mm_hip(x, qdata, scale, bias, out_dtype)`), with the
weights quantised through its loader path (comfy_feather/quant.py:116-136: fp32 weight -> per-tensor scale amax/57344 ->
e5m2 -> (K/16, N, 16)).

Block (pre-norm, residual):
    h = rmsnorm(x);  q, k, v = Wq h, Wk h, Wv h;  q, k = rmsnorm_per_head(q), rmsnorm_per_head(k)
    x = x + Wo sdpa(q, k, v)
    h = rmsnorm(x);  x = x + Wdown gelu(Wup h)

Multi-GPU modes (one process per GPU, the same seeded weights generated on every rank, then sharded):
    "all_gather"   every linear is column-sharded (N) and its output all-gathered, so every rank holds every activation in
                   full and attention runs replicated.  Bitwise the 1-GPU forward.
    "pairs"        tensor-parallel pairs: Wq/Wk/Wv and Wup column-sharded with NO exchange (a rank's columns are its heads /
                   its slice of the FFN), attention on the rank's own heads, Wo and Wdown row-sharded (K) with the
                   reduce-scatter fused into the GEMM and one reduce + all-gather kernel.  Two exchanges per block instead
                   of six, attention divided by the number of ranks.  Not bitwise (K is split across ranks): within the
                   GEMM gate per linear, tolerance end to end.

    "tokens"       token rows sharded, weights replicated (an e5m2 weight is small against the activations): every linear is
                   a local GEMM over the rank's T/g rows with no exchange at all; the one thing that needs every token,
                   attention's keys and values, is all-gathered per block by copy engines while the value and query
                   projections run.  Half the bytes of "pairs", none of them on the critical path of a linear.  Every linear
                   is bitwise the 1-GPU linear on the same input; attention runs on another query partition, so the forward
                   is compared within tolerance.

`linear_factory` exists so tests can run the same forward on CPU ranks with the CPU oracle standing in for the CUDA GEMM;
the default factory is the CUDA path and raises without a GPU.
"""

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import native
from .sharded import ColumnShardedLinear, ReplicatedLinear, RowGather, RowShardedLinear


@dataclass
class DitConfig:
    hidden: int = 5120
    heads: int = 40
    head_dim: int = 128
    ffn: int = 13824
    blocks: int = 4
    eps: float = 1e-6

    def linear_flops(self, tokens):
        return 2.0 * tokens * (4 * self.hidden * self.hidden + 2 * self.hidden * self.ffn) * self.blocks

    def attention_flops(self, tokens):
        return 4.0 * tokens * tokens * self.heads * self.head_dim * self.blocks


class CudaLinearFactory:
    """Builds the sharded CUDA linears from an fp32 weight: quantise + prepack on the GPU (loader path), then shard."""

    def __init__(self, rank, world, device, exchange="peer_store", group=None):
        self.rank, self.world, self.device, self.exchange, self.group = rank, world, device, exchange, group

    def to_fp16(self, x):
        """bf16 -> fp16 with the library's cast kernel (same bits as `x.to(torch.float16)`)."""
        return native.bf16_to_fp16(x.contiguous())

    def _quantised(self, w):
        qdata, scale = native.quantize_prepack(w.to(self.device, torch.float32).contiguous())
        return qdata, scale.reshape(1)

    def column(self, w, bias, gather=True):
        q, s = self._quantised(w)
        exchange = self.exchange if gather else "none"
        return ColumnShardedLinear(q, s, bias.to(torch.bfloat16), self.rank, self.world, self.device, group=self.group, exchange=exchange)

    def row(self, w, bias):
        q, s = self._quantised(w)
        return RowShardedLinear(q, s, bias.to(torch.bfloat16), self.rank, self.world, self.device, group=self.group)

    def full(self, w, bias):
        q, s = self._quantised(w)
        return ReplicatedLinear(q, s, bias.to(torch.bfloat16), self.device)

    def row_gather(self, total_rows, cols, dtype):
        return RowGather(total_rows, cols, dtype, self.device, self.rank, self.world, self.group)

    def gather_rows(self, local_rows):
        """[T/g, C] on every rank -> [T, C] on every rank (the forward's result)."""
        if self.world == 1:
            return local_rows
        import torch.distributed as dist
        out = torch.empty((self.world * local_rows.shape[0], local_rows.shape[1]), dtype=local_rows.dtype, device=local_rows.device)
        dist.all_gather_into_tensor(out, local_rows.contiguous(), group=self.group)
        return out


def rmsnorm(x, gain, eps):
    return F.rms_norm(x, (x.shape[-1],), gain, eps)


class FeatherDiT:
    def __init__(self, cfg, rank=0, world=1, device=None, mode="all_gather", exchange="peer_store", seed=0, linear_factory=None,
                 init_device=None, group=None):
        if mode not in ("all_gather", "pairs", "tokens"):
            raise ValueError(f"unknown mode {mode!r}")
        if cfg.hidden != cfg.heads * cfg.head_dim:
            raise ValueError("hidden must equal heads x head_dim")
        if mode == "pairs" and (cfg.heads % world or cfg.ffn % (16 * world) or cfg.hidden % (16 * world)):
            raise ValueError("pairs mode needs heads, ffn/16 and hidden/16 divisible by the number of ranks")
        self.cfg, self.rank, self.world, self.mode = cfg, rank, world, mode
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.factory = linear_factory if linear_factory is not None else CudaLinearFactory(rank, world, self.device, exchange, group)
        # the random stream lives on `init_device`: the CPU for tests that compare a CUDA and a CPU model, the GPU for the benchmark
        init_device = init_device if init_device is not None else self.device
        gen = torch.Generator(device=init_device).manual_seed(seed)
        h, f = cfg.hidden, cfg.ffn
        pairs = mode == "pairs"
        self._gathers = {}

        def weight(n, k):
            return torch.randn((n, k), generator=gen, device=init_device, dtype=torch.float32) / k ** 0.5

        def vector(n, spread):
            return (torch.randn((n,), generator=gen, device=init_device, dtype=torch.float32) * spread)

        self.blocks = []
        for _ in range(cfg.blocks):
            b = {}
            b["norm1"] = (1.0 + vector(h, 0.1)).to(self.device, torch.bfloat16)
            b["norm2"] = (1.0 + vector(h, 0.1)).to(self.device, torch.bfloat16)
            q_gain, k_gain = (1.0 + vector(h, 0.1)), (1.0 + vector(h, 0.1))
            if mode == "tokens":
                # the same draws in the same order as the other modes, every weight whole
                for name, n, k in (("q", h, h), ("k", h, h), ("v", h, h), ("o", h, h), ("up", f, h), ("down", h, f)):
                    b[name] = self.factory.full(weight(n, k), vector(n, 0.1))
            else:
                for name, n, k in (("q", h, h), ("k", h, h), ("v", h, h)):
                    b[name] = self.factory.column(weight(n, k), vector(n, 0.1), gather=not pairs)
                b["o"] = self.factory.row(weight(h, h), vector(h, 0.1)) if pairs else self.factory.column(weight(h, h), vector(h, 0.1))
                b["up"] = self.factory.column(weight(f, h), vector(f, 0.1), gather=not pairs)
                b["down"] = self.factory.row(weight(h, f), vector(h, 0.1)) if pairs else self.factory.column(weight(h, f), vector(h, 0.1))
            # per-head gains of the q/k norm, [heads, head_dim]; a rank in pairs mode keeps the gains of its own heads
            heads = slice(rank * cfg.heads // world, (rank + 1) * cfg.heads // world) if pairs else slice(None)
            b["q_gain"] = q_gain.view(cfg.heads, cfg.head_dim)[heads].to(self.device, torch.bfloat16)
            b["k_gain"] = k_gain.view(cfg.heads, cfg.head_dim)[heads].to(self.device, torch.bfloat16)
            self.blocks.append(b)

    # ------------------------------------------------------------------------------------------
    def _attention(self, q, k, v, blk):
        """q, k, v [T, heads_here * head_dim] bf16 -> [T, heads_here * head_dim]; per-head RMSNorm on q and k first."""
        t = q.shape[0]
        d = self.cfg.head_dim
        q = q.view(t, -1, d)
        k = k.view(t, -1, d)
        v = v.view(t, -1, d)
        q = F.rms_norm(q, (d,), None, self.cfg.eps) * blk["q_gain"]
        k = F.rms_norm(k, (d,), None, self.cfg.eps) * blk["k_gain"]
        out = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0))
        return out.squeeze(0).transpose(0, 1).reshape(t, -1)

    def _forward_tokens(self, x, hook):
        """Token rows sharded, weights replicated: x [T, hidden] (the same on every rank) -> [T, hidden] on every rank."""
        cfg, bf16 = self.cfg, torch.bfloat16
        cast = self.factory.to_fp16
        t, d = x.shape[0], cfg.head_dim
        if t % self.world:
            raise ValueError(f"{t} tokens do not divide over {self.world} ranks")
        rows = t // self.world
        xl = x[self.rank * rows:(self.rank + 1) * rows]
        gathers = self._gathers.get(t)
        if gathers is None:
            gathers = self._gathers[t] = (self.factory.row_gather(t, cfg.hidden, bf16), self.factory.row_gather(t, cfg.hidden, bf16))
        k_all, v_all = gathers

        def call(lin, name, i, a16, **kw):
            y = lin(a16, bf16, total_rows=t, **kw)
            if hook is not None:
                hook(name, i, a16, y)
            return y

        for i, blk in enumerate(self.blocks):
            h16 = cast(rmsnorm(xl, blk["norm1"], cfg.eps))
            # keys first (normalised per head before they travel), then values, each on its way while the next projection runs
            k = call(blk["k"], "k", i, h16)
            k_rows = k_all.begin()
            torch.mul(F.rms_norm(k.view(rows, -1, d), (d,), None, cfg.eps), blk["k_gain"], out=k_rows.view(rows, -1, d))
            k_all.push()
            v_rows = v_all.begin()
            call(blk["v"], "v", i, h16, out=v_rows)
            v_all.push()
            q = call(blk["q"], "q", i, h16)
            q = F.rms_norm(q.view(rows, -1, d), (d,), None, cfg.eps) * blk["q_gain"]
            kf = k_all.wait().view(t, -1, d)
            vf = v_all.wait().view(t, -1, d)
            attn = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), kf.transpose(0, 1).unsqueeze(0), vf.transpose(0, 1).unsqueeze(0))
            attn16 = cast(attn.squeeze(0).transpose(0, 1).reshape(rows, -1))
            xl = call(blk["o"], "o", i, attn16, residual=xl)
            h16 = cast(rmsnorm(xl, blk["norm2"], cfg.eps))
            u16 = cast(F.gelu(call(blk["up"], "up", i, h16), approximate="tanh"))
            xl = call(blk["down"], "down", i, u16, residual=xl)
        return self.factory.gather_rows(xl)

    def forward(self, x, hook=None):
        """x [T, hidden] bf16 (the same on every rank) -> [T, hidden] bf16 (the same on every rank).
        `hook(name, block, input_fp16, output)` sees every linear's input and output (tests use it)."""
        if self.mode == "tokens":
            return self._forward_tokens(x, hook)
        cfg, bf16 = self.cfg, torch.bfloat16
        pairs = self.mode == "pairs"
        cast = self.factory.to_fp16

        def call(lin, name, i, a16, **kw):
            y = lin(a16, bf16, **kw)
            if hook is not None:
                hook(name, i, a16, y)
            return y

        for i, blk in enumerate(self.blocks):
            h16 = cast(rmsnorm(x, blk["norm1"], cfg.eps))
            q = call(blk["q"], "q", i, h16)
            k = call(blk["k"], "k", i, h16)
            v = call(blk["v"], "v", i, h16)
            attn16 = cast(self._attention(q, k, v, blk))
            if pairs:
                x = call(blk["o"], "o", i, attn16, residual=x)
            else:
                x = x + call(blk["o"], "o", i, attn16)
            h16 = cast(rmsnorm(x, blk["norm2"], cfg.eps))
            u16 = cast(F.gelu(call(blk["up"], "up", i, h16), approximate="tanh"))
            if pairs:
                x = call(blk["down"], "down", i, u16, residual=x)
            else:
                x = x + call(blk["down"], "down", i, u16)
        return x

    __call__ = forward

    def linears(self):
        for i, blk in enumerate(self.blocks):
            for name in ("q", "k", "v", "o", "up", "down"):
                yield i, name, blk[name]
