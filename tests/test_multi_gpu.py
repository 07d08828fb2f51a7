"""GPU (2 or more devices): the column-sharded linear, one process per GPU over NCCL / NVLink.  Both exchanges - the fused
peer-store epilogue over symmetric memory and the NCCL all-gather baseline - must reproduce the single-GPU output bit for
bit (K is never split across ranks).  Skipped on a single-GPU box."""

import importlib
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    import __graft_entry__

    __graft_entry__.load_package()
    native = importlib.import_module("feather_b200.kernel.b200.native")
    sharded = importlib.import_module("feather_b200.kernel.b200.sharded")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    g = torch.Generator(device=dev).manual_seed(0)            # same seed on every rank: replicated activations and weights
    M, K, N = 1000, 1024, 1536
    a = torch.randn((M, K), generator=g, device=dev).to(torch.float16)
    w = torch.randn((N, K), generator=g, device=dev) / K ** 0.5
    bias = torch.randn((N,), generator=g, device=dev).to(torch.bfloat16)
    bq, s = native.quantize_prepack(w)
    s = s.reshape(1)
    full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    native.scaled_mm_into(a, bq, s, bias, full)
    ok = True
    for exchange in ("peer_store", "all_gather"):
        lin = sharded.ColumnShardedLinear(bq, s, bias, rank, world, dev, exchange=exchange)
        for _ in range(2):                                    # twice: the symmetric buffer is reused
            out = lin(a, torch.bfloat16)
            torch.cuda.synchronize()
            ok = ok and out.shape == (M, N) and torch.equal(out.view(torch.int16), full.view(torch.int16))
    native.check_device_status(dev)
    with open(os.path.join(tmpdir, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_column_sharded_linear_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / f"ok{r}").read() for r in range(2)] == ["1", "1"]
