"""Row-sharded block scaling on two GPUs over NCCL equals the single-process oracle result
bit for bit (outputs, meta, amax, non-zero count, error sum).  Needs two CUDA devices."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, dtype_name, ss_mode, thr, q, exchange="nccl", calls=1):
    import torch.distributed as dist
    from mor_b200.sharded import KIND_BLOCK, ShardedScaling, shard_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        dtype = getattr(torch, dtype_name)
        g = torch.Generator().manual_seed(11)
        x = torch.randn(1024, 512, generator=g)
        x[3, 5] = 0.0
        x = x.to(dtype)
        r0, r1 = shard_rows(x.shape[0], world, rank, 128)
        xs = x[r0:r1].contiguous().to(dev)
        out = torch.empty_like(xs)
        op = ShardedScaling(r1 - r0, x.shape[1], 128, 128, dtype, dev, KIND_BLOCK, exchange=exchange)
        assert (op.peer is not None) == (exchange == "p2p")
        for _ in range(calls):     # several calls: the epoch flags and the two buffer copies alternate
            res = op(xs, out, ss_mode, thr)
        torch.cuda.synchronize()
        o = out.cpu()
        o = o.view(torch.int16).numpy().view(np.uint16) if dtype == torch.bfloat16 else o.numpy()
        q.put((rank, o.copy(), int(res.meta.item()), float(res.global_amax.item()), int(res.global_nnz.item()),
               float(res.global_error.item())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype_name,ss_mode,thr,exchange,calls", [
    ("bfloat16", 1, 0.045, "nccl", 1), ("float32", 1, 0.045, "nccl", 1), ("float32", 4, 1e-6, "nccl", 1),
    ("bfloat16", 1, 0.045, "p2p", 5), ("float32", 4, 1e-6, "p2p", 2)])
def test_two_gpus_equal_oracle(dtype_name, ss_mode, thr, exchange, calls):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import oracle
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, dtype_name, ss_mode, thr, q, exchange, calls)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=180) for _ in range(2)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g = torch.Generator().manual_seed(11)
    x = torch.randn(1024, 512, generator=g)
    x[3, 5] = 0.0
    x = x.to(getattr(torch, dtype_name))
    xn = x.view(torch.int16).numpy().view(np.uint16) if dtype_name == "bfloat16" else x.numpy()
    full = oracle.block_scaling(xn, 128, 128, thr, ss_mode)
    out = np.concatenate([t[1] for t in got], axis=0)
    assert np.array_equal(out.view(np.uint8), np.ascontiguousarray(full[0]).view(np.uint8))
    for t in got:
        assert t[2] == full[1] and np.float32(t[3]) == full[2] and t[4] == full[3]
        assert np.float32(t[5]).view(np.uint32) == np.float32(full[4]).view(np.uint32)
