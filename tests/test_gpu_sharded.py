"""Row-sharded block scaling on several GPUs equals the single-process oracle result bit for bit
(outputs, meta, amax, non-zero count, error sum), for both exchanges (NCCL collectives, peer stores),
plain and pipelined, over several calls with a different tensor in every call.  Needs two CUDA devices
(four for the four-rank cases); skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS, COLS = 2048, 512


def make_input(dtype_name, call):
    g = torch.Generator().manual_seed(11 + call)
    x = torch.randn(ROWS, COLS, generator=g) * (10.0 ** call if call < 3 else 1.0)
    if call == 1:
        x = x * 10.0 ** (torch.rand(ROWS, COLS, generator=g) * 8 - 4)     # wide range: the tensor falls back to BF16
    x[3, 5] = 0.0
    return x.to(getattr(torch, dtype_name))


def as_np(t):
    t = t.cpu()
    return t.view(torch.int16).numpy().view(np.uint16).copy() if t.dtype == torch.bfloat16 else t.numpy().copy()


def _worker(rank, world, port, dtype_name, ss_mode, thr, q, exchange, calls, overlap):
    import torch.distributed as dist
    from mor_b200.sharded import KIND_BLOCK, ShardedScaling, shard_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        dtype = getattr(torch, dtype_name)
        r0, r1 = shard_rows(ROWS, world, rank, 128)
        # odd numbers of calls: the amax kernel exchanges the scalars itself; even: the exchange kernel of its own
        op = ShardedScaling(r1 - r0, COLS, 128, 128, dtype, dev, KIND_BLOCK, exchange=exchange, overlap=overlap,
                            fused_exchange=calls % 2 == 1)
        assert (op.peer is not None) == (exchange == "p2p")
        xs = [make_input(dtype_name, c)[r0:r1].contiguous().to(dev) for c in range(calls)]
        outs = [torch.empty_like(x) for x in xs]
        results = []
        for x, o in zip(xs, outs):     # several calls back to back: epoch flags, buffer copies and scratch sets alternate
            res = op(x, o, ss_mode, thr)
            # the scalar tensors are reused by later calls: copy them on the stream that completes them
            res.wait()
            results.append([t.clone() for t in (res.meta, res.global_amax, res.global_nnz, res.global_error)])
        torch.cuda.synchronize()
        q.put((rank, [(as_np(o), int(r[0].item()), float(r[1].item()), int(r[2].item()), float(r[3].item()))
                      for o, r in zip(outs, results)]))
        op.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dtype_name,ss_mode,thr,exchange,calls,overlap", [
    ("bfloat16", 1, 0.045, "nccl", 1, False), ("float32", 1, 0.045, "nccl", 3, True), ("float32", 4, 1e-6, "nccl", 1, False),
    ("bfloat16", 1, 0.045, "p2p", 5, False), ("float32", 4, 1e-6, "p2p", 2, False),
    ("float32", 1, 0.045, "p2p", 6, True), ("bfloat16", 4, 0.045, "p2p", 5, True)])
def test_ranks_equal_oracle(world, dtype_name, ss_mode, thr, exchange, calls, overlap):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import oracle
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, dtype_name, ss_mode, thr, q, exchange, calls, overlap))
             for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=240) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    metas = set()
    for c in range(calls):
        full = oracle.block_scaling(as_np(make_input(dtype_name, c)), 128, 128, thr, ss_mode)
        out = np.concatenate([g[1][c][0] for g in got], axis=0)
        assert np.array_equal(out.view(np.uint8), np.ascontiguousarray(full[0]).view(np.uint8)), f"call {c}: output"
        for g in got:
            _, meta, amax, nnz, err = g[1][c]
            assert meta == full[1] and np.float32(amax) == full[2] and nnz == full[3], f"call {c} rank {g[0]}"
            assert np.float32(err).view(np.uint32) == np.float32(full[4]).view(np.uint32), f"call {c} rank {g[0]}: error sum"
        metas.add(full[1])
    if calls >= 2 and thr == 0.045:
        assert metas == {1, 3}, "the calls should cover both a kept and a fallen-back tensor"


def test_second_device_in_the_same_process():
    """kernels that opt in to more than 48 KiB of shared memory do so once per device: the float32 tile kernel
    (64 KiB), the single-launch kernel and the streaming kernels must also launch on a second GPU of the process"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mor
    import oracle
    from mor_b200 import cabi
    g = torch.Generator().manual_seed(5)
    x = torch.randn(512, 768, generator=g)
    xb = x.to(torch.bfloat16)
    exp32 = oracle.block_scaling(x.numpy(), 128, 128, 0.045, 1)
    exp16 = oracle.channel_scaling(oracle.bf16_bits(xb), 1, 32, 0.045, 2)
    for mask in (0, 2):      # the single-launch kernel, then the launch sequence with the TMA-staged tile kernel
        cabi.lib().mor_b200_debug_kernel_selection(mask)
        try:
            for d in (0, 1, 0):
                dev = torch.device("cuda", d)
                out = mor.ops.fake_quantize_block_scaling(x.to(dev), 512, 768, 128, 128, 0.045, 1)
                assert np.array_equal(out[0].cpu().numpy().view(np.uint32), exp32[0].view(np.uint32)), (mask, d)
                assert out[1].item() == exp32[1] and out[3].item() == exp32[3]
                o16 = mor.ops.fake_quantize_channel_scaling(xb.to(dev), 512, 768, 1, 32, 0.045, 2)
                assert np.array_equal(oracle.bf16_bits(o16[0].cpu()), exp16[0]), (mask, d)
        finally:
            cabi.lib().mor_b200_debug_kernel_selection(0)
