"""Host logic of the row-sharded pipeline on two CPU ranks over gloo: the partition,
the order and kind of the collectives, and that the sharded result equals the
single-process result bit for bit.  The kernels are replaced by the CPU oracle here
(a test stand-in handed in explicitly; the product has no such path)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mor_b200.sharded import KIND_BLOCK, ShardedScaling, shard_rows

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """CPU stand-in for CudaBackend with the same four phases."""

    def __init__(self, rows, cols, brows, bcols):
        self.rows, self.cols, self.brows, self.bcols = rows, cols, brows, bcols
        self.n_err = (rows // brows) * (cols // bcols)
        self.stride = 1
        self.launches = 0

    @staticmethod
    def _np(t):
        return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()

    def amax_nnz(self, x, amax_out, nnz_out):
        a, n = oracle.amax_nnz(self._np(x))
        amax_out[0], nnz_out[0] = float(a), n

    def cast(self, x, out, ss_mode, global_amax, block_err):
        res = oracle.block_scaling(self._np(x), self.brows, self.bcols, 3e38, ss_mode,
                                   global_amax=float(global_amax[0]), want_blocks=True)
        self._np(out)[...] = res[0]
        block_err.copy_(torch.from_numpy(res[6]))

    def finalize(self, all_err, global_nnz, threshold, meta, global_error):
        m, e = oracle.finalize(all_err.numpy(), self.stride, int(global_nnz[0]), threshold)
        meta[0], global_error[0] = m, float(e)

    def fallback(self, x, out, meta):
        if int(meta[0]) == 3:
            out.copy_(x)


def make_input(dtype, rows=512, cols=256, wide=False):
    g = torch.Generator().manual_seed(11)
    t = torch.randn(rows, cols, generator=g)
    if wide:
        t = t * 10.0 ** (torch.rand(rows, cols, generator=g) * 8 - 4)
    t[3, 5] = 0.0
    return t.to(dtype)


def worker(rank, world, port, dtype_name, ss_mode, thr, wide, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dtype = getattr(torch, dtype_name)
        x = make_input(dtype, wide=wide)
        r0, r1 = shard_rows(x.shape[0], world, rank, 128)
        xs = x[r0:r1].contiguous()
        out = torch.empty_like(xs)
        op = ShardedScaling(r1 - r0, x.shape[1], 128, 128, dtype, torch.device("cpu"), KIND_BLOCK,
                            backend=OracleBackend(r1 - r0, x.shape[1], 128, 128))
        res = op(xs, out, ss_mode, thr)
        q.put((rank, r0, r1, OracleBackend._np(out).copy(), int(res.meta[0]), float(res.global_amax[0]),
               int(res.global_nnz[0]), float(res.global_error[0]), op.collectives))
    finally:
        dist.destroy_process_group()


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
@pytest.mark.parametrize("ss_mode,thr,wide", [(1, 0.045, False), (4, 0.045, False), (1, 0.045, True), (3, 3e38, True)])
def test_two_ranks_equal_one_process(dtype_name, ss_mode, thr, wide):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, dtype_name, ss_mode, thr, wide, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = make_input(getattr(torch, dtype_name), wide=wide)
    full = oracle.block_scaling(OracleBackend._np(x), 128, 128, thr, ss_mode)
    out = np.concatenate([g[3] for g in got], axis=0)
    assert np.array_equal(out.view(np.uint8), np.ascontiguousarray(full[0]).view(np.uint8))
    for g in got:
        assert g[4] == full[1]                                # meta identical on every rank
        assert np.float32(g[5]) == full[2] and g[6] == full[3]
        assert np.float32(g[7]).view(np.uint32) == np.float32(full[4]).view(np.uint32)
        assert g[8] == 3                                      # amax MAX, nnz SUM, error all-gather
    assert (full[1] == 3) == wide or thr > 1.0


def uneven_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        r0, r1 = shard_rows(384, world, rank, 128)            # three block rows on two ranks: 256 and 128 rows
        try:
            ShardedScaling(r1 - r0, 256, 128, 128, torch.float32, torch.device("cpu"), KIND_BLOCK,
                           backend=OracleBackend(r1 - r0, 256, 128, 128))
            q.put((rank, "accepted"))
        except ValueError as e:
            q.put((rank, "refused: " + str(e)))
    finally:
        dist.destroy_process_group()


def test_uneven_slabs_are_refused_on_every_rank():
    """The gathered error arrays are fixed-size and every rank computes its offsets from its own slab: slabs of
    different heights must be refused before anything is exchanged, and by all ranks alike."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=uneven_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(g[1].startswith("refused") and "slab shape" in g[1] for g in got), got


def test_shard_rows_partition():
    for rows, world, mult in ((131072, 8, 128), (1024, 3, 128), (256, 4, 128), (4096, 5, 32)):
        spans = [shard_rows(rows, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == rows
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0
        assert all((b - a) % mult == 0 for a, b in spans)
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard_rows(1000, 2, 0, 128)


def test_product_backend_refuses_cpu():
    """Without a CUDA device the product backend cannot be built: no silent CPU path."""
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    from mor_b200.sharded import CudaBackend
    b = CudaBackend(KIND_BLOCK, 256, 256, 128, 128, torch.bfloat16, torch.device("cpu"))
    x = torch.zeros(256, 256, dtype=torch.bfloat16)
    with pytest.raises(Exception):
        b.amax_nnz(x, torch.zeros(1), torch.zeros(1, dtype=torch.int64))
