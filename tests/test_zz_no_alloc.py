"""mor_b200_block_scaling_static: the block-scaling pipeline for callers that cannot hand
over (or allocate) a workspace -- its scratch is an array built into the library.

Checked against the workspace form of the same operator, bit for bit (outputs, meta, amax,
non-zero count and error sum: the tolerance of the other GPU tests, i.e. none), on two calls
in a row with different inputs, because the built-in scratch keeps the previous call's
contents and the second call must not see them.  The file sorts last on purpose: a run
that stops at the first failure has by then run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(x, bx, by, thr, ss):
    import gpu_harness as H
    from mor_b200 import cabi
    rows, cols = x.shape
    d = H.to_dev(x)
    out = torch.empty_like(d)
    f32 = x.dtype == np.float32
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    gamax = torch.zeros(1, dtype=torch.float32, device="cuda")
    gnnz = torch.zeros(1, dtype=torch.int64 if f32 else torch.int32, device="cuda")
    gerr = torch.zeros(1, dtype=torch.float32, device="cuda")
    cabi.call("mor_b200_block_scaling_static", d.data_ptr(), out.data_ptr(), H.dtype_of(x), rows, cols, bx, by,
              float(thr), ss, meta.data_ptr(), gamax.data_ptr(), gnnz.data_ptr(), 1 if f32 else 0, gerr.data_ptr(),
              H.stream())
    torch.cuda.synchronize()
    return {"out": H.to_np(out), "meta": H.to_np(meta), "gamax": gamax.item(), "gnnz": int(gnnz.item()),
            "gerr": gerr.item()}


def _same(a, b):
    assert np.array_equal(a["out"].view(np.uint8), b["out"].view(np.uint8))
    assert np.array_equal(a["meta"], b["meta"]) and a["gnnz"] == b["gnnz"]
    for k in ("gamax", "gerr"):
        assert np.float32(a[k]).view(np.uint32) == np.float32(b[k]).view(np.uint32), k


def test_static_scratch_matches_workspace_form_twice_in_a_row():
    import gpu_harness as H
    g = torch.Generator().manual_seed(2024)
    first = (torch.randn(512, 768, generator=g)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    # second call: other shape, wide range (tensor falls back to BF16), fewer blocks than the first
    wide = 10.0 ** (torch.rand(256, 256, generator=g) * 8 - 4)
    second = wide.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    third = torch.randn(384, 512, generator=g).numpy()  # float32, int64 non-zero count
    for x, bx, by, thr, ss in ((first, 128, 128, 0.045, 1), (second, 128, 128, 0.045, 1), (third, 64, 128, 3e38, 3)):
        _same(_call_static(x, bx, by, thr, ss), H.block_scaling(x, bx, by, thr, ss))


def test_static_scratch_rejects_what_does_not_fit():
    from mor_b200 import cabi
    d = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    # 65537 blocks of 32 x 64: one more than the built-in scratch holds; refused before any launch
    rc = cabi.lib().mor_b200_block_scaling_static(d.data_ptr(), d.data_ptr(), cabi.BF16, 32 * 65537, 64, 32, 64, 0.045,
                                                  1, d.data_ptr(), d.data_ptr(), d.data_ptr(), 0, d.data_ptr(), None)
    assert rc == -6 and b"65536" in cabi.lib().mor_b200_status_string(rc)
