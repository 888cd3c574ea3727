"""mor_b200 -- B200 (sm_100a) implementation of the MoR fake-quantization operators.

``import mor_b200`` loads ``libmor_b200.so`` (CUDA kernels behind a C ABI) and the
``_C`` PyTorch shim, which registers ``torch.ops.mor.*`` with the operator schemas of
boryiings/mor, and exposes ``mor_b200.ops`` with the signatures of ``mor/ops.py``.
Both native artefacts must have been built (``python mor_b200/build.py``); importing
fails loudly otherwise, and the operators exist for CUDA tensors only.
"""
import torch  # noqa: F401  (the shim links against libtorch)

from . import cabi

cabi.lib()  # fail here, not at first use, if the kernels are not built

try:
    from . import _C  # noqa: F401  registers torch.ops.mor.*
except ImportError as e:  # pragma: no cover
    raise ImportError(
        "mor_b200._C (the PyTorch shim) is not built: run `python mor_b200/build.py`. "
        "There is no pure-Python or CPU fallback for torch.ops.mor.*") from e

from . import ops  # noqa: E402

__all__ = ["ops", "cabi"]
