"""Drop-in alias: ``import mor`` / ``mor.ops.fake_quantize(...)`` as with boryiings/mor
(mor/__init__.py:1-2 there), served by the mor_b200 kernels."""
import torch  # noqa: F401
from mor_b200 import _C, ops  # noqa: F401
