"""B200 (sm_100a) backend for Lattice's Q4 weight-only linear layer (+LoRA, +QuaRot rotation).

The compute lives in ``liblattice_q4.so`` (hand-written CUDA behind the C ABI of
``include/lattice_q4.h``); this package is the thin host-side mirror of the reference's
call sites.  PyTorch is used for device memory and streams only.
"""
from . import _lib
from ._lib import Lq4Error
from .backend import CudaQ4Backend, LoraLayerData, Q4WeightBuf

__all__ = ["CudaQ4Backend", "LoraLayerData", "Q4WeightBuf", "Lq4Error", "_lib"]
