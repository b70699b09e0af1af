"""berth_b200: the EXL3 trellis-linear / A3B-MoE hot path of berth for NVIDIA B200.

The product is ``libberth_b200.so`` (hand-written sm_100a CUDA behind the C ABI declared in
``include/berth_b200.h``).  This package is the host-side mirror of the interface berth's Rust
crates put on top of that ABI (``berth-kernels`` wrappers, ``berth-engine``'s ``Exl3Linear`` and
``MlpLayer``); it holds no arithmetic of its own and fails loudly when the CUDA library is
missing -- there is no CPU path.
"""
from . import kernels  # noqa: F401
from .kernels import Codebook, Error, OutDtype  # noqa: F401
