"""strixite_b200: the quantized mixture-of-experts FFN path of strixite, written for NVIDIA B200 (sm_100a).

The product is libstrix_b200.so (CUDA kernels behind the C ABI of include/strix_b200.h).  This package binds it:
`kernels` mirrors the reference's strix::kernels launchers, `layer` composes them into the MoE sublayer as the
reference's forward does, `ep` runs that sublayer expert-parallel over torch.distributed.
"""
from . import _lib  # noqa: F401
from .kernels import Act, Error, GpuFatalError, MoeMath, QDeviceView  # noqa: F401

__version__ = "0.1"
