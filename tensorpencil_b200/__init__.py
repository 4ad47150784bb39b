"""tensorpencil_b200 -- B200-native (sm_100a) quantized-linear path for TensorPencil.

The product is the C-ABI shared library ``libtpb200.so`` (declared in
``include/tpb200.h``, sources under ``csrc/``).  The Python modules here are the
host-side mirror of the reference's ``cuda.Backend`` op surface for this path
(``backend.Backend``), built on that library through ``ctypes``; PyTorch only
provides device memory, streams and ``torch.distributed``.

There is no CPU fallback: every op raises if the library is missing or if no
CUDA device is present.
"""
__version__ = "0.1.0"
