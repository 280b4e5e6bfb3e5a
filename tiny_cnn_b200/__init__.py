"""B200 (sm_100a) implementation of tiny-dnn's training hot path.

`tiny_cnn_b200._lib`     ctypes binding of the C ABI (include/tinycnn_b200.h)
`tiny_cnn_b200.ops`      operator-level mirror of the reference's op kernels
`tiny_cnn_b200.network`  mirror of network<sequential> over the device-resident step
`tiny_cnn_b200.build`    nvcc build recipe of csrc/libtinycnn_b200.so

Importing the package does not load the native library; the first call does,
and fails loudly when it is missing (there is no CPU path).
"""
from ._lib import B200Error  # noqa: F401

__version__ = "0.1"
