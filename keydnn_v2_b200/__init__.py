"""B200 (sm_100a) operator library for KeyDNN's pool / reduce / elementwise / optimizer path.

``libkeydnn_b200.so`` (sources in ``csrc/``) exports the reference DLL's C ABI for that path;
this package is the host-side mirror of the reference's ops / Tensor layers that drives it.
There is no CPU fallback: importing is cheap, the first device call needs the built library.
"""
from ._native import NativeLibraryError, load  # noqa: F401
from .tensor import Context, Device, Parameter, Tensor, no_grad  # noqa: F401

__all__ = ["load", "NativeLibraryError", "Tensor", "Parameter", "Context", "Device", "no_grad"]
