"""B200 (sm_100a) implementation of apache/singa's training backward path:
the gradient kernels behind ``singa::Tensor`` math and the BN / pooling /
softmax-cross-entropy operation handles, the SGD-momentum update, and the
data-parallel gradient synchronisation of ``io::Communicator``.

``singa_b200.singa_wrap``  the reference's SWIG-level names over the C ABI
``singa_b200.opt``         SGD / DistOpt drivers (python in the reference too)
``singa_b200._lib``        ctypes binding of ``libsgb.so`` (``include/sgb.h``)
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
