"""opennn_b200: B200 (sm_100a) kernels for OpenNN's transformer training path.

The product is the C ABI in include/onn_b200.h (libonn_b200.so) and the C++ host mirror of
the OpenNN interfaces above it (libonn_b200_host.so).  This Python package only builds,
loads and drives them; it holds no compute of its own and no fallback path.
"""

from ._build import build  # noqa: F401

__all__ = ["build"]
