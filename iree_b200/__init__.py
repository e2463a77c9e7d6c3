"""iree_b200: B200-native (sm_100a) mmt4d / pack / unpack behind the IREE ukernel surface.

``iree_b200.abi``      flag constants and ctypes parameter structs (no native code needed)
``iree_b200.ukernel``  the operations (loads ``libiree_uk_b200.so``; no fallback)
``iree_b200.build``    in-tree nvcc build of the shared library
"""
from . import abi  # noqa: F401

__all__ = ["abi"]
