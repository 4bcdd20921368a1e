"""Loads the native library.  There is no Python or CPU fallback: if the library is
missing the import fails with the command that builds it."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libtreebeard-runtime.so")

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m treebeard_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib
