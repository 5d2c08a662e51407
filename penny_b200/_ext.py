"""Loader of the native extension `penny_cpp` (built in-tree by setup.py).

The extension is the product: on a machine with a GPU a missing or stale build
is an error, never a silent PyTorch fallback.  On a CPU-only machine the module
still imports (it links no driver library), which is what the CPU test tier and
the build check rely on.
"""
import importlib
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load():
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    try:
        return importlib.import_module("penny_cpp")
    except ImportError:
        if _ROOT not in sys.path:
            sys.path.insert(0, _ROOT)
        try:
            return importlib.import_module("penny_cpp")
        except ImportError as e:  # pragma: no cover - depends on the build state
            raise ImportError(
                "penny_cpp is not built. Run `python setup.py build_ext --inplace` in "
                f"{_ROOT} (nvcc, sm_100a). Original error: {e}") from e


ops = load()
