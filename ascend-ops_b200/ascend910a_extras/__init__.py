"""Drop-in `ascend910a_extras` package backed by hand-written sm_100a CUDA kernels.

The reference's package init (ascend910a_extras/__init__.py:7-27) loads its op library
`libcust_opapi.so` and points CANN at the custom operator path.  The counterpart here is
loading the compiled torch extension `ascend910a_extras_C`, which links the C-ABI library
`lib/libb200ops.so`.  There is no fallback: if the extension has not been built the import
fails with instructions instead of silently computing somewhere else.
"""
import os as _os

import torch as _torch  # noqa: F401  (the extension needs libtorch loaded first)

_PKG_DIR = _os.path.dirname(_os.path.abspath(__file__))

try:
    from . import ascend910a_extras_C  # noqa: F401
except ImportError as _exc:  # pragma: no cover - exercised only on a broken install
    raise ImportError(
        "ascend910a_extras: the CUDA extension is not built. Run "
        f"`python {_os.path.join(_os.path.dirname(_PKG_DIR), 'build.py')}` "
        "(needs nvcc with sm_100a support). There is no CPU or eager fallback. "
        f"Original error: {_exc}"
    ) from _exc

LIB_PATH = _os.path.join(_PKG_DIR, "lib", "libb200ops.so")
