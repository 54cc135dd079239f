"""splitrpc_b200: a control/data-path-splitting RPC stack for ML inference serving
on B200 GPUs.

The native core (``splitrpc_b200._C``) holds the C++ host runtime (wire format,
request pools, transports, server threads, load generator) and the sm_100a CUDA
kernels.  It is built in-tree by :mod:`splitrpc_b200._build`; importing the
package builds it when it is missing or stale and ``nvcc`` is available, and
fails loudly otherwise.
"""
from __future__ import annotations

import importlib
import os

from . import _build

__version__ = "0.1.0"


def _load_native():
    if not _build.up_to_date():
        if os.environ.get("SPLITRPC_NO_BUILD") == "1":
            if not _build.TARGET.exists():
                raise ImportError("splitrpc_b200._C is not built and SPLITRPC_NO_BUILD=1")
        else:
            _build.build()
    return importlib.import_module("splitrpc_b200._C")


_C = _load_native()

from .utils.config import AppPreset, APP_PRESETS, set_app_config  # noqa: E402
