"""App presets and environment configuration.

The stack is configured through ``P2P_RPC_*`` environment variables with the
same names and defaults as the original system (reference
``src/utils/config_utils.h:15-100``); ``set_app_config`` is the Python form of
``SETAPPCONFIGS`` (reference ``conf_scripts/app_config.sh:3-70``) and exports
MTU, request size and response size for a named app.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class AppPreset:
    mtu: int
    req_size: int
    resp_size: int
    model: str | None = None


APP_PRESETS: dict[str, AppPreset] = {
    "echo": AppPreset(1024, 1024, 1024),
    "resnet18": AppPreset(8192, 602112, 4000, "resnet18v2batchedtrt.onnx"),
    "resnet50": AppPreset(8192, 602112, 4000, "resnet50v2batchedtrt.onnx"),
    "bert": AppPreset(8192, 6152, 2056, "bertsquad10-symbolic.onnx"),
    "vecadd1k": AppPreset(1024, 1024, 1024),
    "vecadd1M": AppPreset(8192, 1 << 20, 1 << 20),
    "lenet": AppPreset(784, 784, 40),
    "lstm": AppPreset(8192, 8192, 1024),
    "matmul16": AppPreset(2048, 2048, 1024),
    "matmul32": AppPreset(8192, 8192, 4096),
    "matmul": AppPreset(8192, 32768, 16384),
    # configurations added by this framework
    "lenet5": AppPreset(8192, 3136, 40),
    "bert_base_cls": AppPreset(8192, 512, 8),
    "bert_large_tp": AppPreset(8192, 1536, 8),
}


def set_app_config(name: str) -> AppPreset:
    """Exports ``P2P_RPC_{MTU,REQ_SIZE,RESP_SIZE,ORT_MODEL_NAME}`` for ``name``."""
    p = APP_PRESETS[name]
    os.environ["P2P_RPC_MTU"] = str(p.mtu)
    os.environ["P2P_RPC_REQ_SIZE"] = str(p.req_size)
    os.environ["P2P_RPC_RESP_SIZE"] = str(p.resp_size)
    if p.model:
        os.environ["P2P_RPC_ORT_MODEL_NAME"] = p.model
    from .. import _C

    _C.set_rpc_mtu(p.mtu)
    return p
