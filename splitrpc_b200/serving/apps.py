"""What the command-line mains can serve: the built-in apps and the models, by name."""
from __future__ import annotations

from .. import _C

# name -> (request bytes, response bytes, payload generator of the load generator)
BUILTIN = {
    "echo": (1024, 1024, "echo"),
    "vec_add": (1024, 1024, "vec_add"),
    "matmul": (4096, 4096, "matmul"),
    "lenet5": (3136, 40, "uniform"),
}
MODELS = {"resnet50": "normal", "bert_base": "ids"}


def build_model(name: str, device: int, max_batch: int):
    if name == "resnet50":
        from ..models import ResNet50

        return ResNet50(device=device, max_batch=max_batch)
    if name == "bert_base":
        from ..models import BERT_BASE, BertClassifier

        return BertClassifier(BERT_BASE, seq=128, device=device, max_batch=max_batch)
    raise SystemExit(f"unknown model '{name}' (models: {sorted(MODELS)}, apps: {sorted(BUILTIN)})")


def sizes(name: str, req_size: int | None, resp_size: int | None) -> tuple[int, int, str]:
    """Request size, response size and payload kind of an app or model."""
    if name in BUILTIN:
        rq, rs, kind = BUILTIN[name]
        return req_size or rq, resp_size or rs, kind
    if name == "resnet50":
        return 3 * 224 * 224 * 4, 4000, MODELS[name]
    if name == "bert_base":
        return 128 * 4, 8, MODELS[name]
    raise SystemExit(f"unknown app '{name}'")


def make_builtin(name: str, device: int, req_size: int, resp_size: int, pool: int, max_batch: int):
    """A built-in app on `device` (-1 = CPU) with its scatter-gather engine."""
    return _C.make_app(name, device, req_size, resp_size, [], pool, 1, max_batch, "cpu" if device < 0 else "gpu", 2)
