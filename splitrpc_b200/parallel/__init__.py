"""Multi-GPU layer: one process per GPU, ``torch.distributed`` (NCCL) for bootstrap,
symmetric peer memory over NVLink for the data path, and the fused
all-gather->GEMM / GEMM->reduce-scatter kernels for tensor parallelism."""
from .symm import init_distributed, SymmetricArena  # noqa: F401
from .tp import TensorParallel  # noqa: F401
