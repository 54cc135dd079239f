"""Tensor-parallel building blocks on the fused NVLink kernels.

Activations between blocks are sharded by rows (sequence-parallel layout).  A
column-parallel linear is ``ag_gemm`` (all-gather of the row shards fused into
the GEMM that consumes them); a row-parallel linear is ``gemm_rs`` (the GEMM's
epilogue stores partial tiles into the owner ranks' slots) followed by
``ln_reduce`` (sum of the slots + bias + residual + LayerNorm on the owner).
Ranks run in lockstep; step numbers ("epochs") written into peer-visible flag
words order producers and consumers, and every device-side wait on them is
bounded.
"""
from __future__ import annotations

import torch

from .. import _C
from ..ops import ACT, _ptr, _stream, status_word
from .symm import SymmetricArena


class TensorParallel:
    """Buffers, flags and kernel launchers of one tensor-parallel group for activations ``[tokens, hidden]``."""

    N_SITES = 5  # A (input of the first column-parallel GEMM), B (input of the second), RS1, RS2, DONE

    def __init__(self, tokens: int, hidden: int, device: torch.device, n_copy: int | None = None, group=None):
        import torch.distributed as dist

        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert tokens % (128 * self.tp) == 0, "tokens must be a multiple of 128 * tp"
        # Copier blocks of the all-gather kernels.  One moves about 25 GB/s (16 KB bulk copies through its shared memory),
        # so a shard of several MB wants a few dozen of them; with many ranks the GEMMs are small and can spare the SMs.
        if n_copy is None:
            n_copy = 32 if self.tp <= 2 else 64
        self.tokens, self.hidden, self.device, self.n_copy = tokens, hidden, device, n_copy
        self.rows = tokens // self.tp
        bf = 2
        nbytes = 2 * tokens * hidden * bf + 2 * self.tp * self.rows * hidden * bf + 4096 + 64 * 1024
        self.arena = SymmetricArena(nbytes, device, group)
        a = self.arena
        self.gathered = {"A": a.alloc("gA", (tokens, hidden), torch.bfloat16), "B": a.alloc("gB", (tokens, hidden), torch.bfloat16)}
        self.slots = {"RS1": a.alloc("rs1", (self.tp, self.rows, hidden), torch.bfloat16),
                      "RS2": a.alloc("rs2", (self.tp, self.rows, hidden), torch.bfloat16)}
        self.flags = a.alloc("flags", (self.N_SITES, 8), torch.int32)  # [site][source rank]
        self._site = {"A": 0, "B": 1, "RS1": 2, "RS2": 3, "DONE": 4}
        self.mblock_ready = {k: torch.zeros(tokens // 128, dtype=torch.int32, device=device) for k in ("A", "B")}
        self.owner_count = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=device)
        self.done_count = torch.zeros(1, dtype=torch.int32, device=device)
        a.barrier()

    # ------------------------------------------------------------------ helpers
    def shard(self, which: str) -> torch.Tensor:
        """This rank's row shard inside gathered buffer ``which`` (where producers write their output)."""
        return self.gathered[which][self.rank * self.rows:(self.rank + 1) * self.rows]

    def _flag_ptr(self, site: str, on_rank: int, source: int) -> int:
        return self.arena.ptr("flags", on_rank, (self._site[site] * 8 + source) * 4)

    STEP = 64  # step numbers reserved per forward pass

    def begin_step(self) -> None:
        """Start of a forward pass: waits until every peer has finished the previous pass (they may still be reading
        this rank's buffers), then advances the step-number base.  Captured into graphs like any other launch."""
        # Pass f ends by publishing DONE = base(f) (the base after its own bump); before bumping, the current base is
        # exactly that value (0 before the first pass, which the zero-initialised flags satisfy).
        _C.tp_begin(self.flags[self._site["DONE"]].data_ptr(), self.tp, self.epoch_base.data_ptr(), self.STEP,
                    status_word().data_ptr(), _stream())

    def end_step(self) -> None:
        """End of a forward pass: tells every peer that this rank no longer reads their buffers."""
        self.signal("DONE", 0)

    def signal(self, which: str, epoch: int) -> None:
        """Tells every peer that this rank's shard of gathered buffer ``which`` holds step ``epoch``."""
        _C.tp_signal([self._flag_ptr(which, p, self.rank) for p in range(self.tp)], epoch, _stream(), self.epoch_base.data_ptr())

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, which: str, w: torch.Tensor | None, epoch: int, bias: torch.Tensor | None = None, act: str | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor | None:
        """``act(allgather(shards of which) @ w.T + bias)``; ``w is None`` performs only the all-gather."""
        g = self.gathered[which]
        T, K = g.shape
        N = 0 if w is None else w.shape[0]
        if w is not None and out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
        src = [self.arena.ptr("g" + which, r, r * self.rows * K * 2) for r in range(self.tp)]
        _C.gemm_tp(g.data_ptr(), K, _ptr(w) or g.data_ptr(), K if w is None else w.stride(0), T, N, K,
                   _ptr(out), 0 if out is None else out.stride(0), _ptr(bias), ACT[act], self.tp, self.rank, epoch,
                   self.mblock_ready[which].data_ptr() if self.tp > 1 else 0, self.n_copy if self.tp > 1 else 0, src,
                   g.data_ptr(), self.flags[self._site[which]].data_ptr(), 0, [], [], 0, status_word().data_ptr(), _stream(),
                   self.epoch_base.data_ptr())
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, site: str, epoch: int) -> None:
        """Partial ``a @ w.T`` (a: ``[tokens, K_local]``) pushed tile by tile into the owners' ``site`` slots."""
        T, K = a.shape
        N = w.shape[0]
        dst = [self.arena.ptr("rs1" if site == "RS1" else "rs2", o, self.rank * self.rows * N * 2) for o in range(self.tp)]
        dflag = [self._flag_ptr(site, o, self.rank) for o in range(self.tp)]
        _C.gemm_tp(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), T, N, K, self.slots[site].data_ptr(), N, 0, 0, self.tp,
                   self.rank, epoch, 0, 0, [], 0, 0, 1, dst, dflag, self.owner_count.data_ptr(), status_word().data_ptr(),
                   _stream(), self.epoch_base.data_ptr())

    def ln_reduce(self, site: str, epoch: int, bias: torch.Tensor, residual: torch.Tensor | None, gamma: torch.Tensor,
                  beta: torch.Tensor, out: torch.Tensor, eps: float = 1e-12, signal: tuple[str, int] | None = None) -> torch.Tensor:
        """``out = LN(sum over source ranks of the site's slots + bias + residual)`` on this rank's rows.

        ``signal=(which, epoch)`` makes the kernel's last block tell every peer that this rank's shard of gathered
        buffer ``which`` (normally ``out``) holds that step, instead of a separate :meth:`signal` launch."""
        s = self.slots[site]
        slot_ptrs = [s[r].data_ptr() for r in range(self.tp)]
        sig_flags, sig_epoch, done = [], 0, 0
        if signal is not None:
            sig_flags = [self._flag_ptr(signal[0], p, self.rank) for p in range(self.tp)]
            sig_epoch, done = signal[1], self.done_count.data_ptr()
        _C.layernorm_reduce(slot_ptrs, self.flags[self._site[site]].data_ptr(), epoch, _ptr(bias), _ptr(residual),
                            gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), self.rows, self.hidden, eps,
                            status_word().data_ptr(), _stream(), self.epoch_base.data_ptr(), sig_flags, sig_epoch, done)
        return out
