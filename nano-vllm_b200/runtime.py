"""Per-process tensor-parallel runtime: owns the b2_ctx (symmetric buffers,
split-K workspace, status word) and exchanges the buffer handles between ranks.

It takes the place of what the reference sets up around NCCL in
nanovllm/engine/model_runner.py:26-27 (process group + device) and tears down
in :50-59.  The torch.distributed group is still used, but only to bootstrap:
the 64-byte handles travel over it once; no collective of the layer path does.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _abi


class TPRuntime:
    def __init__(self, rank: int, world: int, device: int, max_tokens: int, hidden: int, oneshot_tokens: int = 1024,
                 vocab: int = 0, max_seqs: int = 0, timeout_ms: int = 5000, group=None):
        if not torch.cuda.is_available():
            raise RuntimeError("nanovllm_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.rank, self.world, self.device = rank, world, device
        self.vocab, self.max_seqs, self.hidden, self.max_tokens = vocab, max_seqs, hidden, max_tokens
        self.oneshot_tokens = min(oneshot_tokens if oneshot_tokens > 0 else 1024, max_tokens)
        # the library's default (b2_ctx_create)
        self.default_twoshot_min_tokens = (min(1023 if world >= 8 else 511, self.oneshot_tokens) if world >= 4 else min(1024, self.oneshot_tokens)) + 1
        cfg = _abi.Config(rank, world, device, max_tokens, hidden, oneshot_tokens, vocab, max_seqs, timeout_ms)
        ctx = C.c_void_p()
        torch.cuda.set_device(device)
        _abi.check(_abi.lib.b2_ctx_create(C.byref(cfg), C.byref(ctx)), "b2_ctx_create")
        self.ctx = ctx
        self.poisoned = False
        if world > 1:
            handle = (C.c_ubyte * _abi.HANDLE_BYTES)()
            _abi.check(_abi.lib.b2_symm_export(self.ctx, handle), "b2_symm_export")
            gathered: list = [None] * world
            dist.all_gather_object(gathered, bytes(handle), group=group)
            blob = b"".join(gathered)
            assert len(blob) == world * _abi.HANDLE_BYTES
            _abi.check(_abi.lib.b2_symm_import(self.ctx, blob), "b2_symm_import")
            dist.barrier(group=group)  # every rank's buffers are mapped before anyone pushes

    def check_status(self) -> None:
        """Raise if a bounded device-side wait has expired since the last check.
        No CUDA call is made; call it after the step's own synchronisation.
        After an expired wait the runtime refuses further checks until every
        rank has called reset() (or the runtime has been re-created): the
        buffers and launch counters of the ranks no longer agree."""
        if self.poisoned:
            raise _abi.B2Error(f"rank {self.rank}: a device-side wait expired earlier; call reset() on every rank")
        code, detail = C.c_int(), C.c_int()
        _abi.lib.b2_status(self.ctx, C.byref(code), C.byref(detail))
        if code.value != _abi.OK:
            self.poisoned = True
            raise _abi.B2Error(f"rank {self.rank}: {_abi.WAIT_NAMES.get(detail.value, detail.value)} (code {code.value})")

    def set_option(self, option: int, value: int) -> None:
        """b2_ctx_set_option (see _abi.OPT_*); every rank must set the same values."""
        _abi.check(_abi.lib.b2_ctx_set_option(self.ctx, option, value), "b2_ctx_set_option")

    def reset(self, group=None) -> None:
        """Collective over the ranks: back to the state right after creation (see b2_ctx_reset).  Every rank must
        call it, with none of its kernels in flight."""
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=group)
        _abi.check(_abi.lib.b2_ctx_reset(self.ctx), "b2_ctx_reset")
        if self.world > 1:
            dist.barrier(group=group)
        self.poisoned = False

    def close(self) -> None:
        if self.ctx:
            from . import ops
            ops._LOGIT_VIEWS.clear()  # views of the buffer that is about to be freed
            torch.cuda.synchronize()
            _abi.lib.b2_ctx_destroy(self.ctx)
            self.ctx = None


_RUNTIME: TPRuntime | None = None


def init_runtime(max_tokens: int, hidden: int, **kw) -> TPRuntime:
    """Create the runtime from the default process group, which must exist even
    at world size 1 (the reference's layers read rank and world from it,
    nanovllm/layers/linear.py:23-24)."""
    global _RUNTIME
    if _RUNTIME is not None:
        raise RuntimeError("runtime already initialised")
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = kw.pop("device", torch.cuda.current_device())
    _RUNTIME = TPRuntime(rank, world, device, max_tokens, hidden, **kw)
    return _RUNTIME


def get_runtime() -> TPRuntime:
    if _RUNTIME is None:
        raise RuntimeError("call nanovllm_b200.init_runtime(...) after torch.distributed.init_process_group and set_device")
    return _RUNTIME


def shutdown_runtime() -> None:
    global _RUNTIME
    if _RUNTIME is not None:
        _RUNTIME.close()
        _RUNTIME = None
