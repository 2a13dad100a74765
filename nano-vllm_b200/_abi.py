"""ctypes binding of libb200tp.so (the C ABI declared in include/b200tp.h).

There is no fallback: if the library has not been built, importing this module
raises, and so does every layer that would have used it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200tp.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python nano-vllm_b200/build.py` (nvcc, sm_100a). "
        "There is no CPU or PyTorch fallback for this path."
    )

lib = C.CDLL(LIB_PATH)

OK, ERR_ARG, ERR_SHAPE, ERR_CUDA, ERR_STATE, ERR_TIMEOUT, ERR_UNSUPPORTED = range(7)
HANDLE_BYTES = 64
FORM_AUTO, FORM_ONESHOT, FORM_OWNER, FORM_TWOSHOT = range(4)
OPT_ROWPAR_FORM, OPT_OWNER_MAX_TOKENS, OPT_TWOSHOT_MIN_TOKENS, OPT_WHOLE_TILES, OPT_OWNER_MIN_TOKENS = 1, 2, 3, 4, 5
_ERR_NAMES = {1: "bad argument", 2: "shape outside what the context was created for", 3: "CUDA error",
              4: "bad state (peers not imported?)", 5: "device-side wait timed out", 6: "unsupported"}
WAIT_NAMES = {0: "none", 1: "GEMM: TMA stage never filled", 2: "GEMM: stage never freed", 3: "GEMM: accumulator never completed",
              4: "GEMM: accumulator never drained", 5: "fused row-parallel: partial rows never arrived",
              6: "embedding: owner row never arrived", 7: "LM head: a peer's logits never arrived",
              8: "token broadcast: rank 0's tokens never arrived", 9: "two-shot row-parallel: rows owned by other ranks never arrived"}


class Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("rank", "world", "device", "max_tokens", "hidden", "oneshot_tokens", "vocab", "max_seqs", "timeout_ms")]


class B2Error(RuntimeError):
    pass


class GemmPlan(C.Structure):
    """b2_gemm_plan: what the launch planner decides for one GEMM (host arithmetic only)."""
    _fields_ = [(n, C.c_int) for n in ("swap", "bn", "tiles_p", "tiles_q", "kblocks", "gemm_ctas", "round_robin", "grid", "cluster_split")]


_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

SIGNATURES = {
    "b2_ctx_create": [C.POINTER(Config), C.POINTER(_p)],
    "b2_symm_export": [_p, _p],
    "b2_symm_import": [_p, _p],
    "b2_ctx_destroy": [_p],
    "b2_status": [_p, C.POINTER(_i), C.POINTER(_i)],
    "b2_status_clear": [_p],
    "b2_ctx_reset": [_p],
    "b2_trace": [_p, _i, _p, _i],
    "b2_gemm": [_p, _p, _i64, _p, _i64, _p, _p, _i64, _i, _i, _i, _p],
    "b2_qkv_fused": [_p, _p, _i64, _p, _i64, _p, _p, _i64, _i, _i, _i, _i, _i, _p, _p, _f, _p, _p, _p, _p, _p, _p],
    "b2_gemm_silu_mul": [_p, _p, _i64, _p, _i64, _p, _i64, _i, _i, _i, _p],
    "b2_gemm_static_scratch": [_p, _i64, _p, _i64, _p, _p, _i64, _i, _i, _i, _p],
    "b2_rowpar_fused": [_p, _p, _i64, _p, _i64, _p, _i, _i, _i, _p, _p, _f, _p, _p, _p],
    "b2_ctx_set_option": [_p, _i, _i64],
    "b2_rowpar_form": [_p, _i, _i],
    "b2_rowpar_fused_twoshot": [_p, _p, _i64, _p, _i64, _p, _i, _i, _i, _p, _p, _f, C.POINTER(_p), _p, _p],
    "b2_rmsnorm": [_p, _i64, _p, _f, _i, _i, _p, _i64, _p],
    "b2_add_rmsnorm": [_p, _p, _p, _f, _i, _i, _p, _p, _p],
    "b2_store_kvcache": [_p, _i64, _p, _i64, _p, _p, _p, _i, _i, _p],
    "b2_embed": [_p, _p, _p, _i64, _i64, _i, _i, _p, _p],
    "b2_lm_head": [_p, _p, _i64, _p, _p, _i64, _i, _i, _i, C.POINTER(_p), _p],
    "b2_lm_head_sample": [_p, _p, _i64, _p, _p, _i64, _i, _i, _i, _p, C.c_uint64, _p, _p],
    "b2_sampler_noise_bits": [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)],
    "b2_philox4x32_10": [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)],
    "b2_silu_and_mul": [_p, _i64, _i, _i, _p, _p],
    "b2_qk_norm_rope_store": [_p, _i64, _i, _i, _i, _i, _p, _p, _f, _p, _p, _p, _p, _p, _p],
    "b2_argmax": [_p, _i64, _i, _i, _p, _p],
    "b2_broadcast_tokens": [_p, _p, _i, _p],
    "b2_advance_decode": [_p, _p, _p, _p, _p, _p, _i64, _i, _i, _i64, _i, _p],
    # the planner as data: no CUDA call, usable without a GPU
    "b2_plan_gemm": [_i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(GemmPlan)],
    "b2_plan_gemm_opts": [_i, _i, _i, _i, _i, C.POINTER(_i), _i, C.POINTER(GemmPlan)],
    "b2_plan_cta_units": [C.POINTER(GemmPlan), _i, C.POINTER(_i), _i],
    "b2_plan_tile_contributors": [C.POINTER(GemmPlan), _i, C.POINTER(_i), C.POINTER(_i)],
    "b2_last_gemm_kernel": [],
    "b2_row_owner": [_i, _i, C.POINTER(_i)],
    "b2_owned_rows": [_i, _i, _i],
    "b2_owner_form_row": [_i, _i, C.POINTER(_i)],
    "b2_owner_form_rows": [_i, _i, _i],
}
for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _i
lib.b2_last_error.restype = C.c_char_p
lib.b2_last_error.argtypes = []
lib.b2_launch_count.restype = _i64
lib.b2_launch_count.argtypes = []

EXPORTED = list(SIGNATURES) + ["b2_last_error", "b2_launch_count"]


def check(rc: int, what: str) -> None:
    if rc != OK:
        msg = _ERR_NAMES.get(rc, f"code {rc}")
        if rc == ERR_CUDA:
            msg += ": " + (lib.b2_last_error() or b"").decode()
        raise B2Error(f"{what}: {msg}")


def launch_count() -> int:
    return int(lib.b2_launch_count())
