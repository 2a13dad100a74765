"""B200-native tensor-parallel layer path for nano-vllm.

The directory name is not a Python identifier; load the package with
`__graft_entry__.load_package()` (it registers it as `nanovllm_b200`).
Layout mirrors the part of the reference it replaces:

    csrc/      CUDA kernels (sm_100a) and the C ABI (include/b200tp.h)
    _abi.py    ctypes binding
    runtime.py per-process tensor-parallel context (symmetric buffers)
    ops.py     tensor-level wrappers over the C ABI
    layers/    drop-in layer classes (linear, layernorm, embed_head, attention, ...)
    models/    Qwen3 wiring that uses the fused row-parallel entry
    engine/    the part of the model runner that hosts the path
    utils/     per-step context
"""
from . import _abi  # noqa: F401  (fails loudly when the CUDA library is missing)
from .runtime import TPRuntime, get_runtime, init_runtime, shutdown_runtime  # noqa: F401
