"""b2_gemm_static_scratch: the GEMM for callers that cannot allocate.

Some users of the library are not in a position to call cudaMalloc - for
example a plug-in that is loaded after the serving engine has given all free
HBM to its KV cache, or code that is handed only a stream and tensors and has
no context to create.  For them the library keeps the kernel's scratch (split
tile partials and arrival counters) in a fixed device array compiled into the
.so.  This test calls that entry point straight through the C ABI, twice in a
row (the second call finds the first call's leftovers in the shared array),
and checks each result against the ordinary b2_gemm entry point on the same
inputs, with the bf16 tolerance the other GEMM tests use.

The file name sorts last on purpose: a run that stops at the first failure
has already been through every other test.
"""
import ctypes as C

import pytest
import torch

from tests.gpu_util import assert_close_bf16, ensure_group

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture()
def ordinary_gemm(pkg):
    """The existing context-based entry point, with a context of its own when
    no other test has one open (so the file also passes alone, in a fresh process)."""
    ensure_group()
    from nanovllm_b200 import ops, runtime
    created = runtime._RUNTIME is None
    if created:
        runtime.init_runtime(max_tokens=256, hidden=1024, oneshot_tokens=256)
    yield ops.gemm
    if created:
        runtime.shutdown_runtime()


def _static_gemm(x: torch.Tensor, w: torch.Tensor, bias=None) -> tuple[int, torch.Tensor]:
    from nanovllm_b200 import _abi
    out = torch.empty(x.shape[0], w.shape[0], dtype=torch.bfloat16, device=x.device)
    rc = _abi.lib.b2_gemm_static_scratch(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), bias.data_ptr() if bias is not None else None,
                                         out.data_ptr(), out.stride(0), x.shape[0], w.shape[0], x.shape[1],
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_scratch_gemm_matches_the_ordinary_entry_point(ordinary_gemm):
    from nanovllm_b200 import _abi
    g = torch.Generator().manual_seed(77)
    # both shapes split output tiles over several CTAs, so the shared scratch is really used
    for m, n, k in [(64, 4096, 4096), (17, 1024, 12288)]:
        x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
        w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(DEV)
        bias = torch.randn(n, generator=g).bfloat16().to(DEV)
        want = ordinary_gemm(x, w, bias)
        rc1, first = _static_gemm(x, w, bias)
        rc2, second = _static_gemm(x, w, bias)  # straight after, on the scratch the first call left behind
        torch.cuda.synchronize()
        assert rc1 == _abi.OK and rc2 == _abi.OK, _abi.lib.b2_last_error()
        assert_close_bf16(first, want.float(), f"first call {m}x{n}x{k}", abs_tol=2e-2, rel_tol=1e-2)
        assert_close_bf16(second, want.float(), f"second call {m}x{n}x{k}", abs_tol=2e-2, rel_tol=1e-2)
        assert_close_bf16(first, x.float() @ w.float().t() + bias.float(), f"against fp32 {m}x{n}x{k}")


def test_static_scratch_gemm_rejects_what_does_not_fit(pkg):
    from nanovllm_b200 import _abi
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    rc, _ = _static_gemm(x, w)
    assert rc == _abi.ERR_SHAPE
    assert b"64 token rows" in _abi.lib.b2_last_error()
