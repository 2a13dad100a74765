"""The LM head fused with the sampler (b2_lm_head_sample) on one B200: greedy picks against the stored-logits
path, temperature draws against the oracle fed with the same counter-based noise, the distribution of many
draws, and replays of a captured graph."""
import pytest
import torch

from oracle import tp_path as O
from tests.gpu_util import check_sampler_picks as _check_picks, ensure_group

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SEED = 0x5EED0123456789


@pytest.fixture()
def fresh_runtime(pkg):
    """A runtime per test: the sampler's call counter (part of its noise counter) starts at zero."""
    ensure_group()
    from nanovllm_b200 import ops
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    made = []

    def make(vocab, hidden, max_seqs=256):
        made.append(init_runtime(max_tokens=max(256, max_seqs), hidden=hidden, oneshot_tokens=256, vocab=vocab, max_seqs=max_seqs))
        return ops, made[-1]

    yield make
    torch.cuda.synchronize()
    shutdown_runtime()


def _case(rows, vocab, hidden, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    h = (torch.randn(rows, hidden, generator=g) * scale).bfloat16()
    w = (torch.randn(vocab, hidden, generator=g) * 0.05).bfloat16()
    return h, w


@pytest.mark.parametrize("rows,vocab,hidden", [(1, 512, 128), (7, 1000, 256), (64, 4096, 1024), (33, 151936, 1024), (200, 8192, 512), (256, 2048, 64)])
def test_greedy_matches_stored_logits(fresh_runtime, rows, vocab, hidden):
    ops, rt = fresh_runtime(vocab, hidden)
    h, w = _case(rows, vocab, hidden, seed=rows + vocab)
    hd, wd = h.to(DEV), w.to(DEV)
    logits = ops.lm_head(hd, wd, None).clone()
    tokens = ops.lm_head_sample(hd, wd, None, None, SEED)
    torch.cuda.synchronize()
    rt.check_status()
    assert tokens.dtype == torch.int64 and tokens.shape == (rows,)
    assert int(tokens.min()) >= 0 and int(tokens.max()) < vocab
    _check_picks(tokens, logits, None, None, "greedy")
    # the same call again: the table of best keys was left clean
    again = ops.lm_head_sample(hd, wd, None, None, SEED)
    torch.cuda.synchronize()
    _check_picks(again, logits, None, None, "greedy, second call")


@pytest.mark.parametrize("rows,vocab,hidden", [(5, 640, 128), (64, 4096, 512), (40, 151936, 1024), (130, 3000, 256)])
def test_temperature_draws_match_oracle_noise(fresh_runtime, rows, vocab, hidden):
    ops, rt = fresh_runtime(vocab, hidden)
    h, w = _case(rows, vocab, hidden, seed=7 * rows + vocab, scale=2.0)
    hd, wd = h.to(DEV), w.to(DEV)
    g = torch.Generator().manual_seed(rows)
    temps = (torch.rand(rows, generator=g) * 1.4 + 0.1).to(DEV)
    logits = ops.lm_head(hd, wd, None).clone()
    draws = []
    for call in range(3):                      # the call number is part of the noise counter
        tokens = ops.lm_head_sample(hd, wd, None, temps, SEED).clone()
        torch.cuda.synchronize()
        _check_picks(tokens, logits, temps, O.fused_sampler_noise(SEED, call, rows, vocab), f"call {call}")
        draws.append(tokens.cpu())
    rt.check_status()
    if rows >= 40:
        assert not torch.equal(draws[0], draws[1]) and not torch.equal(draws[1], draws[2])
    # the last-token selection of prefill (row_index) draws with the noise of rows 0 .. n-1 of the selection
    idx = torch.arange(0, rows, 2, dtype=torch.int32)
    tokens = ops.lm_head_sample(hd, wd, idx.to(DEV), temps[::2].contiguous(), SEED)
    torch.cuda.synchronize()
    _check_picks(tokens, logits[::2], temps[::2], O.fused_sampler_noise(SEED, 3, idx.numel(), vocab), "row_index")


def test_draw_frequencies_follow_softmax(fresh_runtime):
    vocab, hidden, rows, calls, temp = 512, 128, 64, 60, 0.7
    ops, rt = fresh_runtime(vocab, hidden, max_seqs=64)
    g = torch.Generator().manual_seed(11)
    h1 = torch.randn(1, hidden, generator=g).bfloat16()
    w = (torch.randn(vocab, hidden, generator=g) * 0.25).bfloat16()
    hd, wd = h1.expand(rows, hidden).contiguous().to(DEV), w.to(DEV)
    temps = torch.full((rows,), temp, device=DEV)
    logits = ops.lm_head(hd, wd, None)[0].float().cpu()
    p = torch.softmax(logits / temp, -1).double()
    counts = torch.zeros(vocab, dtype=torch.float64)
    out = torch.empty(rows, dtype=torch.int64, device=DEV)
    for _ in range(calls):
        ops.lm_head_sample(hd, wd, None, temps, SEED, out=out)
        counts += torch.bincount(out.cpu(), minlength=vocab).double()
    rt.check_status()
    n = rows * calls
    top = p.argsort(descending=True)[:12]
    sigma = torch.sqrt(p * (1 - p) / n)
    assert p[top].sum() > 0.5                                   # the test distribution is concentrated enough to say something
    assert ((counts[top] / n - p[top]).abs() <= 4.5 * sigma[top] + 1e-3).all(), ((counts / n - p) / sigma)[top]
    rest = 1.0 - p[top].sum().item()
    got_rest = 1.0 - counts[top].sum().item() / n
    assert abs(got_rest - rest) <= 4.5 * (rest * (1 - rest) / n) ** 0.5 + 1e-3


def test_graph_replays_draw_afresh(fresh_runtime):
    rows, vocab, hidden = 48, 4096, 256
    ops, rt = fresh_runtime(vocab, hidden, max_seqs=64)
    h, w = _case(rows, vocab, hidden, seed=5, scale=2.0)
    hd, wd = h.to(DEV), w.to(DEV)
    temps = torch.full((rows,), 0.9, device=DEV)
    logits = ops.lm_head(hd, wd, None).clone()
    out = torch.empty(rows, dtype=torch.int64, device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ops.lm_head_sample(hd, wd, None, temps, SEED, out=out)   # call 0: warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.lm_head_sample(hd, wd, None, temps, SEED, out=out)   # captured, not executed
    seen = []
    for call in (1, 2, 3):
        graph.replay()
        torch.cuda.synchronize()
        _check_picks(out, logits, temps, O.fused_sampler_noise(SEED, call, rows, vocab), f"replay {call}")
        seen.append(out.cpu().clone())
    rt.check_status()
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])


def test_more_than_256_rows_is_refused(fresh_runtime):
    ops, rt = fresh_runtime(1024, 128, max_seqs=512)
    from nanovllm_b200._abi import B2Error
    h, w = _case(300, 1024, 128, seed=1)
    with pytest.raises(B2Error, match="shape"):
        ops.lm_head_sample(h.to(DEV), w.to(DEV), None, None, SEED)
