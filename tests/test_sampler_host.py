"""The sampler on the CPU: the oracle's two formulations against the reference's own draw (golden fixture), the
generator behind the fused LM-head sampler against published known answers and against the library's host copy,
and the distribution of the fused formulation."""
import ctypes as C
import os

import numpy as np
import torch

from oracle import tp_path as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors): counter, key, output
PHILOX_KAT = [
    ([0, 0, 0, 0], (0, 0), [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
    ([0xffffffff] * 4, (0xffffffff, 0xffffffff), [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
    ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], (0xa4093822, 0x299f31d0), [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
]


def test_reference_sampler_golden():
    """nanovllm/layers/sampler.py run on the CPU with a seeded generator: the restatement with the same noise picks
    the same tokens, and so does the softmax-free form the fused kernel evaluates."""
    d = torch.load(os.path.join(GOLDEN, "sampler.pt"))
    assert torch.equal(O.sampler_with_noise(d["logits"], d["temperatures"], d["noise"]), d["tokens"])
    assert torch.equal(O.sampler_scores(d["logits"], d["temperatures"], d["noise"]).argmax(-1), d["tokens"])
    # greedy = the reference at a temperature far below the logit spacing (its own lower limit is 1e-10)
    cold = torch.full_like(d["temperatures"], 1e-4)
    assert torch.equal(O.sampler_with_noise(d["logits"], cold, d["noise"]), O.sampler_scores(d["logits"], None, None).argmax(-1))


def test_philox_known_answers(pkg):
    from nanovllm_b200 import _abi
    for ctr, key, want in PHILOX_KAT:
        assert O.philox4x32_10(np.array(ctr, dtype=np.uint32), key).tolist() == want
        out = (C.c_uint32 * 4)()
        assert _abi.lib.b2_philox4x32_10((C.c_uint32 * 4)(*ctr), (C.c_uint32 * 2)(*key), out) == 0
        assert list(out) == want


def test_library_noise_matches_oracle(pkg):
    """The host copy of the device generator (b2_sampler_noise_bits) and the oracle's vectorised one agree on the
    counter layout: (vocab id, row // 4, call, tag), word row % 4."""
    from nanovllm_b200 import _abi
    rng = np.random.default_rng(3)
    for seed in (0, 1234, 0xDEADBEEFCAFEF00D):
        for call in (0, 1, 77):
            rows, vocab = 11, 300
            E = O.fused_sampler_noise(seed, call, rows, vocab)
            for _ in range(40):
                row, v = int(rng.integers(rows)), int(rng.integers(vocab))
                bits = C.c_uint32()
                assert _abi.lib.b2_sampler_noise_bits(seed, v, row, call, C.byref(bits)) == 0
                u = ((bits.value >> 9) + 0.5) * 2.0 ** -23
                assert 0.0 < u < 1.0 and np.float32(u) == u        # exact in fp32, ends excluded
                assert abs(-np.log(u) - E[row, v].item()) < 1e-12


def test_fused_formulation_has_the_reference_distribution():
    """argmax(logit / T - log E) with the fused sampler's own noise draws token i with probability softmax(logit / T)_i."""
    vocab, rows, calls, temp = 24, 64, 150, 0.8
    g = torch.Generator().manual_seed(9)
    logits = (torch.randn(vocab, generator=g) * 2).bfloat16()
    p = torch.softmax(logits.float() / temp, -1).double()
    counts = torch.zeros(vocab, dtype=torch.float64)
    batch = logits.unsqueeze(0).expand(rows, vocab)
    temps = torch.full((rows,), temp)
    for call in range(calls):
        E = O.fused_sampler_noise(seed=2024, call=call, rows=rows, vocab=vocab)
        tok = O.sampler_scores(batch, temps, E).argmax(-1)
        counts += torch.bincount(tok, minlength=vocab).double()
    n = rows * calls
    sigma = torch.sqrt(p * (1 - p) / n)
    assert ((counts / n - p).abs() <= 4.5 * sigma + 1e-4).all(), (counts / n - p) / sigma
    # rows and calls draw independently: no token repeats across a whole call more often than chance allows
    chi2 = (((counts - n * p) ** 2) / (n * p)).sum().item()
    assert chi2 < 70.0, chi2          # 23 degrees of freedom: mean 23, P(chi2 > 70) < 1e-6
