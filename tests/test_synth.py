"""The synthetic-weight quantizers (torch) write blocks the reference's dequantizers read back: the oracle's
dequantize_row (pinned to the reference by the golden fixtures) recovers the input within the format's step."""
import numpy as np
import pytest


@pytest.mark.parametrize("qtype,tid,levels", [("q4_K", 12, 15), ("q5_K", 13, 31), ("q6_K", 14, 63)])
def test_synth_blocks_dequantize(b200, oracle, qtype, tid, levels):
    import torch
    from llama_cpp_b200 import synth
    k, rows = 512, 6
    raw = synth.make_tensor(tid, k, rows, seed=3, sigma=0.02)
    assert raw.size == rows * oracle.row_size(qtype, k)
    gen = torch.Generator(device="cpu"); gen.manual_seed(3)
    x = (0.02 * torch.randn(rows, k, generator=gen, dtype=torch.float32)).numpy()
    y = oracle.dequantize_rows(qtype, raw.reshape(rows, -1), k)
    # per 32-value (Q6_K: 16-value) group the error is at most about one quantization step
    step = (x.max() - x.min()) / levels
    assert np.abs(y - x).max() <= 1.5 * step
    assert oracle.nmse(x, y) < {"q4_K": 2e-2, "q5_K": 5e-3, "q6_K": 1.5e-3}[qtype]


@pytest.mark.parametrize("qtype,tid", [("q4_0", 2), ("q8_0", 8)])
def test_synth_q4_0_q8_0_equal_reference_quantizer(b200, oracle, qtype, tid):
    """For the two simple formats the torch generator is the reference's own rounding rule: same bytes as the oracle's
    quantize_row (pinned to the reference by the golden fixtures)."""
    import torch
    from llama_cpp_b200 import synth
    k, rows = 512, 6
    raw = synth.make_tensor(tid, k, rows, seed=3, sigma=0.02).reshape(rows, -1)
    gen = torch.Generator(device="cpu"); gen.manual_seed(3)
    x = (0.02 * torch.randn(rows, k, generator=gen, dtype=torch.float32)).numpy()
    assert np.array_equal(raw, oracle.quantize_rows(qtype, x))
