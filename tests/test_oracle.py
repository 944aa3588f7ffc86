"""Pins the CPU oracle (oracle/ggml_oracle.c) to the reference: against the golden
fixtures produced by the unmodified reference, and, where the reference build is
present, against the reference libraries directly.  CPU only."""
import numpy as np
import pytest

QT = ["q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q2_K", "q3_K", "q4_K", "q5_K", "q6_K", "iq4_nl", "iq4_xs"]
SIMPLE_QT = ["q4_0", "q4_1", "q5_0", "q5_1", "q8_0"]


@pytest.mark.parametrize("qt", QT)
def test_dequantize_bit_exact_vs_golden(oracle, golden, qt):
    q = golden[f"quant.q.{qt}"]
    want = golden[f"quant.dq.{qt}"]
    got = oracle.dequantize_rows(qt, q[None, :], want.size)[0]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("qt", SIMPLE_QT)
def test_quantize_bit_exact_vs_golden(oracle, golden, qt):
    x = golden["quant.input"]
    got = oracle.quantize_rows(qt, x[None, :])[0]
    assert np.array_equal(got, golden[f"quant.q.{qt}"])


def test_f16_rounding_vs_golden(oracle, golden):
    got = oracle.f32_to_f16(golden["f16.input"])
    assert np.array_equal(got.view(np.uint16), golden["f16.output"].view(np.uint16))


@pytest.mark.parametrize("qt", QT)
def test_mul_mat_vs_golden(oracle, golden, qt):
    # same integer algorithm as the CPU backend; only the float summation order differs
    got = oracle.mul_mat(qt, golden[f"mul_mat.w.{qt}"], golden["mul_mat.x"])
    assert oracle.nmse(golden[f"mul_mat.y.{qt}"], got) < 1e-10


@pytest.mark.parametrize("qt", QT)
def test_mul_mat_quantization_error_is_small(oracle, golden, qt):
    # the int8-activation product stays within test-backend-ops' 5e-4 of the float product
    w, x = golden[f"mul_mat.w.{qt}"], golden["mul_mat.x"]
    assert oracle.nmse(oracle.mul_mat(qt, w, x, exact_f32=True), oracle.mul_mat(qt, w, x)) < 5e-4


def test_flash_attn_vs_golden(oracle, golden):
    got = oracle.flash_attn(golden["fattn.q"], golden["fattn.k"], golden["fattn.v"], golden["fattn.mask"], 1.0 / np.sqrt(128.0))
    assert oracle.nmse(golden["fattn.y"], got) < 1e-8


def test_glue_ops_vs_golden(oracle, golden):
    x, w, g = golden["glue.x"], golden["glue.w"], golden["glue.g"]
    assert oracle.nmse(golden["glue.rms_norm"], oracle.rms_norm(x, 1e-5)) < 1e-12
    assert oracle.nmse(golden["glue.rms_norm_mul"], oracle.rms_norm(x, 1e-5, w)) < 1e-12
    assert oracle.nmse(golden["glue.silu_mul"], oracle.silu_mul(g, x)) < 1e-12
    assert oracle.nmse(golden["glue.soft_max"], oracle.soft_max(x, 0.125)) < 1e-12


@pytest.mark.parametrize("mode", [0, 2])
def test_rope_vs_golden(oracle, golden, mode):
    got = oracle.rope(golden["rope.x"], golden["rope.pos"], golden["rope.ff"], 128, mode, 8192, 500000.0)
    assert oracle.nmse(golden[f"rope.y.mode{mode}"], got) < 1e-10


@pytest.mark.parametrize("qt", SIMPLE_QT)
def test_quantize_vs_reference_library(oracle, qt):
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 512)).astype(np.float32) * 0.02
    x[3] = 0.0                                             # all-zero blocks
    x[4, :32] = np.float32(1e-30)
    assert np.array_equal(oracle.quantize_rows(qt, x), oracle.ref_quantize_rows(qt, x))


@pytest.mark.parametrize("qt", QT)
def test_dequantize_vs_reference_quantizer_output(oracle, qt):
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    rng = np.random.default_rng(6)
    x = rng.standard_normal((3, 1024)).astype(np.float32) * 0.02
    q = oracle.ref_quantize_rows(qt, x)
    dq = oracle.dequantize_rows(qt, q, 1024)
    # reconstruction error bound used by the reference (tests/test-quantize-fns.cpp:17-25, :152-158), scaled to
    # sigma: the 2-bit and 3-bit formats are allowed 3.75x and 2x the default
    rmse = float(np.sqrt(np.mean((dq - x) ** 2)))
    assert rmse < 0.02 * 0.2 * {"q2_K": 3.75, "q3_K": 2.0}.get(qt, 1.0)
