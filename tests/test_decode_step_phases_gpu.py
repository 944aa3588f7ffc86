"""Each phase of the persistent decode-step kernel (csrc/kernels/decode_step.cu) on its own, through the flat C-ABI
(b200_decode_step_*_host), against the oracle of the op sequence it replaces and against the one-kernel-per-op
entry points of the same library."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
NMSE_MM = 5e-4          # the reference's MUL_MAT / FLASH_ATTN_EXT criterion (tests/test-backend-ops.cpp:1916-1918, 3137-3139)


def weights(oracle, qt, m, k, seed):
    rng = np.random.default_rng(seed)
    return oracle.quantize_rows(qt, (rng.standard_normal((m, k)) * 0.02).astype(np.float32)) if qt in ("q4_0", "q8_0") else \
        oracle_k_quant(oracle, qt, m, k, rng)


def oracle_k_quant(oracle, qt, m, k, rng):
    """K-quant rows: the reference's own quantizer when oracle/_ref is built, else random well-formed blocks
    (every byte pattern of a K-quant block is a valid block; d / dmin are set to small finite halves)."""
    if oracle.ref_available():
        return oracle.ref_quantize_rows(qt, (rng.standard_normal((m, k)) * 0.02).astype(np.float32))
    rb = oracle.row_size(qt, k)
    w = rng.integers(0, 256, (m, rb), dtype=np.uint8)
    bs = {"q4_K": 144, "q5_K": 176, "q6_K": 210}[qt]
    blocks = w.reshape(m, rb // bs, bs)
    d = np.float16(0.001).view(np.uint16)
    if qt == "q6_K":
        blocks[:, :, 208] = d & 0xff; blocks[:, :, 209] = d >> 8
    else:
        for off in (0, 2):
            blocks[:, :, off] = d & 0xff; blocks[:, :, off + 1] = d >> 8
    return w


# (type, K, M): one and several ring-slot segments per row, both rows of a pair in one slot, Q6_K's half-block lanes,
# row counts that do not fill the grid evenly
SHAPES = [("q4_K", 2048, 512), ("q4_K", 4096, 4096), ("q4_K", 14336, 1024), ("q4_K", 8192, 1000), ("q4_K", 4096, 1001),
          ("q6_K", 2048, 512), ("q6_K", 4096, 2048), ("q6_K", 14336, 1024), ("q5_K", 4096, 1024), ("q5_K", 8192, 1024), ("q5_K", 2048, 514),
          ("q4_0", 2048, 512), ("q4_0", 4096, 4096), ("q4_0", 14336, 1024), ("q4_0", 8192, 1001),
          ("q8_0", 2048, 512), ("q8_0", 4096, 2048), ("q8_0", 14336, 1024), ("q8_0", 4096, 1001)]


@pytest.mark.parametrize("qt,k,m", SHAPES)
def test_mat_vec_phase_plain(b200, oracle, qt, k, m):
    w = weights(oracle, qt, m, k, seed=1)
    x = np.random.default_rng(2).standard_normal(k).astype(np.float32)
    got, _ = b200.decode_step_mul_mat(qt, w, x)
    assert np.isfinite(got).all()
    rows = np.random.default_rng(3).choice(m, min(m, 96), replace=False)
    rows[:2] = [0, m - 1]
    assert oracle.nmse(oracle.mul_mat(qt, w[rows], x[None, :])[0], got[rows]) <= NMSE_MM
    # and the one-kernel-per-op path of the same library (same int8 activation scheme): every row
    assert oracle.nmse(b200.mul_mat_q(qt, w, x[None, :])[0], got) <= 1e-5


@pytest.mark.parametrize("qt,k,m", [("q4_K", 4096, 2048), ("q6_K", 4096, 512), ("q4_K", 8192, 512), ("q4_0", 4096, 1024), ("q8_0", 4096, 1024)])
def test_mat_vec_phase_residual_and_norm(b200, oracle, qt, k, m):
    rng = np.random.default_rng(5)
    w = weights(oracle, qt, m, k, seed=4)
    x, r = rng.standard_normal(k).astype(np.float32), rng.standard_normal(k).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    got, s = b200.decode_step_mul_mat(qt, w, x, x_add=r, norm_w=nw, eps=1e-5)
    assert np.array_equal(s, x + r)                                  # the residual stream is an exact F32 sum
    y = oracle.rms_norm((x + r)[None, :], 1e-5, nw)
    assert oracle.nmse(oracle.mul_mat(qt, w, y)[0], got) <= NMSE_MM


@pytest.mark.parametrize("k,m", [(2048, 512), (4096, 14336), (8192, 1024)])
def test_gate_up_phase(b200, oracle, k, m):
    wg, wu = weights(oracle, "q4_K", m, k, seed=6), weights(oracle, "q4_K", m, k, seed=7)
    x = np.random.default_rng(8).standard_normal(k).astype(np.float32)
    got = b200.decode_step_gate_up("q4_K", wg, wu, x)
    rows = np.random.default_rng(9).choice(m, 128, replace=False)
    want = oracle.silu_mul(oracle.mul_mat("q4_K", wg[rows], x[None, :]), oracle.mul_mat("q4_K", wu[rows], x[None, :]))[0]
    assert oracle.nmse(want, got[rows]) <= NMSE_MM


@pytest.mark.parametrize("qt_v", ["q4_K", "q6_K"])
@pytest.mark.parametrize("pos,n_dims,ff", [(0, 128, False), (517, 128, False), (4000, 64, True)])
def test_qkv_rope_phase(b200, oracle, qt_v, pos, n_dims, ff):
    k, n_head, n_head_kv = 2048, 8, 2
    rng = np.random.default_rng(10)
    wq, wk, wv = weights(oracle, "q4_K", n_head * 128, k, 11), weights(oracle, "q4_K", n_head_kv * 128, k, 12), weights(oracle, qt_v, n_head_kv * 128, k, 13)
    x = rng.standard_normal(k).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    factors = (1.0 + rng.random(n_dims // 2)).astype(np.float32) if ff else None
    q, kk, vv = b200.decode_step_qkv("q4_K", qt_v, wq, wk, wv, n_head, n_head_kv, x, nw, 1e-5, pos, n_dims, 500000.0, factors)
    y = oracle.rms_norm(x[None, :], 1e-5, nw)
    p = np.array([pos], dtype=np.int32)
    want_q = oracle.rope(oracle.mul_mat("q4_K", wq, y).reshape(1, n_head, 128), p, factors, n_dims, 0, 8192, 500000.0)[0]
    want_k = oracle.rope(oracle.mul_mat("q4_K", wk, y).reshape(1, n_head_kv, 128), p, factors, n_dims, 0, 8192, 500000.0)[0]
    want_v = oracle.mul_mat(qt_v, wv, y).reshape(n_head_kv, 128)
    assert oracle.nmse(want_q, q) <= NMSE_MM
    assert oracle.nmse(want_k, kk.astype(np.float32)) <= NMSE_MM + 1e-6      # + F16 rounding of the cache row
    assert oracle.nmse(want_v, vv.astype(np.float32)) <= NMSE_MM + 1e-6


@pytest.mark.parametrize("n_kv,n_slices,next_merges", [(256, 1, False), (256, 2, False), (256, 2, True), (768, 4, True), (4096, 18, False),
                                                       (1000, 3, False), (2048, 8, True), (768, 12, True), (1024, 16, True)])
@pytest.mark.parametrize("n_head,n_head_kv", [(32, 8), (16, 2)])
def test_attention_phase(b200, oracle, n_kv, n_slices, next_merges, n_head, n_head_kv):
    rng = np.random.default_rng(n_kv + n_slices)
    q = rng.standard_normal((n_head, 128)).astype(np.float32)
    k = rng.standard_normal((n_head_kv, n_kv, 128)).astype(np.float16)
    v = rng.standard_normal((n_head_kv, n_kv, 128)).astype(np.float16)
    n_valid = n_kv - 37                                           # causal: the tail of the padded cache is masked out
    mask = np.zeros(n_kv, dtype=np.float16); mask[n_valid:] = -np.inf
    scale = 1.0 / np.sqrt(128.0)
    got = b200.decode_step_attention(q, k, v, mask, scale, n_slices, merge_in_next_phase=next_merges)
    # exact attention in float64
    kq = np.einsum("hd,hkd->hk", q.astype(np.float64), np.repeat(k, n_head // n_head_kv, axis=0).astype(np.float64)) * scale
    kq[:, n_valid:] = -np.inf
    pr = np.exp(kq - kq.max(axis=1, keepdims=True)); pr /= pr.sum(axis=1, keepdims=True)
    exact = np.einsum("hk,hkd->hd", pr, np.repeat(v, n_head // n_head_kv, axis=0).astype(np.float64))
    assert oracle.nmse(exact, got) <= 1e-6                        # FP32 softmax and accumulation
    want = oracle.flash_attn(q[:, None, :], k, v, mask[None, :], scale)[0]
    assert oracle.nmse(want, got) <= NMSE_MM
    # the op-level kernel of the same library
    assert oracle.nmse(b200.flash_attn(q[:, None, :], k, v, mask[None, :], scale)[0], got) <= 1e-6
