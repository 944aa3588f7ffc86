"""FLASH_ATTN_EXT for batches of queries at head size 128 (the tcgen05 kernel, csrc/kernels/fattn_tc.cu): ragged query and
key counts around its 128 x 128 tiles, no mask, causal masks, masks with arbitrary holes and rows with nothing visible,
against exact float64 attention (tolerance: the reference's NMSE criterion for FLASH_ATTN_EXT,
tests/test-backend-ops.cpp:3137-3139) and, on a sample, against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
NMSE = 5e-4
D = 128


def exact_attention(q, k, v, mask, scale):
    """q [nh, nq, D] f32, k/v [nhkv, nkv, D] f16, mask [nq, nkv] f16 or None -> [nq, nh, D] float64"""
    nh, nq, _ = q.shape
    gqa = nh // k.shape[0]
    out = np.zeros((nq, nh, D))
    m = None if mask is None else mask[:nq].astype(np.float64)
    for h in range(nh):
        s = q[h].astype(np.float64) @ k[h // gqa].astype(np.float64).T * scale
        if m is not None:
            s = s + m
        mx = s.max(axis=1, keepdims=True)
        mx[~np.isfinite(mx)] = 0.0
        p = np.exp(s - mx)
        l = p.sum(axis=1, keepdims=True)
        l[l == 0] = 1.0
        out[:, h] = (p / l) @ v[h // gqa].astype(np.float64)
    return out


def causal(n_q, n_kv):
    m = np.full((n_q, n_kv), -np.inf, dtype=np.float32)
    for i in range(n_q):
        m[i, : n_kv - n_q + i + 1] = 0.0
    return m.astype(np.float16)


def nmse(a, b):
    return float(np.sum((a - b) ** 2) / max(np.sum(a ** 2), 1e-30))


@pytest.mark.parametrize("n_q,n_kv", [(64, 128), (100, 200), (128, 128), (130, 520), (257, 1000), (512, 512), (300, 2048)])
@pytest.mark.parametrize("kind", ["causal", "none", "holes"])
def test_prefill_attention_shapes_and_masks(b200, n_q, n_kv, kind):
    if kind == "causal" and n_q > n_kv:
        pytest.skip("a causal mask needs at least as many keys as queries")
    rng = np.random.default_rng(n_q * 7919 + n_kv)
    nh, nhkv = 8, 2
    q = rng.standard_normal((nh, n_q, D)).astype(np.float32)
    k = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    if kind == "causal":
        mask = causal(n_q, n_kv)
    elif kind == "none":
        mask = None
    else:
        # arbitrary holes, finite biases, whole 64-key runs hidden, and a few rows that see nothing at all
        m = np.where(rng.random((n_q, n_kv)) < 0.3, -np.inf, 0.0).astype(np.float32)
        m += np.where(np.isfinite(m), rng.standard_normal((n_q, n_kv)) * 0.5, 0.0).astype(np.float32)
        m[:, 64:128] = -np.inf
        m[3] = -np.inf
        m[n_q - 1] = -np.inf
        mask = m.astype(np.float16)
    scale = 1.0 / np.sqrt(D)
    got = b200.flash_attn(q, k, v, mask, scale)
    assert np.isfinite(got).all()
    want = exact_attention(q, k, v, mask, scale)
    assert nmse(want, got) <= NMSE, (n_q, n_kv, kind, nmse(want, got))
    if kind == "holes":                                   # rows with nothing visible give zeros (the CPU path: sum 0 -> 0 output)
        assert np.all(got[3] == 0.0) and np.all(got[n_q - 1] == 0.0)


def test_prefill_attention_against_oracle_sample(b200, oracle):
    rng = np.random.default_rng(11)
    nh, nhkv, n_q, n_kv = 8, 2, 192, 640
    q = rng.standard_normal((nh, n_q, D)).astype(np.float32)
    k = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    mask = causal(n_q, n_kv)
    got = b200.flash_attn(q, k, v, mask, 1.0 / np.sqrt(D))
    rows = np.array([0, 1, 63, 64, 127, 128, 129, 191])
    want = oracle.flash_attn(q[:, rows], k, v, mask[rows], 1.0 / np.sqrt(D))
    assert oracle.nmse(want, got[rows]) <= NMSE


def test_prefill_attention_large_logits(b200):
    """Scores far from zero (the running maximum moves between tiles and the accumulator is rescaled)."""
    rng = np.random.default_rng(5)
    nh, nhkv, n_q, n_kv = 4, 1, 128, 768
    q = (rng.standard_normal((nh, n_q, D)) * 4.0).astype(np.float32)
    k = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    k[:, 700:] *= 3.0                                     # the largest scores come in the last tile
    v = rng.standard_normal((nhkv, n_kv, D)).astype(np.float16)
    got = b200.flash_attn(q, k, v, None, 1.0 / np.sqrt(D))
    want = exact_attention(q, k, v, None, 1.0 / np.sqrt(D))
    assert np.isfinite(got).all() and nmse(want, got) <= NMSE
