"""b200_mul_mat_q_noalloc: the MUL_MAT entry point for callers that may not allocate device memory
(a serving loop under a frozen memory budget, a host that forbids cudaMalloc after start-up, a
process whose device allocator belongs to another framework).  Its activation scratch is a fixed array inside the library.  The test calls it through
the C-ABI twice in a row -- the second call reuses the array the first one dirtied -- and checks
both results against the ordinary entry point, which uses the same kernels on a caller-provided
scratch buffer.  It lives in a file of its own that is collected last."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_pair(b200, torch, qt, w, x):
    l = b200.lib()
    n, k = x.shape
    m = w.shape[0]
    t = b200.TYPES[qt]
    rb = b200.row_size(qt, k)
    dw = torch.from_numpy(w).cuda()
    dx = torch.from_numpy(x).cuda()
    ref = torch.zeros(n, m, device="cuda", dtype=torch.float32)
    out = torch.full((n, m), float("nan"), device="cuda", dtype=torch.float32)
    sb = int(l.b200_mul_mat_q_scratch_bytes(t, m, k, n))
    scratch = torch.empty(sb + 256, device="cuda", dtype=torch.uint8)
    st = torch.cuda.current_stream().cuda_stream
    rc = l.b200_mul_mat_q(t, dw.data_ptr(), rb, m, k, dx.data_ptr(), k, n, ref.data_ptr(), m, scratch.data_ptr(), sb, st)
    assert rc == 0, l.b200_last_error()
    rc = l.b200_mul_mat_q_noalloc(t, dw.data_ptr(), rb, m, k, dx.data_ptr(), k, n, out.data_ptr(), m, st)
    assert rc == 0, l.b200_noalloc_last_error()
    torch.cuda.synchronize()
    return ref.cpu().numpy(), out.cpu().numpy()


def test_noalloc_matches_regular_entry_point_twice(b200, oracle, golden):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    # first call: Q4_K, 5 columns; second call: Q6_K, 1 column of a different length -> other scratch contents
    for qt, n, reps in (("q4_K", 5, 4), ("q6_K", 1, 8)):
        w = np.ascontiguousarray(np.tile(golden[f"mul_mat.w.{qt}"], (3, reps)))           # [96, row_size(512*reps)]
        x = rng.standard_normal((n, 512 * reps)).astype(np.float32)
        ref, out = run_pair(b200, torch, qt, w, x)
        assert np.isfinite(out).all()
        assert oracle.nmse(ref, out) <= 5e-4                     # the tolerance of the MUL_MAT parity tests
        assert np.array_equal(ref, out)                          # same kernels, same inputs: identical bits
        assert oracle.nmse(oracle.mul_mat(qt, w, x), out) <= 5e-4


def test_noalloc_at_the_scratch_limit_and_eight_columns(b200, oracle):
    """8 columns of 104832 values need 1,048,320 of the 1,048,576 scratch bytes; one more activation block per column is refused."""
    torch = pytest.importorskip("torch")
    l = b200.lib()
    rng = np.random.default_rng(1)
    n, m = 8, 16
    for k, fits in ((104832, True), (104960, False)):
        w = oracle.quantize_rows("q8_0", (rng.standard_normal((m, k)) * 0.02).astype(np.float32))
        x = rng.standard_normal((n, k)).astype(np.float32)
        if fits:
            ref, out = run_pair(b200, torch, "q8_0", w, x)
            assert np.array_equal(ref, out)
            assert oracle.nmse(oracle.mul_mat("q8_0", w, x), out) <= 5e-4
        else:
            dw, dx = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
            out = torch.zeros(n, m, device="cuda")
            rc = l.b200_mul_mat_q_noalloc(b200.TYPES["q8_0"], dw.data_ptr(), b200.row_size("q8_0", k), m, k, dx.data_ptr(), k, n, out.data_ptr(), m, None)
            assert rc == -4 and b"scratch" in l.b200_noalloc_last_error()


def test_noalloc_second_call_allocates_nothing_and_status_is_clean(b200, golden):
    torch = pytest.importorskip("torch")
    l = b200.lib()
    w = np.ascontiguousarray(np.tile(golden["mul_mat.w.q4_K"], (3, 4)))
    x = np.random.default_rng(2).standard_normal((2, 2048)).astype(np.float32)
    dw, dx = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    out = torch.zeros(2, w.shape[0], device="cuda")
    args = (b200.TYPES["q4_K"], dw.data_ptr(), b200.row_size("q4_K", 2048), w.shape[0], 2048, dx.data_ptr(), 2048, 2, out.data_ptr(), w.shape[0], None)
    assert l.b200_mul_mat_q_noalloc(*args) == 0           # warm-up: module and kernel variant are materialised here
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert l.b200_mul_mat_q_noalloc(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0          # not a byte of device memory taken by the second call
    assert l.b200_noalloc_status(None) == 0               # no kernel gave up a wait
    # arguments a kernel would fault on come back as B200_E_BAD_ARG without a launch
    bad = list(args); bad[5] = dx.data_ptr() + 2
    assert l.b200_mul_mat_q_noalloc(*bad) == -2
    bad = list(args); bad[6] = 1024
    assert l.b200_mul_mat_q_noalloc(*bad) == -2


def test_noalloc_rejects_oversize(b200):
    torch = pytest.importorskip("torch")
    l = b200.lib()
    buf = torch.zeros(1024, device="cuda")
    big_k = 256 * 4096                                           # 8 columns of 1M values: 10 MiB of activation blocks
    rc = l.b200_mul_mat_q_noalloc(b200.TYPES["q4_K"], buf.data_ptr(), 144 * 4096, 1, big_k, buf.data_ptr(), big_k, 8,
                                  buf.data_ptr(), 1, None)
    assert rc == -4 and b"scratch" in l.b200_noalloc_last_error()
    rc = l.b200_mul_mat_q_noalloc(b200.TYPES["q4_K"], buf.data_ptr(), 144, 1, 256, buf.data_ptr(), 256, 9, buf.data_ptr(), 1, None)
    assert rc == -1
