"""Row-split over ranks: the split rule (C-ABI against its Python mirror and the reference's rule), the slice and
gather logic on two gloo ranks on CPU, and - on a box with two or more B200s - a row-split model through the
backend's peer-store exchange compared with the same model on one GPU."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
WORKER = ROOT / "tests" / "rank_worker.py"


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(world, mode, out_path, timeout=600):
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(WORKER), mode, str(out_path)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()                       # the exact child started above
            o, _ = p.communicate()
        outs.append(o)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"


SHAPES = [4096, 1024, 14336, 128256, 8192, 28672, 1000, 128, 100, 1]


def test_row_range_matches_c_abi_and_reference_rule(b200):
    import ctypes as C
    from llama_cpp_b200 import row_split
    l = b200.lib()
    l.b200_row_split_range.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    l.b200_row_split_range.restype = None
    for n_rows in SHAPES:
        for n in (1, 2, 4, 8):
            prev = 0
            for r in range(n):
                lo, hi = C.c_int64(), C.c_int64()
                l.b200_row_split_range(n_rows, r, n, C.byref(lo), C.byref(hi))
                assert (lo.value, hi.value) == row_split.row_range(n_rows, r, n)
                # get_row_split (ggml-cuda.cu:725-742) with tensor_split[r] = r / n and rounding 128
                exp_lo = 0 if r == 0 else int(n_rows * (r / n)) // 128 * 128
                exp_hi = n_rows if r == n - 1 else int(n_rows * ((r + 1) / n)) // 128 * 128
                assert (lo.value, hi.value) == (exp_lo, exp_hi)
                assert lo.value == prev and hi.value >= lo.value     # ranges tile [0, n_rows) in rank order
                prev = hi.value
            assert prev == n_rows


def test_slice_rows():
    from llama_cpp_b200 import row_split
    data = np.arange(10 * 6, dtype=np.uint8)
    assert row_split.slice_rows(data, 10, 3, 4).tolist() == list(range(18, 42))
    assert row_split.slice_rows(data, 10, 5, 0).size == 0            # a rank with an empty range
    with pytest.raises(ValueError):
        row_split.slice_rows(data[:-1], 10, 0, 1)


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_gather_equals_unsplit(tmp_path, oracle, world):
    """1000 rows over 2 ranks ([0, 384), [384, 1000)) and over 4 ([0, 128), [128, 384), [384, 640), [640, 1000))."""
    sys.path.insert(0, str(ROOT / "tests"))
    import rank_worker as w
    out = tmp_path / "gathered.npy"
    run_ranks(world, "cpu_gather", out, timeout=300)
    c = w.CPU_CASE
    rng = np.random.default_rng(c["seed"])
    wq = oracle.quantize_rows("q8_0", rng.standard_normal((c["m"], c["k"])).astype(np.float32) * 0.02)
    x = rng.standard_normal((c["n"], c["k"])).astype(np.float32)
    full = oracle.mul_mat("q8_0", wq, x)
    assert np.array_equal(np.load(out), full)                         # row results do not depend on who computed them


@pytest.mark.gpu
def test_row_split_two_gpus_matches_one_gpu(tmp_path, b200, oracle, monkeypatch):
    if b200.device_count() < 2:
        pytest.skip("needs two B200s")
    # Both runs on the one-launch-per-node path with K undivided, so that every output row is computed by the same kernel
    # with the same order of sums whether its matrix is whole or one rank's slice (the persistent decode step does not take
    # row-split graphs, and the tile plan of the tensor-core GEMM depends on the row count).
    monkeypatch.setenv("GGML_B200_MEGA", "0")
    monkeypatch.setenv("GGML_B200_TC_NO_SPLIT", "1")
    sys.path.insert(0, str(ROOT / "tests"))
    import rank_worker as w
    from llama_cpp_b200 import llama
    out = tmp_path / "split.npy"
    run_ranks(2, "gpu_llama", out)
    split = np.load(out)
    m = llama.Llama(n_ctx=512, n_ubatch=64, **w.SPLIT_ARCH)
    try:
        w.fill(m, b200)
        single = w.run_llama(m)
    finally:
        m.close()
    assert split.shape == single.shape and np.isfinite(split).all()
    for a, b in zip(split, single):
        assert oracle.nmse(b, a) <= 1e-6                               # same kernels, same per-row arithmetic


@pytest.mark.gpu
def test_barrier_wait_runs_out_and_the_context_stays_usable(b200, oracle, golden):
    """Failure detection without a fault: the cross-GPU barrier kernel as rank 0 of 2 on one GPU, its peer's flag never
    written.  The bounded wait gives up after the (test-size) limit, the status word says ERR_PEER_TIMEOUT, the kernel
    returns; afterwards the same context computes a MUL_MAT correctly and a barrier whose peer has arrived passes."""
    import ctypes as C
    l = b200.lib()
    st = C.c_int(-1)
    assert l.b200_peer_barrier_probe_host(2000, 0, C.byref(st)) == 0, l.b200_last_error()
    assert st.value == 3                                         # ERR_PEER_TIMEOUT
    got = b200.mul_mat_q("q4_K", golden["mul_mat.w.q4_K"], golden["mul_mat.x"])
    assert oracle.nmse(oracle.mul_mat("q4_K", golden["mul_mat.w.q4_K"], golden["mul_mat.x"]), got) <= 5e-4
    assert l.b200_peer_barrier_probe_host(2000, 1, C.byref(st)) == 0 and st.value == 0
