"""The in-process row-split buffer type (csrc/host/split.cpp; ggml_backend_split_buffer_type by name, what libllama
asks a device registry for in split-mode row: src/llama-model.cpp:304-326) through the reference's own API: the
graph-cases tool for the buffer type and MUL_MAT, the reference's libllama (llama-logits) and llama-bench with
`-sm row` for whole models.  With one GPU all rows land on it (the code path is the same: per-tensor slices, scatter /
gather, the sliced MUL_MAT); with two or more the rows are divided and the second half of the layers has the other
GPU as main device."""
import json
import os
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
LIB = ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so"
NMSE = 5e-4          # tests/test-backend-ops.cpp:1916-1918 (MUL_MAT)
ARCH = dict(n_layer=4, n_embd=2048, n_head=16, n_head_kv=4, n_ff=4096, n_vocab=2048, rope_theta=500000.0, rms_eps=1e-5)


def n_gpus():
    import torch
    return torch.cuda.device_count()


def test_split_buffer_round_trip_and_mul_mat():
    """Scatter / gather of the weight bytes is the identity, and MUL_MAT on split weights equals the reference CPU
    backend for Q4_K, Q6_K, Q8_0 and F16 at N in {1, 8, 64, 512}, equal and 3:1:1... splits, row counts that are and are
    not multiples of the 128-row rounding."""
    exe = REF / "graph-cases"
    if not exe.exists():
        pytest.skip("oracle/_ref/graph-cases not built (make -f oracle/ref.mk tools)")
    env = dict(os.environ, GGML_BACKEND_PATH=str(LIB))
    r = subprocess.run([str(exe), "B200_0", "split", str(os.cpu_count() or 8)], cwd=REF, env=env, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "SPLIT unavailable" not in r.stdout and "NONFINITE" not in r.stdout, r.stdout[-2000:]
    m = re.search(r"SPLIT devices=(\d+) main=(\d+)", r.stdout)
    assert m and int(m.group(1)) == n_gpus()
    assert re.search(r"SPLIT buffer type B200_0_Split", r.stdout)
    trips = re.findall(r"ROUNDTRIP w (\w+)", r.stdout)
    assert trips and all(t == "identical" for t in trips), r.stdout[-2000:]
    cases = {m.group(1): float(m.group(2)) for m in re.finditer(r"CASE (\S+) nmse=(\S+)", r.stdout)}
    assert len(cases) == 2 * 4 * 4, sorted(cases)
    bad = {k: v for k, v in cases.items() if v > NMSE}
    assert not bad, bad


def logits(tmp_path, model, tag, split_mode, visible=None):
    env = dict(os.environ, GGML_BACKEND_PATH=str(LIB), GGML_B200_VERBOSE="1")
    if visible is not None:
        env["CUDA_VISIBLE_DEVICES"] = visible
    out = tmp_path / f"logits_{tag}.bin"
    r = subprocess.run([str(REF / "llama-logits"), str(model), str(out), "99", "37", "6", "5", "1", split_mode], cwd=REF, env=env,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return np.fromfile(out, dtype=np.float32).reshape(7, -1), r.stderr


def nmse(a, b):
    a = a.astype(np.float64)
    return float(np.sum((a - b) ** 2) / np.sum(a ** 2))


def test_libllama_split_mode_row(tmp_path, b200):
    """libllama with split_mode = row places the layer matrices in the split buffer type of the plugin and its logits
    are those of the unsplit run (prompt batch and six generated tokens)."""
    if not (REF / "llama-logits").exists():
        pytest.skip("oracle/_ref/llama-logits not built (make -f oracle/ref.mk tools)")
    from llama_cpp_b200 import gguf_synth
    model = tmp_path / "m.gguf"
    gguf_synth.write_llama_gguf(model, ARCH, device="cuda")
    base, _ = logits(tmp_path, model, "none", "none", visible="0")
    row, err = logits(tmp_path, model, "row", "row")
    assert re.search(r"B200_\d_Split model buffer size", err), err[-3000:]
    assert np.isfinite(row).all()
    # same kernels on the same rows of the same matrices; the split path does not group mat-vecs that share an input,
    # which changes the order of a few sums (see tests/test_decode_step_gpu.py on how a random-init network amplifies that)
    for i, (x, y) in enumerate(zip(base, row)):
        assert nmse(x, y) <= 5e-3, (i, nmse(x, y))
    if n_gpus() >= 2:
        assert re.search(r"B200_1_Split model buffer size", err), err[-3000:]


def test_llama_bench_split_mode_row(tmp_path, b200):
    """The reference's llama-bench runs `-sm row -ngl 99` through the plugin and reports the split mode it used."""
    if not (REF / "llama-bench").exists():
        pytest.skip("oracle/_ref/llama-bench not built (make -f oracle/ref.mk tools)")
    from llama_cpp_b200 import gguf_synth
    model = tmp_path / "m.gguf"
    gguf_synth.write_llama_gguf(model, ARCH, device="cuda")
    env = dict(os.environ, GGML_BACKEND_PATH=str(LIB))
    r = subprocess.run([str(REF / "llama-bench"), "-m", str(model), "-p", "64", "-n", "8", "-ngl", "99", "-fa", "1", "-sm", "row", "-r", "1", "-o", "json"],
                       cwd=REF, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    rows = json.loads(r.stdout)
    assert len(rows) == 2 and all(x["split_mode"] == "row" and x["avg_ts"] > 0 for x in rows), rows
    assert all("B200" in x["backends"] for x in rows)
