"""Drop-in check at the application level: the reference's own, unmodified llama-bench + libllama (built by
oracle/ref.mk) load libggml-b200.so through GGML_BACKEND_PATH, offload a synthetic Llama model (written by
llama.cpp_b200/gguf_synth.py) to device B200_0 and run prefill and decode through it."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
TINY = dict(n_layer=4, n_embd=1024, n_head=8, n_head_kv=2, n_ff=2048, n_vocab=2048, rope_theta=500000.0, rms_eps=1e-5)


def run_llama_bench(model, *args, plugin=True, timeout=900):
    if not (REF / "llama-bench").exists():
        pytest.skip("oracle/_ref/llama-bench not built (make -f oracle/ref.mk all)")
    env = dict(os.environ)
    if plugin:
        env["GGML_BACKEND_PATH"] = str(ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so")
    r = subprocess.run([str(REF / "llama-bench"), "-m", str(model), "-o", "json", *args], cwd=REF, env=env, capture_output=True, text=True,
                       timeout=timeout)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return json.loads(r.stdout), r.stderr


def test_reference_llama_bench_runs_on_the_plugin(tmp_path, b200):
    from llama_cpp_b200 import gguf_synth
    model = tmp_path / "tiny.gguf"
    gguf_synth.write_llama_gguf(model, TINY, device="cuda")
    res, log = run_llama_bench(model, "-p", "64", "-n", "16", "-fa", "1", "-ngl", "99", "-r", "2")
    assert len(res) == 2
    for r in res:
        assert "B200" in r["backends"], r
        assert r["n_gpu_layers"] == 99 and r["flash_attn"] and r["avg_ts"] > 0
    # the same file on the reference CPU backend alone (no plugin): the loader and the graph are the reference's own
    cpu, _ = run_llama_bench(model, "-p", "64", "-n", "16", "-fa", "1", "-ngl", "0", "-r", "1", "-t", "4", plugin=False)
    assert all(r["avg_ts"] > 0 for r in cpu)


def run_logits(model, out, ngl, plugin, n_prompt=37, n_gen=6, fa=1):
    if not (REF / "llama-logits").exists():
        pytest.skip("oracle/_ref/llama-logits not built (make -f oracle/ref.mk tools)")
    env = dict(os.environ)
    if plugin:
        env["GGML_BACKEND_PATH"] = str(ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so")
    r = subprocess.run([str(REF / "llama-logits"), str(model), str(out), str(ngl), str(n_prompt), str(n_gen), "5", str(fa)], cwd=REF, env=env,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    import numpy as np
    return np.fromfile(out, dtype=np.float32).reshape(n_gen + 1, -1), r.stderr


@pytest.mark.parametrize("fa", [1, 0])
def test_libllama_logits_plugin_vs_reference_cpu(tmp_path, b200, oracle, fa):
    """libllama itself (loader, graph builder, scheduler: all the reference's) evaluates the same tokens on the
    reference CPU backend and on the plugin; the logits agree within the per-op criterion times the depth.
    fa=1: FLASH_ATTN_EXT; fa=0: llama-bench's default path (K.q and V.p as F16 MUL_MATs, SOFT_MAX, transposed V
    cache).  Six generated tokens: the decode graph runs directly, is captured, and is then replayed."""
    from llama_cpp_b200 import gguf_synth
    model = tmp_path / "tiny.gguf"
    gguf_synth.write_llama_gguf(model, TINY, device="cuda")
    cpu, _ = run_logits(model, tmp_path / "cpu.bin", 0, plugin=False, fa=fa)
    gpu, log = run_logits(model, tmp_path / "gpu.bin", 99, plugin=True, fa=fa)
    assert "B200" in log                                   # the layers were offloaded to the device
    n_mul_mat = 7 * TINY["n_layer"] + 1
    for a, b in zip(cpu, gpu):
        assert oracle.nmse(a, b) <= 5e-4 * n_mul_mat


def test_gguf_loader_and_driver_agree_with_libllama(tmp_path, b200, oracle):
    """The same model file evaluated twice on the B200 kernels: by the reference's libllama (its loader, its graph)
    through the plugin, and by this package's own GGUF loader and graph driver.  Same tokens (std::mt19937 and
    numpy's RandomState are the same generator).  The two graphs are not node for node the same (views, batching,
    which kernel serves an op), so the bound is the per-op criterion of test-backend-ops, 5e-4, once -- not times
    the depth as against the CPU backend; a wrong hyper-parameter, tensor placement or rope convention in the loader
    gives an NMSE near 1."""
    import numpy as np
    from llama_cpp_b200 import gguf_synth, llama
    model = tmp_path / "tiny.gguf"
    gguf_synth.write_llama_gguf(model, TINY, device="cuda")
    n_prompt, n_gen, seed = 37, 6, 5
    ref, log = run_logits(model, tmp_path / "gpu.bin", 99, plugin=True, n_prompt=n_prompt, n_gen=n_gen, fa=1)
    assert "B200" in log
    toks = (np.random.RandomState(seed).randint(0, 2 ** 32, size=n_prompt + n_gen, dtype=np.uint64) % TINY["n_vocab"]).astype(np.int32)
    m = llama.Llama.from_gguf(model, n_ctx=512, n_ubatch=64)
    try:
        mine = [m.decode(toks[:n_prompt], 0).copy()]
        for i in range(n_gen):
            mine.append(m.decode(toks[n_prompt + i:n_prompt + i + 1], n_prompt + i).copy())
    finally:
        m.close()
    for a, b in zip(ref, mine):
        assert oracle.nmse(a, b) <= 5e-4
