"""The persistent decode step (one cooperative launch for a whole run of Llama layers, csrc/kernels/decode_step.cu)
against the one-launch-per-node path of the same backend, the reference CPU backend, and through libllama's own graph."""
import os
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
# head size 128 and row lengths that are multiples of 2048 (what the kernel takes); Q4_K_M mixture: Q4_K and Q6_K matrices
ARCH = dict(n_layer=4, n_embd=2048, n_head=16, n_head_kv=4, n_ff=4096, n_vocab=2048, rope_theta=500000.0, rms_eps=1e-5)


def make_model(b200, reg, mega, arch=ARCH, n_ctx=1024, n_ubatch=512, n_threads=8):
    from llama_cpp_b200 import llama, synth
    old = os.environ.get("GGML_B200_MEGA")
    os.environ["GGML_B200_MEGA"] = "1" if mega else "0"          # read when the backend instance is created
    try:
        m = llama.Llama(n_ctx=n_ctx, n_ubatch=n_ubatch, reg=reg, n_threads=n_threads, **arch)
    finally:
        if old is None:
            del os.environ["GGML_B200_MEGA"]
        else:
            os.environ["GGML_B200_MEGA"] = old
    for t in m.tensors():
        m.set_tensor(t["index"], synth.make_tensor(t["type"], t["ne0"], t["ne1"], seed=t["index"], sigma=0.05))
    return m


def run_tokens(m, n_prompt, n_gen, seed=0):
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, m.cfg.n_vocab, n_prompt + n_gen).astype(np.int32)
    outs = [m.decode(toks[:n_prompt], 0).copy()]
    launches = []
    for i in range(n_gen):
        l0 = m.launch_count
        outs.append(m.decode(toks[n_prompt + i:n_prompt + i + 1], n_prompt + i).copy())
        launches.append(m.launch_count - l0)
    return outs, launches


def check_against(oracle, cpu_outs, node_outs, fused_outs):
    """The two device paths use the same int8 activation scheme and the same dot products, but sum in a different
    order; a difference in the last bit flips an int8 rounding now and then, and a random-init network amplifies
    that from layer to layer.  What must hold: the persistent path is as close to the reference CPU backend as the
    per-node path is, and the two device paths are far closer to each other than either is to the CPU."""
    for i, (y, z) in enumerate(zip(node_outs, fused_outs)):
        assert np.isfinite(z).all()
        d_paths = oracle.nmse(y, z)
        if cpu_outs is None:
            assert d_paths <= 5e-3, (i, d_paths)
            continue
        d_node, d_fused = oracle.nmse(cpu_outs[i], y), oracle.nmse(cpu_outs[i], z)
        assert d_fused <= 1.25 * d_node + 1e-4, (i, d_node, d_fused)
        assert d_paths <= 0.25 * d_node + 1e-6, (i, d_node, d_paths)


@pytest.mark.parametrize("n_prompt", [37, 300])        # 2 and 3 KV slices per head
def test_decode_step_matches_per_node_path(b200, oracle, n_prompt):
    per_node = make_model(b200, None, mega=False)
    fused = make_model(b200, None, mega=True)
    cpu = make_model(b200, oracle.ref_cpu_backend_reg(), mega=False) if oracle.ref_available() else None
    try:
        # 8 generated tokens: the first runs directly, the second is captured into a CUDA graph, the rest replay it
        a, la = run_tokens(per_node, n_prompt, 8)
        b, lb = run_tokens(fused, n_prompt, 8)
        c = run_tokens(cpu, n_prompt, 8)[0] if cpu else None
        assert max(lb) <= 8 < min(la), (la, lb)           # the whole run of layers is one launch
        assert np.array_equal(a[0], b[0])                 # the prompt batch takes the same kernels in both
        check_against(oracle, c, a, b)
    finally:
        per_node.close(); fused.close()
        if cpu:
            cpu.close()


def test_decode_step_gqa8(b200, oracle):
    """8 query heads per KV head (two passes over the row tile of the attention phase)."""
    arch = dict(ARCH, n_head=16, n_head_kv=2)
    per_node = make_model(b200, None, mega=False, arch=arch)
    fused = make_model(b200, None, mega=True, arch=arch)
    cpu = make_model(b200, oracle.ref_cpu_backend_reg(), mega=False, arch=arch) if oracle.ref_available() else None
    try:
        a, _ = run_tokens(per_node, 50, 4, seed=3)
        b, lb = run_tokens(fused, 50, 4, seed=3)
        c = run_tokens(cpu, 50, 4, seed=3)[0] if cpu else None
        assert max(lb) <= 8
        check_against(oracle, c, a, b)
    finally:
        per_node.close(); fused.close()
        if cpu:
            cpu.close()


@pytest.mark.parametrize("flash_attn,weight_type", [("1", None), ("0", None), ("1", 2), ("1", 8)])      # None: Q4_K_M mixture; 2 Q4_0; 8 Q8_0
def test_libllama_graph_takes_the_decode_step(tmp_path, b200, flash_attn, weight_type):
    """libllama's own graph (the reference's builder, allocator and scheduler) is recognised: the plugin reports
    persistent launches, and the logits equal those of the per-node path.  With and without FLASH_ATTN_EXT in the graph
    (without it: MUL_MAT / SOFT_MAX / MUL_MAT on a V cache kept transposed, an F32 mask)."""
    if not (REF / "llama-logits").exists():
        pytest.skip("oracle/_ref/llama-logits not built (make -f oracle/ref.mk tools)")
    from llama_cpp_b200 import gguf_synth
    model = tmp_path / "m.gguf"
    gguf_synth.write_llama_gguf(model, ARCH, device="cuda", weight_type=weight_type)
    outs = {}
    for mega in ("0", "1"):
        env = dict(os.environ, GGML_BACKEND_PATH=str(ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so"), GGML_B200_MEGA=mega, GGML_B200_VERBOSE="1")
        out = tmp_path / f"logits{mega}.bin"
        r = subprocess.run([str(REF / "llama-logits"), str(model), str(out), "99", "37", "6", "5", flash_attn], cwd=REF, env=env,
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
        outs[mega] = (np.fromfile(out, dtype=np.float32).reshape(7, -1), r.stderr)
    m = re.findall(r"(\d+) of them persistent decode steps", outs["1"][1])
    assert m and max(int(x) for x in m) >= 5, outs["1"][1][-2000:]
    assert all(int(x) == 0 for x in re.findall(r"(\d+) of them persistent decode steps", outs["0"][1]))
    a, b = outs["0"][0], outs["1"][0]
    assert np.array_equal(a[0], b[0])                     # the prompt batch
    for x, y in zip(a[1:], b[1:]):
        d = float(np.sum((x.astype(np.float64) - y) ** 2) / np.sum(x.astype(np.float64) ** 2))
        assert np.isfinite(y).all() and d <= 5e-3         # same scheme, different summation order (see check_against)
