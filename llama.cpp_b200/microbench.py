#!/usr/bin/env python
"""Per-op timing of the hot-path kernels through the flat C-ABI, cold cache.

The counterpart of the reference's `test-backend-ops perf` (tests/test-backend-ops.cpp:681-693) for the
ops this backend accelerates.  Each case cycles through enough distinct copies of its large operand
(>= 600 MB in total, several times the L2) that every launch reads it from HBM, and is timed with CUDA
events on the launching stream.  Bytes and flops follow the reference's accounting
(tests/test-backend-ops.cpp:1924-1927 for MUL_MAT, :3141-3146 for FLASH_ATTN_EXT).

  python llama.cpp_b200/microbench.py mul_mat --type q4_K -k 4096 -m 14336 -n 1
  python llama.cpp_b200/microbench.py mul_mat --type q4_K -k 4096 -m 14336 -n 512
  python llama.cpp_b200/microbench.py flash_attn --n-kv 32768 --n-q 1
  python llama.cpp_b200/microbench.py sweep          # the projection shapes of Llama-3-8B
  python llama.cpp_b200/microbench.py i8_probe -k 4096                # the int8-MMA-plus-drain form of the GEMM, per 32-deep step
  python llama.cpp_b200/microbench.py load --path m.gguf     # model-file load time (file mapping -> HBM)

`--copies C --reps R` bound the work (for a profiler capture: `--copies 4 --reps 1`).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

QK_TYPES = ("q4_0", "q8_0", "q4_K", "q5_K", "q6_K", "q2_K", "q3_K", "iq4_nl", "iq4_xs")
# byte offsets of the F16 scale fields inside one block of the types filled with random bytes below
_SCALE_FIELDS = {"q2_K": (84, (80, 82)), "q3_K": (110, (108,)), "iq4_nl": (18, (0,)), "iq4_xs": (136, (0,))}


def _weights(pkg, torch, qtype, k, m, copies):
    """`copies` distinct device copies of one synthetic quantized [k x m] weight matrix."""
    from llama_cpp_b200 import synth
    l = pkg.lib()
    t = pkg.TYPES[qtype]
    rb = int(l.b200_row_size(t, k))
    rows = min(m, 4096)
    if qtype in ("q4_K", "q6_K"):
        base = torch.from_numpy(synth.make_tensor(t, k, rows, 1, device="cuda")).cuda()
    elif qtype == "q5_K":       # a Q4_K block with 32 random high-bit bytes spliced in after its 16-byte header
        q4 = torch.from_numpy(synth.make_tensor(pkg.TYPES["q4_K"], k, rows, 1, device="cuda")).cuda().reshape(-1, 144)
        qh = torch.randint(0, 256, (q4.shape[0], 32), dtype=torch.uint8, device="cuda")
        base = torch.cat([q4[:, :16], qh, q4[:, 16:]], 1).reshape(-1)
    elif qtype in _SCALE_FIELDS:   # timing only: random quant bytes, block scales set to small positive F16 numbers
        bb, fields = _SCALE_FIELDS[qtype]
        blk = torch.randint(0, 256, (rows * rb // bb, bb), dtype=torch.uint8, device="cuda")
        for f in fields:
            blk[:, f] = torch.randint(0, 256, (blk.shape[0],), dtype=torch.uint8, device="cuda")
            blk[:, f + 1] = 0x1C        # F16 0x1Cxx: about 4e-3 .. 8e-3
        base = blk.reshape(-1)
    else:                       # Q4_0 / Q8_0 through the device quantizers (CPY F32 -> quantized)
        import numpy as np
        x = (0.02 * torch.randn(rows, k, device="cuda")).cpu().numpy()
        base = torch.from_numpy(pkg.quantize_rows(qtype, x).reshape(-1)).cuda()
    w = torch.empty((copies, rb * m + 256), dtype=torch.uint8, device="cuda")
    for c in range(copies):
        for r0 in range(0, m, 4096):
            n = min(4096, m - r0)
            w[c, r0 * rb:(r0 + n) * rb] = base[:n * rb]
    return w, rb, t


def _time(torch, run, reps, graph=True):
    """Average device milliseconds of run(), replayed from a CUDA graph so host launch cost is excluded."""
    run()
    torch.cuda.synchronize()
    replay = run
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        replay = g.replay
        replay()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def bench_mul_mat(pkg, torch, qtype, k, m, n, copies=None, reps=20, whole=False):
    l = pkg.lib()
    rb = int(l.b200_row_size(pkg.TYPES[qtype], k))
    copies = copies or max(2, int(600e6 // (rb * m)) + 1)
    w, rb, t = _weights(pkg, torch, qtype, k, m, copies)
    x = torch.randn(n, k, device="cuda")
    dst = torch.empty(n, m, device="cuda")
    if n <= 8 and not whole:   # decode: activations quantized once, then the mat-vec kernel alone
        xq = torch.empty(int(l.b200_act_bytes(k, n)), dtype=torch.uint8, device="cuda")
        assert l.b200_quantize_act(x.data_ptr(), k, k, n, xq.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0

        def run():
            s = torch.cuda.current_stream().cuda_stream
            for c in range(copies):
                rc = l.b200_mul_mat_vec_q(t, w[c].data_ptr(), rb, m, k, xq.data_ptr(), n, dst.data_ptr(), m, s)
                assert rc == 0, l.b200_last_error()
        graph = True
    else:               # the whole MUL_MAT as the graph path runs it (activation conversion + the kernel the library picks)
        sb = int(l.b200_mul_mat_q_scratch_bytes(t, m, k, n))
        sc = torch.empty(sb + 256, dtype=torch.uint8, device="cuda")

        def run():
            s = torch.cuda.current_stream().cuda_stream
            for c in range(copies):
                rc = l.b200_mul_mat_q(t, w[c].data_ptr(), rb, m, k, x.data_ptr(), k, n, dst.data_ptr(), m, sc.data_ptr(), sb, s)
                assert rc == 0, l.b200_last_error()
        graph = False
    us = _time(torch, run, reps, graph) * 1e3 / copies
    nbytes = rb * m + 4 * k * n + 4 * m * n
    flops = 2.0 * m * n * k
    print(f"MUL_MAT {qtype:5s} K={k:6d} M={m:7d} N={n:4d}  {us:9.2f} us  {nbytes / us / 1e3:8.1f} GB/s  {flops / us / 1e6:8.1f} TFLOP/s"
          f"  ({copies} copies, {rb * m / 1e6:.1f} MB each)", flush=True)
    return us


def bench_flash_attn(pkg, torch, n_kv, n_q, n_head=32, n_head_kv=8, d=128, copies=None, reps=20, layout="token"):
    l = pkg.lib()
    kv_bytes = 2 * 2 * d * n_kv * n_head_kv
    copies = copies or max(2, int(600e6 // kv_bytes) + 1)
    # cache layout of the reference's KV views: a token's heads are adjacent (nb1 = n_head_kv * d * 2, nb2 = d * 2)
    # (layout "head": each head's rows contiguous, nb1 = d * 2, nb2 = n_kv * d * 2 -- the contiguous tensors of test-backend-ops)
    shape = (copies, n_kv, n_head_kv, d) if layout == "token" else (copies, n_head_kv, n_kv, d)
    kc = torch.randn(*shape, device="cuda").half()
    vc = torch.randn(*shape, device="cuda").half()
    nb1, nb2 = (n_head_kv * d * 2, d * 2) if layout == "token" else (d * 2, n_kv * d * 2)
    q = torch.randn(n_head, n_q, d, device="cuda")
    n_pad = (n_q + 63) // 64 * 64
    mask = torch.full((n_pad, n_kv), float("-inf"), device="cuda", dtype=torch.float16)
    qi = torch.arange(n_q, device="cuda")[:, None]
    ki = torch.arange(n_kv, device="cuda")[None, :]
    mask[:n_q] = torch.where(ki <= n_kv - n_q + qi, 0.0, float("-inf")).half()
    dst = torch.empty(n_q, n_head, d, device="cuda")
    sb = int(l.b200_flash_attn_scratch_bytes(d, n_q, n_head, n_kv))
    sc = torch.empty(sb + 256, dtype=torch.uint8, device="cuda")

    def run():
        s = torch.cuda.current_stream().cuda_stream
        for c in range(copies):
            rc = l.b200_flash_attn(q.data_ptr(), d * 4, n_q * d * 4, kc[c].data_ptr(), nb1, nb2,
                                   vc[c].data_ptr(), nb1, nb2, mask.data_ptr(), n_kv * 2, dst.data_ptr(),
                                   d, n_q, n_head, n_kv, n_head_kv, d ** -0.5, 0.0, 0.0, sc.data_ptr(), sb, s)
            assert rc == 0, l.b200_last_error()
    us = _time(torch, run, reps, graph=n_q <= 8) * 1e3 / copies
    nbytes = kv_bytes + 2 * 4 * d * n_q * n_head + 2 * n_kv * n_q
    flops = 4.0 * n_head * n_q * d * n_kv
    print(f"FLASH_ATTN_EXT D={d} heads {n_head}/{n_head_kv} n_kv={n_kv:6d} n_q={n_q:4d}  {us:9.2f} us  {nbytes / us / 1e3:8.1f} GB/s"
          f"  {flops / us / 1e6:8.1f} TFLOP/s  ({copies} copies, K/V rows by {layout})", flush=True)
    return us


def bench_load(pkg, path, reps=3):
    """Wall time of b200_llama_load_gguf (parse, allocate, copy every tensor to the device) and one decoded token."""
    import time
    import numpy as np
    from llama_cpp_b200 import llama
    size = Path(path).stat().st_size
    for r in range(reps):
        t0 = time.perf_counter()
        m = llama.Llama.from_gguf(path, n_ctx=1024, n_ubatch=512)
        t1 = time.perf_counter()
        logits = m.decode(np.array([1], dtype=np.int32), 0)
        t2 = time.perf_counter()
        assert np.isfinite(logits).all()
        m.close()
        print(f"LOAD {path}  {size / 1e9:.2f} GB  load {t1 - t0:7.3f} s  {size / (t1 - t0) / 1e9:6.2f} GB/s  first token {1e3 * (t2 - t1):7.1f} ms"
              f"  ({'page cache warm' if r else 'first pass'})", flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["mul_mat", "flash_attn", "sweep", "load", "i8_probe"])
    ap.add_argument("--path", default=None, help="load: a Llama-architecture GGUF file (llama.cpp_b200/gguf_synth.py writes one)")
    ap.add_argument("--type", default="q4_K", choices=QK_TYPES)
    ap.add_argument("-k", type=int, default=4096)
    ap.add_argument("-m", type=int, default=14336)
    ap.add_argument("-n", type=int, default=1)
    ap.add_argument("--n-kv", type=int, default=4096)
    ap.add_argument("--n-q", type=int, default=1)
    ap.add_argument("--whole", action="store_true", help="mul_mat with N <= 8: time the whole MUL_MAT entry point (quantization + the kernel the library picks) instead of the mat-vec kernel alone")
    ap.add_argument("--kv-layout", default="token", choices=["token", "head"], help="flash_attn: K/V rows of one token adjacent (the cache views of libllama) or of one head")
    ap.add_argument("--copies", type=int, default=None)
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    pkg = entry.load_package()
    import torch
    if pkg.device_count() < 1:
        raise SystemExit("no sm_100 device visible: these kernels have no CPU fallback")
    if a.op == "i8_probe":
        # the int8 form of the prefill GEMM (one kind::i8 MMA per 32-deep step, drained and scaled in FP32), nothing else
        import ctypes as C
        us, chk, exp = C.c_float(), C.c_float(), C.c_float()
        rc = pkg.lib().b200_tc_i8_probe_host(a.k // 32, a.reps, C.byref(us), C.byref(chk), C.byref(exp))
        if rc != 0:
            raise SystemExit(f"probe failed ({rc}): {pkg.lib().b200_last_error().decode()}")
        steps = a.k // 32
        print(f"kind::i8 128x256x32 + drain: {us.value:.4f} us per 32-deep step ({us.value * 2:.4f} us per 64 values of K; "
              f"{2 * 128 * 256 * 32 / us.value / 1e6:.1f} TFLOP/s per SM-resident CTA x 148), K = {a.k} ({steps} steps), "
              f"element check {chk.value:.3f} (expected {exp.value:.3f})", flush=True)
    elif a.op == "load":
        bench_load(pkg, a.path, reps=min(a.reps, 3))
    elif a.op == "mul_mat":
        bench_mul_mat(pkg, torch, a.type, a.k, a.m, a.n, a.copies, a.reps, whole=a.whole)
    elif a.op == "flash_attn":
        bench_flash_attn(pkg, torch, a.n_kv, a.n_q, copies=a.copies, reps=a.reps, layout=a.kv_layout)
    else:
        shapes = [(4096, 4096), (4096, 14336), (14336, 4096)]
        for n in (1, 8, 32, 128, 512):
            for qt in ("q4_K", "q6_K", "q8_0"):
                for k, m in shapes:
                    bench_mul_mat(pkg, torch, qt, k, m, n, reps=a.reps if n <= 8 else 5)
        for qt in ("q4_K", "q6_K", "q8_0"):
            for n in (1, 512):
                bench_mul_mat(pkg, torch, qt, 4096, 128256, n, copies=2, reps=5)
        bench_mul_mat(pkg, torch, "q4_0", 4096, 4096, 1)
        bench_mul_mat(pkg, torch, "q4_0", 4096, 4096, 512, reps=5)
        for qt in ("q2_K", "q3_K", "iq4_nl", "iq4_xs", "q5_K"):       # types served by the generic kernels
            for n in (1, 512):
                bench_mul_mat(pkg, torch, qt, 4096, 14336, n, reps=a.reps if n == 1 else 5)
        for n_kv in (512, 4096, 32768):
            for n_q in (1, 512):
                bench_flash_attn(pkg, torch, n_kv, n_q, reps=a.reps if n_q == 1 else 5)


if __name__ == "__main__":
    main()
