#!/usr/bin/env python
"""Benchmark: Llama-3-8B architecture, Q4_K_M, pp512 + tg128 per step, through the B200 ggml backend.

One step = what one repetition of the reference's llama-bench does (examples/llama-bench/llama-bench.cpp:
1430-1468): a 512-token prompt evaluated as one batch at an empty KV cache, then 128 single-token decodes
(here they continue from the prompt, i.e. at KV positions 512..639; llama-bench's own tg test starts from an
empty cache).  Weights are random-init (seeded N(0, 0.02), quantized to the Q4_K_M tensor-type mixture); token
ids are uniform random, as llama-bench feeds them.  The model (4.6 GB of weights) is far larger than L2, so
every timed token re-reads it from HBM; no L2 flush is needed.

  value      tg128 tokens/s from the device time of graph_compute (CUDA events on the backend's stream;
             inputs already resident), summed over the 128 decodes of each timed step
  e2e        the same tokens/s by host clock around the driver's decode call: token ids and mask copied
             host->device, logits copied device->host, every token
  roofline   the persistent decode-step kernel (one launch per token): weight bytes + attended K/V bytes of a
             token over the CUDA-event time of the token's graph, against the measured HBM copy bandwidth
  llama_bench  the reference's own, unmodified llama-bench + libllama driving the plugin on the same
             architecture (a GGUF written by llama.cpp_b200/gguf_synth.py): the number a user of the drop-in gets
  cpu_baseline  the reference's ggml CPU backend (oracle/_ref) running the same graph on the same weights
             on a bounded sample (pp128 + tg16), one thread per physical core

`--impl reference` runs the stock reference path alone: oracle/_ref/llama-bench -ngl 0 (the reference's CPU
backend, its own graph builder and scheduler) at pp512 + tg128 on a GGUF of the same architecture, one thread
per physical core; it neither loads this repository's library nor touches a GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

N_PROMPT, N_GEN = 512, 128
LLAMA3_8B = dict(n_layer=32, n_embd=4096, n_head=32, n_head_kv=8, n_ff=14336, n_vocab=128256, rope_theta=500000.0, rms_eps=1e-5)
LLAMA3_70B = dict(n_layer=80, n_embd=8192, n_head=64, n_head_kv=8, n_ff=28672, n_vocab=128256, rope_theta=500000.0, rms_eps=1e-5)
CPU_PROMPT, CPU_GEN = 128, 16
# DRAM bytes moved per algorithmic byte by the decode-step kernel, from an ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum) of an 8-layer model with the same layer shapes; traffic grows with the number of layers
DRAM_TRAFFIC_RATIO = 1.0247       # 1,531,302,400 DRAM bytes for 1,494,425,600 algorithmic ones
METRIC = "llama3-8b-q4_k_m tg128 tokens/s (pp512+tg128 per step)"   # --model 70b replaces the model name


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def physical_cores() -> int:
    """Cores x sockets as lscpu reports them (hyper-threads do not count); falls back to the logical CPU count."""
    try:
        out = subprocess.run(["lscpu"], capture_output=True, text=True, timeout=10).stdout
        f = {l.split(":")[0].strip(): l.split(":")[1].strip() for l in out.splitlines() if ":" in l}
        n = int(f["Core(s) per socket"]) * int(f["Socket(s)"])
        if n > 0:
            return min(n, os.cpu_count() or n)
    except Exception:
        pass
    return os.cpu_count() or 1


REF_DIR = ROOT / "oracle" / "_ref"


def synth_gguf(arch_name: str, arch: dict, device: str, share_layers: bool) -> Path:
    """The synthetic model as a GGUF file under the system's temporary directory (written once per machine)."""
    import tempfile
    from llama_cpp_b200 import gguf_synth
    path = Path(tempfile.gettempdir()) / f"b200-bench-llama3-{arch_name}-q4_k_m{'-shared' if share_layers else ''}.gguf"
    if not path.exists():
        t0 = time.time()
        tmp = path.with_suffix(".part")
        n = gguf_synth.write_llama_gguf(tmp, arch, device=device, share_layers=share_layers)
        tmp.rename(path)
        log(f"[bench] wrote {path} ({n / 1e9:.2f} GB) in {time.time() - t0:.1f} s")
    return path


def run_llama_bench(gguf: Path, n_prompt: int, n_gen: int, reps: int, keep: int, plugin: bool, threads: int):
    """The reference's llama-bench (built unmodified by oracle/ref.mk).  Runs `reps` repetitions after llama-bench's own
    warm-up run and averages the last `keep`.  Returns {"pp": tokens/s, "tg": tokens/s} or raises."""
    exe = REF_DIR / "llama-bench"
    if not exe.exists():
        raise RuntimeError("oracle/_ref/llama-bench is not built (make -f oracle/ref.mk all)")
    env = {k: v for k, v in os.environ.items() if k != "GGML_BACKEND_PATH"}
    cmd = [str(exe), "-m", str(gguf), "-p", str(n_prompt), "-n", str(n_gen), "-fa", "1", "-r", str(reps), "-o", "json"]
    if plugin:
        env["GGML_BACKEND_PATH"] = str(ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so")
        cmd += ["-ngl", "99"]
    else:
        cmd += ["-ngl", "0", "-t", str(threads)]
    r = subprocess.run(cmd, cwd=REF_DIR, env=env, capture_output=True, text=True, timeout=3000)
    if r.returncode != 0:
        raise RuntimeError(f"llama-bench failed: {(r.stdout + r.stderr)[-500:]}")
    out = {}
    for t in json.loads(r.stdout):
        ts = t["samples_ts"][-keep:]
        out["pp" if t["n_prompt"] else "tg"] = float(np.mean(ts))
        out["backends"] = t.get("backends")
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def fill_weights(models, device):
    """Random-init weights, generated once per tensor and handed to every model as host bytes.  A row-split
    model (models[0] on rank r of n) takes its rows of the same full tensor every rank generates."""
    from llama_cpp_b200 import row_split, synth
    t0 = time.time()
    total = 0
    infos = [m.tensors() for m in models]
    for i, t in enumerate(infos[0]):
        data = synth.make_tensor(t["type"], t["ne0"], t["full_rows"], seed=1000 + t["index"], device=device)
        for m, info in zip(models, infos):
            ti = info[i]
            m.set_tensor(ti["index"], row_split.slice_rows(data, ti["full_rows"], ti["row_low"], ti["ne1"]))
        total += data.size
    log(f"[bench] weights: {total / 1e9:.2f} GB generated and uploaded in {time.time() - t0:.1f} s")


def run_step(m, tokens, n_prompt, n_gen):
    """pp + tg pass; returns (pp_wall_s, tg_wall_s, pp_dev_ms, tg_dev_ms)."""
    t0 = time.perf_counter()
    m.decode(tokens[:n_prompt], 0)
    t1 = time.perf_counter()
    pp_dev = m.last_compute_ms
    tg_dev = 0.0
    for i in range(n_gen):
        m.decode(tokens[n_prompt + i:n_prompt + i + 1], n_prompt + i)
        tg_dev += m.last_compute_ms
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1, pp_dev, tg_dev


def io_bytes_per_step(n_prompt, n_gen, n_vocab):
    h2d = d2h = 0
    for n_tok, pos0 in [(n_prompt, 0)] + [(1, n_prompt + i) for i in range(n_gen)]:
        n_kv = (pos0 + n_tok + 255) // 256 * 256
        n_pad = (n_tok + 63) // 64 * 64
        h2d += n_tok * 4 * 2 + n_kv * n_pad * 4 + 4
        d2h += n_vocab * 4
    return h2d, d2h


def gemv_roofline(pkg, m, torch):
    """Times the decode mat-vec kernel over every weight matrix of the model, in graph order, with CUDA events."""
    l = pkg.lib()
    mats = [t for t in m.tensors() if t["type"] != 0 and t["name"] != "token_embd.weight"]
    order = sorted(mats, key=lambda t: (t["name"] == "output.weight", t["index"]))
    kmax = max(t["ne0"] for t in order)
    x = torch.randn(kmax, device="cuda", dtype=torch.float32)
    xq = {k: torch.empty(int(l.b200_act_bytes(k, 1)), device="cuda", dtype=torch.uint8) for k in {t["ne0"] for t in order}}
    dst = torch.empty(max(t["ne1"] for t in order), device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    for k, buf in xq.items():
        assert l.b200_quantize_act(x.data_ptr(), k, k, 1, buf.data_ptr(), stream) == 0
    algo = 0
    # as inside the backend's graphs: each kernel's first weight loads overlap its predecessor's tail
    l.b200_set_dependent_launch.argtypes = [C.c_int]
    l.b200_set_dependent_launch.restype = None
    l.b200_set_dependent_launch(1)

    def one_pass():
        nonlocal algo
        algo = 0
        st = torch.cuda.current_stream().cuda_stream
        for t in order:
            rb = t["nbytes"] // t["ne1"]
            rc = l.b200_mul_mat_vec_q(t["type"], m.tensor_data(t["index"]), rb, t["ne1"], t["ne0"], xq[t["ne0"]].data_ptr(), 1,
                                      dst.data_ptr(), t["ne1"], st)
            assert rc == 0, l.b200_last_error()
            algo += t["nbytes"] + 4 * t["ne0"] + 4 * t["ne1"]        # weights + F32 activations in + F32 out
    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    # the launches of one pass are captured into a CUDA graph so that the host's launch cost
    # (a Python call per kernel) does not sit between kernels while they are being timed
    replay = one_pass
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_pass()
        replay = g.replay
        replay(); torch.cuda.synchronize()
    except Exception as e:
        log(f"[bench] CUDA graph capture of the mat-vec pass failed ({e}); timing direct launches")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    l.b200_set_dependent_launch(0)
    return algo, ms, len(order)


def cpu_model(arch, n_threads):
    from llama_cpp_b200 import llama
    orc = entry.load_oracle()
    if not orc.ref_available():
        raise RuntimeError("oracle/_ref (the reference CPU backend) is not built")
    return llama.Llama(n_ctx=256, n_ubatch=CPU_PROMPT, reg=orc.ref_cpu_backend_reg(), n_threads=n_threads, **arch)


def time_cpu(m, tokens, steps, warmup):
    """Bounded sample on the reference CPU backend: pp128 + tg16 per step."""
    for _ in range(warmup):
        m.decode(tokens[:8], 0, want_logits=False)
        m.decode(tokens[8:9], 8, want_logits=False)
    pp_s = tg_s = 0.0
    for _ in range(steps):
        pp, tg, _, _ = run_step(m, tokens, CPU_PROMPT, CPU_GEN)
        pp_s += pp; tg_s += tg
    return steps * CPU_PROMPT / pp_s, steps * CPU_GEN / tg_s, (pp_s + tg_s) / steps


def emit(line: str):
    """The one JSON line goes to the process's original stdout; everything else any library prints
    (NCCL's version banner, for one) was redirected to stderr at start-up."""
    os.write(_REAL_STDOUT, (line + "\n").encode())


_REAL_STDOUT = 1


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--n-prompt", type=int, default=512, help="prompt tokens per step (smaller only for profiler captures)")
    ap.add_argument("--n-gen", type=int, default=128, help="generated tokens per step (smaller only for profiler captures)")
    ap.add_argument("--no-roofline", action="store_true", help="skip the separate per-op mat-vec pass (profiler captures)")
    ap.add_argument("--no-llama-bench", action="store_true", help="skip the run of the reference's llama-bench on the plugin")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (profiler captures only; the line says so)")
    ap.add_argument("--model", default="8b", choices=["8b", "70b"],
                    help="8b: the configuration the metric is quoted on; 70b: the row-split parity configuration (no CPU baseline)")
    args = ap.parse_args()
    global N_PROMPT, N_GEN
    N_PROMPT, N_GEN = args.n_prompt, args.n_gen

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    arch = dict(LLAMA3_8B if args.model == "8b" else LLAMA3_70B)
    if args.layers > 0:
        arch["n_layer"] = args.layers
    cores = physical_cores()
    rng = np.random.default_rng(1234)
    tokens = rng.integers(0, arch["n_vocab"], N_PROMPT + N_GEN).astype(np.int32)
    config = {"workload": f"llama3-{args.model}-arch q4_k_m pp512+tg128, random-init weights, uniform-random token ids", "n_prompt": N_PROMPT, "n_gen": N_GEN,
              "flash_attn": True, "kv_type": "f16", "l2": "every token re-reads all weights (4.6 GB for 8b, 42 GB for 70b) >> L2, no flush needed"}
    if args.layers > 0:
        config["layers_cut_to"] = args.layers          # not the benchmark configuration: a profiler capture

    if args.impl == "reference":
        if rank != 0:
            return
        entry.load_package()                           # the Python package only (synthetic weights, GGUF writer): the CUDA library is never opened here
        try:
            gguf = synth_gguf(args.model, arch, "cpu", share_layers=True)
            warm = max(args.warmup, 1)
            t0 = time.perf_counter()
            res = run_llama_bench(gguf, N_PROMPT, N_GEN, reps=args.steps + warm - 1, keep=args.steps, plugin=False, threads=cores)
            wall = time.perf_counter() - t0
        except Exception as e:
            emit(json.dumps({"impl": "reference", "unavailable": f"the reference's llama-bench could not be run here: {e}"[:300]}))
            return
        sample = (f"oracle/_ref/llama-bench -ngl 0 -fa 1 -t {cores} -p {N_PROMPT} -n {N_GEN}: the reference's CPU backend, {cores} threads "
                  f"(one per physical core), last {args.steps} of {args.steps + warm - 1} repetitions after llama-bench's own warm-up run; "
                  "synthetic GGUF of the same architecture whose layers share one set of random weights")
        emit(json.dumps({"impl": "reference", "metric": METRIC.replace("8b", args.model), "value": res["tg"], "unit": "tokens/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": warm, "ms_per_step": (N_PROMPT / res["pp"] + N_GEN / res["tg"]) * 1e3,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int4/6 dot, f32 accumulate",
                          "data": "synthetic", "config": config, "pp512_tokens_per_s": res["pp"], "tg128_tokens_per_s": res["tg"], "wall_s": wall,
                          "cpu_baseline": {"value": res["tg"], "unit": "tokens/s", "cores": cores, "kind": "reference", "sample": sample},
                          "e2e": {"value": res["tg"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    pkg = entry.load_package()   # registers the package under the alias llama_cpp_b200
    from llama_cpp_b200 import llama
    import torch
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if pkg.device_count() <= local:
        raise SystemExit("no sm_100 device visible for this rank: the B200 path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        # one process per GPU; NCCL carries set-up data and the timing reductions, the row-split exchange itself
        # is done by the backend's kernels with stores into peer memory
        import torch.distributed as dist
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
        config["parallelism"] = f"row-split x{world} (weight rows over ranks, peer stores + barrier per MUL_MAT group)"

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if dist is None:
            return list(vals)
        t = torch.tensor(vals, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    m = llama.Llama(n_ctx=1024, n_ubatch=N_PROMPT, device_index=local, rank=rank, n_ranks=world, **arch)
    cpu = None
    if not args.no_cpu_baseline and rank == 0 and world == 1 and args.model == "8b":
        try:
            cpu = cpu_model(arch, cores)
        except Exception as e:  # the baseline is reported, never required for the GPU number
            log(f"[bench] cpu baseline unavailable: {e}")
    fill_weights([m] + ([cpu] if cpu else []), "cuda")
    if dist is not None:
        from llama_cpp_b200 import row_split
        m.attach_peers(row_split.gather_bytes(dist))

    sync_all()
    for _ in range(max(args.warmup, 3)):
        run_step(m, tokens, N_PROMPT, N_GEN)
    sync_all()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = m.launch_count
    pp_wall = tg_wall = pp_dev = tg_dev = 0.0
    t_start = time.perf_counter()
    for _ in range(args.steps):
        a, b, c, d = run_step(m, tokens, N_PROMPT, N_GEN)
        pp_wall += a; tg_wall += b; pp_dev += c; tg_dev += d
    sync_all()
    wall = time.perf_counter() - t_start
    clocks = sampler.stop()
    launches = m.launch_count - launches0
    # the slowest rank sets the job's time (device times by CUDA events on each rank's stream)
    pp_wall, tg_wall, pp_dev, tg_dev, wall = max_over_ranks(pp_wall, tg_wall, pp_dev, tg_dev, wall)
    l_a = m.launch_count
    m.decode(tokens[N_PROMPT:N_PROMPT + 1], N_PROMPT, want_logits=False)
    launches_per_token = m.launch_count - l_a
    nodes_per_token = m.last_n_nodes
    logits = m.decode(tokens[:8], 0).copy()
    assert np.isfinite(logits).all(), "non-finite logits"

    n_tg, n_pp = args.steps * N_GEN, args.steps * N_PROMPT
    tg_tps_dev, pp_tps_dev = n_tg / (tg_dev / 1e3), n_pp / (pp_dev / 1e3)
    tg_tps_e2e, pp_tps_e2e = n_tg / tg_wall, n_pp / pp_wall
    h2d, d2h = io_bytes_per_step(N_PROMPT, N_GEN, arch["n_vocab"])

    if rank != 0:                 # rank 0 reports; the others wait for it to finish the single-GPU roofline pass
        sync_all()
        m.close()
        dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    # The dominant kernel is the persistent decode step: one launch per token that reads every weight matrix once and
    # the attended part of the KV cache.  Its duration is the CUDA-event time of the token's graph on the backend's
    # stream (the graph also holds the token's embedding-row gather and the mask cast: two launches, < 1 % of the time).
    n_embd_kv = arch["n_embd"] // arch["n_head"] * arch["n_head_kv"]
    kv_bytes = sum(2 * 2 * n_embd_kv * (N_PROMPT + i + 1) for i in range(N_GEN)) / N_GEN * arch["n_layer"]     # K and V rows up to the token, F16
    bytes_per_token = m.weight_bytes + kv_bytes
    ms_per_token = tg_dev / n_tg
    achieved = bytes_per_token / (ms_per_token / 1e3) / 1e9
    persistent = launches_per_token <= 16
    roofline = {"bound": "hbm",
                "kernel": ("decode_step_kernel (one persistent launch per token: all layers' mat-vecs, norms, rope, KV store, attention)" if persistent
                           else "the token's graph of per-op kernels (mmvq_*, fattn_dec, glue)"),
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "traffic": bytes_per_token * DRAM_TRAFFIC_RATIO if persistent else None,
                "traffic_unit": "DRAM bytes per launch (ncu capture of an 8-layer model of the same layer shapes, scaled by layers)",
                "bytes_per_launch": bytes_per_token, "weight_bytes_per_token": m.weight_bytes, "kv_bytes_per_token": kv_bytes,
                "us_per_launch": ms_per_token * 1e3, "launches_per_token": launches_per_token,
                "whole_decode_step": {"weight_bytes_per_token_per_gpu": m.weight_bytes, "achieved_gbs_per_gpu": m.weight_bytes * tg_tps_dev / 1e9,
                                      "frac": m.weight_bytes * tg_tps_dev / 1e9 / peak}}
    if not args.no_roofline:
        algo, gemv_ms, n_mats = gemv_roofline(pkg, m, torch)
        roofline["per_op_mat_vec_kernels"] = {"what": "the one-kernel-per-op decode mat-vec (mmvq_k / mmvq_q6k), every weight matrix in graph order, cold L2",
                                              "achieved": algo / (gemv_ms / 1e3) / 1e9, "frac": algo / (gemv_ms / 1e3) / 1e9 / peak,
                                              "launches_per_pass": n_mats, "ms_per_pass": gemv_ms}
    # the drop-in path: the reference's own llama-bench + libllama on the plugin, same architecture
    llama_bench = None
    if world == 1 and args.model == "8b" and not args.no_llama_bench:
        try:
            gguf = synth_gguf(args.model, arch, "cuda", share_layers=False)
            lb = run_llama_bench(gguf, N_PROMPT, N_GEN, reps=3, keep=3, plugin=True, threads=cores)
            llama_bench = {"pp512_tokens_per_s": lb["pp"], "tg128_tokens_per_s": lb["tg"], "backends": lb.get("backends"),
                           "command": "oracle/_ref/llama-bench -p 512 -n 128 -fa 1 -ngl 99 -r 3 with GGML_BACKEND_PATH=libggml-b200.so"}
        except Exception as e:
            log(f"[bench] llama-bench through the plugin unavailable: {e}")
    cpu_baseline = None
    if cpu is not None:
        c_pp, c_tg, _ = time_cpu(cpu, tokens, 1, 1)
        # parity on the same weights and tokens: logits of an 8-token prompt
        ref_logits = cpu.decode(tokens[:8], 0).copy()
        den = float(np.sum(ref_logits.astype(np.float64) ** 2))
        nmse = float(np.sum((ref_logits.astype(np.float64) - logits) ** 2)) / den
        cpu_baseline = {"value": c_tg, "unit": "tokens/s", "cores": cores, "kind": "reference",
                        "sample": f"pp{CPU_PROMPT}+tg{CPU_GEN} on the reference ggml CPU backend, {cores} threads",
                        "pp_tokens_per_s": c_pp, "logits_nmse_vs_b200": nmse}
        cpu.close()
    out = {"metric": METRIC.replace("8b", args.model), "value": tg_tps_dev, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
           "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "int8 x int4/6 dot, f32 accumulate", "data": "synthetic", "config": config,
           "pp512_tokens_per_s": pp_tps_dev, "tg128_tokens_per_s": tg_tps_dev,
           "e2e": {"value": tg_tps_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "pp512_tokens_per_s": pp_tps_e2e},
           "gpu_launches": launches * world, "launches_per_token": launches_per_token, "graph_nodes_per_token": nodes_per_token, "clocks": clocks,
           "roofline": roofline, "llama_bench": llama_bench, "cpu_baseline": cpu_baseline}
    if dist is not None:
        sync_all()
    m.close()
    if dist is not None:
        dist.destroy_process_group()
    emit(json.dumps(out))


if __name__ == "__main__":
    main()
