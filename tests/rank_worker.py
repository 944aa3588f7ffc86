"""Child process of the multi-rank tests: one rank of a torch.distributed job (RANK / WORLD_SIZE / MASTER_* in the
environment, rendezvous on 127.0.0.1).  Not collected by pytest.

  python tests/rank_worker.py cpu_gather OUT.npy     gloo ranks on CPU: each rank multiplies its row slice of a seeded
                                                     Q8_0 matrix with the CPU oracle, the slices are all-gathered
  python tests/rank_worker.py gpu_llama OUT.npy      one GPU per rank: a small row-split Llama through the B200
                                                     backend (peer stores + barrier kernels); rank 0 saves the logits
"""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

SPLIT_ARCH = dict(n_layer=3, n_embd=1024, n_head=8, n_head_kv=2, n_ff=2048, n_vocab=4096, rope_theta=500000.0, rms_eps=1e-5)
CPU_CASE = dict(k=256, m=1000, n=3, seed=7)        # 1000 rows over 2 ranks: [0, 384) and [384, 1000)


def seeded_tokens(n_vocab, n):
    return np.random.default_rng(0).integers(0, n_vocab, n).astype(np.int32)


def fill(m, pkg):
    """Every rank generates each full tensor from the same seed and uploads its own rows."""
    from llama_cpp_b200 import row_split, synth
    for t in m.tensors():
        full = synth.make_tensor(t["type"], t["ne0"], t["full_rows"], seed=t["index"], sigma=0.05)
        m.set_tensor(t["index"], row_split.slice_rows(full, t["full_rows"], t["row_low"], t["ne1"]))


def run_llama(m, n_prompt=37, n_gen=4):
    toks = seeded_tokens(m.cfg.n_vocab, n_prompt + n_gen)
    outs = [m.decode(toks[:n_prompt], 0).copy()]
    for i in range(n_gen):
        outs.append(m.decode(toks[n_prompt + i:n_prompt + i + 1], n_prompt + i).copy())
    # again from the start: the decode graphs are now replayed from captured CUDA graphs
    outs.append(m.decode(toks[:n_prompt], 0).copy())
    for i in range(n_gen):
        outs.append(m.decode(toks[n_prompt + i:n_prompt + i + 1], n_prompt + i).copy())
    return np.stack(outs)


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    pkg = entry.load_package()
    from llama_cpp_b200 import llama, row_split
    if mode == "cpu_gather":
        dist.init_process_group("gloo", rank=rank, world_size=world)
        orc = entry.load_oracle()
        c = CPU_CASE
        rng = np.random.default_rng(c["seed"])
        w = orc.quantize_rows("q8_0", rng.standard_normal((c["m"], c["k"])).astype(np.float32) * 0.02)
        x = rng.standard_normal((c["n"], c["k"])).astype(np.float32)
        lo, hi = row_split.row_range(c["m"], rank, world)
        mine = row_split.slice_rows(w, c["m"], lo, hi - lo).reshape(hi - lo, -1)
        part = orc.mul_mat("q8_0", mine, x) if hi > lo else np.empty((c["n"], 0), np.float32)
        full = row_split.gather_rows(dist, part, c["m"])
        if rank == 0:
            np.save(out_path, full)
    elif mode == "gpu_llama":
        import torch
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("gloo", rank=rank, world_size=world)     # set-up data only; the data path is peer stores
        m = llama.Llama(n_ctx=512, n_ubatch=64, device_index=local, rank=rank, n_ranks=world, **SPLIT_ARCH)
        fill(m, pkg)
        m.attach_peers(row_split.gather_bytes(dist))
        dist.barrier()
        outs = run_llama(m)
        dist.barrier()
        m.close()
        if rank == 0:
            np.save(out_path, outs)
    else:
        raise SystemExit(f"unknown mode {mode}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
