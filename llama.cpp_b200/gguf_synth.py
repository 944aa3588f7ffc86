#!/usr/bin/env python
"""Writes a synthetic Llama-architecture model as a GGUF file the unmodified reference can load.

The file format is GGUF version 3 (ggml/include/gguf.h:41-46 and the layout comment at its top: header, key/value
metadata, tensor infos, padding to `general.alignment` = 32, tensor data).  Weights are random-init (seeded
N(0, 0.02)), already quantized to the reference's Q4_K_M tensor-type mixture (src/llama-quant.cpp:129-131, 235-243,
291-298) by this package's own quantizers, i.e. the same bytes `bench.py` feeds through the C-ABI driver.  The
tokenizer section says `no_vocab`, which makes libllama create `<arch>.vocab_size` dummy tokens
(src/llama-vocab.cpp:1350-1368): all that llama-bench, which feeds random token ids, needs.

    python llama.cpp_b200/gguf_synth.py llama3-8b-q4_k_m.gguf --model 8b
    GGML_BACKEND_PATH=llama.cpp_b200/lib/libggml-b200.so oracle/_ref/llama-bench -m /tmp/llama3-8b-q4_k_m.gguf \
        -p 512 -n 128 -fa 1 -ngl 99
"""
from __future__ import annotations

import argparse
import struct
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ALIGN = 32
T_F32, T_Q4_0, T_Q8_0, T_Q4_K, T_Q5_K, T_Q6_K = 0, 2, 8, 12, 13, 14
# gguf_type ids (ggml/include/gguf.h:53-68)
G_U32, G_F32, G_STR = 4, 6, 8


def use_more_bits(il: int, n: int) -> bool:        # src/llama-quant.cpp:129-131
    return il < n // 8 or il >= 7 * n // 8 or (il - n // 8) % 3 == 2


def tensor_list(arch: dict, rope_freqs: bool = False, weight_type: int | None = None):
    """(name, ggml type, ne0, ne1) in file order; 1-D tensors have ne1 = 1.  weight_type None: the Q4_K_M mixture;
    T_Q4_0 / T_Q8_0: every matrix in that type, output.weight in Q6_K for Q4_0 as the reference's quantizer leaves it
    (src/llama-quant.cpp:196-204)."""
    E, F, L = arch["n_embd"], arch["n_ff"], arch["n_layer"]
    KV = E // arch["n_head"] * arch["n_head_kv"]
    out = [("token_embd.weight", T_Q4_K, E, arch["n_vocab"]), ("output_norm.weight", T_F32, E, 1),
           ("output.weight", T_Q6_K, E, arch["n_vocab"])]
    for il in range(L):
        more = T_Q6_K if use_more_bits(il, L) else T_Q4_K
        v_type = T_Q5_K if (L == 80 and more == T_Q4_K) else more        # 70B-class: src/llama-quant.cpp:238-243
        p = f"blk.{il}."
        out += [(p + "attn_norm.weight", T_F32, E, 1), (p + "attn_q.weight", T_Q4_K, E, E), (p + "attn_k.weight", T_Q4_K, E, KV),
                (p + "attn_v.weight", v_type, E, KV), (p + "attn_output.weight", T_Q4_K, E, E), (p + "ffn_norm.weight", T_F32, E, 1),
                (p + "ffn_gate.weight", T_Q4_K, E, F), (p + "ffn_up.weight", T_Q4_K, E, F), (p + "ffn_down.weight", more, F, E)]
    if rope_freqs:                                                        # as Llama-3.1 conversions carry it
        out.append(("rope_freqs.weight", T_F32, E // arch["n_head"] // 2, 1))
    if weight_type is not None:
        out = [(n, t if t == T_F32 else (T_Q6_K if (n == "output.weight" and weight_type == T_Q4_0) else weight_type), a, b) for n, t, a, b in out]
    return out


def row_bytes(t: int, ne0: int) -> int:
    return {T_F32: 4 * ne0, T_Q4_0: ne0 // 32 * 18, T_Q8_0: ne0 // 32 * 34, T_Q4_K: ne0 // 256 * 144, T_Q5_K: ne0 // 256 * 176, T_Q6_K: ne0 // 256 * 210}[t]


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, gtype: int, value) -> bytes:
    head = _s(key) + struct.pack("<I", gtype)
    if gtype == G_U32:
        return head + struct.pack("<I", value)
    if gtype == G_F32:
        return head + struct.pack("<f", value)
    return head + _s(value)


def write_llama_gguf(path, arch: dict, n_ctx_train: int = 8192, seed_base: int = 1000, device: str = "cpu", make_tensor=None,
                     rope_freqs: np.ndarray | None = None, share_layers: bool = False, dequantize=None, weight_type: int | None = None) -> int:
    """Returns the number of bytes written.  make_tensor(type, ne0, ne1, seed, device) -> flat uint8 array.
    rope_freqs: head_dim / 2 frequency factors written as rope_freqs.weight (none by default).
    share_layers: every layer gets the bytes of the first layer that has the same tensor (name suffix, type, shape):
    for timing runs on hosts where quantizing 8 billion random weights on the CPU would take minutes; speed does
    not depend on the values.
    dequantize(type, bytes, ne0) -> float32 [rows, ne0]: when given, every quantized tensor is written as the F32 values
    its blocks decode to -- the same model with exact weights, for parity checks against an unquantized evaluation."""
    if make_tensor is None:
        from llama_cpp_b200 import synth
        make_tensor = synth.make_tensor
    a = "llama"
    head_dim = arch["n_embd"] // arch["n_head"]
    kvs = [_kv("general.architecture", G_STR, a), _kv("general.name", G_STR, "synthetic llama (random init)"),
           _kv("general.file_type", G_U32, {None: 15, T_Q4_0: 2, T_Q8_0: 7}[weight_type]),       # LLAMA_FTYPE_MOSTLY_Q4_K_M / Q4_0 / Q8_0
           _kv("general.alignment", G_U32, ALIGN),
           _kv(f"{a}.context_length", G_U32, n_ctx_train), _kv(f"{a}.embedding_length", G_U32, arch["n_embd"]),
           _kv(f"{a}.block_count", G_U32, arch["n_layer"]), _kv(f"{a}.feed_forward_length", G_U32, arch["n_ff"]),
           _kv(f"{a}.attention.head_count", G_U32, arch["n_head"]), _kv(f"{a}.attention.head_count_kv", G_U32, arch["n_head_kv"]),
           _kv(f"{a}.attention.layer_norm_rms_epsilon", G_F32, arch["rms_eps"]), _kv(f"{a}.rope.freq_base", G_F32, arch["rope_theta"]),
           _kv(f"{a}.rope.dimension_count", G_U32, head_dim), _kv(f"{a}.vocab_size", G_U32, arch["n_vocab"]),
           _kv("tokenizer.ggml.model", G_STR, "no_vocab")]
    tensors = tensor_list(arch, rope_freqs is not None, weight_type)
    src_types = [t for _, t, _, _ in tensors]
    if dequantize is not None:
        tensors = [(name, T_F32, ne0, ne1) for name, _, ne0, ne1 in tensors]
    infos, off = [], 0
    for name, t, ne0, ne1 in tensors:
        dims = [ne0] if ne1 == 1 else [ne0, ne1]
        infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", t, off))
        off += (row_bytes(t, ne0) * ne1 + ALIGN - 1) // ALIGN * ALIGN
    header = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs) + b"".join(infos)
    header += b"\0" * (-len(header) % ALIGN)
    written = 0
    shared = {}
    with open(path, "wb") as f:
        f.write(header)
        written += len(header)
        for i, (name, t, ne0, ne1) in enumerate(tensors):
            key = (name.split(".", 2)[-1] if name.startswith("blk.") else name, t, ne0, ne1)
            if name == "rope_freqs.weight":
                data = np.ascontiguousarray(rope_freqs, dtype=np.float32).view(np.uint8).reshape(-1)
            elif share_layers and key in shared:
                data = shared[key]
            else:
                data = np.ascontiguousarray(make_tensor(src_types[i], ne0, ne1, seed=seed_base + i, device=device)).view(np.uint8).reshape(-1)
                if dequantize is not None and src_types[i] != T_F32:
                    data = np.ascontiguousarray(dequantize(src_types[i], data, ne0), dtype=np.float32).view(np.uint8).reshape(-1)
                if share_layers:
                    shared[key] = data
            assert data.size == row_bytes(t, ne0) * ne1, name
            f.write(data.tobytes())
            f.write(b"\0" * (-data.size % ALIGN))
            written += data.size + (-data.size % ALIGN)
    return written


def main():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    entry.load_package()
    from llama_cpp_b200 import llama
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("path")
    ap.add_argument("--model", default="8b", choices=["8b", "70b", "tiny"])
    ap.add_argument("--weight-type", default="q4_k_m", choices=["q4_k_m", "q4_0", "q8_0"])
    a = ap.parse_args()
    arch = {"8b": llama.LLAMA3_8B, "70b": llama.LLAMA3_70B,
            "tiny": dict(n_layer=4, n_embd=1024, n_head=8, n_head_kv=2, n_ff=2048, n_vocab=2048, rope_theta=500000.0, rms_eps=1e-5)}[a.model]
    n = write_llama_gguf(a.path, arch, device="cuda" if torch.cuda.is_available() else "cpu",
                         weight_type={"q4_k_m": None, "q4_0": T_Q4_0, "q8_0": T_Q8_0}[a.weight_type])
    print(f"wrote {a.path}: {n / 1e9:.2f} GB")


if __name__ == "__main__":
    main()
