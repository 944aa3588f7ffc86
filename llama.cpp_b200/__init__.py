"""ctypes binding of libggml-b200.so: the flat C-ABI of include/b200_kernels.h.

The package directory name contains a dot, so import it through
``__graft_entry__.load_package()`` (importlib with the alias ``llama_cpp_b200``).

Nothing here computes on the CPU: every function forwards to the CUDA library
and raises if the library is missing or no sm_100 device is visible.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libggml-b200.so"

# ggml_type numbers (ggml/include/ggml.h:351-392)
TYPES = {"f32": 0, "f16": 1, "q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8,
         "q2_K": 10, "q3_K": 11, "q4_K": 12, "q5_K": 13, "q6_K": 14, "iq4_nl": 20, "iq4_xs": 23, "i32": 26, "bf16": 30}
BLOCK = {"f32": (1, 4), "f16": (1, 2), "q4_0": (32, 18), "q4_1": (32, 20), "q5_0": (32, 22), "q5_1": (32, 24),
         "q8_0": (32, 34), "q2_K": (256, 84), "q3_K": (256, 110), "q4_K": (256, 144), "q5_K": (256, 176), "q6_K": (256, 210),
         "iq4_nl": (32, 18), "iq4_xs": (256, 136)}

EXPORTS = [
    "b200_device_count", "b200_last_error", "b200_row_size",
    "b200_mul_mat_q_scratch_bytes", "b200_mul_mat_q", "b200_mul_mat_q_host",
    "b200_act_bytes", "b200_quantize_act", "b200_mul_mat_vec_q", "b200_set_dependent_launch",
    "b200_mul_mat_q_noalloc", "b200_noalloc_last_error", "b200_noalloc_status",
    "b200_decode_step_mul_mat_host", "b200_decode_step_gate_up_host", "b200_decode_step_qkv_host",
    "b200_decode_step_attention_host", "b200_decode_step_last_error", "b200_peer_barrier_probe_host", "b200_tc_i8_probe_host",
    "b200_flash_attn_scratch_bytes", "b200_flash_attn", "b200_flash_attn_host",
    "b200_dequantize_rows_host", "b200_get_rows_host", "b200_quantize_rows_host", "b200_f32_to_f16_host",
    "b200_rms_norm_host", "b200_rope_host", "b200_silu_mul_host", "b200_soft_max_host",
    "ggml_backend_init", "ggml_backend_score",
    "b200_llama_create", "b200_llama_free", "b200_llama_error", "b200_llama_n_tensors", "b200_llama_tensor_info",
    "b200_llama_set_tensor", "b200_llama_tensor_data", "b200_llama_decode", "b200_llama_last_n_nodes",
    "b200_llama_last_compute_ms", "b200_llama_launch_count", "b200_llama_weight_bytes",
    "b200_row_split_range", "b200_llama_tensor_rows", "b200_llama_ipc_handle", "b200_llama_attach_peers",
    "b200_llama_load_gguf", "b200_llama_get_config",
    "b200_gguf_open", "b200_gguf_close", "b200_gguf_error", "b200_gguf_version", "b200_gguf_alignment", "b200_gguf_data_offset",
    "b200_gguf_n_kv", "b200_gguf_n_tensors", "b200_gguf_key", "b200_gguf_get_u32", "b200_gguf_get_f32", "b200_gguf_get_str",
    "b200_gguf_tensor_info", "b200_gguf_find_tensor", "b200_gguf_tensor_data",
]


class B200Error(RuntimeError):
    pass


def build(ref: str | None = None, jobs: int = 8) -> Path:
    """Compile lib/libggml-b200.so for sm_100a (needs nvcc and the reference headers)."""
    env = dict(os.environ)
    cmd = ["make", "-C", str(PKG_DIR), f"-j{jobs}"]
    if ref:
        cmd.append(f"REF={ref}")
    subprocess.run(cmd, check=True, env=env)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    """The loaded CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise B200Error(f"{LIB_PATH} is missing: build it with __graft_entry__.build() (there is no CPU fallback)")
        l = C.CDLL(str(LIB_PATH))
        i64, f32, vp, sz = C.c_int64, C.c_float, C.c_void_p, C.c_size_t
        l.b200_last_error.restype = C.c_char_p
        l.b200_row_size.restype = sz
        l.b200_row_size.argtypes = [C.c_int, i64]
        l.b200_mul_mat_q_scratch_bytes.restype = sz
        l.b200_mul_mat_q_scratch_bytes.argtypes = [C.c_int, i64, i64, i64]
        l.b200_mul_mat_q.argtypes = [C.c_int, vp, i64, i64, i64, vp, i64, i64, vp, i64, vp, sz, vp]
        l.b200_mul_mat_q_host.argtypes = [C.c_int, vp, i64, i64, vp, i64, vp]
        l.b200_act_bytes.restype = sz
        l.b200_act_bytes.argtypes = [i64, i64]
        l.b200_quantize_act.argtypes = [vp, i64, i64, i64, vp, vp]
        l.b200_mul_mat_vec_q.argtypes = [C.c_int, vp, i64, i64, i64, vp, i64, vp, i64, vp]
        l.b200_mul_mat_q_noalloc.argtypes = [C.c_int, vp, i64, i64, i64, vp, i64, i64, vp, i64, vp]
        l.b200_noalloc_last_error.restype = C.c_char_p
        l.b200_noalloc_status.argtypes = [vp]
        l.b200_decode_step_last_error.restype = C.c_char_p
        l.b200_decode_step_mul_mat_host.argtypes = [C.c_int, vp, i64, i64, vp, vp, vp, f32, vp, vp]
        l.b200_decode_step_gate_up_host.argtypes = [C.c_int, vp, vp, i64, i64, vp, vp]
        l.b200_decode_step_qkv_host.argtypes = [C.c_int, C.c_int, vp, vp, vp, i64, i64, i64, vp, vp, f32, C.c_int32, C.c_int, f32, vp, vp, vp, vp]
        l.b200_decode_step_attention_host.argtypes = [vp, vp, vp, vp, i64, i64, i64, f32, C.c_int, C.c_int, vp]
        l.b200_peer_barrier_probe_host.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_int)]
        l.b200_tc_i8_probe_host.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        l.b200_flash_attn_scratch_bytes.restype = sz
        l.b200_flash_attn_scratch_bytes.argtypes = [i64, i64, i64, i64]
        l.b200_flash_attn.argtypes = [vp, i64, i64, vp, i64, i64, vp, i64, i64, vp, i64, vp,
                                      i64, i64, i64, i64, i64, f32, f32, f32, vp, sz, vp]
        l.b200_flash_attn_host.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, f32, f32]
        l.b200_dequantize_rows_host.argtypes = [C.c_int, vp, i64, i64, vp]
        l.b200_get_rows_host.argtypes = [C.c_int, vp, i64, i64, vp, i64, vp]
        l.b200_quantize_rows_host.argtypes = [C.c_int, vp, i64, i64, vp]
        l.b200_f32_to_f16_host.argtypes = [vp, i64, vp]
        l.b200_rms_norm_host.argtypes = [vp, i64, i64, f32, vp, vp]
        l.b200_rope_host.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, C.c_int, f32, f32, f32, f32, f32, f32, vp]
        l.b200_silu_mul_host.argtypes = [vp, vp, i64, vp]
        l.b200_soft_max_host.argtypes = [vp, i64, i64, vp, f32, vp]
        _lib = l
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise B200Error(f"libggml-b200 call failed (code {rc}): {lib().b200_last_error().decode()}")


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def device_count() -> int:
    return int(lib().b200_device_count())


def row_size(qtype: str, k: int) -> int:
    return int(lib().b200_row_size(TYPES[qtype], k))


def mul_mat_q(qtype: str, w: np.ndarray, x: np.ndarray) -> np.ndarray:
    """w: uint8 [M, row_size(K)] quantized rows; x: float32 [N, K]; returns float32 [N, M]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    m = w.shape[0]
    assert w.shape[1] == row_size(qtype, k), (w.shape, row_size(qtype, k))
    out = np.empty((n, m), dtype=np.float32)
    _check(lib().b200_mul_mat_q_host(TYPES[qtype], _p(w), m, k, _p(x), n, _p(out)))
    return out


def flash_attn(q: np.ndarray, k: np.ndarray, v: np.ndarray, mask: np.ndarray | None, scale: float,
               max_bias: float = 0.0, softcap: float = 0.0) -> np.ndarray:
    """q f32 [n_head, n_q, D]; k, v f16 [n_head_kv, n_kv, D]; mask f16 [>=n_q, n_kv]; returns f32 [n_q, n_head, D]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float16)
    v = np.ascontiguousarray(v, dtype=np.float16)
    nh, nq, d = q.shape
    nhkv, nkv, _ = k.shape
    if mask is not None:
        mask = np.ascontiguousarray(mask[:nq], dtype=np.float16)
        assert mask.shape == (nq, nkv)
    out = np.empty((nq, nh, d), dtype=np.float32)
    _check(lib().b200_flash_attn_host(_p(q), _p(k), _p(v), _p(mask), _p(out), d, nq, nh, nkv, nhkv, scale, max_bias, softcap))
    return out


def _check_ds(rc: int) -> None:
    if rc != 0:
        raise B200Error(f"decode-step phase failed (code {rc}): {lib().b200_decode_step_last_error().decode()}")


def decode_step_mul_mat(qtype: str, w: np.ndarray, x: np.ndarray, x_add: np.ndarray | None = None,
                        norm_w: np.ndarray | None = None, eps: float = 1e-5):
    """One mat-vec phase of the persistent decode-step kernel: w uint8 [M, row_size(K)], x f32 [K].
    Returns (dst [M], x + x_add or None)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    k, m = x.size, w.shape[0]
    assert w.shape[1] == row_size(qtype, k)
    xa = None if x_add is None else np.ascontiguousarray(x_add, dtype=np.float32).reshape(-1)
    nw = None if norm_w is None else np.ascontiguousarray(norm_w, dtype=np.float32).reshape(-1)
    out = np.empty(m, dtype=np.float32)
    s = None if xa is None else np.empty(k, dtype=np.float32)
    _check_ds(lib().b200_decode_step_mul_mat_host(TYPES[qtype], _p(w), m, k, _p(x), _p(xa), _p(nw), eps, _p(out), _p(s)))
    return out, s


def decode_step_gate_up(qtype: str, wg: np.ndarray, wu: np.ndarray, x: np.ndarray) -> np.ndarray:
    wg = np.ascontiguousarray(wg, dtype=np.uint8); wu = np.ascontiguousarray(wu, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.empty(wg.shape[0], dtype=np.float32)
    _check_ds(lib().b200_decode_step_gate_up_host(TYPES[qtype], _p(wg), _p(wu), wg.shape[0], x.size, _p(x), _p(out)))
    return out


def decode_step_qkv(qt_qk: str, qt_v: str, wq, wk, wv, n_head: int, n_head_kv: int, x, norm_w, eps: float, pos: int,
                    n_dims: int, freq_base: float, freq_factors=None):
    """Returns (q f32 [n_head, 128], k f16 [n_head_kv, 128], v f16 [n_head_kv, 128])."""
    wq, wk, wv = (np.ascontiguousarray(a, dtype=np.uint8) for a in (wq, wk, wv))
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    nw = np.ascontiguousarray(norm_w, dtype=np.float32).reshape(-1)
    ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, dtype=np.float32)
    q = np.empty((n_head, 128), dtype=np.float32)
    k = np.empty((n_head_kv, 128), dtype=np.float16); v = np.empty((n_head_kv, 128), dtype=np.float16)
    _check_ds(lib().b200_decode_step_qkv_host(TYPES[qt_qk], TYPES[qt_v], _p(wq), _p(wk), _p(wv), n_head, n_head_kv, x.size, _p(x), _p(nw), eps,
                                             pos, n_dims, freq_base, _p(ff), _p(q), _p(k), _p(v)))
    return q, k, v


def decode_step_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, mask: np.ndarray | None, scale: float, n_slices: int,
                          merge_in_next_phase: bool = False) -> np.ndarray:
    """q f32 [n_head, 128]; k, v f16 [n_head_kv, n_kv, 128]; mask f16 [n_kv] or None; returns f32 [n_head, 128]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float16); v = np.ascontiguousarray(v, dtype=np.float16)
    m = None if mask is None else np.ascontiguousarray(mask, dtype=np.float16).reshape(-1)
    nh, nhkv, nkv = q.shape[0], k.shape[0], k.shape[1]
    out = np.empty((nh, 128), dtype=np.float32)
    _check_ds(lib().b200_decode_step_attention_host(_p(q), _p(k), _p(v), _p(m), nkv, nh, nhkv, scale, n_slices, int(merge_in_next_phase), _p(out)))
    return out


def dequantize_rows(qtype: str, rows: np.ndarray, k: int) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.uint8).reshape(-1, row_size(qtype, k))
    out = np.empty((rows.shape[0], k), dtype=np.float32)
    _check(lib().b200_dequantize_rows_host(TYPES[qtype], _p(rows), rows.shape[0], k, _p(out)))
    return out


def get_rows(qtype: str, rows: np.ndarray, k: int, idx: np.ndarray) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.uint8).reshape(-1, row_size(qtype, k))
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty((idx.size, k), dtype=np.float32)
    _check(lib().b200_get_rows_host(TYPES[qtype], _p(rows), rows.shape[0], k, _p(idx), idx.size, _p(out)))
    return out


def quantize_rows(qtype: str, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    out = np.empty((n, row_size(qtype, k)), dtype=np.uint8)
    _check(lib().b200_quantize_rows_host(TYPES[qtype], _p(x), n, k, _p(out)))
    return out


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.float16)
    _check(lib().b200_f32_to_f16_host(_p(x), x.size, _p(out)))
    return out


def rms_norm(x: np.ndarray, eps: float, weight: np.ndarray | None = None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    out = np.empty_like(x)
    _check(lib().b200_rms_norm_host(_p(x), x.shape[0], x.shape[1], eps, _p(w), _p(out)))
    return out


def rope(x: np.ndarray, pos: np.ndarray, freq_factors: np.ndarray | None, n_dims: int, mode: int, n_ctx_orig: int,
         freq_base: float, freq_scale: float = 1.0, ext_factor: float = 0.0, attn_factor: float = 1.0,
         beta_fast: float = 32.0, beta_slow: float = 1.0) -> np.ndarray:
    """x f32 [n_tok, n_head, head_dim]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, dtype=np.float32)
    nt, nh, hd = x.shape
    out = np.empty_like(x)
    _check(lib().b200_rope_host(_p(x), hd, nh, nt, _p(pos), _p(ff), n_dims, mode, n_ctx_orig, freq_base, freq_scale,
                                ext_factor, attn_factor, beta_fast, beta_slow, _p(out)))
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    _check(lib().b200_silu_mul_host(_p(gate), _p(up), gate.size, _p(out)))
    return out


def soft_max(x: np.ndarray, scale: float = 1.0, mask: np.ndarray | None = None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = None if mask is None else np.ascontiguousarray(mask, dtype=np.float16)
    out = np.empty_like(x)
    _check(lib().b200_soft_max_host(_p(x), x.shape[0], x.shape[1], _p(m), scale, _p(out)))
    return out
