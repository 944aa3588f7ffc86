"""ctypes wrapper of the CPU oracle (oracle/ggml_oracle.c) and, when present, of the
unmodified reference libraries built by oracle/ref.mk into oracle/_ref.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke test and the CPU-baseline
leg of bench.py as the checker; never by the product path.
"""
from __future__ import annotations

import ctypes as C
import struct
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "ggml_oracle.c"
LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"

TYPES = {"f32": 0, "f16": 1, "q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8, "q2_K": 10, "q3_K": 11, "q4_K": 12, "q5_K": 13, "q6_K": 14, "iq4_nl": 20, "iq4_xs": 23}
QUANT_TYPES = ["q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q2_K", "q3_K", "q4_K", "q5_K", "q6_K", "iq4_nl", "iq4_xs"]


def build() -> Path:
    """Compile the C restatement (gcc, no SIMD flags, no FMA contraction)."""
    if not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-fvisibility=hidden", "-ffp-contract=off",
                        str(SRC), "-o", str(LIB), "-lm"], check=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(str(LIB))
        i64, f32, vp = C.c_int64, C.c_float, C.c_void_p
        l.oracle_row_size.restype = i64
        l.oracle_row_size.argtypes = [C.c_int, i64]
        l.oracle_dequantize_row.argtypes = [C.c_int, vp, vp, i64]
        l.oracle_quantize_row.argtypes = [C.c_int, vp, vp, i64]
        l.oracle_mul_mat.argtypes = [C.c_int, vp, i64, i64, vp, i64, vp]
        l.oracle_mul_mat_f32.argtypes = [C.c_int, vp, i64, i64, vp, i64, vp]
        l.oracle_flash_attn.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, f32, f32]
        l.oracle_rms_norm.argtypes = [vp, i64, i64, f32, vp, vp]
        l.oracle_silu_mul.argtypes = [vp, vp, i64, vp]
        l.oracle_soft_max.argtypes = [vp, i64, i64, vp, f32, vp]
        l.oracle_rope.argtypes = [vp, i64, i64, i64, vp, vp, C.c_int, C.c_int, C.c_int, f32, f32, f32, f32, f32, f32, vp]
        l.oracle_f32_to_f16.argtypes = [vp, vp, i64]
        _lib = l
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def row_size(qtype: str, k: int) -> int:
    return int(lib().oracle_row_size(TYPES[qtype], k))


def dequantize_rows(qtype: str, rows: np.ndarray, k: int) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.uint8).reshape(-1, row_size(qtype, k))
    out = np.empty((rows.shape[0], k), dtype=np.float32)
    for i in range(rows.shape[0]):
        assert lib().oracle_dequantize_row(TYPES[qtype], _p(rows[i]), _p(out[i]), k) == 0
    return out


def quantize_rows(qtype: str, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty((x.shape[0], row_size(qtype, x.shape[1])), dtype=np.uint8)
    for i in range(x.shape[0]):
        assert lib().oracle_quantize_row(TYPES[qtype], _p(x[i]), _p(out[i]), x.shape[1]) == 0, qtype
    return out


def mul_mat(qtype: str, w: np.ndarray, x: np.ndarray, exact_f32: bool = False) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    m = w.shape[0]
    out = np.empty((n, m), dtype=np.float32)
    fn = lib().oracle_mul_mat_f32 if exact_f32 else lib().oracle_mul_mat
    assert fn(TYPES[qtype], _p(w), m, k, _p(x), n, _p(out)) == 0
    return out


def flash_attn(q, k, v, mask, scale, max_bias=0.0, softcap=0.0) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float16)
    v = np.ascontiguousarray(v, dtype=np.float16)
    nh, nq, d = q.shape
    nhkv, nkv, _ = k.shape
    if mask is not None:
        mask = np.ascontiguousarray(mask[:nq], dtype=np.float16)
    out = np.empty((nq, nh, d), dtype=np.float32)
    assert lib().oracle_flash_attn(_p(q), _p(k), _p(v), _p(mask), _p(out), d, nq, nh, nkv, nhkv, scale, max_bias, softcap) == 0
    return out


def rms_norm(x, eps, weight=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    out = np.empty_like(x)
    lib().oracle_rms_norm(_p(x), x.shape[0], x.shape[1], eps, _p(w), _p(out))
    return out


def silu_mul(g, u):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    out = np.empty_like(g)
    lib().oracle_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


def soft_max(x, scale=1.0, mask=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = None if mask is None else np.ascontiguousarray(mask, dtype=np.float16)
    out = np.empty_like(x)
    lib().oracle_soft_max(_p(x), x.shape[0], x.shape[1], _p(m), scale, _p(out))
    return out


def rope(x, pos, ff, n_dims, mode, n_ctx_orig, freq_base, freq_scale=1.0, ext_factor=0.0, attn_factor=1.0,
         beta_fast=32.0, beta_slow=1.0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    f = None if ff is None else np.ascontiguousarray(ff, dtype=np.float32)
    nt, nh, hd = x.shape
    out = np.empty_like(x)
    lib().oracle_rope(_p(x), hd, nh, nt, _p(pos), _p(f), n_dims, mode, n_ctx_orig, freq_base, freq_scale, ext_factor,
                      attn_factor, beta_fast, beta_slow, _p(out))
    return out


def f32_to_f16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_f16(_p(x), _p(out), x.size)
    return out.view(np.float16)


def nmse(a: np.ndarray, b: np.ndarray) -> float:
    """sum((a-b)^2)/sum(a^2), the criterion of tests/test-backend-ops.cpp:175-188 (a = reference)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    den = float(np.sum(a * a))
    return float(np.sum((a - b) ** 2)) / (den if den > 0 else 1.0)


# ---- golden fixtures (tests/golden/golden.bin, written by tests/golden/make_golden.cpp) ----
def load_golden(path: Path | None = None) -> dict[str, np.ndarray]:
    path = path or (HERE.parent / "tests" / "golden" / "golden.bin")
    data = path.read_bytes()
    assert data[:4] == b"GOLD"
    (n,) = struct.unpack_from("<I", data, 4)
    off, out = 8, {}
    dtypes = {0: np.float32, 1: np.uint8, 2: np.int32, 3: np.float16}
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", data, off); off += 4
        name = data[off:off + nl].decode(); off += nl
        dt, nd = struct.unpack_from("<II", data, off); off += 8
        dims = struct.unpack_from(f"<{nd}Q", data, off); off += 8 * nd
        dtype = np.dtype(dtypes[dt])
        count = int(np.prod(dims))
        out[name] = np.frombuffer(data, dtype=dtype, count=count, offset=off).reshape(dims).copy()
        off += count * dtype.itemsize
    return out


# ---- the unmodified reference (only where oracle/_ref was built) ----
_ref = None


def ref_available() -> bool:
    return (REF_DIR / "libggml-base.so").exists()


def ref_base() -> C.CDLL:
    """libggml-base.so of the reference build: reference quantizers and dequantizers."""
    global _ref
    if _ref is None:
        l = C.CDLL(str(REF_DIR / "libggml-base.so"))
        l.ggml_quantize_chunk.restype = C.c_size_t
        l.ggml_quantize_chunk.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
        l.ggml_row_size.restype = C.c_size_t
        l.ggml_row_size.argtypes = [C.c_int, C.c_int64]
        _ref = l
    return _ref


def ref_quantize_rows(qtype: str, x: np.ndarray) -> np.ndarray:
    """quantize_row_*_ref through ggml_quantize_chunk (ggml/src/ggml.c:6410)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    l = ref_base()
    out = np.empty((n, l.ggml_row_size(TYPES[qtype], k)), dtype=np.uint8)
    l.ggml_quantize_chunk(TYPES[qtype], _p(x), _p(out), 0, n, k, None)
    return out


_cpu_lib = None


def ref_cpu_backend_reg() -> int:
    """Address of the reference CPU backend's ggml_backend_reg: the best-scoring libggml-cpu-*.so variant of
    oracle/_ref is dlopen'ed and its ggml_backend_init() called, as ggml_backend_load_best does
    (ggml/src/ggml-backend-reg.cpp:487-551)."""
    global _cpu_lib
    if _cpu_lib is None:
        C.CDLL(str(REF_DIR / "libggml-base.so"), mode=C.RTLD_GLOBAL)
        best, best_score = None, 0
        for p in sorted(REF_DIR.glob("libggml-cpu-*.so")):
            l = C.CDLL(str(p))
            s = l.ggml_backend_score()
            if s > best_score:
                best, best_score = l, s
        if best is None:
            raise RuntimeError("no usable reference CPU backend variant in oracle/_ref")
        best.ggml_backend_init.restype = C.c_void_p
        _cpu_lib = best
    return int(_cpu_lib.ggml_backend_init())


def ref_gguf_directory(path) -> dict:
    """What the reference's own GGUF reader (gguf_init_from_file, ggml/src/gguf.cpp:288) sees in a file:
    version, alignment, data offset, keys with their types, tensors with type, offset and size."""
    l = ref_base()

    class Params(C.Structure):
        _fields_ = [("no_alloc", C.c_bool), ("ctx", C.c_void_p)]

    vp, i64 = C.c_void_p, C.c_int64
    l.gguf_init_from_file.restype = vp
    l.gguf_init_from_file.argtypes = [C.c_char_p, Params]
    for fn, rt in (("gguf_get_version", C.c_uint32), ("gguf_get_alignment", C.c_size_t), ("gguf_get_data_offset", C.c_size_t),
                   ("gguf_get_n_kv", i64), ("gguf_get_n_tensors", i64)):
        getattr(l, fn).restype = rt
        getattr(l, fn).argtypes = [vp]
    for fn, rt in (("gguf_get_key", C.c_char_p), ("gguf_get_kv_type", C.c_int), ("gguf_get_tensor_name", C.c_char_p),
                   ("gguf_get_tensor_offset", C.c_size_t), ("gguf_get_tensor_type", C.c_int), ("gguf_get_tensor_size", C.c_size_t)):
        getattr(l, fn).restype = rt
        getattr(l, fn).argtypes = [vp, i64]
    l.gguf_free.argtypes = [vp]
    g = l.gguf_init_from_file(str(path).encode(), Params(True, None))
    if not g:
        return None
    try:
        return dict(version=l.gguf_get_version(g), alignment=l.gguf_get_alignment(g), data_offset=l.gguf_get_data_offset(g),
                    keys=[(l.gguf_get_key(g, i).decode(), l.gguf_get_kv_type(g, i)) for i in range(l.gguf_get_n_kv(g))],
                    tensors=[dict(name=l.gguf_get_tensor_name(g, i).decode(), type=l.gguf_get_tensor_type(g, i),
                                  offset=l.gguf_get_tensor_offset(g, i), nbytes=l.gguf_get_tensor_size(g, i))
                             for i in range(l.gguf_get_n_tensors(g))])
    finally:
        l.gguf_free(g)
