"""ctypes binding of the GGUF reader (b200_gguf_* in include/b200_llama.h): metadata and tensor directory of a
model file in the reference's on-disk format (ggml/include/gguf.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import B200Error, lib

_bound = False


def _bind():
    global _bound
    l = lib()
    if not _bound:
        vp, cp = C.c_void_p, C.c_char_p
        l.b200_gguf_open.restype = vp
        l.b200_gguf_open.argtypes = [cp]
        l.b200_gguf_close.argtypes = [vp]
        l.b200_gguf_error.restype = cp
        l.b200_gguf_version.restype = C.c_uint32
        l.b200_gguf_version.argtypes = [vp]
        l.b200_gguf_alignment.restype = C.c_uint32
        l.b200_gguf_alignment.argtypes = [vp]
        l.b200_gguf_data_offset.restype = C.c_uint64
        l.b200_gguf_data_offset.argtypes = [vp]
        l.b200_gguf_n_kv.restype = C.c_int64
        l.b200_gguf_n_kv.argtypes = [vp]
        l.b200_gguf_n_tensors.restype = C.c_int64
        l.b200_gguf_n_tensors.argtypes = [vp]
        l.b200_gguf_key.argtypes = [vp, C.c_int64, cp, C.c_size_t, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
        l.b200_gguf_get_u32.argtypes = [vp, cp, C.POINTER(C.c_uint32)]
        l.b200_gguf_get_f32.argtypes = [vp, cp, C.POINTER(C.c_float)]
        l.b200_gguf_get_str.argtypes = [vp, cp, cp, C.c_size_t]
        l.b200_gguf_tensor_info.argtypes = [vp, C.c_int64, cp, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                            C.POINTER(C.c_int64), C.POINTER(C.c_uint64), C.POINTER(C.c_size_t)]
        l.b200_gguf_find_tensor.restype = C.c_int64
        l.b200_gguf_find_tensor.argtypes = [vp, cp]
        l.b200_gguf_tensor_data.restype = vp
        l.b200_gguf_tensor_data.argtypes = [vp, C.c_int64]
        _bound = True
    return l


class GGUF:
    """An open model file.  Raises B200Error for a malformed, truncated or unsupported file."""

    def __init__(self, path):
        self.l = _bind()
        self.h = self.l.b200_gguf_open(str(path).encode())
        if not self.h:
            raise B200Error(self.l.b200_gguf_error().decode())

    def close(self):
        if self.h:
            self.l.b200_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def version(self) -> int:
        return int(self.l.b200_gguf_version(self.h))

    @property
    def alignment(self) -> int:
        return int(self.l.b200_gguf_alignment(self.h))

    @property
    def data_offset(self) -> int:
        return int(self.l.b200_gguf_data_offset(self.h))

    def keys(self):
        """[(key, gguf_type, array element type, array count)] in file order."""
        out = []
        name = C.create_string_buffer(256)
        t, et, n = C.c_uint32(), C.c_uint32(), C.c_uint64()
        for i in range(self.l.b200_gguf_n_kv(self.h)):
            self.l.b200_gguf_key(self.h, i, name, 256, C.byref(t), C.byref(et), C.byref(n))
            out.append((name.value.decode(), t.value, et.value, n.value))
        return out

    def get_u32(self, key: str):
        v = C.c_uint32()
        return v.value if self.l.b200_gguf_get_u32(self.h, key.encode(), C.byref(v)) == 0 else None

    def get_f32(self, key: str):
        v = C.c_float()
        return v.value if self.l.b200_gguf_get_f32(self.h, key.encode(), C.byref(v)) == 0 else None

    def get_str(self, key: str):
        buf = C.create_string_buffer(1024)
        return buf.value.decode() if self.l.b200_gguf_get_str(self.h, key.encode(), buf, 1024) == 0 else None

    def tensors(self):
        out = []
        name = C.create_string_buffer(256)
        t, nd, off, nb = C.c_int32(), C.c_int32(), C.c_uint64(), C.c_size_t()
        ne = (C.c_int64 * 4)()
        for i in range(self.l.b200_gguf_n_tensors(self.h)):
            self.l.b200_gguf_tensor_info(self.h, i, name, 256, C.byref(t), C.byref(nd), ne, C.byref(off), C.byref(nb))
            out.append(dict(index=i, name=name.value.decode(), type=t.value, n_dims=nd.value, ne=list(ne), offset=off.value, nbytes=nb.value))
        return out

    def find(self, name: str) -> int:
        return int(self.l.b200_gguf_find_tensor(self.h, name.encode()))

    def tensor_bytes(self, i: int, nbytes: int) -> np.ndarray:
        """A copy of tensor i's bytes."""
        p = self.l.b200_gguf_tensor_data(self.h, i)
        if not p:
            raise B200Error("no such tensor")
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(nbytes,)).copy()
