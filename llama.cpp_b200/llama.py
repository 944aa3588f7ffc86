"""ctypes binding of the Llama graph driver (include/b200_llama.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import B200Error, lib


class Config(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
                ("n_ff", C.c_int32), ("n_vocab", C.c_int32), ("n_ctx", C.c_int32), ("n_ubatch", C.c_int32),
                ("rope_theta", C.c_float), ("rms_eps", C.c_float), ("n_threads", C.c_int32),
                ("n_ranks", C.c_int32), ("rank", C.c_int32)]

IPC_HANDLE_BYTES = 64


LLAMA3_8B = dict(n_layer=32, n_embd=4096, n_head=32, n_head_kv=8, n_ff=14336, n_vocab=128256, rope_theta=500000.0, rms_eps=1e-5)
LLAMA3_70B = dict(n_layer=80, n_embd=8192, n_head=64, n_head_kv=8, n_ff=28672, n_vocab=128256, rope_theta=500000.0, rms_eps=1e-5)

_bound = False


def _bind():
    global _bound
    l = lib()
    if not _bound:
        vp = C.c_void_p
        l.b200_llama_create.restype = vp
        l.b200_llama_create.argtypes = [vp, C.c_int32, C.POINTER(Config)]
        l.b200_llama_free.argtypes = [vp]
        l.b200_llama_error.restype = C.c_char_p
        l.b200_llama_n_tensors.argtypes = [vp]
        l.b200_llama_tensor_info.argtypes = [vp, C.c_int32, C.c_char_p, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.c_int64),
                                             C.POINTER(C.c_int64), C.POINTER(C.c_size_t)]
        l.b200_llama_set_tensor.argtypes = [vp, C.c_int32, vp, C.c_size_t]
        l.b200_llama_tensor_data.restype = vp
        l.b200_llama_tensor_data.argtypes = [vp, C.c_int32]
        l.b200_llama_decode.argtypes = [vp, vp, C.c_int32, C.c_int32, vp]
        l.b200_llama_last_n_nodes.argtypes = [vp]
        l.b200_llama_last_compute_ms.restype = C.c_double
        l.b200_llama_last_compute_ms.argtypes = [vp]
        l.b200_llama_launch_count.restype = C.c_uint64
        l.b200_llama_launch_count.argtypes = [vp]
        l.b200_llama_weight_bytes.restype = C.c_size_t
        l.b200_llama_weight_bytes.argtypes = [vp]
        l.b200_llama_tensor_rows.argtypes = [vp, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        l.b200_llama_ipc_handle.argtypes = [vp, vp]
        l.b200_llama_attach_peers.argtypes = [vp, vp]
        l.b200_llama_load_gguf.restype = vp
        l.b200_llama_load_gguf.argtypes = [vp, C.c_int32, C.c_char_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
        l.b200_llama_get_config.argtypes = [vp, C.POINTER(Config)]
        _bound = True
    return l


class Llama:
    """A Llama-architecture model evaluated through a ggml backend's C-ABI.

    reg: address of a ggml_backend_reg (another backend library's ggml_backend_init() result) or None for the B200 plugin.
    rank / n_ranks: row-split over n_ranks processes with one GPU each; after construction (and before the first
    decode) every rank calls attach_peers() with a gather function, e.g. the one row_split.gather_bytes builds
    on torch.distributed.
    """

    def __init__(self, n_ctx: int, n_ubatch: int, reg: int | None = None, device_index: int = 0, n_threads: int = 0,
                 rank: int = 0, n_ranks: int = 1, **arch):
        self.l = _bind()
        self.cfg = Config(n_ctx=n_ctx, n_ubatch=n_ubatch, n_threads=n_threads, n_ranks=n_ranks, rank=rank, **arch)
        self.h = self.l.b200_llama_create(reg, device_index, C.byref(self.cfg))
        if not self.h:
            raise B200Error(f"b200_llama_create failed: {self.l.b200_llama_error().decode()}")
        self.logits = np.empty(self.cfg.n_vocab, dtype=np.float32)

    @classmethod
    def from_gguf(cls, path, n_ctx: int, n_ubatch: int, reg: int | None = None, device_index: int = 0, n_threads: int = 0,
                  rank: int = 0, n_ranks: int = 1) -> "Llama":
        """Loads a Llama-architecture GGUF file: hyper-parameters and tensor types from the file, weights copied
        into the backend's buffer (this rank's rows only when n_ranks > 1)."""
        self = cls.__new__(cls)
        self.l = _bind()
        self.h = self.l.b200_llama_load_gguf(reg, device_index, str(path).encode(), n_ctx, n_ubatch, n_threads, n_ranks, rank)
        if not self.h:
            raise B200Error(f"b200_llama_load_gguf failed: {self.l.b200_llama_error().decode()}")
        self.cfg = Config()
        self.l.b200_llama_get_config(self.h, C.byref(self.cfg))
        self.logits = np.empty(self.cfg.n_vocab, dtype=np.float32)
        return self

    def close(self):
        if self.h:
            self.l.b200_llama_free(self.h)
            self.h = None

    def tensors(self):
        out = []
        name = C.create_string_buffer(128)
        t, n0, n1, nb = C.c_int32(), C.c_int64(), C.c_int64(), C.c_size_t()
        lo, full = C.c_int64(), C.c_int64()
        for i in range(self.l.b200_llama_n_tensors(self.h)):
            self.l.b200_llama_tensor_info(self.h, i, name, 128, C.byref(t), C.byref(n0), C.byref(n1), C.byref(nb))
            self.l.b200_llama_tensor_rows(self.h, i, C.byref(lo), C.byref(full))
            # ne1 rows starting at row_low of a full_rows-row tensor are stored on this rank
            out.append(dict(index=i, name=name.value.decode(), type=t.value, ne0=n0.value, ne1=n1.value, nbytes=nb.value,
                            row_low=lo.value, full_rows=full.value))
        return out

    def attach_peers(self, gather):
        """gather(handle: bytes) -> list of every rank's bytes in rank order (a collective call)."""
        if self.cfg.n_ranks < 2:
            return
        h = C.create_string_buffer(IPC_HANDLE_BYTES)
        if self.l.b200_llama_ipc_handle(self.h, h) != 0:
            raise B200Error(self.l.b200_llama_error().decode())
        allh = gather(h.raw)
        if len(allh) != self.cfg.n_ranks or any(len(x) != IPC_HANDLE_BYTES for x in allh):
            raise B200Error("attach_peers: gather must return one handle per rank")
        if self.l.b200_llama_attach_peers(self.h, b"".join(allh)) != 0:
            raise B200Error(self.l.b200_llama_error().decode())

    def set_tensor(self, i: int, data: np.ndarray):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        if self.l.b200_llama_set_tensor(self.h, i, data.ctypes.data_as(C.c_void_p), data.size) != 0:
            raise B200Error(self.l.b200_llama_error().decode())

    def tensor_data(self, i: int) -> int:
        return int(self.l.b200_llama_tensor_data(self.h, i) or 0)

    def decode(self, tokens: np.ndarray, pos0: int, want_logits: bool = True) -> np.ndarray | None:
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        out = self.logits.ctypes.data_as(C.c_void_p) if want_logits else None
        if self.l.b200_llama_decode(self.h, tokens.ctypes.data_as(C.c_void_p), tokens.size, pos0, out) != 0:
            raise B200Error(self.l.b200_llama_error().decode())
        return self.logits if want_logits else None

    @property
    def last_compute_ms(self) -> float:
        return float(self.l.b200_llama_last_compute_ms(self.h))

    @property
    def last_n_nodes(self) -> int:
        return int(self.l.b200_llama_last_n_nodes(self.h))

    @property
    def launch_count(self) -> int:
        return int(self.l.b200_llama_launch_count(self.h))

    @property
    def weight_bytes(self) -> int:
        return int(self.l.b200_llama_weight_bytes(self.h))
