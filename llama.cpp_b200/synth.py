"""Synthetic model data: random-init weights of a Llama architecture written as valid
ggml quant blocks (Q4_K, Q5_K, Q6_K, Q4_0, Q8_0) or F32, generated with torch on whatever device is given.

This is an input generator for benchmarks and tests, not part of the compute path.  The
quantizers here are plain min/max (Q4_K) and abs-max (Q6_K) rounding to the block formats
of ggml/src/ggml-common.h:279-320; they produce well-formed blocks whose dequantized
values follow the requested N(0, sigma) weights, but they are not the reference's
search-based quantize_row_q4_K_ref / q6_K_ref.
"""
from __future__ import annotations

import numpy as np
import torch


def _f16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16)


def quantize_q4_K(x: torch.Tensor) -> torch.Tensor:
    """x float32 [rows, K] (K % 256 == 0) -> uint8 [rows, K/256*144]."""
    R, K = x.shape
    nb = K // 256
    xb = x.reshape(R, nb, 8, 32)
    mn = xb.amin(-1).clamp(max=0.0)
    mx = xb.amax(-1)
    scale_f = (mx - mn) / 15.0
    min_f = -mn
    d16 = _f16_round(scale_f.amax(-1) / 63.0)
    dmin16 = _f16_round(min_f.amax(-1) / 63.0)
    d, dmin = d16.float().unsqueeze(-1), dmin16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale_f / d.clamp(min=1e-30)), torch.zeros_like(scale_f)).clamp(0, 63)
    m = torch.where(dmin > 0, torch.round(min_f / dmin.clamp(min=1e-30)), torch.zeros_like(min_f)).clamp(0, 63)
    eff_s, eff_m = (d * sc).unsqueeze(-1), (dmin * m).unsqueeze(-1)
    q = torch.where(eff_s > 0, torch.round((xb + eff_m) / eff_s.clamp(min=1e-30)), torch.zeros_like(xb)).clamp(0, 15).to(torch.uint8)
    sc, m = sc.to(torch.uint8), m.to(torch.uint8)
    out = torch.empty(R, nb, 144, dtype=torch.uint8, device=x.device)
    out[..., 0:2] = d16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 2:4] = dmin16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 4:8] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 8:12] = m[..., 0:4] | ((m[..., 4:8] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:8] & 0xF) | ((m[..., 4:8] & 0xF) << 4)
    qq = q.reshape(R, nb, 4, 2, 32)
    out[..., 16:144] = (qq[..., 0, :] | (qq[..., 1, :] << 4)).reshape(R, nb, 128)
    return out.reshape(R, nb * 144)


def quantize_q5_K(x: torch.Tensor) -> torch.Tensor:
    """x float32 [rows, K] (K % 256 == 0) -> uint8 [rows, K/256*176]: Q4_K's layout with 32 levels, the fifth
    bit of value l of sub-block s in bit s of qh[l] (dequantize_row_q5_K, ggml/src/ggml-quants.c:1482-1508)."""
    R, K = x.shape
    nb = K // 256
    xb = x.reshape(R, nb, 8, 32)
    mn = xb.amin(-1).clamp(max=0.0)
    mx = xb.amax(-1)
    scale_f = (mx - mn) / 31.0
    min_f = -mn
    d16 = _f16_round(scale_f.amax(-1) / 63.0)
    dmin16 = _f16_round(min_f.amax(-1) / 63.0)
    d, dmin = d16.float().unsqueeze(-1), dmin16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale_f / d.clamp(min=1e-30)), torch.zeros_like(scale_f)).clamp(0, 63)
    m = torch.where(dmin > 0, torch.round(min_f / dmin.clamp(min=1e-30)), torch.zeros_like(min_f)).clamp(0, 63)
    eff_s, eff_m = (d * sc).unsqueeze(-1), (dmin * m).unsqueeze(-1)
    q = torch.where(eff_s > 0, torch.round((xb + eff_m) / eff_s.clamp(min=1e-30)), torch.zeros_like(xb)).clamp(0, 31).to(torch.uint8)
    sc, m = sc.to(torch.uint8), m.to(torch.uint8)
    out = torch.empty(R, nb, 176, dtype=torch.uint8, device=x.device)
    out[..., 0:2] = d16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 2:4] = dmin16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 4:8] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 8:12] = m[..., 0:4] | ((m[..., 4:8] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:8] & 0xF) | ((m[..., 4:8] & 0xF) << 4)
    hi = (q >> 4) & 1                                              # [R, nb, 8, 32]
    qh = torch.zeros(R, nb, 32, dtype=torch.uint8, device=x.device)
    for sblk in range(8):
        qh |= hi[:, :, sblk, :] << sblk
    out[..., 16:48] = qh
    qq = (q & 0xF).reshape(R, nb, 4, 2, 32)
    out[..., 48:176] = (qq[..., 0, :] | (qq[..., 1, :] << 4)).reshape(R, nb, 128)
    return out.reshape(R, nb * 176)


def quantize_q6_K(x: torch.Tensor) -> torch.Tensor:
    """x float32 [rows, K] (K % 256 == 0) -> uint8 [rows, K/256*210]."""
    R, K = x.shape
    nb = K // 256
    xb = x.reshape(R, nb, 16, 16)
    scale_f = xb.abs().amax(-1) / 31.0
    d16 = _f16_round(scale_f.amax(-1) / 127.0)
    d = d16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale_f / d.clamp(min=1e-30)), torch.zeros_like(scale_f)).clamp(0, 127)
    eff = (d * sc).unsqueeze(-1)
    q = torch.where(eff > 0, torch.round(xb / eff.clamp(min=1e-30)), torch.zeros_like(xb)).clamp(-32, 31) + 32
    q = q.to(torch.uint8).reshape(R, nb, 2, 4, 32)           # [half n][group t of 32][l]
    lo, hi = q & 0xF, q >> 4
    out = torch.empty(R, nb, 210, dtype=torch.uint8, device=x.device)
    ql = torch.empty(R, nb, 2, 64, dtype=torch.uint8, device=x.device)
    ql[..., 0:32] = lo[..., 0, :] | (lo[..., 2, :] << 4)
    ql[..., 32:64] = lo[..., 1, :] | (lo[..., 3, :] << 4)
    qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
    out[..., 0:128] = ql.reshape(R, nb, 128)
    out[..., 128:192] = qh.reshape(R, nb, 64)
    out[..., 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = d16.view(torch.uint8).reshape(R, nb, 2)
    return out.reshape(R, nb * 210)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    """x float32 [rows, K] (K % 32 == 0) -> uint8 [rows, K/32*18]: d = (value of largest magnitude) / -8, q = x / d + 8
    in [0, 15], value l in the low nibble of qs[l], value l + 16 in the high one (ggml/src/ggml-quants.c:67-100)."""
    R, K = x.shape
    nb = K // 32
    xb = x.reshape(R, nb, 32)
    idx = xb.abs().argmax(-1, keepdim=True)
    d = torch.gather(xb, -1, idx) / -8.0
    d16 = _f16_round(d)
    inv = torch.where(d != 0, 1.0 / torch.where(d != 0, d, torch.ones_like(d)), torch.zeros_like(d))
    q = torch.floor(xb * inv + 8.5).clamp(0, 15).to(torch.uint8)
    out = torch.empty(R, nb, 18, dtype=torch.uint8, device=x.device)
    out[..., 0:2] = d16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 2:18] = q[..., 0:16] | (q[..., 16:32] << 4)
    return out.reshape(R, nb * 18)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    """x float32 [rows, K] (K % 32 == 0) -> uint8 [rows, K/32*34]: d = amax / 127, q = round(x / d)
    (ggml/src/ggml-quants.c:204-230)."""
    R, K = x.shape
    nb = K // 32
    xb = x.reshape(R, nb, 32)
    d = xb.abs().amax(-1, keepdim=True) / 127.0
    d16 = _f16_round(d)
    inv = torch.where(d != 0, 1.0 / torch.where(d != 0, d, torch.ones_like(d)), torch.zeros_like(d))
    q = torch.round(xb * inv).clamp(-127, 127).to(torch.int8)
    out = torch.empty(R, nb, 34, dtype=torch.uint8, device=x.device)
    out[..., 0:2] = d16.view(torch.uint8).reshape(R, nb, 2)
    out[..., 2:34] = q.view(torch.uint8)
    return out.reshape(R, nb * 34)


QUANTIZERS = {2: quantize_q4_0, 8: quantize_q8_0, 12: quantize_q4_K, 13: quantize_q5_K, 14: quantize_q6_K}


def make_tensor(ggml_type: int, ne0: int, ne1: int, seed: int, device: str | torch.device = "cpu", sigma: float = 0.02,
                rows_per_chunk: int = 8192) -> np.ndarray:
    """Random-init tensor [ne1 rows, ne0] as host bytes in the given ggml type (0 F32, 2 Q4_0, 8 Q8_0, 12 Q4_K, 13 Q5_K, 14 Q6_K).
    1-row F32 tensors (norm weights) are 1 + N(0, sigma)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    if ggml_type == 0:
        w = 1.0 + sigma * torch.randn(ne1, ne0, generator=gen, device=device, dtype=torch.float32)
        return w.cpu().numpy().view(np.uint8).reshape(-1)
    fn = QUANTIZERS[ggml_type]
    parts = []
    for r0 in range(0, ne1, rows_per_chunk):
        r = min(rows_per_chunk, ne1 - r0)
        w = sigma * torch.randn(r, ne0, generator=gen, device=device, dtype=torch.float32)
        parts.append(fn(w).cpu())
    return torch.cat(parts, 0).numpy().reshape(-1)
