"""Round-to-nearest GGML quantizers in numpy (Q8_0, Q4_0, Q4_K, Q6_K).

They manufacture valid packed ``[N, bytesPerRow]`` uint8 weights from float32 matrices, for
benchmarks, demos and tests.  They are not part of the parity surface: every consumer (CUDA
kernels and CPU checker alike) reads the packed bytes.  Block layouts follow the GGML formats the
reference consumes (gomlx/gomlx ml/ggml/dequant.go:56-115 for Q8_0 / Q4_0; 144-byte Q4_K and
210-byte Q6_K super-blocks for the k-quants).
"""
from __future__ import annotations

import numpy as np

from .ggml import GGMLQuantType


def _f16_bytes(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a.astype("<f2")).view(np.uint8).reshape(*a.shape, 2)


def _f16_round(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).astype(np.float32)


def _inv(a: np.ndarray) -> np.ndarray:
    with np.errstate(divide="ignore"):
        return np.where(a != 0, np.float32(1.0) / a, np.float32(0.0)).astype(np.float32)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 32, 32)
    d = _f16_round(np.abs(b).max(axis=2) / np.float32(127.0))
    q = np.clip(np.rint(b * _inv(d)[..., None]), -127, 127).astype(np.int8)
    out = np.empty((n, k // 32, 34), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(n, -1)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 32, 32)
    idx = np.abs(b).argmax(axis=2)
    vmax = np.take_along_axis(b, idx[..., None], axis=2)[..., 0]
    d = _f16_round(vmax / np.float32(-8.0))
    q = np.clip(np.rint(b * _inv(d)[..., None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((n, k // 32, 18), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(n, -1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 256, 8, 32)
    lo = np.minimum(b.min(axis=3), 0)
    scale = (b.max(axis=3) - lo) / np.float32(15.0)
    mins = -lo
    d = _f16_round(scale.max(axis=2) / np.float32(63.0))
    dmin = _f16_round(mins.max(axis=2) / np.float32(63.0))
    sc = np.clip(np.rint(scale * _inv(d)[..., None]), 0, 63).astype(np.uint8)
    mn = np.clip(np.rint(mins * _inv(dmin)[..., None]), 0, 63).astype(np.uint8)
    ds = d[..., None] * sc.astype(np.float32)
    dm = dmin[..., None] * mn.astype(np.float32)
    q = np.clip(np.rint((b + dm[..., None]) * _inv(ds)[..., None]), 0, 15).astype(np.uint8)
    out = np.zeros((n, k // 256, 144), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    s = out[..., 4:16]
    s[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    s[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    q = q.reshape(n, k // 256, 4, 2, 32)
    out[..., 16:] = (q[:, :, :, 0] | (q[:, :, :, 1] << 4)).reshape(n, k // 256, 128)
    return out.reshape(n, -1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 256, 16, 16)
    idx = np.abs(b).argmax(axis=3)
    vmax = np.take_along_axis(b, idx[..., None], axis=3)[..., 0]
    sub = vmax / np.float32(-32.0)
    d = _f16_round(np.abs(sub).max(axis=2) / np.float32(127.0))
    sc = np.clip(np.rint(sub * _inv(d)[..., None]), -128, 127).astype(np.int8)
    ds = d[..., None] * sc.astype(np.float32)
    q = np.clip(np.rint(b * _inv(ds)[..., None]) + 32, 0, 63).astype(np.uint8)
    q = q.reshape(n, k // 256, 2, 4, 32)  # [half][group of 32][l]
    out = np.empty((n, k // 256, 210), np.uint8)
    ql = out[..., 0:128].reshape(n, k // 256, 2, 2, 32)
    ql[:, :, :, 0] = (q[:, :, :, 0] & 0x0F) | ((q[:, :, :, 2] & 0x0F) << 4)
    ql[:, :, :, 1] = (q[:, :, :, 1] & 0x0F) | ((q[:, :, :, 3] & 0x0F) << 4)
    out[..., 0:128] = ql.reshape(n, k // 256, 128)
    qh = (q[:, :, :, 0] >> 4) | ((q[:, :, :, 1] >> 4) << 2) | ((q[:, :, :, 2] >> 4) << 4) | ((q[:, :, :, 3] >> 4) << 6)
    out[..., 128:192] = qh.reshape(n, k // 256, 64)
    out[..., 192:208] = sc.view(np.uint8)
    out[..., 208:210] = _f16_bytes(d)
    return out.reshape(n, -1)


_QUANTIZERS = {GGMLQuantType.Q8_0: quantize_q8_0, GGMLQuantType.Q4_0: quantize_q4_0,
               GGMLQuantType.Q4_K: quantize_q4_k, GGMLQuantType.Q6_K: quantize_q6_k}


def quantize(ggml_type: GGMLQuantType, w: np.ndarray) -> np.ndarray:
    """float32 ``[N, K]`` -> packed uint8 ``[N, bytesPerRow]``."""
    ggml_type = GGMLQuantType(ggml_type)
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2 or w.shape[1] % ggml_type.values_per_block():
        raise ValueError(f"weights must be [N, K] with K a multiple of {ggml_type.values_per_block()}")
    return np.ascontiguousarray(_QUANTIZERS[ggml_type](w))


def synthetic_weights(ggml_type: GGMLQuantType, n: int, k: int, sigma: float = 0.02, seed: int = 0,
                      band: int = 1024) -> np.ndarray:
    """Packed weights for a benchmark: a seeded N(0, sigma) band of up to ``band`` rows is quantized
    and repeated down the N rows (full-size bytes and shapes; values repeat every ``band`` rows)."""
    rng = np.random.default_rng(seed)
    rows = min(n, band)
    packed = quantize(ggml_type, rng.standard_normal((rows, k), dtype=np.float32) * np.float32(sigma))
    reps = -(-n // rows)
    return np.ascontiguousarray(np.tile(packed, (reps, 1))[:n])
