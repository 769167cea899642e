"""Host-side storage helpers for the element types numpy lacks.

bf16 travels as ``uint16`` bit patterns, fp8-e4m3 (OCP "e4m3fn": bias 7, no infinities, max
finite 448, 0x7F/0xFF = NaN) and fp8-e5m2 (OCP: bias 15, the upper byte of an IEEE half, max
finite 57344; "bf8" in the reference's MFMA names) as ``uint8``.  8-bit integers are ``int8``
and their sums ``int32``.  Conversions are round-to-nearest-even, the rounding the GPU epilogue
(``cvt.rn``) and the tensor cores' operand formats assume.
"""

from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0
E5M2_MAX = 57344.0


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round-to-nearest-even, NaN -> quiet NaN."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    out = rounded.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32 (exact)."""
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bf16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            val = np.nan
        elif exp == 0:
            val = man * 2.0 ** -9
        else:
            val = (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        t[code] = sign * val
    return t


E4M3_TABLE = _e4m3_table()


def e4m3_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """fp8-e4m3 bit patterns (uint8) -> float32 (exact)."""
    return E4M3_TABLE[np.ascontiguousarray(b, dtype=np.uint8)]


def f32_to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> fp8-e4m3 bit patterns (uint8), round-to-nearest-even.

    Magnitudes beyond the largest finite value saturate to 448 (the per-tensor scaling
    ``amax / 448`` used on this path never produces them); NaN -> 0x7F.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    _, ex = np.frexp(a)
    e = np.maximum(ex - 1, -6)  # exponent of the value's binade; subnormals share binade -6
    step = np.ldexp(1.0, e - 3)
    q = np.minimum(np.rint(a / step) * step, E4M3_MAX)
    _, ex2 = np.frexp(q)
    e2 = ex2 - 1
    sub = (q < 2.0 ** -6)
    exp_field = np.where(sub, 0, e2 + 7).astype(np.int64)
    man_field = np.where(sub, np.rint(q * 2.0 ** 9), np.rint((q / np.ldexp(1.0, e2) - 1.0) * 8.0)).astype(np.int64)
    bits = (exp_field << 3) | man_field
    bits = np.where(q == 0.0, 0, bits)
    bits = bits | np.where(np.signbit(x), 0x80, 0)
    bits = np.where(np.isnan(x), 0x7F, bits)
    return bits.astype(np.uint8)


def e5m2_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """fp8-e5m2 bit patterns (uint8) -> float32 (exact): the byte is the top half of an f16."""
    b = np.ascontiguousarray(b, dtype=np.uint8)
    return (b.astype(np.uint16) << np.uint16(8)).view(np.float16).astype(np.float32)


def f32_to_e5m2_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> fp8-e5m2 bit patterns (uint8), round-to-nearest-even in one step (not through
    f16, which would round twice).  Magnitudes beyond 57344 saturate to it; NaN -> 0x7F."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    a = np.where(np.isnan(a), 0.0, a)
    _, ex = np.frexp(a)
    e = np.maximum(ex - 1, -14)  # subnormals share binade -14
    step = np.ldexp(1.0, e - 2)
    q = np.minimum(np.rint(a / step) * step, E5M2_MAX)
    bits = (q.astype(np.float16).view(np.uint16) >> np.uint16(8)).astype(np.int64)  # q is exact in f16
    bits = bits | np.where(np.signbit(x), 0x80, 0)
    bits = np.where(np.isnan(x), 0x7F, bits)
    return bits.astype(np.uint8)


def quantize_e4m3(x: np.ndarray) -> tuple[np.ndarray, np.float32]:
    """Per-tensor scaled quantisation: ``scale = amax / 448``, ``q = e4m3(x / scale)``.

    Returns ``(bits, scale)`` with ``x ~= e4m3_bits_to_f32(bits) * scale``.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    amax = np.float32(np.max(np.abs(x))) if x.size else np.float32(0.0)
    scale = np.float32(amax / np.float32(E4M3_MAX)) if amax > 0 else np.float32(1.0)
    return f32_to_e4m3_bits(x / scale), scale


MX_BLOCK = 32  # elements of K that share one E8M0 scale
_MX_ELEM = {"e4m3": (8, f32_to_e4m3_bits, e4m3_bits_to_f32), "e5m2": (15, f32_to_e5m2_bits, e5m2_bits_to_f32)}


def quantize_mx(x: np.ndarray, elem: str = "e4m3") -> tuple[np.ndarray, np.ndarray]:
    """Block-scaled ("MX") quantisation along the last axis, after the OCP microscaling rule:
    per block of 32 values the shared exponent is ``floor(log2(amax)) - emax`` (emax = 8 for
    e4m3, 15 for e5m2), clamped to [-127, 127]; elements are ``x / 2**exponent`` rounded to
    nearest even with saturation.  Returns ``(bits [..., K], scales [..., K/32])``, both uint8;
    a scale byte is the biased exponent (127 = 1.0).  An all-zero block gets scale 127."""
    emax, enc, _ = _MX_ELEM[elem]
    x = np.ascontiguousarray(x, dtype=np.float32)
    K = x.shape[-1]
    if K % MX_BLOCK:
        raise ValueError(f"last axis {K} is not a multiple of {MX_BLOCK}")
    blocks = x.reshape(*x.shape[:-1], K // MX_BLOCK, MX_BLOCK)
    amax = np.abs(blocks).max(axis=-1)
    _, ex = np.frexp(amax)  # amax = m * 2**ex with m in [0.5, 1): floor(log2(amax)) = ex - 1
    shared = np.clip(np.where(amax > 0, ex - 1 - emax, 0), -127, 127).astype(np.int32)
    scaled = blocks / np.ldexp(np.float32(1.0), shared)[..., None]
    return enc(scaled.astype(np.float32)).reshape(x.shape), (shared + 127).astype(np.uint8)


def dequantize_mx(bits: np.ndarray, scales: np.ndarray, elem: str = "e4m3") -> np.ndarray:
    """float32 values of block-scaled data (exact unless the product leaves the f32 range)."""
    _, _, dec = _MX_ELEM[elem]
    vals = dec(bits)
    factor = np.ldexp(np.float32(1.0), np.asarray(scales, dtype=np.int32) - 127)
    return (vals.reshape(*scales.shape, MX_BLOCK) * factor[..., None]).reshape(vals.shape).astype(np.float32)


def to_f32(arr: np.ndarray, dtype: str) -> np.ndarray:
    """Decode a stored operand (see module docstring) to float32."""
    if dtype == "f16":
        return np.asarray(arr, dtype=np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(arr)
    if dtype == "e4m3":
        return e4m3_bits_to_f32(arr)
    if dtype == "e5m2":
        return e5m2_bits_to_f32(arr)
    if dtype in ("i8", "i32"):
        return np.asarray(arr).astype(np.float32)
    if dtype == "f32":
        return np.asarray(arr, dtype=np.float32)
    raise ValueError(f"unknown dtype {dtype!r}")


def from_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    """Encode float32 values into the storage type of ``dtype`` (no scaling)."""
    if dtype == "f16":
        return np.asarray(x, dtype=np.float32).astype(np.float16)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    if dtype == "e4m3":
        return f32_to_e4m3_bits(x)
    if dtype == "e5m2":
        return f32_to_e5m2_bits(x)
    if dtype == "i8":
        return np.clip(np.rint(np.asarray(x, dtype=np.float32)), -128, 127).astype(np.int8)
    if dtype == "i32":
        return np.rint(np.asarray(x, dtype=np.float64)).astype(np.int32)
    if dtype == "f32":
        return np.ascontiguousarray(x, dtype=np.float32)
    raise ValueError(f"unknown dtype {dtype!r}")


STORAGE = {"f16": np.float16, "bf16": np.uint16, "e4m3": np.uint8, "e5m2": np.uint8, "i8": np.int8, "i32": np.int32,
           "f32": np.float32, "mxe4m3": np.uint8, "mxe5m2": np.uint8, "e5m2_e4m3": np.uint8, "e4m3_e5m2": np.uint8}
