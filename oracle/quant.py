"""CPU restatement of the reference's group-wise block-scale quantizer.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows, function by function, the reference's own CPU models and the kernel
they model (paths are relative to the reference project):

* UE8M0 scale with the fast-math ``log2f`` quirk .. ``tests/test_group_wise_quant.py:40-53``
  (same model in ``tests/utils/gemm_utils.py:392-407``); kernel expression
  ``csrc/common/mx_quant.cuh:104-110``.
* MXFP8 group math ............................... ``tests/test_group_wise_quant.py:56-79``;
  kernel ``csrc/common/mx_quant.cuh:113-131``.
* NVFP4 group math ............................... ``tests/test_group_wise_quant.py:97-157``;
  kernel ``csrc/kernel/gemm/group_wise_quant.cu:180-212``.
* MXFP4 group math ............................... ``tests/test_group_wise_quant.py:165-213``.
* E2M1 round-half-away + packing ................. ``tests/utils/fp4_utils.py:20-37``;
  kernel ``csrc/kernel/gemm/group_wise_quant.cu:63-83``.
* SfAtom 128x4 swizzle ........................... ``tests/test_group_wise_quant.py:221-255``,
  ``tests/utils/gemm_utils.py:55-65``; kernel ``csrc/common/mx_quant.cuh:143-150``.

Where the reference's test model and its kernel disagree the kernel wins: the
amax floor is the kernel's 1e-10 (``mx_quant.cuh:50``), not the models' 1e-4 /
1e-12 clips.  The two only differ for all-zero or vanishingly small groups.
"""

from __future__ import annotations

import numpy as np

MODES = ("w8a8-mxfp8", "w4a4-mxfp4", "w4a4-nvfp4")
GROUP_SIZE = {"w8a8-mxfp8": 32, "w4a4-mxfp4": 32, "w4a4-nvfp4": 16}

E4M3_MAX = np.float32(448.0)
E2M1_MAX = np.float32(6.0)
AMAX_FLOOR = np.float32(1e-10)  # mx_quant.cuh:50

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MIDPOINTS = ((E2M1_VALUES[:-1] + E2M1_VALUES[1:]) / 2).astype(np.float32)

SF_ATOM_ROWS = 128
SF_ATOM_COLS = 4
SF_ATOM_BYTES = 512


# --------------------------------------------------------------------------
# 8-bit float codecs
# --------------------------------------------------------------------------

def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for c in range(256):
        e, m = (c >> 3) & 0xF, c & 7
        if e == 0:
            v = (m / 8.0) * 2.0 ** -6
        elif e == 15 and m == 7:
            v = np.nan
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[c] = -v if c & 0x80 else v
    return t


_E4M3_TABLE = _e4m3_table()


def decode_e4m3(codes: np.ndarray) -> np.ndarray:
    """float8_e4m3fn bit patterns -> float32."""
    return _E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def decode_ue4m3(codes: np.ndarray) -> np.ndarray:
    """UE4M3 scale bytes (e4m3 with the sign bit clear) -> float32."""
    return _E4M3_TABLE[np.asarray(codes, dtype=np.uint8) & 0x7F]


def decode_ue8m0(codes: np.ndarray) -> np.ndarray:
    """UE8M0 scale bytes -> float32 ``2^(byte - 127)``."""
    return np.exp2(np.asarray(codes, dtype=np.int32).astype(np.float32) - 127.0).astype(np.float32)


def encode_e4m3_rn_satfinite(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 byte, round-to-nearest-even, finite values saturate at
    +-448 (the ``cvt.rn.satfinite.e4m3x2.f32`` the kernel uses).  NaN is not
    expected here; the callers clamp first, as the kernel does."""
    x = np.asarray(x, dtype=np.float32)
    sign = (x.view(np.uint32) >> 24).astype(np.uint8) & 0x80
    a = np.minimum(np.abs(x), E4M3_MAX).astype(np.float32)
    # normal range: round the 23-bit mantissa to 3 bits, ties to even
    bits = a.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 20) & 1
    r = (bits + 0x7FFFF + lsb) & ~np.uint64(0xFFFFF)
    exp = (r >> 23).astype(np.int64) - 127 + 7
    man = (r >> 20) & 7
    normal = ((exp << 3) | man.astype(np.int64)).astype(np.int64)
    # subnormal range (< 2^-6): multiples of 2^-9, ties to even
    sub = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)
    code = np.where(a < np.float32(2.0 ** -6), sub, normal)
    code = np.minimum(code, 0x7E)
    return (code.astype(np.uint8) | sign).astype(np.uint8)


# --------------------------------------------------------------------------
# scale recipes
# --------------------------------------------------------------------------

def ue8m0_from_scale(scale: np.ndarray) -> np.ndarray:
    """UE8M0 byte of the smallest power of two >= scale, as the kernel's
    fast-math ``ceilf(log2f(scale)) + 127`` produces it: an exact power of two
    below 1 comes out one exponent higher
    (reference ``tests/test_group_wise_quant.py:40-53``)."""
    x = np.clip(np.abs(np.asarray(scale, dtype=np.float32)), np.float32(1e-38), None)
    x = x.astype(np.float32)
    lg = np.log2(x).astype(np.float32)
    raw = x.view(np.uint32)
    bump = ((raw & 0x007FFFFF) == 0) & (x < 1.0)
    lg[bump] = np.nextafter(lg[bump], np.float32(np.inf))
    return np.clip(np.ceil(lg) + 127.0, 0.0, 254.0).astype(np.uint8)


def ue8m0_from_scale_closed_form(scale: np.ndarray) -> np.ndarray:
    """The same function written on the float's bit fields (what the CUDA
    quantizer executes): biased exponent, plus one when the mantissa is
    non-zero or the value is below 1.  Equal to :func:`ue8m0_from_scale` for
    every scale that is ``amax / 448`` or ``amax / 6`` of a bf16 or fp16 amax
    (checked exhaustively in ``tests/test_oracle_golden.py``)."""
    s = np.asarray(scale, dtype=np.float32)
    raw = s.view(np.uint32)
    exp = ((raw >> 23) & 0xFF).astype(np.int32)
    man = raw & 0x007FFFFF
    e = exp + ((man != 0) | (exp < 127)).astype(np.int32)
    return np.clip(e, 0, 254).astype(np.uint8)


def _to_f32(x) -> np.ndarray:
    try:
        import torch
        if isinstance(x, torch.Tensor):
            return x.detach().to("cpu").to(torch.float32).numpy()
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(x, dtype=np.float32)


def _group_amax(xg: np.ndarray) -> np.ndarray:
    # fmaxf chain seeded with the floor; NaN operands are ignored by fmaxf
    a = np.abs(xg)
    a = np.where(np.isnan(a), np.float32(0), a)
    return np.maximum(a.max(axis=-1), AMAX_FLOOR).astype(np.float32)


def _e2m1_codes(x_scaled: np.ndarray) -> np.ndarray:
    """4-bit E2M1 codes: magnitude to the nearest grid value with exact
    midpoints going to the larger one, sign taken from the scaled value."""
    idx = np.searchsorted(E2M1_MIDPOINTS, np.abs(x_scaled), side="right").astype(np.uint8)
    return ((x_scaled < 0).astype(np.uint8) << 3) | idx


def _pack_nibbles(codes: np.ndarray) -> np.ndarray:
    return ((codes[..., 1::2] << 4) | codes[..., 0::2]).astype(np.uint8)


# --------------------------------------------------------------------------
# SfAtom swizzle
# --------------------------------------------------------------------------

def sf_rows(rows: int) -> int:
    """Scale rows padded to whole 128-row atoms."""
    return -(-rows // SF_ATOM_ROWS) * SF_ATOM_ROWS


def sf_atom_offsets(rows: int, kb_dim: int) -> np.ndarray:
    """[rows, kb_dim] byte offsets of the logical scales in the swizzled
    buffer: 512-byte atoms of 128 rows x 4 K-blocks, K-fastest, then row
    tiles; inside an atom ``(row % 32) * 16 + (row % 128) // 32 * 4 + kb % 4``."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    kb = np.arange(kb_dim, dtype=np.int64)[None, :]
    return (
        ((r // SF_ATOM_ROWS) * (kb_dim // SF_ATOM_COLS) + kb // SF_ATOM_COLS) * SF_ATOM_BYTES
        + (r % 32) * 16
        + ((r % SF_ATOM_ROWS) // 32) * 4
        + kb % SF_ATOM_COLS
    )


def swizzle_sf(sf_logical: np.ndarray) -> np.ndarray:
    """[rows, kb_dim] logical scales -> [ceil128(rows), kb_dim] array whose
    flat bytes are in SfAtom order; padding rows are zero."""
    sf_logical = np.asarray(sf_logical, dtype=np.uint8)
    rows, kb_dim = sf_logical.shape
    assert kb_dim % SF_ATOM_COLS == 0
    m_sf = sf_rows(rows)
    padded = np.zeros((m_sf, kb_dim), dtype=np.uint8)
    padded[:rows] = sf_logical
    out = np.empty(m_sf * kb_dim, dtype=np.uint8)
    out[sf_atom_offsets(m_sf, kb_dim).ravel()] = padded.ravel()
    return out.reshape(m_sf, kb_dim)


def unswizzle_sf(sf_swizzled: np.ndarray, rows: int) -> np.ndarray:
    """Inverse of :func:`swizzle_sf`: the first ``rows`` logical scale rows."""
    sf_swizzled = np.asarray(sf_swizzled, dtype=np.uint8)
    kb_dim = sf_swizzled.shape[-1]
    flat = sf_swizzled.reshape(-1)
    return flat[sf_atom_offsets(rows, kb_dim)]


# --------------------------------------------------------------------------
# the quantizer
# --------------------------------------------------------------------------

def quant_group_wise(x, mode: str = "w8a8-mxfp8", use_swizzle: bool = True):
    """Quantize ``x`` ([m, k] bf16/fp16 tensor or float32 array holding such
    values) group-wise along k.  Returns ``(q, sf)`` as uint8 arrays:
    ``q`` is [m, k] e4m3 bytes (mxfp8) or [m, k/2] packed e2m1 (even index in
    the low nibble); ``sf`` is [m, k/g] (linear) or [ceil128(m), k/g] with
    flat bytes in SfAtom order (swizzled)."""
    if mode not in MODES:
        raise ValueError(f"Unsupported quantization mode: {mode}")
    g = GROUP_SIZE[mode]
    xf = _to_f32(x)
    m, k = xf.shape
    if k % g:
        raise ValueError("k must be divisible by the quantization group size")
    kb = k // g
    if use_swizzle and kb % 4:
        raise ValueError("scale kb_dim must be divisible by 4")
    xg = xf.reshape(m, kb, g)
    amax = _group_amax(xg)

    with np.errstate(invalid="ignore", over="ignore"):
        if mode == "w8a8-mxfp8":
            sf = ue8m0_from_scale(amax / E4M3_MAX)
            # 2^(127 - e); e = 254 gives 2^-127, which the kernel's FTZ exp2f flushes to 0
            inv = np.where(sf == 254, np.float32(0), np.exp2(127.0 - sf.astype(np.float32))).astype(np.float32)
            xs = (xg * inv[..., None]).astype(np.float32)
            # fminf(fmaxf(x, -448), 448): NaN -> -448
            xs = np.where(np.isnan(xs), -E4M3_MAX, np.clip(xs, -E4M3_MAX, E4M3_MAX)).astype(np.float32)
            q = encode_e4m3_rn_satfinite(xs).reshape(m, k)
        else:
            scale = (amax / E2M1_MAX).astype(np.float32)
            if mode == "w4a4-nvfp4":
                sf = encode_e4m3_rn_satfinite(np.clip(scale, 0, E4M3_MAX))
                sf = np.where((sf == 0) & (amax > 0), np.uint8(1), sf).astype(np.uint8)
                inv = (np.float32(1.0) / decode_ue4m3(sf)).astype(np.float32)
            else:
                sf = ue8m0_from_scale(scale)
                inv = np.where(sf == 254, np.float32(0), np.exp2(127.0 - sf.astype(np.float32))).astype(np.float32)
            xs = (xg * inv[..., None]).astype(np.float32)
            xs = np.where(np.isnan(xs), -E2M1_MAX, np.clip(xs, -E2M1_MAX, E2M1_MAX)).astype(np.float32)
            q = _pack_nibbles(_e2m1_codes(xs.reshape(m, k)))

    sf = sf.astype(np.uint8)
    if use_swizzle:
        sf = swizzle_sf(sf) if m else np.zeros((0, kb), dtype=np.uint8)
    return q, sf


def decode_e2m1_packed(packed: np.ndarray) -> np.ndarray:
    """[m, k/2] packed e2m1 bytes -> [m, k] float32 values on the E2M1 grid."""
    packed = np.asarray(packed, dtype=np.uint8)
    m, half = packed.shape
    codes = np.empty((m, half * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    vals = E2M1_VALUES[codes & 7]
    return np.where(codes & 8, -vals, vals).astype(np.float32)


def rms_norm_ref(x, weight, eps: float = 1e-6):
    """fp32 RMSNorm rounded to bf16: ``x * rsqrt(mean(x^2) + eps) * weight``, the
    reference's ``ref_rms_norm`` (``tests/test_rms_norm_quant.py:36-40``).  Returns
    a torch bfloat16 tensor."""
    import torch

    xf = x.detach().to("cpu").float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.detach().to("cpu").float()
    return y.to(torch.bfloat16)
