"""CPU restatement of the float8_experimental Float8Linear arithmetic (numpy only).

TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import this module; the shipped package
never does and has no CPU execution path of its own.

Every function restates one step of the reference library and cites the reference
file:line it follows.  The arithmetic itself lives in PyTorch (an un-vendored
dependency of the reference, `torch >= 2.3`; pinned here against torch 2.11.0 CPU
eager), so the rounding points below restate PyTorch's eager semantics:

* elementwise ops on bf16/fp16 tensors compute in fp32 and round the result back
  to the tensor dtype after EVERY op;
* a 0-dim tensor does not take part in dtype promotion against a dimensioned
  tensor of the same category, a 1-element 1-D tensor does;
* `python_scalar / tensor` is `tensor.reciprocal() * python_scalar`.

Parity pinning: `tests/golden/make_golden.py` imports the reference itself and
records its outputs; `tests/test_oracle.py` checks this module against those
records and (when torch is importable) against torch's own fp8 conversion for
every bf16 bit pattern.

High-precision tensors are passed as numpy arrays: `float32` arrays for fp32,
`uint16` bit patterns for bf16 and fp16 (numpy has no bf16).  fp8 tensors are
`uint8` bit patterns.
"""
from __future__ import annotations

import numpy as np

BF16 = "bf16"
FP16 = "fp16"
FP32 = "fp32"
E4M3 = "e4m3fn"
E5M2 = "e5m2"

# float8_experimental/float8_utils.py:19
EPS = 1e-12

# torch.finfo(torch.float8_e4m3fn).max / torch.finfo(torch.float8_e5m2).max
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}
FP16_MAX = 65504.0

# (exponent bits, mantissa bits, bias) of the two OCP formats
_FP8_FMT = {E4M3: (4, 3, 7), E5M2: (5, 2, 15)}


# ---------------------------------------------------------------------------
# dtype plumbing
# ---------------------------------------------------------------------------
def to_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    """Widen a tensor given as bit patterns to float32 (exact)."""
    if dtype == FP32:
        return np.asarray(x, dtype=np.float32)
    x = np.asarray(x, dtype=np.uint16)
    if dtype == BF16:
        return (x.astype(np.uint32) << np.uint32(16)).view(np.float32)
    if dtype == FP16:
        return x.view(np.float16).astype(np.float32)
    raise ValueError(dtype)


def round_f32_to(v: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to `dtype` (RNE) and return them widened back to float32."""
    v = np.asarray(v, dtype=np.float32)
    if dtype == FP32:
        return v
    if dtype == FP16:
        with np.errstate(over="ignore"):
            return v.astype(np.float16).astype(np.float32)
    if dtype == BF16:
        return to_f32(f32_to_bf16_bits(v), BF16)
    raise ValueError(dtype)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round-to-nearest-even, NaN kept quiet."""
    u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    rounded = (u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    out = np.where(nan, np.uint32(0x7FC0), rounded)
    return out.astype(np.uint16)


def from_f32(v: np.ndarray, dtype: str) -> np.ndarray:
    """Inverse of `to_f32` after rounding: float32 values -> storage of `dtype`."""
    if dtype == FP32:
        return np.asarray(v, dtype=np.float32)
    if dtype == BF16:
        return f32_to_bf16_bits(v)
    if dtype == FP16:
        with np.errstate(over="ignore"):
            return np.asarray(v, dtype=np.float32).astype(np.float16).view(np.uint16)
    raise ValueError(dtype)


# ---------------------------------------------------------------------------
# fp8 encode / decode (OCP e4m3fn and e5m2)
# ---------------------------------------------------------------------------
def fp8_decode(b: np.ndarray, fp8: str) -> np.ndarray:
    """fp8 bit patterns -> float32 (exact).  `_data.float()` in
    float8_experimental/float8_aten_api.py:24-25 and float8_tensor.py:208."""
    ebits, mbits, bias = _FP8_FMT[fp8]
    b = np.asarray(b, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> mbits) & ((1 << ebits) - 1)
    m = b & ((1 << mbits) - 1)
    normal = np.ldexp(1.0 + m / float(1 << mbits), e - bias)
    subnormal = np.ldexp(m / float(1 << mbits), 1 - bias)
    val = np.where(e == 0, subnormal, normal)
    if fp8 == E4M3:
        val = np.where((e == 15) & (m == 7), np.nan, val)
    else:
        val = np.where((e == 31) & (m != 0), np.nan, val)
        val = np.where((e == 31) & (m == 0), np.inf, val)
    return (sign * val).astype(np.float32)


def fp8_encode_rne(v: np.ndarray, fp8: str) -> np.ndarray:
    """float32 -> fp8 bit patterns, round-to-nearest-even including subnormals.

    Restates the conversion `x.to(float8_dtype)` at float8_experimental/float8_utils.py:137
    for inputs already clamped to the finite fp8 range (:135-136), which is the only
    way the reference reaches it.  NaN encodes as 0x7F in both formats, -0.0 as 0x80.
    Values beyond the finite range (never produced after the clamp) saturate.
    """
    ebits, mbits, bias = _FP8_FMT[fp8]
    v = np.asarray(v, dtype=np.float32)
    a = np.abs(v).astype(np.float64)
    neg = np.signbit(v)
    nan = np.isnan(v)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, FP8_MAX[fp8])
    # exponent of the binade, floored at the smallest normal exponent
    mant, ex = np.frexp(a)  # a = mant * 2**ex, mant in [0.5, 1)
    e_unb = np.maximum(ex - 1, 1 - bias)
    quantum = np.ldexp(1.0, e_unb - mbits)
    q = np.rint(a / quantum)  # ties to even
    r = q * quantum  # rounded magnitude, exactly representable
    mant2, ex2 = np.frexp(r)
    e2 = ex2 - 1
    is_norm = r >= np.ldexp(1.0, 1 - bias)
    efield = np.where(is_norm, e2 + bias, 0)
    frac_norm = np.rint((r / np.ldexp(1.0, np.where(is_norm, e2, 0)) - 1.0) * (1 << mbits))
    frac_sub = np.rint(r / np.ldexp(1.0, 1 - bias - mbits))
    mfield = np.where(is_norm, frac_norm, frac_sub)
    bits = (efield.astype(np.int64) << mbits) | mfield.astype(np.int64)
    bits = np.where(neg, bits | 0x80, bits)
    bits = np.where(nan, 0x7F, bits)
    return bits.astype(np.uint8)


# ---------------------------------------------------------------------------
# amax and scale
# ---------------------------------------------------------------------------
def tensor_to_amax(x: np.ndarray, dtype: str) -> np.float32:
    """`torch.max(torch.abs(x))`, float8_experimental/float8_utils.py:102-112.

    Result is a value of `dtype` (returned widened to float32); NaN propagates.
    The optional cross-rank MAX (:109-110) is `np.maximum.reduce` over ranks and
    is done by the caller."""
    a = np.abs(to_f32(x, dtype))
    if a.size == 0:
        raise ValueError("amax of an empty tensor is undefined (torch.max raises)")
    if np.isnan(a).any():
        return np.float32(np.nan)
    return np.float32(a.max())


def amax_to_scale(amax, fp8: str, orig_dtype: str, amax_dtype: str) -> np.ndarray:
    """float8_experimental/float8_utils.py:35-57.

    `finfo(fp8).max / clamp(amax, min=EPS)` evaluated as reciprocal-then-multiply
    (`Tensor.__rtruediv__`) in `amax_dtype`, with a rounding after each of the three
    ops; clamp to 65504 when `orig_dtype` is fp16 (:54-55); stored as fp32 (:45,56).
    `amax` holds values of `amax_dtype` widened to float32; any shape."""
    amax = np.asarray(amax, dtype=np.float32)
    eps_t = round_f32_to(np.float32(EPS), amax_dtype)
    # torch.clamp(min=) propagates NaN
    c = np.where(np.isnan(amax), amax, np.maximum(amax, eps_t))
    with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
        r = round_f32_to(np.float32(1.0) / c, amax_dtype)
        s = round_f32_to(r * np.float32(FP8_MAX[fp8]), amax_dtype)
    if orig_dtype == FP16:
        s = np.where(np.isnan(s), s, np.minimum(s, np.float32(FP16_MAX)))
    return s.astype(np.float32)


def tensor_to_scale(x: np.ndarray, dtype: str, fp8: str) -> np.float32:
    """float8_experimental/float8_utils.py:115-120 (amax and scale both in x's dtype)."""
    return np.float32(amax_to_scale(tensor_to_amax(x, dtype), fp8, dtype, dtype))


# ---------------------------------------------------------------------------
# the cast
# ---------------------------------------------------------------------------
def cast_to_fp8(x: np.ndarray, dtype: str, scale, fp8: str, product_dtype: str) -> np.ndarray:
    """`to_fp8_saturated(tensor * scale)`:
    float8_experimental/float8_tensor.py:158-159 and float8_utils.py:123-139.

    `product_dtype` is where `tensor * scale` is rounded before the clamp: the
    tensor's own dtype when `scale` is 0-dim (dynamic scaling,
    float8_scaling_utils.py:55-62), fp32 when `scale` has shape [1] (delayed scaling
    buffers, float8_linear.py:201-203) or the tensor is fp32."""
    xf = to_f32(x, dtype)
    s = np.float32(scale)
    with np.errstate(over="ignore", invalid="ignore"):
        p = round_f32_to(xf * s, product_dtype)
    f = np.float32(FP8_MAX[fp8])
    p = np.where(np.isnan(p), p, np.clip(p, -f, f))
    return fp8_encode_rne(p, fp8)


def product_dtype_for(x_dtype: str, scale_ndim: int) -> str:
    """PyTorch type promotion of `tensor * scale` with an fp32 scale."""
    return x_dtype if scale_ndim == 0 else FP32


def cast_dynamic(x: np.ndarray, dtype: str, fp8: str):
    """float8_experimental/float8_scaling_utils.py:33-62: returns (bits, scale, amax)."""
    amax = tensor_to_amax(x, dtype)
    scale = np.float32(amax_to_scale(amax, fp8, dtype, dtype))
    return cast_to_fp8(x, dtype, scale, fp8, dtype), scale, amax


def cast_delayed(x: np.ndarray, dtype: str, stored_scale, fp8: str):
    """float8_experimental/float8_scaling_utils.py:65-96: the amax buffer receives
    amax(x) (as fp32) and the cast uses the scale already stored ([1]-shaped => fp32
    product).  Returns (bits, new_amax_buffer_value)."""
    amax = tensor_to_amax(x, dtype)
    return cast_to_fp8(x, dtype, stored_scale, fp8, FP32), np.float32(amax)


def dequant(bits: np.ndarray, fp8: str, scale, orig_dtype: str) -> np.ndarray:
    """`_data.to(orig_dtype) / _scale`, float8_experimental/float8_tensor.py:208.
    Returns values of `orig_dtype` widened to float32."""
    v = round_f32_to(fp8_decode(bits, fp8), orig_dtype)
    with np.errstate(divide="ignore", invalid="ignore"):
        return round_f32_to(v / np.float32(scale), orig_dtype)


# ---------------------------------------------------------------------------
# RMSNorm as the producer of a cast input
# ---------------------------------------------------------------------------
_NORM_THREADS = 256  # summation order of the row's sum of squares: 256 partial sums of 8-element chunks


def rmsnorm_rstd(x: np.ndarray, dtype: str, eps: float) -> np.ndarray:
    """1 / sqrt(mean(x^2) + eps) per row in fp32 with a FIXED summation order, so that the
    result is reproducible to the bit: partial sum t adds fl(x*x) of the 8-element chunks c with
    c % 256 == t in increasing order, the 256 partial sums are combined by xor butterflies
    (offsets 16, 8, 4, 2, 1 inside each group of 32, then 4, 2, 1 over the 8 group sums).
    `_norm` of float8_experimental/benchmarks/profile_linear_float8.py:69-70 with the
    reduction order pinned."""
    v = to_f32(x, dtype)
    rows, cols = v.shape
    chunks = -(-cols // 8)
    iters = -(-chunks // _NORM_THREADS)
    padded = np.zeros((rows, iters * _NORM_THREADS * 8), dtype=np.float32)
    padded[:, :cols] = v
    sq = (padded * padded).reshape(rows, iters, _NORM_THREADS, 8)  # fl(x*x)
    part = np.zeros((rows, _NORM_THREADS), dtype=np.float32)
    for it in range(iters):
        for j in range(8):
            part = part + sq[:, it, :, j]  # fp32 add, one element per partial sum at a time
    lanes = part.reshape(rows, _NORM_THREADS // 32, 32)
    idx = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        lanes = lanes + lanes[:, :, idx ^ off]
    warp = lanes[:, :, 0]  # every lane of a group holds the same sum
    idx8 = np.arange(_NORM_THREADS // 32)
    for off in (4, 2, 1):
        warp = warp + warp[:, idx8 ^ off]
    total = warp[:, 0]
    mean = total / np.float32(cols)
    with np.errstate(divide="ignore", invalid="ignore"):
        return (np.float32(1.0) / np.sqrt(mean + np.float32(eps))).astype(np.float32)


def rmsnorm(x: np.ndarray, dtype: str, weight: np.ndarray, eps: float):
    """y = RN_T(float(RN_T(x * rstd)) * w): RMSNorm.forward of
    float8_experimental/benchmarks/profile_linear_float8.py:72-74 for x and weight of one
    dtype T.  Returns (y widened to float32, rstd)."""
    rstd = rmsnorm_rstd(x, dtype, eps)
    o = round_f32_to(to_f32(x, dtype) * rstd[:, None], dtype)
    y = round_f32_to(o * to_f32(weight, dtype)[None, :], dtype)
    return y, rstd


def rmsnorm_cast_dynamic(x: np.ndarray, dtype: str, weight: np.ndarray, eps: float, fp8: str):
    """The dynamic cast (float8_experimental/float8_scaling_utils.py:33-62) applied to the
    RMSNorm output without materialising it.  Returns (bits, scale, amax, rstd)."""
    y, rstd = rmsnorm(x, dtype, weight, eps)
    bits, scale, amax = cast_dynamic(from_f32(y, dtype), dtype, fp8)
    return bits, scale, amax, rstd


def swiglu(a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
    """y = RN_T(float(RN_T(silu(a))) * b) with silu(a) = a / (1 + exp(-a)) in fp32:
    `F.silu(self.w1(x)) * self.w3(x)` of
    float8_experimental/benchmarks/profile_linear_float8.py:117-118.  exp is numpy's float32 exp,
    which may differ from another math library's in the last bit.  Returns y widened to float32."""
    a32, b32 = to_f32(a, dtype), to_f32(b, dtype)
    with np.errstate(over="ignore", invalid="ignore"):
        s = a32 / (np.float32(1.0) + np.exp(-a32, dtype=np.float32))
    return round_f32_to(round_f32_to(s.astype(np.float32), dtype) * b32, dtype)


def swiglu_cast_dynamic(a: np.ndarray, b: np.ndarray, dtype: str, fp8: str):
    """The dynamic cast (float8_experimental/float8_scaling_utils.py:33-62) applied to the
    SwiGLU gate output without materialising it.  Returns (bits, scale, amax)."""
    y = swiglu(a, b, dtype)
    return cast_dynamic(from_f32(y, dtype), dtype, fp8)


# ---------------------------------------------------------------------------
# delayed-scaling bookkeeping
# ---------------------------------------------------------------------------
def init_amax_history(amax: np.float32, history: np.ndarray, fp8: str, x_dtype: str):
    """float8_experimental/float8_scaling_utils.py:99-125: first-iteration init.
    history[0] = amax; scale = amax_to_scale(max(history)) in fp32 arithmetic with the
    fp16 clamp keyed on x's dtype.  Returns (cur_amax, history, scale)."""
    h = np.array(history, dtype=np.float32, copy=True)
    h[0] = amax
    hmax = np.float32(np.nan) if np.isnan(h).any() else h.max()
    return np.float32(amax), h, np.float32(amax_to_scale(hmax, fp8, x_dtype, FP32))


def sync_amax_and_scale(amax: np.ndarray, history: np.ndarray, fp8_max_kind, x_dtype: str,
                        write_back_history: bool = False):
    """float8_experimental/float8_linear_utils.py:286-319 with `_update_history_stack`
    (:37-56) and `amax_history_to_scale_stack` (float8_utils.py:80-99).

    amax [R] fp32, history [R, H] fp32, `fp8_max_kind` a list of R format names.
    Per row: rolled = [amax, h[0..H-2]]; scale = amax_to_scale(max(rolled)) in fp32.
    The reference rolls a stacked COPY of the module buffers and never writes it back
    (:291-302), so by default the returned history equals the input history; pass
    `write_back_history=True` for the rolled one."""
    amax = np.asarray(amax, dtype=np.float32)
    history = np.asarray(history, dtype=np.float32)
    rolled = np.roll(history, 1, axis=1)
    rolled[:, 0] = amax
    row_max = np.where(np.isnan(rolled).any(axis=1), np.float32(np.nan), rolled.max(axis=1))
    scales = np.empty_like(amax)
    for kind in set(fp8_max_kind):
        sel = np.array([k == kind for k in fp8_max_kind])
        scales[sel] = amax_to_scale(row_max[sel], kind, x_dtype, FP32)
    return scales, (rolled if write_back_history else history.copy())


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def mm_float8_emulated(a_bits, a_fp8, a_scale, b_bits, b_fp8, b_scale, out_dtype: str) -> np.ndarray:
    """float8_experimental/float8_aten_api.py:16-28:
    `(m1.float()/s1) @ (m2.float()/s2)` in fp32, rounded to the output dtype.
    a_bits [M,K], b_bits [K,N] (any strides).  Returns values widened to float32."""
    with np.errstate(divide="ignore", invalid="ignore"):
        a = fp8_decode(a_bits, a_fp8) / np.float32(a_scale)
        b = fp8_decode(b_bits, b_fp8) / np.float32(b_scale)
    return round_f32_to(a @ b, out_dtype)


def float8_linear_fwd_bwd(x, w, go, dtype: str = BF16):
    """One Float8Linear forward+backward with dynamic scaling for all three tensors
    and no bias: float8_experimental/float8_linear.py:356-373 (forward) and :65-95
    (backward), casts per float8_scaling_utils.py:33-62 and :188-216.

    x [M,K], w [N,K], go [M,N] in `dtype` storage.  Returns a dict with the fp8 bits,
    scales and the three GEMM results (widened to float32)."""
    x8, sx, ax = cast_dynamic(x, dtype, E4M3)
    w8, sw, aw = cast_dynamic(w, dtype, E4M3)
    g8, sg, ag = cast_dynamic(go, dtype, E5M2)
    y = mm_float8_emulated(x8, E4M3, sx, w8.T, E4M3, sw, dtype)
    dx = mm_float8_emulated(g8, E5M2, sg, w8, E4M3, sw, dtype)
    dw = mm_float8_emulated(g8.T, E5M2, sg, x8, E4M3, sx, dtype)
    return dict(x8=x8, w8=w8, g8=g8, sx=sx, sw=sw, sg=sg, ax=ax, aw=aw, ag=ag, y=y, dx=dx, dw=dw)


def sqnr_db(ref: np.ndarray, got: np.ndarray) -> float:
    """float8_experimental/float8_utils.py:142-154 (`compute_error`)."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    return float(20.0 * np.log10(np.linalg.norm(ref) / np.linalg.norm(ref - got)))
