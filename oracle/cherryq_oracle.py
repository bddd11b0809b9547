"""CPU oracle for the CherryQ quantized-linear path (TEST INFRASTRUCTURE ONLY).

This file restates, in plain numpy, the arithmetic of the reference project
wangitu/Mixed-precision-CUDA-kernel for its quantized linear layer.  It is the
checker the GPU kernels are compared against.  It is never imported by the
product package: only the test-suite, the smoke test and the CPU-baseline leg
of the benchmark may use it.

Parity status: PINNED.  Every function here is checked bit-for-bit (integer
and fp16 outputs) against the reference's own Python code executed on seeded
inputs; the frozen results live in tests/golden/*.npz together with the script
that produced them (tests/golden/make_golden.py).

Reference citations are paths inside the reference project:

* llama/quantizer.py:136-170   FullSymQuantizer (iinfo, get_scaling_factor,
                               quantize, dequantize, transform)
* llama/quantizer.py:10-34     get_max_input (row-wise |max|)
* llama/cherry_linear.py:33    num_cherries
* llama/cherry_linear.py:69-75 group scales over the compacted axis
* llama/cherry_linear.py:77-99 fake-quant weight (_adjust_weight)
* llama/qlinear.py:67-118      pack (bit order of the uint8 rows)
* llama/qlinear.py:120-162     unpack (dense fp16 weight)
* llama/qlinear.py:164-199     forward
* csrc/quant_cuda_kernel.cu:718-835 (4-bit) / :558-672 (3-bit) matvec kernels
* csrc/quant_cuda_kernel.cu:869-922 / :956-1010 Dequantize{3,4}Normal
"""
from __future__ import annotations

import math

import numpy as np

F16 = np.float16
F32 = np.float32


# --------------------------------------------------------------------------
# quantizer (llama/quantizer.py:136-170)
# --------------------------------------------------------------------------
def iinfo_min(bits: int) -> int:
    """FullSymQuantizer.iinfo(bits).min  (llama/quantizer.py:141-146)."""
    return -(2 ** (bits - 1))


def num_cherries(in_features: int, cherry_fraction: float) -> int:
    """llama/cherry_linear.py:33 and llama/qlinear.py:37."""
    return math.ceil(in_features * cherry_fraction) // 8 * 8


def _opmath_binary(a, b, op, dtype):
    """torch computes fp16 element-wise arithmetic in fp32 and rounds once to
    fp16; fp32 stays fp32."""
    r = op(a.astype(F32), b.astype(F32) if isinstance(b, np.ndarray) else F32(b))
    return r.astype(dtype)


def get_scaling_factor(w: np.ndarray, bits: int) -> np.ndarray:
    """FullSymQuantizer.get_scaling_factor with layerwise=False, clip_val=None
    (llama/quantizer.py:148-152, 10-34): s = (max|w| + 1e-6) / 2^(bits-1),
    evaluated in w's dtype, one value per row."""
    dt = w.dtype
    mx = np.max(np.abs(w), axis=-1, keepdims=True)
    s = _opmath_binary(mx, 1e-6, np.add, dt)
    s = _opmath_binary(s, float(2 ** (bits - 1)), np.divide, dt)
    return s


def group_scales(normal_w: np.ndarray, bits: int, group_size: int) -> np.ndarray:
    """cherry_linear.QuantLinear._get_scaling_factors (llama/cherry_linear.py:69-75):
    one scale per (row, group) over the compacted axis; the last group may be
    partial.  Returns (out, num_group) in normal_w's dtype."""
    cols = []
    for i in range(0, normal_w.shape[-1], group_size):
        cols.append(get_scaling_factor(normal_w[:, i:i + group_size], bits))
    return np.concatenate(cols, axis=-1)


def expand_scales(s: np.ndarray, group_size: int, width: int) -> np.ndarray:
    """repeat_interleave(group_size)[:, :width] (llama/qlinear.py:81)."""
    return np.repeat(s, group_size, axis=1)[:, :width]


def quantize(w: np.ndarray, s: np.ndarray, bits: int) -> np.ndarray:
    """FullSymQuantizer.quantize (llama/quantizer.py:154-158):
    round(clamp((w / s).float(), -qmax, qmax) - 0.5) as int32, qmax = 2^(b-1) - 0.01.
    The division happens in the promoted dtype of (w, s)."""
    dt = np.result_type(w.dtype, s.dtype)
    q = (w.astype(F32) / s.astype(F32)).astype(dt).astype(F32)
    qmax = F32(2 ** (bits - 1) - 1e-2)
    q = np.clip(q, -qmax, qmax)
    return np.rint(q - F32(0.5)).astype(np.int32)


def dequantize(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    """FullSymQuantizer.dequantize (llama/quantizer.py:160-163): (q + 0.5) * s in s's dtype."""
    dt = s.dtype
    a = _opmath_binary(q.astype(dt), 0.5, np.add, dt)
    return _opmath_binary(a, s, np.multiply, dt)


def transform(w: np.ndarray, s: np.ndarray, bits: int) -> np.ndarray:
    """FullSymQuantizer.transform (llama/quantizer.py:165-170), the fake-quant
    used by the training-side layer; everything in w's dtype."""
    dt = w.dtype
    qmax = 2 ** (bits - 1) - 1e-2
    r = _opmath_binary(w, s, np.divide, dt)
    r = np.clip(r, dt.type(-qmax), dt.type(qmax))
    r = _opmath_binary(r, 0.5, np.subtract, dt)
    r = np.rint(r.astype(F32)).astype(dt)
    r = _opmath_binary(r, 0.5, np.add, dt)
    return _opmath_binary(r, s, np.multiply, dt)


# --------------------------------------------------------------------------
# index handling
# --------------------------------------------------------------------------
def normal_columns(in_features: int, cherry_sorted: np.ndarray) -> np.ndarray:
    """Columns that stay quantized, in original order (llama/qlinear.py:75-76)."""
    mask = np.ones(in_features, dtype=bool)
    mask[cherry_sorted.astype(np.int64)] = False
    return np.nonzero(mask)[0]


def compact_to_original(k: int, cherry_sorted: np.ndarray) -> int:
    """The kernel's upper-bound search (csrc/quant_cuda_kernel.cu:785-795):
    number of cherries with idx[m] - m <= k, added to the compact index k."""
    low, high = 0, len(cherry_sorted)
    while low < high:
        mid = (low + high) >> 1
        if int(cherry_sorted[mid]) - mid <= k:
            low = mid + 1
        else:
            high = mid
    return k + low


# --------------------------------------------------------------------------
# bit packing (llama/qlinear.py:86-118) and unpacking (:124-148)
# --------------------------------------------------------------------------
def pack_codes(u: np.ndarray, bits: int) -> np.ndarray:
    """u: (K', N) unsigned codes (uint8, 0 <= u < 2^bits), K' % 8 == 0.
    Returns the reference's qweight (K'//8*bits, N) uint8.

    4-bit: row r = u[2r] | u[2r+1] << 4                   (qlinear.py:89-94)
    3-bit: each 8 codes form a little-endian 24-bit word, code i at bits
           3i..3i+2, spread over 3 consecutive rows       (qlinear.py:95-114)
    """
    kp, n = u.shape
    assert kp % 8 == 0
    u = u.astype(np.uint32)
    if bits == 4:
        return (u[0::2] | (u[1::2] << 4)).astype(np.uint8)
    if bits == 3:
        g = u.reshape(kp // 8, 8, n)
        word = np.zeros((kp // 8, n), dtype=np.uint32)
        for i in range(8):
            word |= g[:, i, :] << (3 * i)
        out = np.empty((kp // 8, 3, n), dtype=np.uint8)
        out[:, 0] = word & 0xFF
        out[:, 1] = (word >> 8) & 0xFF
        out[:, 2] = (word >> 16) & 0xFF
        return out.reshape(kp // 8 * 3, n)
    raise NotImplementedError(f"{bits} bit")


def unpack_codes(qweight: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of pack_codes: (R, N) uint8 -> (K', N) uint8 codes."""
    r, n = qweight.shape
    q = qweight.astype(np.uint32)
    if bits == 4:
        out = np.empty((r * 2, n), dtype=np.uint8)
        out[0::2] = q & 0xF
        out[1::2] = (q >> 4) & 0xF
        return out
    if bits == 3:
        assert r % 3 == 0
        t = q.reshape(r // 3, 3, n)
        word = t[:, 0] | (t[:, 1] << 8) | (t[:, 2] << 16)
        out = np.empty((r // 3, 8, n), dtype=np.uint8)
        for i in range(8):
            out[:, i] = (word >> (3 * i)) & 0x7
        return out.reshape(r // 3 * 8, n)
    raise NotImplementedError(f"{bits} bit")


def pack(weight: np.ndarray, cherry_indices: np.ndarray, bits: int, group_size: int):
    """qlinear.QuantLinear.pack (llama/qlinear.py:67-118).

    weight: (N, K) fp16 or fp32; cherry_indices: (C,) any order.
    Returns dict(cherry_indices int16 (C,), cherry_weight fp16 (C, N),
    qweight uint8 (K'//8*bits, N), scales fp16 (NG, N))."""
    n, k = weight.shape
    if group_size == -1:
        group_size = k
    idx = np.sort(cherry_indices.astype(np.int64))
    cherry_weight = weight.T[idx].astype(F16)
    ncols = normal_columns(k, idx)
    normal = weight[:, ncols]
    scales = group_scales(normal, bits, group_size).astype(F16)          # (N, NG)
    s_full = expand_scales(scales, group_size, normal.shape[1])
    q = quantize(normal, s_full, bits)                                   # (N, K') int32
    u = (q.T - iinfo_min(bits)).astype(np.uint8)                         # (K', N)
    return dict(
        cherry_indices=idx.astype(np.int16),
        cherry_weight=np.ascontiguousarray(cherry_weight),
        qweight=pack_codes(u, bits),
        scales=np.ascontiguousarray(scales.T),
    )


def unpack(qweight, scales, cherry_weight, cherry_indices, bits, group_size, in_features):
    """qlinear.QuantLinear.unpack (llama/qlinear.py:120-162): dense (N, K) fp16."""
    if group_size == -1:
        group_size = in_features
    n = qweight.shape[1]
    u = unpack_codes(qweight, bits)                                      # (K', N)
    q = u.T.astype(np.int8) + np.int8(iinfo_min(bits))                   # (N, K')
    s = expand_scales(np.ascontiguousarray(scales.T), group_size, q.shape[1])
    deq = dequantize(q, s.astype(F16))
    w = np.zeros((n, in_features), dtype=F16)
    idx = cherry_indices.astype(np.int64)
    w[:, normal_columns(in_features, idx)] = deq
    w[:, idx] = cherry_weight.T
    return w


def fake_quant_weight(weight, cherry_indices, bits, group_size):
    """cherry_linear.QuantLinear._adjust_weight(ste=False) (llama/cherry_linear.py:77-99):
    cherries untouched, the rest fake-quantized with scales in the weight dtype."""
    n, k = weight.shape
    if group_size == -1:
        group_size = k
    idx = cherry_indices.astype(np.int64)
    ncols = normal_columns(k, np.sort(idx))
    normal = weight[:, ncols]
    s = group_scales(normal, bits, group_size)
    s = expand_scales(s, group_size, normal.shape[1])
    out = weight.copy()
    out[:, ncols] = transform(normal, s, bits)
    return out


# --------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------
def forward_dense_fp64(x, dense_w):
    """The parity target for the matvec / GEMM kernels: x.float() @ unpack().float().T
    (llama/qlinear.py:183-195), accumulated in fp64 so the target itself has no
    summation-order noise."""
    return x.astype(np.float64) @ dense_w.astype(np.float64).T


def kernel_forward(x, qweight, cherry_weight, cherry_indices, scales, bits, group_size):
    """What the reference CUDA kernel sums, restated without its fp16 atomics
    (csrc/quant_cuda_kernel.cu:718-835 4-bit, :558-672 3-bit): for every compact
    index k the code u is decoded, (u - off) * scale[group(k)] multiplies
    x[:, compact_to_original(k)], plus the cherry rows times x[:, idx].  fp64."""
    m, kfull = x.shape
    off = 2 ** (bits - 1) - 0.5
    u = unpack_codes(qweight, bits).astype(np.float64)                   # (K', N)
    kp = u.shape[0]
    orig = np.array([compact_to_original(k, cherry_indices) for k in range(kp)])
    grp = np.arange(kp) // group_size
    w = (u - off) * scales.astype(np.float64)[grp]                       # (K', N)
    y = x.astype(np.float64)[:, orig] @ w
    y += x.astype(np.float64)[:, cherry_indices.astype(np.int64)] @ cherry_weight.astype(np.float64)
    return y


def dequantize_normal(qweight, scales_f32, bits, group_size):
    """Intended semantics of Dequantize{3,4}Normal (csrc/quant_cuda_kernel.cu:869-922,
    :956-1010): out[k', n] = (u - off) * scale[k' // group, n] in fp32, compact axis,
    no cherries.  (The reference's 4-bit launcher strides by the 3-bit block height,
    :934 and :964, and is wrong past the first 128 rows; this is the 3-bit kernel's
    behaviour applied to 4-bit codes.)"""
    off = F32(2 ** (bits - 1) - 0.5)
    u = unpack_codes(qweight, bits).astype(F32)
    grp = np.arange(u.shape[0]) // group_size
    return (u - off) * scales_f32.astype(F32)[grp]


# --------------------------------------------------------------------------
# synthetic layers (shapes and distributions of the benchmark configurations)
# --------------------------------------------------------------------------
def make_layer(k, n, bits, group_size, cherry_fraction=1 / 256, seed=1234, dtype=F16):
    """Dense W ~ N(0, 0.02); C cherry columns drawn without replacement and
    overwritten with N(0, 0.2); returns (W, cherry_indices int32 unsorted)."""
    rng = np.random.default_rng(seed)
    w = rng.normal(0.0, 0.02, size=(n, k)).astype(F32)
    c = num_cherries(k, cherry_fraction)
    idx = rng.permutation(k)[:c].astype(np.int32)
    if c:
        w[:, idx] = rng.normal(0.0, 0.2, size=(n, c)).astype(F32)
    return w.astype(dtype), idx
