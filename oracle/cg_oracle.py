"""numpy/ctypes front end of the CPU oracle (oracle/cg_oracle.c).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, from the smoke check and from
the benchmark's host-CPU baseline leg; never from the product package.

All arrays are numpy; 16-bit floats travel as uint16 bit patterns with a dtype
code (0 = fp16, 1 = bf16) so that no conversion happens outside the C code.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcg_oracle.so")
_lib = None

F16, BF16 = 0, 1


def build(force=False):
    src = os.path.join(_HERE, "cg_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libcg_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        i64, i32, p = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        _lib.cgo_quantize.argtypes = [p, i32, i32, i32, i32, p, p, p]
        _lib.cgo_quantize.restype = None
        _lib.cgo_dequantize.argtypes = [p, i64, i64, i64, i32, i32, i32, p, p, i32, p, i64, i64, i64, i32]
        _lib.cgo_dequantize.restype = None
        _lib.cgo_quantize_delta.argtypes = [p, i32, i32, i32, i32, p, p, i32, p, p]
        _lib.cgo_quantize_delta.restype = i32
        _lib.cgo_dequantize_delta.argtypes = [p, i32, i32, i32, p, p, i32, p, i32, p, i64, i64, i64, i32]
        _lib.cgo_dequantize_delta.restype = None
        _lib.cgo_calculate_cdf.argtypes = [p, i64, i64, i64, i32, i32, i32, i32, p]
        _lib.cgo_calculate_cdf.restype = i32
        _lib.cgo_encode_stream.argtypes = [p, i32, p, i64, i32, p, i64, p]
        _lib.cgo_encode_stream.restype = i64
        _lib.cgo_decode_stream.argtypes = [p, i32, p, i64, i32, p, i64]
        _lib.cgo_decode_stream.restype = None
        _lib.cgo_encode_chunk.argtypes = [p, i32, p, i64, i64, i64, i32, i32, i32, p, i64, p, p, i64, i32]
        _lib.cgo_encode_chunk.restype = i64
        _lib.cgo_decode_chunk.argtypes = [p, i32, p, p, i32, i32, i32, p, i64, i64, i64, i32]
        _lib.cgo_decode_chunk.restype = None
        _lib.cgo_decode_dequant_chunk.argtypes = [p, i32, p, p, i32, i32, i32, p, p, i32, p, i64, i64, i64, i32, i32]
        _lib.cgo_decode_dequant_chunk.restype = None
        _lib.cgo_f16_to_f32.argtypes = [p, p, i64, i32]
        _lib.cgo_f32_to_f16.argtypes = [p, p, i64, i32]
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _estrides(a):
    return [s // a.itemsize for s in a.strides]


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def half_to_float(bits, dtype=F16):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().cgo_f16_to_f32(_ptr(bits), _ptr(out), bits.size, dtype)
    return out


def float_to_half(x, dtype=F16):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().cgo_f32_to_f16(_ptr(x), _ptr(out), x.size, dtype)
    return out


def quantize(x_bits, bins, dtype=F16):
    """x_bits uint16 [rows, T, C]; bins float32 [rows] -> (sym int8 [rows,T,C], maxes uint16 [rows,T,1])."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, T, C = x_bits.shape
    bins = np.ascontiguousarray(bins, dtype=np.float32)
    assert bins.shape == (rows,)
    sym = np.empty((rows, T, C), dtype=np.int8)
    maxes = np.empty((rows, T, 1), dtype=np.uint16)
    lib().cgo_quantize(_ptr(x_bits), dtype, rows, T, C, _ptr(bins), _ptr(sym), _ptr(maxes))
    return sym, maxes


def quantize_delta(x_bits, bins, res_bins, group, dtype=F16):
    """Anchor-token delta quantiser (cgo_quantize_delta): rows with res_bins > 0 code every token that is
    not the first of its group of `group` as a residual against the dequantised anchor."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, T, C = x_bits.shape
    bins = np.ascontiguousarray(bins, dtype=np.float32)
    res_bins = np.ascontiguousarray(res_bins, dtype=np.float32)
    assert bins.shape == (rows,) and res_bins.shape == (rows,)
    sym = np.empty((rows, T, C), dtype=np.int8)
    maxes = np.empty((rows, T, 1), dtype=np.uint16)
    rc = lib().cgo_quantize_delta(_ptr(x_bits), dtype, rows, T, C, _ptr(bins), _ptr(res_bins), int(group), _ptr(sym),
                                  _ptr(maxes))
    if rc:
        raise ValueError("bad delta settings (group < 1, or residual bins outside [4, bins])")
    return sym, maxes


def dequantize_delta(sym, bins, res_bins, group, maxes, max_dtype=F16, out_dtype=F16):
    """The decoder's side of quantize_delta: uint16 bits [rows, T, C]."""
    rows, T, C = sym.shape
    sym = np.ascontiguousarray(sym.view(np.uint8))
    bins = np.ascontiguousarray(bins, dtype=np.float32)
    res_bins = np.ascontiguousarray(res_bins, dtype=np.float32)
    maxes = np.ascontiguousarray(maxes, dtype=np.uint16).reshape(rows, T)
    out = np.empty((rows, T, C), dtype=np.uint16)
    st = _estrides(out)
    lib().cgo_dequantize_delta(_ptr(sym), rows, T, C, _ptr(bins), _ptr(res_bins), int(group), _ptr(maxes), max_dtype,
                               _ptr(out), st[0], st[1], st[2], out_dtype)
    return out


def dequantize(sym, bins, maxes, max_dtype=F16, out_dtype=F16, out=None, out_strides=None):
    """sym uint8 [rows,T,C] (any strides) -> uint16 bits; default output [rows,T,C] contiguous."""
    rows, T, C = sym.shape
    sym = sym.view(np.uint8)
    bins = np.ascontiguousarray(bins, dtype=np.float32)
    maxes = np.ascontiguousarray(maxes, dtype=np.uint16).reshape(rows, T)
    if out is None:
        out = np.empty((rows, T, C), dtype=np.uint16)
        out_strides = _estrides(out)
    ss = _estrides(sym)
    lib().cgo_dequantize(_ptr(sym), ss[0], ss[1], ss[2], rows, T, C, _ptr(bins), _ptr(maxes), max_dtype,
                         _ptr(out), out_strides[0], out_strides[1], out_strides[2], out_dtype)
    return out


def calculate_cdf(sym, max_bins):
    """sym int8 [rows,T,C] (any strides) -> int16 [rows, C, max_bins+1]."""
    rows, T, C = sym.shape
    sym = sym.view(np.int8)
    cdf = np.empty((rows, C, max_bins + 1), dtype=np.int16)
    s = _estrides(sym)
    rc = lib().cgo_calculate_cdf(_ptr(sym), s[0], s[1], s[2], rows, T, C, max_bins, _ptr(cdf))
    if rc != 0:
        raise ValueError(f"cgo_calculate_cdf failed: {rc}")
    return cdf


def encode_stream(cdf_row, symbols, cap=None):
    cdf_row = np.ascontiguousarray(cdf_row).view(np.uint16)
    symbols = np.ascontiguousarray(symbols, dtype=np.int8)
    n = symbols.size
    cap = cap if cap is not None else 2 * n + 8
    out = np.zeros(cap, dtype=np.uint8)
    ov = ctypes.c_int(0)
    ln = lib().cgo_encode_stream(_ptr(cdf_row), cdf_row.size, _ptr(symbols), 1, n, _ptr(out), cap, ctypes.byref(ov))
    if ov.value:
        raise OverflowError(f"stream needs {ln} bytes, capacity {cap}")
    return out[:ln].copy()


def decode_stream(cdf_row, stream, n):
    cdf_row = np.ascontiguousarray(cdf_row).view(np.uint16)
    stream = np.ascontiguousarray(stream, dtype=np.uint8)
    out = np.empty(n, dtype=np.uint8)
    lib().cgo_decode_stream(_ptr(cdf_row), cdf_row.size, _ptr(stream), stream.size, n, _ptr(out), 1)
    return out


def encode_chunk(cdf, sym, threads=None, cap=None):
    """One sub-chunk: cdf int16 [rows,C,Lp], sym int8 [rows,T,C] (strided ok).
    Returns (bytes uint8 [sum len], lengths int32 [rows, C])."""
    rows, T, C = sym.shape
    cdf = np.ascontiguousarray(cdf, dtype=np.int16)
    Lp = cdf.shape[2]
    sym = sym.view(np.int8)
    s = _estrides(sym)
    cap = cap if cap is not None else 2 * T + 8
    scratch = np.empty(rows * C * cap, dtype=np.uint8)
    lengths = np.empty((rows, C), dtype=np.int32)
    out = np.empty(rows * C * cap, dtype=np.uint8)
    total = lib().cgo_encode_chunk(_ptr(cdf), Lp, _ptr(sym), s[0], s[1], s[2], rows, T, C, _ptr(scratch), cap,
                                   _ptr(lengths), _ptr(out), out.size, threads or host_threads())
    if total < 0:
        raise OverflowError("a stream exceeded the per-stream capacity")
    return out[:total].copy(), lengths


def decode_chunk(cdf, stream_bytes, lengths, T, threads=None, out=None):
    """Inverse of encode_chunk -> uint8 symbols [rows, T, C] (or into `out`, strided ok)."""
    cdf = np.ascontiguousarray(cdf, dtype=np.int16)
    rows, C, Lp = cdf.shape
    prefsum = np.cumsum(np.asarray(lengths, dtype=np.int64).reshape(-1))
    stream_bytes = np.ascontiguousarray(stream_bytes, dtype=np.uint8)
    if out is None:
        out = np.empty((rows, T, C), dtype=np.uint8)
    o = _estrides(out)
    lib().cgo_decode_chunk(_ptr(cdf), Lp, _ptr(stream_bytes), _ptr(prefsum), rows, T, C, _ptr(out),
                           o[0], o[1], o[2], threads or host_threads())
    return out


def decode_dequant_chunk(cdf, stream_bytes, lengths, T, bins, maxes, out, out_strides, max_dtype=F16,
                         out_dtype=F16, threads=None):
    """Timed CPU baseline body: decode one sub-chunk and write 16-bit KV into `out` (uint16 array) at
    element offset row*os0 + token*os1 + channel*os2."""
    cdf = np.ascontiguousarray(cdf, dtype=np.int16)
    rows, C, Lp = cdf.shape
    prefsum = np.cumsum(np.asarray(lengths, dtype=np.int64).reshape(-1))
    stream_bytes = np.ascontiguousarray(stream_bytes, dtype=np.uint8)
    bins = np.ascontiguousarray(bins, dtype=np.float32)
    maxes = np.ascontiguousarray(maxes, dtype=np.uint16).reshape(rows, T)
    lib().cgo_decode_dequant_chunk(_ptr(cdf), Lp, _ptr(stream_bytes), _ptr(prefsum), rows, T, C, _ptr(bins),
                                   _ptr(maxes), max_dtype, _ptr(out), out_strides[0], out_strides[1],
                                   out_strides[2], out_dtype, threads or host_threads())
    return out
