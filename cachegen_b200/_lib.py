"""ctypes binding of libcachegen_b200.so (declarations follow include/cachegen_b200.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# CACHEGEN_B200_LIB selects another build of the library (same ABI), e.g. one kept outside the package
LIB_PATH = os.environ.get("CACHEGEN_B200_LIB") or os.path.join(_HERE, "libcachegen_b200.so")

CG_F16, CG_BF16 = 0, 1
CG_MAX_TOKENS_PER_STREAM = 256
CG_MAX_LP = 64
CG_GROUP_CHANNELS = 128
CG_MAX_DECODE_JOBS = 40
CG_S_STREAM_OVERFLOW, CG_S_BAD_LENGTHS, CG_S_BAD_SYMBOL, CG_S_COUNT_OVERFLOW, CG_S_BAD_TABLE = 1, 2, 4, 8, 16
CG_TABLES_CDF, CG_TABLES_COUNTS, CG_TABLES_SPARSE = 0, 1, 2
CG_LENGTHS_I32, CG_LENGTHS_U16 = 0, 1
CG_E_CUDA = -8


def stream_capacity(ntokens):
    return 2 * ntokens + 8


class DecodeJob(ctypes.Structure):
    """cg_decode_job"""
    _fields_ = [
        ("tables", ctypes.c_void_p),
        ("bytes", ctypes.c_void_p),
        ("lengths", ctypes.c_void_p),
        ("group_off", ctypes.c_void_p),
        ("scales_k", ctypes.c_void_p),
        ("scales_v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("table_row_off", ctypes.c_void_p),
        ("nbytes", ctypes.c_int64),
        ("tables_nbytes", ctypes.c_int64),
        ("ntokens", ctypes.c_int32),
        ("scale_stride", ctypes.c_int32),
        ("table_kind", ctypes.c_int32),
        ("length_kind", ctypes.c_int32),
    ]


class WorkspaceSizes(ctypes.Structure):
    """cg_workspace_sizes"""
    _fields_ = [(n, ctypes.c_int64) for n in ("nsub", "scratch_stride", "encode_scratch", "encode_lengths",
                                              "encode_group_off", "encode_sub_off", "decode_group_off", "symbols")]


EXPORTS = [
    "cg_version", "cg_status_string", "cg_last_cuda_error", "cg_workspace_bytes",
    "cg_calculate_cdf", "cg_encode_padded", "cg_decode_padded", "cg_decode_prefsum", "cg_decode_prefsum_warp",
    "cg_quantize_cdf", "cg_row_absmax", "cg_quantize_cdf_scaled", "cg_pack_sparse_tables", "cg_encode_chunk", "cg_compact_streams",
    "cg_decode_offsets", "cg_decode_dequant", "cg_decode_dequant_static",
    "cg_quantize_cdf_delta", "cg_decode_dequant_delta",
]
CG_STATIC_OFFSET_ENTRIES = 131072

_lib = None


class CacheGenLibraryMissing(ImportError):
    pass


def lib():
    """Loads the CUDA library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise CacheGenLibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m cachegen_b200.build` "
            "(nvcc, sm_100a); cachegen_b200 has no CPU or PyTorch fallback")
    L = ctypes.CDLL(LIB_PATH)
    p, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    S3 = ctypes.POINTER(ctypes.c_int64)
    L.cg_version.restype = ctypes.c_char_p
    L.cg_status_string.restype = ctypes.c_char_p
    L.cg_status_string.argtypes = [i]
    L.cg_last_cuda_error.restype = ctypes.c_char_p
    L.cg_workspace_bytes.argtypes = [i, i, i, ctypes.POINTER(WorkspaceSizes)]
    L.cg_calculate_cdf.argtypes = [p, S3, i, i, i, i, p, p]
    L.cg_encode_padded.argtypes = [p, p, S3, i, i, i, i, p, i64, p, p, p]
    L.cg_decode_padded.argtypes = [p, p, i64, p, p, S3, i, i, i, i, p, p]
    L.cg_decode_prefsum.argtypes = [p, p, i64, p, p, S3, i, i, i, i, p, p]
    L.cg_decode_prefsum_warp.argtypes = L.cg_decode_prefsum.argtypes
    L.cg_quantize_cdf.argtypes = [p, i, i64, i64, i64, i64, i, i, i, i, p, i, p, p, p, p, p, p, p]
    L.cg_row_absmax.argtypes = [p, i, i64, i64, i64, i64, i, i, i, i, p, p]
    L.cg_quantize_cdf_scaled.argtypes = [p, i, i64, i64, i64, i64, i, i, i, i, p, i, p, p, p, p, p, p, p]
    L.cg_pack_sparse_tables.argtypes = [p, p, p, i, i, p, p, p, p, p]
    L.cg_encode_chunk.argtypes = [p, p, i, i, i, i, p, i64, p, p, p, p, p]
    L.cg_compact_streams.argtypes = [p, i64, p, p, p, i, i, i, p, p]
    L.cg_decode_offsets.argtypes = [ctypes.POINTER(DecodeJob), i, i, i, p, p, p]
    L.cg_decode_dequant.argtypes = [ctypes.POINTER(DecodeJob), i, i, i, i, i, p, i, i, i64, i64, i64, i64, p, p]
    L.cg_decode_dequant_static.argtypes = L.cg_decode_dequant.argtypes
    L.cg_quantize_cdf_delta.argtypes = [p, i, i64, i64, i64, i64, i, i, i, i, p, i, i, p, p, p, p, p, p, p, p]
    L.cg_decode_dequant_delta.argtypes = [ctypes.POINTER(DecodeJob), i, i, i, i, i, p, i, p, i, i, i64, i64, i64, i64, p, p]
    for name in EXPORTS:
        fn = getattr(L, name)
        if name not in ("cg_version", "cg_status_string", "cg_last_cuda_error"):
            fn.restype = i
    _lib = L
    return L


def workspace_sizes(nrows, ntokens, nchannels) -> WorkspaceSizes:
    """cg_workspace_bytes: sizes of the caller-allocated buffers of the fused calls for one chunk."""
    out = WorkspaceSizes()
    check(lib().cg_workspace_bytes(int(nrows), int(ntokens), int(nchannels), ctypes.byref(out)), "cg_workspace_bytes")
    return out


def strides3(t):
    s = t.stride()
    return (ctypes.c_int64 * 3)(s[0], s[1], s[2])


def check(rc, what):
    """Turns a negative return code into the RuntimeError a torch extension would raise."""
    if rc == 0:
        return
    L = lib()
    msg = L.cg_status_string(rc).decode()
    if rc == CG_E_CUDA:
        msg += " (" + L.cg_last_cuda_error().decode() + ")"
    raise RuntimeError(f"{what}: {msg} [code {rc}]")


def status_text(bits):
    names = []
    if bits & CG_S_STREAM_OVERFLOW:
        names.append("an encoded stream outgrew its scratch row")
    if bits & CG_S_BAD_LENGTHS:
        names.append("stream lengths are negative or do not match the byte array")
    if bits & CG_S_BAD_SYMBOL:
        names.append("a symbol outside the table was met while encoding")
    if bits & CG_S_COUNT_OVERFLOW:
        names.append("a histogram count does not fit the byte-count tables")
    if bits & CG_S_BAD_TABLE:
        names.append("sparse table offsets reach past the table set")
    return "; ".join(names) if names else "ok"
