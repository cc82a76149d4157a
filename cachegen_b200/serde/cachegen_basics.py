"""CacheGenConfig and the wire dataclasses
(reference: LMCache/lmcache/storage_backend/serde/cachegen_basics.py:8-156).

The blob format is the reference's: `pickle` of a CacheGenGPUEncoderOutput whose tensors are CUDA
tensors.  So that blobs travel both ways between this package and the reference, the two wire
classes pickle under the reference's module path `lmcache.storage_backend.serde.cachegen_basics`;
when no `lmcache` package is importable, alias modules of that name are registered at import time
(see cachegen_b200.compat).
"""
import io
import os
import pickle
import threading
from dataclasses import dataclass, replace
from typing import List

import torch

CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK = 256

REFERENCE_MODULE = "lmcache.storage_backend.serde.cachegen_basics"


@dataclass
class CacheGenConfig:
    """Per-layer-group bin counts: keys in three groups, values in two (cachegen_basics.py:10-21)."""
    key_first_layers: int
    key_second_layers: int
    key_third_layers: int
    key_first_bins: int
    key_second_bins: int
    key_third_bins: int
    value_first_layers: int
    value_first_bins: int
    value_second_bins: int

    def __getitem__(self, key: str) -> int:
        return getattr(self, key)

    @property
    def num_layers(self) -> int:
        return self.key_third_layers

    @property
    def max_bins(self) -> int:
        return max(self.key_first_bins, self.key_second_bins, self.key_third_bins,
                   self.value_first_bins, self.value_second_bins)

    def with_bins_divided(self, divisor: int, minimum: int = 4) -> "CacheGenConfig":
        """A lower quality level: every bin count divided by `divisor`, not below `minimum`."""
        d = lambda b: max(minimum, b // divisor)
        return replace(self, key_first_bins=d(self.key_first_bins), key_second_bins=d(self.key_second_bins),
                       key_third_bins=d(self.key_third_bins), value_first_bins=d(self.value_first_bins),
                       value_second_bins=d(self.value_second_bins))

    def layer_slice(self, start: int, stop: int) -> "CacheGenConfig":
        """The settings of layers [start, stop) as a configuration of their own (layer-sharded runs)."""
        n = stop - start
        if not 0 <= start < stop <= self.key_third_layers:
            raise ValueError(f"bad layer range [{start}, {stop}) of {self.key_third_layers}")
        clip = lambda b: min(max(b - start, 0), n)
        return replace(self, key_first_layers=clip(self.key_first_layers), key_second_layers=clip(self.key_second_layers),
                       key_third_layers=n, value_first_layers=clip(self.value_first_layers))

    @staticmethod
    def from_model_name(model_name: str) -> "CacheGenConfig":
        """Same lookup as cachegen_basics.py:23-96: any name containing "Mistral-7B" reads the
        QUANT_LEVEL environment variable ("1", "2" or "3"; KeyError when unset), the 7B and 70B
        families have fixed settings, anything else raises ValueError."""
        family_7b = ["mistralai/Mistral-7B-Instruct-v0.2", "mistral-community/Mistral-7B-v0.2",
                     "lmsys/longchat-7b-16k"]
        family_70b = ["Yukang/LongAlpaca-70B-16k"]
        if "Mistral-7B" in model_name:
            level = os.environ["QUANT_LEVEL"]
            if level == "1":
                return CacheGenConfig(10, 20, 32, 16, 16, 12, 2, 16, 12)
            if level == "2":
                return CacheGenConfig(10, 20, 32, 32, 16, 16, 2, 32, 16)
            if level == "3":
                return CacheGenConfig(10, 20, 32, 32, 32, 32, 2, 32, 32)
            raise ValueError(f"QUANT_LEVEL must be 1, 2 or 3, got {level!r}")
        elif model_name in family_7b:
            return CacheGenConfig(10, 20, 32, 32, 16, 16, 2, 32, 16)
        elif model_name in family_70b:
            return CacheGenConfig(20, 40, 80, 32, 32, 16, 20, 32, 16)
        else:
            raise ValueError(f"Model {model_name} is not supported")


class DeltaCoding:
    """Settings of anchor-token delta coding (cg_quantize_cdf_delta / cg_decode_dequant_delta; the
    reference has no such step, so chunks written with it are only readable by this package and only by a
    deserializer given the same settings).

    group:    tokens per group, a power of two in 2..256; the first token of a group is the anchor
    divisor:  residual tokens use max(4, bins // divisor) bins
    rows:     "keys" (key rows only: keys are the smooth ones) or "all"
    """

    def __init__(self, group: int, divisor: int = 2, rows: str = "keys"):
        if group < 2 or group > CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK or group & (group - 1):
            raise ValueError(f"delta group must be a power of two in 2..256, got {group}")
        if divisor < 1:
            raise ValueError("delta divisor must be at least 1")
        if rows not in ("keys", "all"):
            raise ValueError(f"delta rows must be 'keys' or 'all', got {rows!r}")
        self.group, self.divisor, self.rows = int(group), int(divisor), rows
        self._res_bins = {}

    def residual_bins(self, key_bins: torch.Tensor, value_bins: torch.Tensor, device) -> torch.Tensor:
        """float32 [2L] on `device`: residual bin counts of the key rows then the value rows, 0 = no delta."""
        key = (str(device), key_bins.numel(), value_bins.numel())
        t = self._res_bins.get(key)
        if t is None:
            kb, vb = key_bins.detach().cpu().float(), value_bins.detach().cpu().float()
            res_k = torch.clamp(torch.div(kb, self.divisor, rounding_mode="floor"), min=4.0)
            res_v = torch.clamp(torch.div(vb, self.divisor, rounding_mode="floor"), min=4.0)
            if self.rows == "keys":
                res_v = torch.zeros_like(res_v)
            t = torch.cat((res_k, res_v)).to(device=device, dtype=torch.float32).contiguous()
            self._res_bins[key] = t
        return t

    def __repr__(self):
        return f"DeltaCoding(group={self.group}, divisor={self.divisor}, rows={self.rows!r})"


def make_key_bins(config: CacheGenConfig, device="cuda") -> torch.Tensor:
    """float32 [L] (cachegen_encoder.py:311-316 / cachegen_decoder.py:122-127)."""
    ret = torch.zeros(config.key_third_layers)
    ret.fill_(config.key_third_bins)
    ret[:config.key_second_layers] = config.key_second_bins
    ret[:config.key_first_layers] = config.key_first_bins
    return ret.to(device)


def make_value_bins(config: CacheGenConfig, device="cuda") -> torch.Tensor:
    """float32 [L] (cachegen_encoder.py:318-322 / cachegen_decoder.py:129-135)."""
    ret = torch.zeros(config.key_third_layers)
    ret.fill_(config.value_second_bins)
    ret[:config.value_first_layers] = config.value_first_bins
    return ret.to(device)


@dataclass
class CacheGenGPUBytestream:
    """One sub-chunk (<= 256 tokens) of encoded streams (cachegen_basics.py:124-131)."""
    bytestream: torch.Tensor          # uint8 [sum of lengths]: streams in (row, channel) order
    bytestream_lengths: torch.Tensor  # int32 [2L, C]
    ntokens: int

    def __getitem__(self, key: str):
        return getattr(self, key)


@dataclass
class CacheGenGPUEncoderOutput:
    """One encoded chunk (cachegen_basics.py:133-156)."""
    data_chunks: List[CacheGenGPUBytestream]
    cdf: torch.Tensor                # int16 [2L, C, Lp]
    max_tensors_key: torch.Tensor    # [L, T, 1], input dtype
    max_tensors_value: torch.Tensor  # [L, T, 1], input dtype
    num_heads: int
    head_size: int

    def __getitem__(self, key: str):
        return getattr(self, key)

    def to_bytes(self) -> bytes:
        try:
            return dump_blob(self)
        except Exception:
            # dump_blob follows torch's legacy storage stream by hand; should a torch release change
            # that format, the plain pickle is still the reference's blob (slower: torch copies every
            # CUDA tensor through pageable memory)
            f = io.BytesIO()
            pickle.dump(self, f)
            return f.getvalue()

    @staticmethod
    def from_bytes(bs: bytes) -> "CacheGenGPUEncoderOutput":
        return load_blob(bs)


# ---- writing a blob ---------------------------------------------------------------------------------------
# pickle.dump of the object gives the reference's blob, but torch pickles a CUDA tensor by copying
# its storage to pageable host memory, writing a legacy `torch.save` stream of it into one buffer,
# copying that into the pickle and the pickle into the result: 34 ms for a 30 MB chunk.  dump_blob
# writes the same bytes -- the same outer pickle, and for each storage the same legacy stream, built
# by _legacy_stream_head -- from one asynchronous copy of all tensors into pinned memory.

class _PersistentId:
    def __init__(self, pid):
        self.pid = pid


class _LegacyPickler(pickle.Pickler):
    def persistent_id(self, obj):
        return obj.pid if isinstance(obj, _PersistentId) else None


def _legacy_stream_head(dtype: torch.dtype, key: str, location: str, numel: int) -> bytes:
    """What torch.save(storage, f, _use_new_zipfile_serialization=False) writes before the storage's
    raw data (torch/serialization.py, _legacy_save): magic number, protocol version and system info
    as three pickles, the storage as a persistent id, the list of storage keys, the element count."""
    import sys
    ser = torch.serialization
    f = io.BytesIO()
    info = {"protocol_version": ser.PROTOCOL_VERSION, "little_endian": sys.byteorder == "little",
            "type_sizes": {"short": ser.SHORT_SIZE, "int": ser.INT_SIZE, "long": ser.LONG_SIZE}}
    for part in (ser.MAGIC_NUMBER, ser.PROTOCOL_VERSION, info):
        pickle.dump(part, f, protocol=ser.DEFAULT_PROTOCOL)
    storage_type = getattr(torch, torch.storage._dtype_to_storage_type_map()[dtype])
    _LegacyPickler(f, protocol=ser.DEFAULT_PROTOCOL).dump(
        _PersistentId(("storage", storage_type, key, location, numel, None)))
    pickle.dump([key], f, protocol=ser.DEFAULT_PROTOCOL)
    f.write(int(numel).to_bytes(8, sys.byteorder))
    return f.getvalue()


class _StreamedStorage:
    """Stands in for a tensor's TypedStorage while pickling: reduces to what the storage itself
    reduces to, (torch.storage._load_from_bytes, (legacy stream,))."""

    def __init__(self, stream: bytes):
        self.stream = stream

    def __reduce__(self):
        return (torch.storage._load_from_bytes, (self.stream,))


def _owns_its_storage(t: torch.Tensor) -> bool:
    return (t.layout == torch.strided and t.is_contiguous() and t.storage_offset() == 0 and not t.requires_grad and
            type(t) is torch.Tensor and t.untyped_storage().nbytes() == t.numel() * t.element_size() and
            t.dtype in torch.storage._dtype_to_storage_type_map())


_PLACEHOLDER_LEN = 1 << 16  # pickle writes byte strings of at least this size outside its frames


class _BlobPickler(pickle.Pickler):
    """Pickles the tensors whose bytes are in `raw_of` (by id) from those bytes; everything else as
    pickle.dump does.  A large storage stream is not built here: a placeholder byte string of
    _PLACEHOLDER_LEN bytes stands in for it (pickle frames it the same way: outside the frames) and
    `deferred` remembers, by the placeholder's id, the stream's head and raw bytes; _assemble puts
    them in place, so the tensor's bytes are copied once, into the final blob."""

    def __init__(self, file, raw_of: dict):
        super().__init__(file)
        self.raw_of = raw_of
        self.deferred = {}
        self.keep = []

    def reducer_override(self, obj):
        if isinstance(obj, torch.Tensor) and id(obj) in self.raw_of:
            from collections import OrderedDict
            head = _legacy_stream_head(obj.dtype, str(obj.untyped_storage()._cdata),
                                       torch.serialization.location_tag(obj.untyped_storage()), obj.numel())
            raw = self.raw_of[id(obj)]
            n = len(head) + len(raw)
            if _PLACEHOLDER_LEN <= n < (1 << 32):
                stream = bytes(_PLACEHOLDER_LEN)
                self.deferred[id(stream)] = (head, raw, n)
                self.keep.append(stream)  # ids must stay unique until the blob is assembled
            else:
                stream = b"".join((head, raw))
            storage = _StreamedStorage(stream)
            return (torch._utils._rebuild_tensor_v2,
                    (storage, 0, tuple(obj.size()), obj.stride(), False, OrderedDict()))
        return NotImplemented


class _PartsWriter:
    """File object that keeps what is written as a list of byte strings: the pickler hands a large
    byte string over as the object it was given, so nothing is copied until the final join."""

    def __init__(self):
        self.parts = []

    def write(self, b):
        self.parts.append(b if isinstance(b, bytes) else bytes(b))
        return len(b)


def _assemble(parts: list, deferred: dict) -> bytes:
    """The blob from the pickler's writes, every placeholder replaced by its stream: the 4-byte length
    before it is corrected, then everything is copied once into a new bytes object -- the large pieces
    by torch's multi-threaded copy, which also spreads the page faults of the fresh allocation."""
    import ctypes
    import struct
    pieces = []  # (bytes-like, length)
    for i, part in enumerate(parts):
        d = deferred.get(id(part))
        if d is None:
            pieces.append(part)
            continue
        head, raw, n = d
        prev = pieces[-1]
        marker = b"B" + struct.pack("<I", _PLACEHOLDER_LEN)  # BINBYTES + length, the last thing written before the payload
        if not prev.endswith(marker):
            raise RuntimeError("unexpected pickle layout around a storage stream")
        pieces[-1] = prev[:-4] + struct.pack("<I", n)
        pieces.append(head)
        pieces.append(raw)
    total = sum(len(x) for x in pieces)
    api = ctypes.pythonapi
    api.PyBytes_FromStringAndSize.restype = ctypes.py_object
    api.PyBytes_FromStringAndSize.argtypes = [ctypes.c_char_p, ctypes.c_ssize_t]
    api.PyBytes_AsString.restype = ctypes.c_void_p
    api.PyBytes_AsString.argtypes = [ctypes.py_object]
    blob = api.PyBytes_FromStringAndSize(None, total)  # uninitialised, ours alone until it is returned
    base = api.PyBytes_AsString(blob)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dst = torch.frombuffer((ctypes.c_ubyte * total).from_address(base), dtype=torch.uint8) if total else None
    pos = 0
    for x in pieces:
        n = len(x)
        if n >= (1 << 20):
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")  # a read-only source buffer, and it is only read
                dst[pos:pos + n].copy_(torch.frombuffer(x, dtype=torch.uint8))
        elif n:
            ctypes.memmove(base + pos, bytes(x) if not isinstance(x, bytes) else x, n)
        pos += n
    return blob


def dump_blob(eo: "CacheGenGPUEncoderOutput") -> bytes:
    """The pickle of an encoded chunk, byte for byte what pickle.dump writes (cachegen_basics.py:146-151).
    Tensors that own their storage are read through pinned memory (one asynchronous copy each, one
    synchronisation) and their legacy streams built here; the others are left to torch."""
    tensors = [eo.cdf, eo.max_tensors_key, eo.max_tensors_value]
    for dc in eo.data_chunks:
        tensors += [dc.bytestream, dc.bytestream_lengths]
    fast = [t for t in tensors if isinstance(t, torch.Tensor) and _owns_its_storage(t)]
    raw_of = {}
    on_gpu = [t for t in fast if t.is_cuda and t.numel()]
    if on_gpu:
        st = staging()
        sizes = [t.numel() * t.element_size() for t in on_gpu]
        st.begin(sum((n + 255) // 256 * 256 for n in sizes))
        pos, slices = 0, []
        for t, n in zip(on_gpu, sizes):
            piece = st.buf[pos:pos + n]
            piece.copy_(t.reshape(-1).view(torch.uint8), non_blocking=True)
            slices.append(piece)
            pos += (n + 255) // 256 * 256
        for dev in {t.device for t in on_gpu}:
            torch.cuda.current_stream(dev).synchronize()
        for t, piece in zip(on_gpu, slices):
            raw_of[id(t)] = memoryview(piece.numpy())
    for t in fast:
        if id(t) not in raw_of:
            raw_of[id(t)] = memoryview(t.reshape(-1).view(torch.uint8).numpy()) if t.numel() else b""
    out = _PartsWriter()
    pickler = _BlobPickler(out, raw_of)
    pickler.dump(eo)
    blob = _assemble(out.parts, pickler.deferred)
    if on_gpu:
        st.end()
    return blob


# `CacheGenEncoderOutput.from_bytes` is what the reference's tests call on a blob
# (LMCache/tests/test_serde.py:43); with pickle it is the same loader.
CacheGenEncoderOutput = CacheGenGPUEncoderOutput


class _StorageRecord(pickle.Unpickler):
    """Reads the one persistent id of a torch legacy storage stream without building the storage."""

    def __init__(self, f):
        super().__init__(f)
        self.seen = []

    def persistent_load(self, saved_id):
        self.seen.append(saved_id)
        return None


def _load_storage_from_bytes(b: bytes):
    """Replacement for torch.storage._load_from_bytes while unpickling a blob.

    Pickling a tensor stores its storage as the bytes of a legacy `torch.save` stream: three small
    pickles (magic, protocol, system info), the pickled storage whose persistent id names type,
    location and size, the list of storage keys, then an int64 element count and the raw data.
    torch's loader copies that data into a CPU storage and then to the GPU; here the data is viewed
    in place inside `b` and copied once, straight to its device.  Anything unexpected falls back to
    torch's own loader."""
    import warnings
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # TypedStorage deprecation notes; read-only buffer note
            return _load_storage_fast(b)
    except Exception:
        return torch.storage._load_from_bytes(bytes(b))


def _load_storage_fast(b):
    f = io.BytesIO(bytes(b[:1 << 16]))  # the stream's head: small pickles, then the raw data (b may be a view)
    if pickle.load(f) != torch.serialization.MAGIC_NUMBER or pickle.load(f) != torch.serialization.PROTOCOL_VERSION:
        raise ValueError("not a legacy stream")
    info = pickle.load(f)
    if not info.get("little_endian", True):
        raise ValueError("big-endian stream")
    rec = _StorageRecord(f)
    rec.load()
    keys = pickle.load(f)
    if len(rec.seen) != 1 or len(keys) != 1:
        raise ValueError("more than one storage")
    typename, storage_type, key, location, numel, view = rec.seen[0]
    if typename != "storage" or view is not None or keys[0] != key:
        raise ValueError("storage view")
    dtype = torch.uint8 if storage_type is torch.UntypedStorage else storage_type.dtype
    esz = torch._utils._element_size(dtype)
    off = f.tell()
    if off + 8 > min(len(b), 1 << 16):
        raise ValueError("header too long")
    count = int.from_bytes(b[off:off + 8], "little")
    nbytes = count * esz
    if count != numel or off + 8 + nbytes != len(b):
        raise ValueError("size mismatch")
    device = torch.device(location)
    if device.type == "cuda" and not (torch.cuda.is_available() and (device.index or 0) < torch.cuda.device_count()):
        raise ValueError("device not present")
    if nbytes == 0:
        raw = torch.empty(0, dtype=torch.uint8, device=device)
    else:
        view_cpu = torch.frombuffer(b, dtype=torch.uint8, count=nbytes, offset=off + 8)  # read-only, only read
        if device.type == "cpu":
            raw = view_cpu.clone()
        else:
            raw = staging().to_device(view_cpu, device)
    return torch.storage.TypedStorage(wrap_storage=raw.untyped_storage(), dtype=dtype, _internal=True)


class _Staging:
    """Pinned host memory that a thread's blob loads and dumps pass through: bytes are copied into it
    by torch's multi-threaded CPU copy and leave it by an asynchronous copy on the current stream
    (or arrive in it from the GPU), several times faster than a copy to or from pageable memory.
    Two buffers per thread, used in turn and grown on demand, so that filling one overlaps the
    copies still leaving the other; `begin` waits until the chosen buffer's last copies are done."""

    def __init__(self):
        self.bufs = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.buf = None
        self.pos = 0

    def begin(self, nbytes: int) -> None:
        self.turn ^= 1
        i = self.turn
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        if self.bufs[i] is None or self.bufs[i].numel() < nbytes:
            self.bufs[i] = None
            self.bufs[i] = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8)
            if torch.cuda.is_available():
                self.bufs[i] = self.bufs[i].pin_memory()
        self.buf = self.bufs[i]
        self.pos = 0

    def end(self) -> None:
        """Storages loaded outside a blob load do not pass through the staging memory."""
        self.buf = None

    def to_device(self, view_cpu: torch.Tensor, device) -> torch.Tensor:
        n = view_cpu.numel()
        if self.buf is None or self.pos + n > self.buf.numel():
            return view_cpu.to(device)  # no load in progress, or more data than the blob announced
        stage = self.buf[self.pos:self.pos + n]
        self.pos += (n + 255) // 256 * 256
        stage.copy_(view_cpu)
        out = torch.empty(n, dtype=torch.uint8, device=device)
        out.copy_(stage, non_blocking=True)
        self.events[self.turn] = torch.cuda.Event()
        self.events[self.turn].record(torch.cuda.current_stream(device))
        return out


    def whole_to_device(self, view_cpu: torch.Tensor, device) -> torch.Tensor:
        """One host buffer (any memory) to the GPU through the staging memory."""
        self.begin(view_cpu.numel())
        try:
            return self.to_device(view_cpu, device)
        finally:
            self.end()

    def whole_from_device(self, t: torch.Tensor) -> bytes:
        """The bytes of a contiguous GPU tensor: one asynchronous copy into the staging memory, one
        synchronisation, one copy into the result."""
        flat = t.reshape(-1).view(torch.uint8)
        self.begin(flat.numel())
        try:
            stage = self.buf[:flat.numel()]
            stage.copy_(flat, non_blocking=True)
            torch.cuda.current_stream(t.device).synchronize()
            return bytes(memoryview(stage.numpy()))
        finally:
            self.end()


_staging_local = threading.local()


def staging() -> _Staging:
    st = getattr(_staging_local, "staging", None)
    if st is None:
        st = _staging_local.staging = _Staging()
    return st


class _ViewReader:
    """File-like reader over a bytes-like object that hands large reads out as memoryview slices
    (no copy) and small ones as bytes."""

    def __init__(self, data):
        self.mv = memoryview(data)
        self.pos = 0

    def read(self, n: int = -1):
        if n is None or n < 0:
            n = len(self.mv) - self.pos
        piece = self.mv[self.pos:self.pos + n]
        self.pos += len(piece)
        return piece if len(piece) >= (1 << 16) else bytes(piece)

    def readline(self):
        end = self.pos
        while end < len(self.mv) and self.mv[end] != 10:
            end += 1
        end = min(end + 1, len(self.mv))
        piece = bytes(self.mv[self.pos:end])
        self.pos = end
        return piece


def _find_wire_class(module, name):
    if name in ("CacheGenGPUEncoderOutput", "CacheGenGPUBytestream") and module in (REFERENCE_MODULE, __name__):
        return globals()[name]
    if module == "torch.storage" and name == "_load_from_bytes":
        return _load_storage_from_bytes
    return None


class _Unpickler(pickle.Unpickler):
    """pickle loader that resolves the two wire classes to this module, whichever module path the
    blob was written under, and reads tensor storages with one copy (see _load_storage_from_bytes)."""

    def find_class(self, module, name):
        return _find_wire_class(module, name) or super().find_class(module, name)


class _ViewUnpickler(pickle._Unpickler):
    """The same loader on the standard library's Python unpickler reading through a _ViewReader: the
    blob's large byte strings (the pickled tensor storages) reach _load_storage_from_bytes as views
    of the blob instead of copies.  A blob has a few hundred opcodes, so the interpreter's speed
    does not matter; copying its 30 MB once more does."""

    def __init__(self, data):
        super().__init__(_ViewReader(data))

    def find_class(self, module, name):
        return _find_wire_class(module, name) or super().find_class(module, name)


def load_blob(bs):
    """Unpickles a CacheGenGPUEncoderOutput written by this package or by the reference."""
    staged = False
    try:
        if torch.cuda.is_available():
            staging().begin(len(bs))
            staged = True
        return _ViewUnpickler(bs).load()
    except Exception:
        with io.BytesIO(bs) as f:
            return _Unpickler(f).load()
    finally:
        if staged:
            staging().end()


def _adopt_reference_module_path():
    from .. import compat
    if compat.install_wire_aliases(__name__):
        CacheGenGPUBytestream.__module__ = REFERENCE_MODULE
        CacheGenGPUEncoderOutput.__module__ = REFERENCE_MODULE


_adopt_reference_module_path()
