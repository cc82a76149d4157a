"""A flat, pickle-free container for one encoded chunk ("CGB2").

The reference's wire format is a pickle of a CacheGenGPUEncoderOutput whose tensors are CUDA tensors
(LMCache/lmcache/storage_backend/serde/cachegen_basics.py:133-156).  It stays the default and the
only format the reference can read.  This container holds the same information in one contiguous
byte buffer that can be copied to the GPU in a single transfer and decoded in place, and it can
carry the tables in a compact form:

  header (little-endian, 128 bytes + 8 * (nsub + 1)):
      magic "CGB2", version, L, H, D, T, Lp, nsub, scale dtype (0 fp16 / 1 bf16),
      table kind (0 = int16 CDF tables, 1 = byte counts, 2 = sparse byte counts), length kind (0 = int32, 1 = uint16),
      a checksum of the encoder's per-row bin counts (0 = not recorded),
      offsets of the four sections and the total size, then the byte offset of every sub-chunk's
      streams inside the payload section
  scales   16-bit [2L, T]: max_tensors_key rows then max_tensors_value rows
  tables   kind 0: int16 [2L, C, Lp] exactly as calculate_cdf returns them
           kind 1: uint8 counts of every non-centre symbol, [row][symbol][channel] with 2*Cq_row
                   symbols per row (CG_TABLES_COUNTS in include/cachegen_b200.h); the decoder
                   rebuilds the tables from them.  Used when no such count exceeds 255.
           kind 2: the same counts without the zeros (CG_TABLES_SPARSE): group offsets, a bit mask
                   per (row, channel) of the symbols that occur, then the non-zero counts.  Used
                   when kind 1 is usable and no row has more than 32 non-centre symbols.
  lengths  [nsub, 2L, C] stream lengths, uint16 (a stream is at most 520 bytes) or int32
  payload  the streams of every sub-chunk, back to back

Sections start on 256-byte boundaries.  Like the reference's blob, the container does not record
the bin settings: encoder and decoder must be configured alike.
"""
import struct
import zlib
from dataclasses import dataclass
from typing import List

import torch

MAGIC = b"CGB2"
VERSION = 1
_FIXED = struct.Struct("<4sI6I3IIQQQQQ")  # 4+4+24+12+4+40 = 88 bytes, padded to 128
HEADER_FIXED_BYTES = 128
ALIGN = 256
TABLES_CDF, TABLES_COUNTS, TABLES_SPARSE = 0, 1, 2
LENGTHS_I32, LENGTHS_U16 = 0, 1
_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1}
_CODE_DTYPE = {0: torch.float16, 1: torch.bfloat16}


def _up(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def is_flat(buf) -> bool:
    return len(buf) >= 4 and bytes(buf[:4]) == MAGIC


def table_row_offsets(bins_cpu: torch.Tensor, nchannels: int) -> List[int]:
    """Offsets of every row's byte counts (and the total) for the given per-row bin counts."""
    offs, acc = [], 0
    for b in bins_cpu.tolist():
        offs.append(acc)
        acc += 2 * (int(b) // 2 - 1) * nchannels
    offs.append(acc)
    return offs


def bins_checksum(bins_cpu: torch.Tensor, delta=None) -> int:
    """Non-zero 32-bit checksum of the per-row bin counts (key rows then value rows) and of the
    anchor-token delta settings, if any.  The byte-count table forms and delta-coded chunks can only be
    read with the settings they were written with; the header carries this so that a decoder
    configured otherwise refuses the container instead of misreading it."""
    raw = struct.pack(f"<{bins_cpu.numel()}H", *[int(b) for b in bins_cpu.tolist()])
    if delta is not None:
        raw += struct.pack("<HHB", delta.group, delta.divisor, 1 if delta.rows == "all" else 0)
    return zlib.crc32(raw) or 1


def mask_row_offsets(bins_cpu: torch.Tensor, nchannels: int) -> List[int]:
    """Offsets of every row's masks inside the mask part of sparse tables (and the part's size): two
    bytes per channel for rows of at most 16 non-centre symbols, else four; rows start 4-byte aligned."""
    offs, acc = [], 0
    for b in bins_cpu.tolist():
        offs.append(acc)
        acc += (nchannels * (2 if 2 * (int(b) // 2 - 1) <= 16 else 4) + 3) // 4 * 4
    offs.append(acc)
    return offs


def sparse_parts(nrows: int, nchannels: int, mask_bytes: int):
    """(offset of the masks, offset of the counts) inside sparse tables: each part starts on a
    16-byte boundary after uint32 [nrows * ceil(C / 128) + 1] group offsets."""
    off_masks = ((nrows * ((nchannels + 127) // 128) + 1) * 4 + 15) // 16 * 16
    return off_masks, off_masks + (mask_bytes + 15) // 16 * 16


def sparse_representable(bins_cpu: torch.Tensor) -> bool:
    return all(2 * (int(b) // 2 - 1) <= 32 for b in bins_cpu.tolist())


@dataclass
class FlatHeader:
    L: int
    H: int
    D: int
    T: int
    lp: int
    nsub: int
    scale_code: int
    table_kind: int
    length_kind: int
    bins_checksum: int
    off_scales: int
    off_tables: int
    off_lengths: int
    off_payload: int
    total: int
    sub_off: List[int]

    @property
    def nbytes_header(self) -> int:
        return HEADER_FIXED_BYTES + 8 * (self.nsub + 1)

    def pack(self) -> bytes:
        fixed = _FIXED.pack(MAGIC, VERSION, self.L, self.H, self.D, self.T, self.lp, self.nsub, self.scale_code,
                            self.table_kind, self.length_kind, self.bins_checksum, self.off_scales, self.off_tables,
                            self.off_lengths, self.off_payload, self.total)
        return fixed.ljust(HEADER_FIXED_BYTES, b"\0") + struct.pack(f"<{self.nsub + 1}Q", *self.sub_off)

    @staticmethod
    def peek_header_bytes(fixed: bytes) -> int:
        """Size of the whole header, from its first HEADER_FIXED_BYTES bytes."""
        if len(fixed) < _FIXED.size or fixed[:4] != MAGIC:
            raise ValueError("not a CGB2 container")
        nsub = _FIXED.unpack(fixed[:_FIXED.size])[7]
        if not 0 < nsub < (1 << 20):
            raise ValueError("corrupt CGB2 header")
        return HEADER_FIXED_BYTES + 8 * (nsub + 1)

    @staticmethod
    def parse(buf) -> "FlatHeader":
        """Parses and validates the header of a complete container (any bytes-like object)."""
        fixed = bytes(buf[:HEADER_FIXED_BYTES])
        return FlatHeader.parse_head(bytes(buf[:FlatHeader.peek_header_bytes(fixed)]), len(buf))

    @staticmethod
    def parse_head(head: bytes, total_len: int) -> "FlatHeader":
        """Parses the header bytes `head` of a container that is `total_len` bytes long."""
        f = _FIXED.unpack(head[:_FIXED.size])
        if f[0] != MAGIC:
            raise ValueError("not a CGB2 container")
        if f[1] != VERSION:
            raise ValueError(f"unsupported CGB2 version {f[1]}")
        L, H, D, T, lp, nsub, scale_code, table_kind, length_kind, bins_sum = f[2:12]
        if min(L, H, D, T, nsub) <= 0 or lp < 2 or lp > 64 or nsub != (T + 255) // 256:
            raise ValueError("corrupt CGB2 header")
        if scale_code not in (0, 1) or table_kind not in (0, 1, 2) or length_kind not in (0, 1):
            raise ValueError("corrupt CGB2 header")
        end = HEADER_FIXED_BYTES + 8 * (nsub + 1)
        if len(head) < end:
            raise ValueError("truncated CGB2 header")
        sub_off = list(struct.unpack(f"<{nsub + 1}Q", head[HEADER_FIXED_BYTES:end]))
        h = FlatHeader(L, H, D, T, lp, nsub, scale_code, table_kind, length_kind, bins_sum, *f[12:17], sub_off)
        C = H * D
        if h.total != total_len or not (end <= h.off_scales <= h.off_tables <= h.off_lengths <= h.off_payload <= h.total):
            raise ValueError("corrupt CGB2 section table")
        if (h.off_tables - h.off_scales < 4 * L * T or
                h.off_payload - h.off_lengths < nsub * 2 * L * C * (2 if length_kind == LENGTHS_U16 else 4) or
                (table_kind == TABLES_CDF and h.off_lengths - h.off_tables < 4 * L * C * lp)):
            raise ValueError("corrupt CGB2 section table")
        if sub_off[0] != 0 or any(a > b for a, b in zip(sub_off, sub_off[1:])) or h.off_payload + sub_off[-1] > h.total:
            raise ValueError("corrupt CGB2 payload table")
        return h


def layout(L: int, H: int, D: int, T: int, lp: int, scale_dtype: torch.dtype, table_kind: int, table_bytes: int,
           length_kind: int, sub_off: List[int], bins_checksum: int = 0) -> FlatHeader:
    nsub = (T + 255) // 256
    C = H * D
    off = _up(HEADER_FIXED_BYTES + 8 * (nsub + 1))
    off_scales = off
    off = _up(off + 2 * L * T * 2)
    off_tables = off
    off = _up(off + table_bytes)
    off_lengths = off
    off = _up(off + nsub * 2 * L * C * (2 if length_kind == LENGTHS_U16 else 4))
    off_payload = off
    total = off + sub_off[-1]
    return FlatHeader(L, H, D, T, lp, nsub, _DTYPE_CODE[scale_dtype], table_kind, length_kind, bins_checksum,
                      off_scales, off_tables, off_lengths, off_payload, total, list(sub_off))


class FlatChunk:
    """A CGB2 container held in one uint8 tensor (on the GPU, or in host memory) with typed views of
    its sections.  Exposes the fields a decode needs."""

    def __init__(self, blob: torch.Tensor, header: FlatHeader = None):
        if blob.dtype != torch.uint8 or blob.dim() != 1 or not blob.is_contiguous():
            raise ValueError("a CGB2 container is a contiguous 1-D uint8 tensor")
        self.blob = blob
        if header is None:
            fixed = blob[:HEADER_FIXED_BYTES].cpu().numpy().tobytes()
            head = blob[:FlatHeader.peek_header_bytes(fixed)].cpu().numpy().tobytes()
            header = FlatHeader.parse_head(head, blob.numel())
        self.header = header

    # -- geometry
    @property
    def num_heads(self) -> int:
        return self.header.H

    @property
    def head_size(self) -> int:
        return self.header.D

    @property
    def num_tokens(self) -> int:
        return self.header.T

    @property
    def scale_dtype(self) -> torch.dtype:
        return _CODE_DTYPE[self.header.scale_code]

    def to(self, device, non_blocking: bool = False) -> "FlatChunk":
        return FlatChunk(self.blob.to(device, non_blocking=non_blocking), self.header)

    def pin_memory(self) -> "FlatChunk":
        return FlatChunk(self.blob.cpu().pin_memory(), self.header)

    def tobytes(self) -> bytes:
        if self.blob.is_cuda:
            from .cachegen_basics import staging
            return staging().whole_from_device(self.blob)  # through pinned memory
        return self.blob.numpy().tobytes()

    # -- section views (same device as the blob)
    def _view(self, off: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        return self.blob[off:off + nbytes].view(dtype)

    def scales(self) -> torch.Tensor:
        h = self.header
        return self._view(h.off_scales, 2 * h.L * h.T * 2, self.scale_dtype).view(2 * h.L, h.T)

    def tables(self) -> torch.Tensor:
        h = self.header
        if h.table_kind == TABLES_CDF:
            n = 2 * h.L * h.H * h.D * h.lp * 2
            return self._view(h.off_tables, n, torch.int16).view(2 * h.L, h.H * h.D, h.lp)
        return self.blob[h.off_tables:h.off_lengths]  # byte counts (dense or sparse); the decoder knows the row offsets

    def lengths(self, j: int) -> torch.Tensor:
        h = self.header
        n = 2 * h.L * h.H * h.D
        if h.length_kind == LENGTHS_U16:
            return self._view(h.off_lengths + j * n * 2, n * 2, torch.int16).view(2 * h.L, h.H * h.D)
        return self._view(h.off_lengths + j * n * 4, n * 4, torch.int32).view(2 * h.L, h.H * h.D)

    def payload(self, j: int) -> torch.Tensor:
        h = self.header
        return self.blob[h.off_payload + h.sub_off[j]:h.off_payload + h.sub_off[j + 1]]

    def sub_tokens(self, j: int) -> int:
        return min(256, self.header.T - 256 * j)

    @property
    def payload_bytes(self) -> int:
        return self.header.sub_off[-1]


def from_bytes(buf, device=None) -> FlatChunk:
    """Wraps a bytes-like CGB2 container; with `device` the bytes are copied there (to a GPU through
    pinned staging memory, straight from `buf`)."""
    header = FlatHeader.parse(buf)
    device = torch.device(device) if device is not None else None
    if device is not None and device.type == "cuda":
        import warnings
        from .cachegen_basics import staging
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # a read-only buffer, and it is only read
            view = torch.frombuffer(buf, dtype=torch.uint8)
        return FlatChunk(staging().whole_to_device(view, device), header)
    t = torch.frombuffer(bytearray(buf) if isinstance(buf, bytes) else buf, dtype=torch.uint8)
    chunk = FlatChunk(t, header)
    return chunk.to(device) if device is not None else chunk
