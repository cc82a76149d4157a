"""CacheGenSerializer (reference: LMCache/lmcache/storage_backend/serde/cachegen_encoder.py:247-348).

`to_bytes` keeps the reference's contract -- KV blob tensor in, pickled CacheGenGPUEncoderOutput out,
byte-identical to what the reference produces from the same input -- with the reference's chain of
torch ops and per-sub-chunk launches replaced by three C-ABI calls:

    cg_quantize_cdf      split K/V + quantise + histogram + tables      (enc.py:257-267)
    cg_encode_chunk      every sub-chunk's streams + offsets            (enc.py:269-292, 225-236)
    cg_compact_streams   gather of the streams                          (enc.py:210-222)

Beside it: encode_many (a whole cache, up to a batch of chunks in flight and no wait in between), encode_levels
(one chunk at several bin settings: cg_row_absmax + cg_quantize_cdf_scaled per level) and encode_flat
(the CGB2 container of flat_format.py, tables packed by cg_pack_sparse_tables).

(enc.py = cachegen_encoder.py of the reference.)
"""
import collections
import ctypes
from typing import Tuple

import torch

from .. import _lib
from ..config import LMCacheEngineConfig, LMCacheEngineMetadata
from ..utils import _lmcache_nvtx_annotate
from . import cachegen_basics as CGBasics
from . import flat_format
from .cachegen_basics import CacheGenConfig, CacheGenGPUBytestream, CacheGenGPUEncoderOutput
from .serde import Serializer

_DTYPES = {torch.float16: _lib.CG_F16, torch.bfloat16: _lib.CG_BF16}


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _split_kv(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[L, 2, T, H, D] -> K and V as [L, T, H*D] (enc.py:72-83)."""
    num_layers, _, num_tokens, num_heads, head_size = tensor.shape
    return torch.unbind(tensor.reshape(num_layers, 2, num_tokens, num_heads * head_size), dim=1)


@_lmcache_nvtx_annotate
def torch_quant_vectorized(bins: torch.Tensor, input_groups: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The reference's quantiser with its own signature (enc.py:42-59), on the quantise kernel: bins
    [R] (any numeric type), input_groups [R, T, C] float16 / bfloat16 on the GPU -> (symbols int8
    [R, T, C], max|x| per (row, token) [R, T, 1] in the input's dtype).  The serializer does not go
    through here (it quantises K and V of the blob in place, tables in the same pass)."""
    if input_groups.dim() != 3 or input_groups.dtype not in _DTYPES or not input_groups.is_cuda:
        raise TypeError("expected a CUDA float16 / bfloat16 tensor [nlayers, ntokens, nchannels]")
    x = input_groups.contiguous()
    R, T, C = x.shape
    if bins.numel() != R:
        raise RuntimeError(f"bins describe {bins.numel()} rows, the input has {R}")
    b = bins.to(device=x.device, dtype=torch.float32).contiguous()
    if R % 2:  # the kernel takes rows in two halves: give an odd count one more row to chew on
        x = torch.cat((x, x[-1:]))
        b = torch.cat((b, b[-1:]))
    half = x.shape[0] // 2
    max_bins = max(int(b.max()), 1)
    sym = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scales = torch.empty(x.shape[:2], dtype=x.dtype, device=x.device)
    cdf = torch.empty((x.shape[0], C, max_bins + 1), dtype=torch.int16, device=x.device)
    null = ctypes.c_void_p(None)
    with torch.cuda.device(x.device):
        rc = _lib.lib().cg_quantize_cdf(_ptr(x), _DTYPES[x.dtype], T * C, half * T * C, C, C, half, T, 1, C, _ptr(b),
                                        max_bins, _ptr(sym), _ptr(scales), _ptr(cdf), null, null, null,
                                        _stream(x.device))
    _lib.check(rc, "cg_quantize_cdf")
    return sym[:R], scales[:R].unsqueeze(-1)


@_lmcache_nvtx_annotate
def concat_max(max1) -> torch.Tensor:
    """A sequence of per-layer max tensors as one tensor with a leading layer axis (enc.py:62-70)."""
    return torch.stack([max1[i] for i in range(len(max1))])


@_lmcache_nvtx_annotate
def collect_bytes(output_buffer: torch.Tensor, output_lengths: torch.Tensor) -> torch.Tensor:
    """The first output_lengths[r, c] bytes of every row output_buffer[r, c, :], back to back in
    (r, c) order, as one uint8 tensor (enc.py:210-222), on the offset and compaction kernels."""
    if output_buffer.dim() != 3 or output_buffer.dtype != torch.uint8 or not output_buffer.is_cuda:
        raise TypeError("expected a CUDA uint8 buffer [nlayers, nchannels, row]")
    buf, lengths = output_buffer.contiguous(), output_lengths.to(torch.int32).contiguous()
    NL, C, stride = buf.shape
    if tuple(lengths.shape) != (NL, C):
        raise RuntimeError("output_lengths must have shape [nlayers, nchannels]")
    dev = buf.device
    total, outside = torch.stack((lengths.sum(dtype=torch.int64),
                                  ((lengths < 0) | (lengths > stride)).sum(dtype=torch.int64))).tolist()
    if outside:
        raise RuntimeError("collect_bytes: a length is negative or exceeds the buffer's row size")
    nslab = (C + _lib.CG_GROUP_CHANNELS - 1) // _lib.CG_GROUP_CHANNELS
    group_off = torch.empty(NL * nslab, dtype=torch.int64, device=dev)
    sub_off = torch.tensor([0, total], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(total, dtype=torch.uint8, device=dev)
    job = _lib.DecodeJob()
    job.lengths, job.nbytes, job.length_kind = lengths.data_ptr(), total, _lib.CG_LENGTHS_I32
    with torch.cuda.device(dev):
        rc = _lib.lib().cg_decode_offsets((_lib.DecodeJob * 1)(job), 1, NL, C, _ptr(group_off), _ptr(status), _stream(dev))
        _lib.check(rc, "cg_decode_offsets")
        rc = _lib.lib().cg_compact_streams(_ptr(buf), stride, _ptr(lengths), _ptr(group_off), _ptr(sub_off), 1, NL, C,
                                           _ptr(out), _stream(dev))
        _lib.check(rc, "cg_compact_streams")
    if int(status.item()):
        raise RuntimeError("collect_bytes: " + _lib.status_text(int(status.item())))
    return out


@_lmcache_nvtx_annotate
def encode_ntokens(cdf_int: torch.Tensor, encode_input: torch.Tensor, output_buffer: torch.Tensor,
                   output_lengths: torch.Tensor) -> torch.Tensor:
    """encode_fast_new into the caller's buffers, then collect_bytes (enc.py:225-242)."""
    from .. import torchac_cuda
    torchac_cuda.encode_fast_new(cdf_int, encode_input, output_buffer, output_lengths)
    torchac_cuda.check_status(cdf_int.device)
    return collect_bytes(output_buffer, output_lengths)


def row_scales(kv: torch.Tensor) -> torch.Tensor:
    """max|x| over the channels of every (row, token): [2L, T] in kv.dtype, key rows then value rows
    (the max1 of torch_quant_vectorized, enc.py:55).  It does not depend on the bin settings."""
    if kv.dim() != 5 or kv.shape[1] != 2 or kv.dtype not in _DTYPES or not kv.is_cuda or kv.stride(4) != 1:
        raise RuntimeError("expected a CUDA float16/bfloat16 KV blob [L, 2, T, H, D] with a unit innermost stride")
    L, _, T, H, D = kv.shape
    scales = torch.empty((2 * L, T), dtype=kv.dtype, device=kv.device)
    with torch.cuda.device(kv.device):
        rc = _lib.lib().cg_row_absmax(_ptr(kv), _DTYPES[kv.dtype], kv.stride(0), kv.stride(1), kv.stride(2),
                                      kv.stride(3), L, T, H, D, _ptr(scales), _stream(kv.device))
    _lib.check(rc, "cg_row_absmax")
    return scales


def quantize_and_tables(kv: torch.Tensor, key_bins: torch.Tensor, value_bins: torch.Tensor, max_bins: int,
                        with_counts: bool = False, scales: torch.Tensor = None, bins_cpu: torch.Tensor = None,
                        delta: "CGBasics.DeltaCoding" = None):
    """Fused torch_quant_vectorized (K and V) + calculate_cdf (K and V) + the two torch.cat of
    encode_function (enc.py:42-59, 257-267).

    kv: CUDA fp16/bf16 blob addressed as [L, 2, T, H, D] (any strides with a unit innermost stride, so
        the permuted view of a "huggingface" blob is read in place).
    Returns (symbols int8 [2L, T, C], scales [2L, T] in kv.dtype, tables int16 [2L, C, max_bins + 1]);
    with_counts adds (byte counts uint8 of the compact table form, int32 status word whose
    CG_S_COUNT_OVERFLOW bit says they are unusable for this chunk).  `scales`: the result of row_scales
    for this blob, when it is already known (encoding one chunk at several bin settings).  `bins_cpu`:
    a host copy of the concatenated bins, to save the transfer.
    """
    if kv.dim() != 5 or kv.shape[1] != 2:
        raise RuntimeError(f"expected a KV blob of shape [L, 2, T, H, D], got {tuple(kv.shape)}")
    if kv.dtype not in _DTYPES:
        raise TypeError(f"the codec takes float16 or bfloat16 KV, got {kv.dtype}")
    if not kv.is_cuda:
        raise RuntimeError("KV must be a CUDA tensor")
    if kv.stride(4) != 1:
        kv = kv.contiguous()
    L, _, T, H, D = kv.shape
    C = H * D
    dev = kv.device
    bins = torch.cat((key_bins, value_bins)).to(device=dev, dtype=torch.float32).contiguous()
    if bins.numel() != 2 * L:
        raise RuntimeError(f"bins describe {bins.numel() // 2} layers, the KV blob has {L}")
    sym = torch.empty((2 * L, T, C), dtype=torch.int8, device=dev)
    given = scales is not None
    if given and (tuple(scales.shape) != (2 * L, T) or scales.dtype != kv.dtype or scales.device != dev or
                  not scales.is_contiguous()):
        raise RuntimeError("scales must be a contiguous [2L, T] tensor of the blob's dtype on its device")
    if not given:
        scales = torch.empty((2 * L, T), dtype=kv.dtype, device=dev)
    cdf = torch.empty((2 * L, C, max_bins + 1), dtype=torch.int16, device=dev)
    counts = row_off = status = None
    if with_counts:
        offs = flat_format.table_row_offsets(bins.cpu() if bins_cpu is None else bins_cpu, C)
        row_off = torch.tensor(offs, dtype=torch.int64, device=dev)
        counts = torch.empty(offs[-1], dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    null = ctypes.c_void_p(None)
    tail = (_ptr(cdf), _ptr(counts) if with_counts else null, _ptr(row_off) if with_counts else null,
            _ptr(status) if with_counts else null, _stream(dev))
    head = (_ptr(kv), _DTYPES[kv.dtype], kv.stride(0), kv.stride(1), kv.stride(2), kv.stride(3), L, T, H, D,
            _ptr(bins), int(max_bins))
    with torch.cuda.device(dev):
        if delta is not None:
            if given:
                raise RuntimeError("precomputed scales cannot be combined with delta coding")
            res_bins = delta.residual_bins(key_bins, value_bins, dev)
            rc = _lib.lib().cg_quantize_cdf_delta(*head, delta.group, _ptr(res_bins), _ptr(sym), _ptr(scales), *tail)
        elif given:
            rc = _lib.lib().cg_quantize_cdf_scaled(*head, _ptr(scales), _ptr(sym), *tail)
        else:
            rc = _lib.lib().cg_quantize_cdf(*head, _ptr(sym), _ptr(scales), *tail)
    _lib.check(rc, "cg_quantize_cdf")
    if with_counts:
        return sym, scales, cdf, counts, status
    return sym, scales, cdf


def encode_streams(cdf: torch.Tensor, sym: torch.Tensor, scratch_stride: int = None, extra_status: torch.Tensor = None):
    """The sub-chunk loop of encode_function in one pass (enc.py:269-292).

    cdf int16 [2L, C, Lp], sym int8 [2L, T, C] contiguous.  Returns (bytes uint8 [total], lengths int32
    [nsub, 2L, C], sub_off: python list of nsub+1 byte offsets of the sub-chunks inside `bytes`).
    Synchronises once, to size the output; `extra_status` (one or more integer words on the GPU) is read
    in the same transfer and appended to the result (an int, or a list of ints for several words).
    """
    NL, T, C = sym.shape
    lp = cdf.shape[2]
    dev = sym.device
    nsub = (T + CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK - 1) // CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK
    stride = scratch_stride or _lib.stream_capacity(min(T, CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK))
    stride = (stride + 3) // 4 * 4
    nslab = (C + _lib.CG_GROUP_CHANNELS - 1) // _lib.CG_GROUP_CHANNELS
    scratch = torch.empty((nsub, NL * C, stride), dtype=torch.uint8, device=dev)
    lengths = torch.empty((nsub, NL, C), dtype=torch.int32, device=dev)
    group_off = torch.empty((nsub, NL * nslab), dtype=torch.int64, device=dev)
    sub_off = torch.empty(nsub + 1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        rc = L.cg_encode_chunk(_ptr(cdf), _ptr(sym), NL, T, C, lp, _ptr(scratch), stride, _ptr(lengths),
                               _ptr(group_off), _ptr(sub_off), _ptr(status), _stream(dev))
        _lib.check(rc, "cg_encode_chunk")
        words = [sub_off, status.to(torch.int64)] + ([extra_status.to(torch.int64)] if extra_status is not None else [])
        host = torch.cat(words).cpu()  # the one synchronisation
        bits = int(host[nsub + 1])
        if bits:
            raise RuntimeError("cachegen encode: " + _lib.status_text(bits))
        offs = [int(v) for v in host[:nsub + 1]]
        out = torch.empty(offs[-1], dtype=torch.uint8, device=dev)
        rc = L.cg_compact_streams(_ptr(scratch), stride, _ptr(lengths), _ptr(group_off), _ptr(sub_off), nsub, NL,
                                  C, _ptr(out), _stream(dev))
        _lib.check(rc, "cg_compact_streams")
    if extra_status is not None:
        extra = [int(v) for v in host[nsub + 2:]]
        return out, lengths, offs, (extra[0] if len(extra) == 1 else extra)
    return out, lengths, offs


def _table_bins(key_bins: torch.Tensor, value_bins: torch.Tensor, max_bins: int = None) -> int:
    """max_bins of the chunk's tables.  The reference builds key and value tables with their own
    maximum and concatenates them, which needs the two to be equal (enc.py:265-267).  `max_bins`
    overrides that: a layer shard of a model must use the whole model's value so that its tables and
    streams are the ones an unsharded encode produces."""
    kmax, vmax = int(key_bins.max()), int(value_bins.max())
    if max_bins is not None:
        if max_bins < max(kmax, vmax):
            raise RuntimeError(f"max_bins {max_bins} is below the largest bin count {max(kmax, vmax)}")
        return int(max_bins)
    if kmax != vmax:
        raise RuntimeError(f"Sizes of tensors must match: key tables have {kmax + 1} entries, value tables {vmax + 1}")
    return kmax


class _PendingChunk:
    """One chunk whose quantise / table / coder kernels are enqueued but whose payload size is not
    yet known on the host."""

    def __init__(self, kv, key_bins, value_bins, max_bins, scales=None, delta=None):
        self.L, _, self.T, self.H, self.D = kv.shape
        self.dtype = kv.dtype
        self.sym, self.scales, self.cdf = quantize_and_tables(kv, key_bins, value_bins, max_bins, scales=scales,
                                                              delta=delta)
        NL, T, C = self.sym.shape
        dev = self.sym.device
        self.nsub = (T + CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK - 1) // CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK
        self.stride = (_lib.stream_capacity(min(T, CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK)) + 3) // 4 * 4
        nslab = (C + _lib.CG_GROUP_CHANNELS - 1) // _lib.CG_GROUP_CHANNELS
        self.scratch = torch.empty((self.nsub, NL * C, self.stride), dtype=torch.uint8, device=dev)
        self.lengths = torch.empty((self.nsub, NL, C), dtype=torch.int32, device=dev)
        self.group_off = torch.empty((self.nsub, NL * nslab), dtype=torch.int64, device=dev)
        # sub_off[0..nsub] then the status word, so that one transfer brings both to the host
        self.tail = torch.zeros(self.nsub + 2, dtype=torch.int64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().cg_encode_chunk(_ptr(self.cdf), _ptr(self.sym), NL, T, C, self.cdf.shape[2],
                                            _ptr(self.scratch), self.stride, _ptr(self.lengths), _ptr(self.group_off),
                                            _ptr(self.tail), _ptr(self.status), _stream(dev))
        _lib.check(rc, "cg_encode_chunk")
        self.tail[self.nsub + 1:].copy_(self.status)
        self.sym = None  # symbols are consumed; free them early

    def finish(self, host_tail) -> CacheGenGPUEncoderOutput:
        bits = int(host_tail[self.nsub + 1])
        if bits:
            raise RuntimeError("cachegen encode: " + _lib.status_text(bits))
        offs = [int(v) for v in host_tail[:self.nsub + 1]]
        dev = self.cdf.device
        NL, C = 2 * self.L, self.H * self.D
        pieces = [torch.empty(offs[j + 1] - offs[j], dtype=torch.uint8, device=dev) for j in range(self.nsub)]
        with torch.cuda.device(dev):
            if self.nsub == 1:
                rc = _lib.lib().cg_compact_streams(_ptr(self.scratch), self.stride, _ptr(self.lengths),
                                                   _ptr(self.group_off), _ptr(self.tail), 1, NL, C, _ptr(pieces[0]),
                                                   _stream(dev))
                _lib.check(rc, "cg_compact_streams")
            else:
                out = torch.empty(offs[-1], dtype=torch.uint8, device=dev)
                rc = _lib.lib().cg_compact_streams(_ptr(self.scratch), self.stride, _ptr(self.lengths),
                                                   _ptr(self.group_off), _ptr(self.tail), self.nsub, NL, C, _ptr(out),
                                                   _stream(dev))
                _lib.check(rc, "cg_compact_streams")
                pieces = [out[offs[j]:offs[j + 1]].clone() for j in range(self.nsub)]
        step = CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK
        data_chunks = [CacheGenGPUBytestream(pieces[j], self.lengths[j] if self.nsub == 1 else self.lengths[j].clone(),
                                             min(step, self.T - j * step)) for j in range(self.nsub)]
        for t in (self.scratch, self.group_off, self.tail):
            t.record_stream(torch.cuda.current_stream(dev))
        return CacheGenGPUEncoderOutput(data_chunks, self.cdf,
                                        max_tensors_key=self.scales[:self.L].clone().unsqueeze(-1),
                                        max_tensors_value=self.scales[self.L:].clone().unsqueeze(-1),
                                        num_heads=self.H, head_size=self.D)


def encode_many(kv: torch.Tensor, key_bins: torch.Tensor, value_bins: torch.Tensor, chunk_tokens: int,
                batch: int = 16, max_bins: int = None, delta=None, streams: int = 3) -> list:
    """Encodes a whole KV cache [L, 2, T, H, D] (GPU, unit innermost stride) chunk by chunk, as
    LMCacheEngine.store does with one to_bytes call per chunk (LMCache/lmcache/cache_engine.py:205-255
    in the reference), but without waiting for a chunk's payload size before the next chunk's kernels
    are enqueued: up to `batch` chunks are in flight; a chunk's sizes come back by an asynchronous copy
    into pinned memory, and its streams are gathered once `batch` later chunks have been enqueued, so
    the host never waits for the GPU except at the end.  Every chunk in flight keeps its own scratch
    (136 MB for a 7B-shape chunk).  Consecutive chunks run on `streams` side streams in turn (see
    _side_streams); the caller's stream waits for them before the call returns.
    Returns the chunks' CacheGenGPUEncoderOutput objects, identical to per-chunk encode_function calls."""
    kmax = _table_bins(key_bins, value_bins, max_bins)
    T = kv.shape[2]
    caller = torch.cuda.current_stream(kv.device)
    lanes = _side_streams(kv.device, streams)
    for side in lanes:
        side.wait_stream(caller)  # the cache is ready on the caller's stream
    result, in_flight = [], collections.deque()

    def finish_oldest():
        p, host, arrived, side = in_flight.popleft()
        arrived.synchronize()
        with torch.cuda.stream(side):
            out = p.finish(host)
        # made on a side stream, used and freed by the caller on its own
        for t in _tensors_of(out):
            t.record_stream(caller)
        result.append(out)

    for i, s in enumerate(range(0, T, chunk_tokens)):
        side = lanes[i % len(lanes)]
        with torch.cuda.stream(side):
            p = _PendingChunk(kv[:, :, s:s + chunk_tokens], key_bins, value_bins, kmax, delta=delta)
            host = torch.empty(p.tail.shape, dtype=p.tail.dtype, pin_memory=True)
            host.copy_(p.tail, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(side)
        in_flight.append((p, host, arrived, side))
        # the oldest chunk's sizes arrived long ago: its gather queues up behind the kernels of the chunks
        # after it, and the host work of finishing it runs while the GPU is busy with them
        if len(in_flight) > batch:
            finish_oldest()
    while in_flight:
        finish_oldest()
    for side in lanes:
        caller.wait_stream(side)
    return result


_SIDE_STREAMS = {}


def _side_streams(device, n):
    """n streams of `device`, made once and kept: consecutive chunks of encode_many go to different
    streams, so that one chunk's kernels fill the SMs that the last, partly filled wave of the previous
    chunk's coder kernel leaves idle (2,048 blocks over 1,480 resident ones: 1.4 waves)."""
    key = (torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device())
    have = _SIDE_STREAMS.setdefault(key, [])
    while len(have) < n:
        have.append(torch.cuda.Stream(device=device))
    return have[:n]


def _tensors_of(out: CacheGenGPUEncoderOutput):
    yield out.cdf
    yield out.max_tensors_key
    yield out.max_tensors_value
    for piece in out.data_chunks:
        yield piece.bytestream
        yield piece.bytestream_lengths


def encode_levels(kv: torch.Tensor, levels: list) -> list:
    """One chunk of KV, [L, 2, T, H, D] on the GPU, encoded at several bin settings: `levels` is a list
    of (key_bins, value_bins) pairs, the result one CacheGenGPUEncoderOutput per pair, each identical
    to what encode_function gives with those bins.  This is what the reference's adaptation scripts
    store per chunk (one blob per QUANT_LEVEL, run_adaptation.py:61-72) so that config_selection can
    pick a level per chunk (src/utils.py:294-314).  The levels share the max|x| pass and one host
    synchronisation; the coder runs once per level, and it is what an encode spends most time in."""
    if kv.stride(4) != 1:
        kv = kv.contiguous()
    scales = row_scales(kv)
    pending = [_PendingChunk(kv, kb, vb, _table_bins(kb, vb), scales=scales) for kb, vb in levels]
    host = torch.cat([p.tail for p in pending]).cpu()  # the one synchronisation
    out, pos = [], 0
    for p in pending:
        out.append(p.finish(host[pos:pos + p.nsub + 2]))
        pos += p.nsub + 2
    return out


@_lmcache_nvtx_annotate
def encode_function(kv: torch.Tensor, config: CacheGenConfig, key_bins: torch.Tensor, value_bins: torch.Tensor,
                    chunk_size: int, max_bins: int = None, delta=None) -> CacheGenGPUEncoderOutput:
    """Encodes one chunk of KV, [L, 2, T, H, D] on the GPU, T == chunk_size (enc.py:247-301)."""
    num_heads, head_size = kv.shape[-2:]
    L = kv.shape[0]
    if kv.shape[2] != chunk_size:
        raise RuntimeError(f"chunk_size {chunk_size} does not match the {kv.shape[2]} tokens of the blob")
    kmax = _table_bins(key_bins, value_bins, max_bins)
    sym, scales, cdf = quantize_and_tables(kv, key_bins, value_bins, kmax, delta=delta)
    stream_bytes, lengths, offs = encode_streams(cdf, sym)
    data_chunks = []
    step = CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK
    nsub = len(offs) - 1
    for j in range(nsub):
        piece = stream_bytes[offs[j]:offs[j + 1]]
        data_chunks.append(CacheGenGPUBytestream(
            bytestream=piece if nsub == 1 else piece.clone(),  # a view would pickle the whole buffer
            bytestream_lengths=lengths[j] if nsub == 1 else lengths[j].clone(),
            ntokens=min(step, chunk_size - j * step)))
    return CacheGenGPUEncoderOutput(
        data_chunks, cdf,
        max_tensors_key=scales[:L].clone().unsqueeze(-1),
        max_tensors_value=scales[L:].clone().unsqueeze(-1),
        num_heads=num_heads, head_size=head_size)


def pack_sparse_tables(counts: torch.Tensor, bins: torch.Tensor, nchannels: int, bins_cpu: torch.Tensor = None):
    """Byte counts of quantize_and_tables -> the parts of the sparse table form (cg_pack_sparse_tables).
    Returns (tables uint8 with room for every count, int32 word holding the number of counts written,
    offset of the counts inside `tables`); the used size is that offset plus that number."""
    dev = counts.device
    bins_cpu = bins.cpu() if bins_cpu is None else bins_cpu
    nrows = bins_cpu.numel()
    count_off = torch.tensor(flat_format.table_row_offsets(bins_cpu, nchannels), dtype=torch.int64, device=dev)
    moffs = flat_format.mask_row_offsets(bins_cpu, nchannels)
    mask_off = torch.tensor(moffs, dtype=torch.int64, device=dev)
    off_masks, off_counts = flat_format.sparse_parts(nrows, nchannels, moffs[-1])
    tables = torch.zeros(off_counts + counts.numel(), dtype=torch.uint8, device=dev)
    ngroups = nrows * ((nchannels + _lib.CG_GROUP_CHANNELS - 1) // _lib.CG_GROUP_CHANNELS)
    with torch.cuda.device(dev):
        rc = _lib.lib().cg_pack_sparse_tables(_ptr(counts), _ptr(count_off), _ptr(bins), nrows, nchannels,
                                              _ptr(tables), ctypes.c_void_p(tables.data_ptr() + off_masks),
                                              _ptr(mask_off), ctypes.c_void_p(tables.data_ptr() + off_counts),
                                              _stream(dev))
    _lib.check(rc, "cg_pack_sparse_tables")
    written = tables[4 * ngroups:4 * ngroups + 4].view(torch.int32)
    return tables, written, off_counts


def encode_flat(kv: torch.Tensor, key_bins: torch.Tensor, value_bins: torch.Tensor,
                compact_tables=True, max_bins: int = None, delta=None) -> flat_format.FlatChunk:
    """Encodes one chunk of KV, [L, 2, T, H, D] on the GPU, into a CGB2 container on the GPU
    (flat_format.py): the same tables, lengths and streams as encode_function, with uint16 lengths and
    the tables in the smallest form that can hold them.  compact_tables: True (sparse byte counts when
    every non-centre histogram count fits a byte and no row has more than 32 of them, else dense byte
    counts when the counts fit, else the int16 tables), "counts" (never sparse) or False (always int16)."""
    L, _, T, H, D = kv.shape
    C = H * D
    kmax = _table_bins(key_bins, value_bins, max_bins)
    bins = torch.cat((key_bins, value_bins)).to(device=kv.device, dtype=torch.float32).contiguous()
    bins_cpu = bins.cpu()
    sym, scales, cdf, counts, qstatus = quantize_and_tables(kv, key_bins, value_bins, kmax, with_counts=True,
                                                            bins_cpu=bins_cpu, delta=delta)
    try_sparse = compact_tables is True and flat_format.sparse_representable(bins_cpu)
    if try_sparse:
        sparse, written, off_counts = pack_sparse_tables(counts, bins, C, bins_cpu)
        extra = torch.cat((qstatus.to(torch.int64), written.to(torch.int64)))
        stream_bytes, lengths, offs, (qbits, nwritten) = encode_streams(cdf, sym, extra_status=extra)
    else:
        stream_bytes, lengths, offs, qbits = encode_streams(cdf, sym, extra_status=qstatus)
    fits = bool(compact_tables) and not (qbits & _lib.CG_S_COUNT_OVERFLOW)
    if fits and try_sparse:
        kind, tables = flat_format.TABLES_SPARSE, sparse[:off_counts + nwritten]
    elif fits:
        kind, tables = flat_format.TABLES_COUNTS, counts
    else:
        kind, tables = flat_format.TABLES_CDF, cdf.view(torch.uint8).reshape(-1)
    header = flat_format.layout(L, H, D, T, kmax + 1, kv.dtype, kind, tables.numel(), flat_format.LENGTHS_U16, offs,
                                bins_checksum=flat_format.bins_checksum(bins_cpu, delta))
    # zeroed, so that the alignment gaps between the sections are defined: the same KV gives the same bytes
    blob = torch.zeros(header.total, dtype=torch.uint8, device=kv.device)
    head = header.pack()
    blob[:len(head)].copy_(torch.frombuffer(bytearray(head), dtype=torch.uint8), non_blocking=True)
    chunk = flat_format.FlatChunk(blob, header)
    chunk.scales().copy_(scales)
    blob[header.off_tables:header.off_tables + tables.numel()].copy_(tables)
    n = 2 * L * C
    blob[header.off_lengths:header.off_lengths + len(offs[:-1]) * n * 2].view(torch.int16).copy_(
        lengths.reshape(-1).to(torch.int16))  # at most 520: fits
    blob[header.off_payload:header.off_payload + offs[-1]].copy_(stream_bytes)
    return chunk


class CacheGenSerializer(Serializer):
    """Reference: enc.py:303-348.  `cachegen_config` may be given instead of looking it up from
    metadata.model_name (quality levels other than the built-in ones).  wire_format: "pickle" (the
    reference's blob, default) or "flat" (the CGB2 container of flat_format.py, which the reference
    cannot read)."""

    def __init__(self, config: LMCacheEngineConfig, metadata: LMCacheEngineMetadata,
                 cachegen_config: CacheGenConfig = None, wire_format: str = "pickle", table_max_bins: int = None,
                 delta: "CGBasics.DeltaCoding" = None):
        if wire_format not in ("pickle", "flat"):
            raise ValueError(f"unknown wire format {wire_format!r}")
        self.wire_format = wire_format
        self.delta = delta  # anchor-token delta coding: off (None) is the reference's behaviour
        self.table_max_bins = table_max_bins  # see _table_bins: set for a layer shard of a model
        _lib.lib()  # fail at construction if the CUDA library is missing
        self.cachegen_config = cachegen_config or CacheGenConfig.from_model_name(metadata.model_name)
        self.chunk_size = config.chunk_size
        self.fmt = metadata.fmt
        self.key_bins = self.make_key_bins(self.cachegen_config)
        self.value_bins = self.make_value_bins(self.cachegen_config)

    def make_key_bins(self, config: CacheGenConfig) -> torch.Tensor:
        return CGBasics.make_key_bins(config, "cuda")

    def make_value_bins(self, config: CacheGenConfig) -> torch.Tensor:
        return CGBasics.make_value_bins(config, "cuda")

    def encode(self, tensor: torch.Tensor) -> CacheGenGPUEncoderOutput:
        """`to_bytes` without the final pickle: the encoded chunk with its tensors on the GPU."""
        if self.fmt == "huggingface":
            tensor = tensor.permute(0, 1, 3, 2, 4)  # a view; the kernels read it through its strides
        ntokens = tensor.shape[2]
        return encode_function(tensor.cuda(), self.cachegen_config, self.key_bins, self.value_bins, ntokens,
                               max_bins=self.table_max_bins, delta=self.delta)

    def encode_many(self, tensor: torch.Tensor, chunk_tokens: int = None, batch: int = 16, streams: int = 3) -> list:
        """A whole KV cache, one encoded chunk per `chunk_tokens` (default: the configured chunk size)
        tokens, with up to `batch` chunks in flight on the GPU, on `streams` streams in turn."""
        if self.fmt == "huggingface":
            tensor = tensor.permute(0, 1, 3, 2, 4)
        tensor = tensor.cuda()
        if tensor.stride(4) != 1:
            tensor = tensor.contiguous()
        return encode_many(tensor, self.key_bins, self.value_bins, chunk_tokens or self.chunk_size, batch,
                           max_bins=self.table_max_bins, delta=self.delta, streams=streams)

    def encode_levels(self, tensor: torch.Tensor, cachegen_configs: list) -> list:
        """The chunk encoded with each of `cachegen_configs` (CacheGenConfig objects, e.g. the three
        QUANT_LEVEL settings) in one go: one CacheGenGPUEncoderOutput per configuration, equal to what
        a serializer built with that configuration returns from `encode`."""
        if self.fmt == "huggingface":
            tensor = tensor.permute(0, 1, 3, 2, 4)
        tensor = tensor.cuda()
        return encode_levels(tensor, [(CGBasics.make_key_bins(c, tensor.device), CGBasics.make_value_bins(c, tensor.device))
                                      for c in cachegen_configs])

    def encode_flat(self, tensor: torch.Tensor, compact_tables=True) -> flat_format.FlatChunk:
        """The chunk as a CGB2 container on the GPU."""
        if self.fmt == "huggingface":
            tensor = tensor.permute(0, 1, 3, 2, 4)
        tensor = tensor.cuda()
        if tensor.stride(4) != 1:
            tensor = tensor.contiguous()
        return encode_flat(tensor, self.key_bins, self.value_bins, compact_tables, max_bins=self.table_max_bins,
                           delta=self.delta)

    @_lmcache_nvtx_annotate
    def to_bytes(self, tensor: torch.Tensor) -> bytes:
        """KV blob ([L,2,T,H,D] for "vllm", [L,2,H,T,D] for "huggingface") -> bytes (enc.py:324-348):
        the reference's pickle, or a CGB2 container when wire_format == "flat"."""
        if self.wire_format == "flat":
            return self.encode_flat(tensor).tobytes()
        return self.encode(tensor).to_bytes()
