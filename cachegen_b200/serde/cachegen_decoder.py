"""CacheGenDeserializer (reference: LMCache/lmcache/storage_backend/serde/cachegen_decoder.py:114-173).

`from_bytes` keeps the reference's contract -- pickled CacheGenGPUEncoderOutput in, KV blob tensor on
the GPU out, bf16 [L,2,T,H,D] for "vllm" and fp16 [L,2,H,T,D] for "huggingface" -- with the
per-sub-chunk launches and the fp32 dequantise / stack / permute / cast chain replaced by two C-ABI
calls: cg_decode_offsets (the cumsum of dec.py:70) and cg_decode_dequant (everything else).
(dec.py = cachegen_decoder.py of the reference.)
"""
import ctypes
from typing import List

import torch

from .. import _lib
from .. import torchac_cuda
from ..config import LMCacheEngineConfig, LMCacheEngineMetadata
from ..utils import _lmcache_nvtx_annotate
from . import cachegen_basics as CGBasics
from . import flat_format
from .cachegen_basics import CacheGenConfig, CacheGenGPUBytestream, CacheGenGPUEncoderOutput
from .serde import Deserializer

_DTYPES = {torch.float16: _lib.CG_F16, torch.bfloat16: _lib.CG_BF16}


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def do_dequantize(t: torch.Tensor, bins: torch.Tensor, maxtensors: torch.Tensor) -> torch.Tensor:
    """The reference's dequantisation formula on torch tensors (dec.py:24-34); the product path
    computes the same values inside cg_decode_dequant.  t [L,T,C] float, bins [L], maxtensors [L,T,1]."""
    C = (bins // 2 - 1)[:, None, None]
    t = t - C
    t = t / C
    t = t * maxtensors
    return t


@_lmcache_nvtx_annotate
def bytes_to_tensor(bs: bytes, device="cuda") -> torch.Tensor:
    """A byte string as a uint8 tensor on `device` (dec.py:37-41); to a GPU through pinned staging."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # a read-only buffer, and it is only read
        view = torch.frombuffer(bs, dtype=torch.uint8)
    device = torch.device(device)
    if device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device() if device.index is None else device.index)
        return CGBasics.staging().whole_to_device(view, device)
    return view.clone()


@_lmcache_nvtx_annotate
def recombine_bytes(bytes_tensor: torch.Tensor, output_lengths: torch.Tensor) -> torch.Tensor:
    """Back-to-back streams as padded rows [nlayers, nchannels, 256] for decode_fast_new
    (dec.py:43-49): row (r, c) holds the 256 bytes that start where stream (r, c) starts, reading
    no further than the last byte of `bytes_tensor`.  The legacy layout; from_bytes does not use it."""
    width = CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK
    lengths = output_lengths.reshape(-1).to(torch.int64)
    starts = lengths.cumsum(0) - lengths
    index = starts[:, None] + torch.arange(width, device=starts.device)
    index.clamp_(max=bytes_tensor.numel() - 1)
    return bytes_tensor[index].reshape(*output_lengths.shape, width)


@_lmcache_nvtx_annotate
def decode_chunk(cdf: torch.Tensor, data_chunk: CacheGenGPUBytestream, target_buffer: torch.Tensor) -> None:
    """Symbols of one sub-chunk into target_buffer [2L, ntokens, C] uint8, strided ok (dec.py:53-75)."""
    lengths = data_chunk.bytestream_lengths
    length_prefsum = lengths.flatten().cumsum(0).reshape(lengths.shape)
    torchac_cuda.decode_fast_prefsum(cdf, data_chunk.bytestream, length_prefsum, target_buffer)


@_lmcache_nvtx_annotate
def decode_function_gpu(cdf: torch.Tensor, data_chunks: List[CacheGenGPUBytestream], layers_in_key: int,
                        chunk_size: int, output: torch.Tensor):
    """Symbol-level decode with the reference's signature (dec.py:78-112): fills `output`
    (uint8 [chunk_size, 2L*C]) and returns (key, value) symbols as float32 [L, chunk_size, C]."""
    nlayers, nchannels, _ = cdf.shape
    output = output.reshape((nlayers, chunk_size, nchannels))
    start = 0
    for data_chunk in data_chunks:
        end = start + data_chunk.ntokens
        decode_chunk(cdf, data_chunk, output[:, start:end, :])
        start = end
    out = output.reshape((2, layers_in_key, chunk_size, nchannels))
    key, value = out.float()
    return key, value


def _check_chunk(eo: CacheGenGPUEncoderOutput):
    """Shape checks of an unpickled reference blob -> (L, C, lp, T)."""
    cdf = eo.cdf
    if cdf.dim() != 3 or cdf.dtype != torch.int16:
        raise RuntimeError("CDF must be an int16 tensor [2L, C, Lp]")
    NL, C, lp = cdf.shape
    L = NL // 2
    mk, mv = eo.max_tensors_key, eo.max_tensors_value
    T = mk.shape[1]
    if eo.num_heads * eo.head_size != C or mk.shape[0] != L or mv.shape[0] != L or mv.shape[1] != T:
        raise RuntimeError("inconsistent shapes in the encoded chunk")
    if mk.dtype not in _DTYPES or mk.dtype != mv.dtype:
        raise TypeError(f"scales must be float16 or bfloat16, got {mk.dtype} / {mv.dtype}")
    if sum(dc.ntokens for dc in eo.data_chunks) != T:
        raise RuntimeError("sub-chunk token counts do not add up to the chunk's tokens")
    return L, C, lp, T


def _to_device(t: torch.Tensor, dev) -> torch.Tensor:
    """Encoded chunks may arrive with their tensors in (pinned) host memory: stage them on `dev`."""
    if t.device == dev:
        return t
    return t.to(dev, non_blocking=True)


class _ChunkView:
    """What a decode needs from one encoded chunk, whichever container it came in, on the GPU."""

    def __init__(self, eo, dev, bins_cpu, delta=None):
        self.keep = []
        if isinstance(eo, flat_format.FlatChunk):
            fc = eo if eo.blob.device == dev else eo.to(dev, non_blocking=True)
            h = fc.header
            self.L, self.H, self.D, self.T, self.lp = h.L, h.H, h.D, h.T, h.lp
            self.C = h.H * h.D
            self.scale_dtype = fc.scale_dtype
            sc = fc.scales()
            self.mk, self.mv = sc[:h.L], sc[h.L:]
            self.tables = fc.tables()
            self.table_kind = h.table_kind
            if ((h.table_kind != flat_format.TABLES_CDF or delta is not None) and h.bins_checksum and
                    h.bins_checksum != flat_format.bins_checksum(bins_cpu, delta)):
                raise RuntimeError("the container was written with other bin or delta settings")
            if (delta is None and h.table_kind == flat_format.TABLES_CDF and h.bins_checksum and
                    h.bins_checksum != flat_format.bins_checksum(bins_cpu)):
                # int16 tables decode with any bins, but a chunk written with delta coding does not
                raise RuntimeError("the container was written with other bin or delta settings")
            if h.table_kind == flat_format.TABLES_COUNTS:
                need = flat_format.table_row_offsets(bins_cpu, self.C)[-1]
                if h.off_lengths - h.off_tables < need:
                    raise RuntimeError("the container's byte-count tables are smaller than the configured bins need")
            elif h.table_kind == flat_format.TABLES_SPARSE:
                if not flat_format.sparse_representable(bins_cpu):
                    raise RuntimeError("sparse tables cannot describe the configured bins")
                need = flat_format.sparse_parts(2 * h.L, self.C, flat_format.mask_row_offsets(bins_cpu, self.C)[-1])[1]
                if h.off_lengths - h.off_tables < need:
                    raise RuntimeError("the container's sparse tables are smaller than the configured bins need")
            self.length_kind = h.length_kind
            self.subs = [(fc.payload(j), fc.lengths(j), fc.sub_tokens(j)) for j in range(h.nsub)]
            self.table_bytes = h.off_lengths - h.off_tables
            self.length_bytes = h.off_payload - h.off_lengths
            self.keep.append(fc.blob)
        else:
            L, C, lp, T = _check_chunk(eo)
            self.L, self.C, self.lp, self.T = L, C, lp, T
            self.H, self.D = eo.num_heads, eo.head_size
            self.scale_dtype = eo.max_tensors_key.dtype
            self.mk = _to_device(eo.max_tensors_key, dev).reshape(L, T).contiguous()
            self.mv = _to_device(eo.max_tensors_value, dev).reshape(L, T).contiguous()
            self.tables = _to_device(eo.cdf, dev).contiguous()
            self.table_kind = _lib.CG_TABLES_CDF
            self.length_kind = _lib.CG_LENGTHS_I32
            self.subs = []
            for dc in eo.data_chunks:
                if dc.bytestream.dtype != torch.uint8 or dc.bytestream.dim() != 1:
                    raise RuntimeError("bytestream must be a 1-D uint8 tensor")
                if dc.bytestream_lengths.dtype != torch.int32 or dc.bytestream_lengths.numel() != 2 * L * C:
                    raise RuntimeError("bytestream_lengths must be int32 [2L, C]")
                self.subs.append((_to_device(dc.bytestream, dev).contiguous(),
                                  _to_device(dc.bytestream_lengths, dev).contiguous(), dc.ntokens))
            self.table_bytes = self.tables.numel() * 2
            self.length_bytes = len(self.subs) * 2 * L * C * 4
            self.keep += [self.mk, self.mv, self.tables] + [t for s in self.subs for t in s[:2]]
        if sum(s[2] for s in self.subs) != self.T:
            raise RuntimeError("sub-chunk token counts do not add up to the chunk's tokens")
        for _, _, ntok in self.subs:
            if not 0 < ntok <= CGBasics.CACHEGEN_GPU_MAX_TOKENS_PER_CHUNK:
                raise RuntimeError("a sub-chunk holds 1..256 tokens")


def _on_gpu(eo) -> bool:
    return eo.blob.is_cuda if isinstance(eo, flat_format.FlatChunk) else eo.cdf.is_cuda


def _device_of(eo):
    return eo.blob.device if isinstance(eo, flat_format.FlatChunk) else eo.cdf.device


class DecodePlan:
    """Everything cg_decode_offsets / cg_decode_dequant need for a list of encoded chunks, built once:
    device-resident inputs, the job descriptors, the output blob and the launch arguments.  Chunks are
    CacheGenGPUEncoderOutput objects (the reference's blob, unpickled) or flat_format.FlatChunk
    containers, on the GPU or in (pinned) host memory."""

    def __init__(self, encoder_outputs: list, bins: torch.Tensor, fmt: str,
                 out_dtype: torch.dtype, out: torch.Tensor = None, workspace: dict = None, device=None,
                 peer_out: bool = False, delta=None):
        if not encoder_outputs:
            raise RuntimeError("nothing to decode")
        if fmt not in ("vllm", "huggingface"):
            raise ValueError(f"unknown KV format {fmt!r}")
        first = encoder_outputs[0]
        dev = torch.device(device) if device is not None else (
            _device_of(first) if _on_gpu(first) else torch.device("cuda", torch.cuda.current_device()))
        ws = workspace if workspace is not None else {}
        bins_cpu = ws.get("bins_cpu")
        if bins_cpu is None or bins_cpu.numel() != bins.numel():
            bins_cpu = bins.cpu()
            ws["bins_cpu"] = bins_cpu
        with torch.cuda.device(dev):
            views = [_ChunkView(eo, dev, bins_cpu, delta) for eo in encoder_outputs]
        v0 = views[0]
        L, C, lp, H, D, scale_dtype = v0.L, v0.C, v0.lp, v0.H, v0.D, v0.scale_dtype
        NL = 2 * L
        for v in views:
            if (v.L, v.C, v.lp, v.H, v.scale_dtype) != (L, C, lp, H, scale_dtype):
                raise RuntimeError("chunks of one decode call must share layers, channels, table length and dtype")
        if scale_dtype not in _DTYPES:
            raise TypeError(f"scales must be float16 or bfloat16, got {scale_dtype}")
        total_T = sum(v.T for v in views)
        if bins.numel() != NL:
            raise RuntimeError(f"bins describe {bins.numel() // 2} layers, the blob has {L}")
        shape = (L, 2, total_T, H, D) if fmt == "vllm" else (L, 2, H, total_T, D)
        if out is None:
            out = torch.empty(shape, dtype=out_dtype, device=dev)
        elif (tuple(out.shape) != shape or out.dtype != out_dtype or out.stride(4) != 1 or
              (out.device != dev and not peer_out)):
            # peer_out: `out` is memory of another GPU of the box that this GPU can address
            # (cachegen_b200.parallel.buffer_on_root); the kernel stores into it over NVLink
            raise RuntimeError("output tensor has the wrong shape, dtype, device or innermost stride")
        if fmt == "vllm":
            o_layer, o_kv, o_token, o_head = out.stride(0), out.stride(1), out.stride(2), out.stride(3)
        else:
            o_layer, o_kv, o_head, o_token = out.stride(0), out.stride(1), out.stride(2), out.stride(3)
        nslab = (C + _lib.CG_GROUP_CHANNELS - 1) // _lib.CG_GROUP_CHANNELS
        ngroups = NL * nslab
        njobs_total = sum(len(v.subs) for v in views)
        goff = ws.get("group_off")
        if goff is None or goff.numel() < njobs_total * ngroups or goff.device != dev:
            goff = torch.empty(njobs_total * ngroups, dtype=torch.int64, device=dev)
            ws["group_off"] = goff
        status = ws.get("status")
        if status is None or status.device != dev:
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            ws["status"] = status
        row_offs = {}
        for kind, name, fn in ((_lib.CG_TABLES_COUNTS, "table_row_off", flat_format.table_row_offsets),
                               (_lib.CG_TABLES_SPARSE, "mask_row_off", flat_format.mask_row_offsets)):
            if any(v.table_kind == kind for v in views):
                t = ws.get(name)
                if t is None or t.device != dev or ws.get(name + "_c") != C:
                    t = torch.tensor(fn(bins_cpu, C), dtype=torch.int64, device=dev)
                    ws[name], ws[name + "_c"] = t, C
                row_offs[kind] = t

        esz = out.element_size()
        self.keep = list(row_offs.values())  # tensors that must outlive the launches
        jobs_all = []
        self.payload_bytes = self.table_bytes = self.length_bytes = 0
        t0 = 0
        for v in views:
            self.keep += v.keep
            self.table_bytes += v.table_bytes
            self.length_bytes += v.length_bytes
            tc = 0
            for bs, ln, ntok in v.subs:
                self.payload_bytes += bs.numel()
                job = _lib.DecodeJob()
                job.tables = v.tables.data_ptr()
                job.bytes = bs.data_ptr()
                job.lengths = ln.data_ptr()
                job.group_off = goff.data_ptr() + 8 * len(jobs_all) * ngroups
                job.scales_k = v.mk.data_ptr() + v.mk.element_size() * tc
                job.scales_v = v.mv.data_ptr() + v.mv.element_size() * tc
                job.out = out.data_ptr() + esz * (t0 + tc) * o_token
                job.table_row_off = row_offs[v.table_kind].data_ptr() if v.table_kind in row_offs else None
                job.nbytes = bs.numel()
                job.tables_nbytes = v.table_bytes
                job.ntokens = ntok
                job.scale_stride = v.T
                job.table_kind = v.table_kind
                job.length_kind = v.length_kind
                jobs_all.append(job)
                tc += ntok
            t0 += v.T
        self.batches = []
        for b in range(0, njobs_total, _lib.CG_MAX_DECODE_JOBS):
            batch = jobs_all[b:b + _lib.CG_MAX_DECODE_JOBS]
            self.batches.append(((_lib.DecodeJob * len(batch))(*batch), len(batch),
                                 ctypes.c_void_p(goff.data_ptr() + 8 * b * ngroups)))
        self.delta_group, self.res_bins = 0, None
        if delta is not None:
            self.delta_group = delta.group
            self.res_bins = delta.residual_bins(bins[:L], bins[L:], dev)
            self.keep.append(self.res_bins)
        self.out, self.dev, self.bins, self.status, self.goff = out, dev, bins, status, goff
        self.dims = (L, H, D, C, lp, NL, total_T)
        self.strides = (o_layer, o_kv, o_token, o_head)
        self.dtypes = (_DTYPES[scale_dtype], _DTYPES[out_dtype])
        self.njobs = njobs_total
        # bytes one decode pass must move: 16-bit KV out, payload, tables, lengths, scales in
        self.scale_bytes = NL * total_T * 2
        self.output_bytes = NL * total_T * C * esz

    # launches per call: 2 per batch
    def run_offsets(self) -> None:
        lib = _lib.lib()
        L, H, D, C, lp, NL, _ = self.dims
        with torch.cuda.device(self.dev):
            st = _stream(self.dev)
            for arr, n, goff in self.batches:
                rc = lib.cg_decode_offsets(arr, n, NL, C, goff, ctypes.c_void_p(self.status.data_ptr()), st)
                _lib.check(rc, "cg_decode_offsets")

    # launches per call: 1 per batch
    def run_decode(self) -> None:
        lib = _lib.lib()
        L, H, D, C, lp, NL, _ = self.dims
        o_layer, o_kv, o_token, o_head = self.strides
        with torch.cuda.device(self.dev):
            st = _stream(self.dev)
            for arr, n, _ in self.batches:
                if self.delta_group:
                    rc = lib.cg_decode_dequant_delta(arr, n, L, H, D, lp, ctypes.c_void_p(self.bins.data_ptr()),
                                                     self.delta_group, ctypes.c_void_p(self.res_bins.data_ptr()),
                                                     self.dtypes[0], self.dtypes[1], o_layer, o_kv, o_token, o_head,
                                                     ctypes.c_void_p(self.status.data_ptr()), st)
                else:
                    rc = lib.cg_decode_dequant(arr, n, L, H, D, lp, ctypes.c_void_p(self.bins.data_ptr()),
                                               self.dtypes[0], self.dtypes[1], o_layer, o_kv, o_token, o_head,
                                               ctypes.c_void_p(self.status.data_ptr()), st)
                _lib.check(rc, "cg_decode_dequant")

    def run(self) -> torch.Tensor:
        self.run_offsets()
        self.run_decode()
        cur = torch.cuda.current_stream(self.dev)
        for t in self.keep:
            t.record_stream(cur)
        return self.out

    @property
    def launches(self) -> int:
        return 3 * len(self.batches)


def decode_many(encoder_outputs: List[CacheGenGPUEncoderOutput], bins: torch.Tensor, fmt: str,
                out_dtype: torch.dtype, out: torch.Tensor = None, workspace: dict = None, delta=None) -> torch.Tensor:
    """Fused decode of consecutive encoded chunks of one KV cache into one blob.

    The chunks' tokens are laid one after the other along the token axis of the result, which has
    shape [L,2,T,H,D] ("vllm") or [L,2,H,T,D] ("huggingface"), T the total token count -- what
    LMCacheEngine.retrive builds with torch.cat from per-chunk from_bytes calls
    (LMCache/lmcache/cache_engine.py:282-320 in the reference).  All sub-chunks of all chunks go
    through cg_decode_offsets + cg_decode_dequant in batches of up to 40 per launch.

    The chunks' tensors may live on the GPU or in (pinned) host memory; host tensors are copied to the
    GPU on the current stream first.  bins: float32 [2L] on the GPU (key bins then value bins).
    `out`, when given, must have the result's shape and dtype with a unit innermost stride (any other
    strides).  `workspace` caches the small offset / status buffers between calls.
    """
    return DecodePlan(encoder_outputs, bins, fmt, out_dtype, out=out, workspace=workspace, delta=delta).run()


_copy_streams = {}


def _chunk_tokens(eo) -> int:
    return eo.num_tokens if isinstance(eo, flat_format.FlatChunk) else eo.max_tensors_key.shape[1]


def decode_many_pipelined(encoder_outputs: List[CacheGenGPUEncoderOutput], bins: torch.Tensor, fmt: str,
                          out_dtype: torch.dtype, out: torch.Tensor = None, groups: int = 4,
                          workspaces: list = None, delta=None) -> torch.Tensor:
    """decode_many for encoded chunks held in pinned host memory, with the host-to-device copies of
    one group of chunks overlapped with the decode of the previous group (a copy stream per device;
    the decode launches stay on the caller's current stream).  `workspaces`: one dict per group."""
    n = len(encoder_outputs)
    groups = max(1, min(groups, n))
    first = encoder_outputs[0]
    dev = _device_of(first) if _on_gpu(first) else torch.device("cuda", torch.cuda.current_device())
    if groups == 1 or _on_gpu(first):
        return decode_many(encoder_outputs, bins, fmt, out_dtype, out=out,
                           workspace=workspaces[0] if workspaces else None)
    L, H, D = bins.numel() // 2, first.num_heads, first.head_size
    total_T = sum(_chunk_tokens(eo) for eo in encoder_outputs)
    shape = (L, 2, total_T, H, D) if fmt == "vllm" else (L, 2, H, total_T, D)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=dev)
    elif tuple(out.shape) != shape:
        raise RuntimeError("output tensor has the wrong shape")
    copy_stream = _copy_streams.get(dev)
    if copy_stream is None:
        copy_stream = torch.cuda.Stream(device=dev)
        _copy_streams[dev] = copy_stream
    cur = torch.cuda.current_stream(dev)
    copy_stream.wait_stream(cur)
    if workspaces is None:
        workspaces = [dict() for _ in range(groups)]
    per = (n + groups - 1) // groups
    t0 = 0
    for g in range(groups):
        part = encoder_outputs[g * per:(g + 1) * per]
        if not part:
            break
        tg = sum(_chunk_tokens(eo) for eo in part)
        view = out[:, :, t0:t0 + tg] if fmt == "vllm" else out[:, :, :, t0:t0 + tg]
        with torch.cuda.stream(copy_stream):
            part = _stage_flat(part, workspaces[g], dev)
            plan = DecodePlan(part, bins, fmt, out_dtype, out=view, workspace=workspaces[g], device=dev, delta=delta)
            ready = torch.cuda.Event()
            ready.record(copy_stream)
        cur.wait_event(ready)
        plan.run()
        t0 += tg
    return out


def _stage_flat(part: list, ws: dict, dev) -> list:
    """Copies a group's CGB2 containers from host memory into one device buffer that the workspace
    keeps between calls (no allocation per call, nothing for the caching allocator to hold back while
    the previous call's kernels still run).  Chunks of other kinds are returned as they are."""
    if not all(isinstance(eo, flat_format.FlatChunk) and not eo.blob.is_cuda for eo in part):
        return part
    starts, need = [], 0
    for eo in part:
        starts.append(need)
        need += (eo.blob.numel() + flat_format.ALIGN - 1) // flat_format.ALIGN * flat_format.ALIGN
    arena = ws.get("arena")
    if arena is None or arena.device != dev or arena.numel() < need:
        arena = torch.empty(need, dtype=torch.uint8, device=dev)
        ws["arena"] = arena
    staged = []
    for eo, a in zip(part, starts):
        dst = arena[a:a + eo.blob.numel()]
        dst.copy_(eo.blob, non_blocking=True)
        staged.append(flat_format.FlatChunk(dst, eo.header))
    return staged


def decode_to_kv(encoder_output: CacheGenGPUEncoderOutput, bins: torch.Tensor, fmt: str, out_dtype: torch.dtype,
                 out: torch.Tensor = None, workspace: dict = None, delta=None) -> torch.Tensor:
    """Fused decode of one encoded chunk into its KV blob (see decode_many)."""
    return decode_many([encoder_output], bins, fmt, out_dtype, out=out, workspace=workspace, delta=delta)


class CacheGenDeserializer(Deserializer):
    """Reference: dec.py:114-173.  `out_dtype` overrides the reference's fixed choice (bf16 for "vllm",
    fp16 for "huggingface"); `cachegen_config` replaces the lookup by model name."""

    def __init__(self, config: LMCacheEngineConfig, metadata: LMCacheEngineMetadata,
                 cachegen_config: CacheGenConfig = None, out_dtype: torch.dtype = None,
                 delta: "CGBasics.DeltaCoding" = None):
        _lib.lib()  # fail at construction if the CUDA library is missing
        self.delta = delta  # anchor-token delta coding: must be what the serializer was given
        self.cachegen_config = cachegen_config or CacheGenConfig.from_model_name(metadata.model_name)
        self.chunk_size = config.chunk_size
        self.fmt = metadata.fmt
        if self.fmt not in ("vllm", "huggingface"):
            raise ValueError(f"unknown KV format {self.fmt!r}")
        self.out_dtype = out_dtype or (torch.bfloat16 if self.fmt == "vllm" else torch.float16)
        self.key_bins = self.make_key_bins(self.cachegen_config)
        self.value_bins = self.make_value_bins(self.cachegen_config)
        self._bins = torch.cat((self.key_bins, self.value_bins)).contiguous()
        self._workspace = {}

    def make_key_bins(self, config: CacheGenConfig) -> torch.Tensor:
        return CGBasics.make_key_bins(config, "cuda")

    def make_value_bins(self, config: CacheGenConfig) -> torch.Tensor:
        return CGBasics.make_value_bins(config, "cuda")

    def decode(self, encoder_output: CacheGenGPUEncoderOutput, out: torch.Tensor = None) -> torch.Tensor:
        """`from_bytes` without the unpickling."""
        ntokens = _chunk_tokens(encoder_output)
        if ntokens > self.chunk_size:
            # the reference slices a chunk_size-row buffer and fails in its reshape (dec.py:138-141,101)
            raise RuntimeError(f"blob holds {ntokens} tokens, more than chunk_size = {self.chunk_size}")
        return decode_to_kv(encoder_output, self._bins_on(_device_of(encoder_output)), self.fmt, self.out_dtype,
                            out=out, workspace=self._workspace, delta=self.delta)

    def decode_many(self, encoder_outputs: List[CacheGenGPUEncoderOutput], out: torch.Tensor = None) -> torch.Tensor:
        """Consecutive chunks of one KV cache into one blob, in as few launches as possible."""
        for eo in encoder_outputs:
            if _chunk_tokens(eo) > self.chunk_size:
                raise RuntimeError(f"a blob holds more tokens than chunk_size = {self.chunk_size}")
        return decode_many(encoder_outputs, self._bins_on(_device_of(encoder_outputs[0])), self.fmt, self.out_dtype,
                           out=out, workspace=self._workspace, delta=self.delta)

    def decode_many_host(self, encoder_outputs: List[CacheGenGPUEncoderOutput], out: torch.Tensor = None,
                         groups: int = None) -> torch.Tensor:
        """decode_many for chunks whose tensors sit in pinned host memory: copies and decodes overlap.
        groups: how many parts the chunks are split into (default: up to 32); the decode of a part
        runs while the next one is copied, so the last part's decode is all that is not hidden."""
        if groups is None:
            groups = min(32, len(encoder_outputs))
        ws = self._workspace.setdefault("groups", [dict() for _ in range(groups)])
        if len(ws) < groups:
            ws += [dict() for _ in range(groups - len(ws))]
        return decode_many_pipelined(encoder_outputs, self._bins_on(_device_of(encoder_outputs[0])), self.fmt,
                                     self.out_dtype, out=out, groups=groups, workspaces=ws, delta=self.delta)

    def group_status_words(self):
        """Status words of the pipelined path's per-group workspaces."""
        return [w["status"] for w in self._workspace.get("groups", []) if "status" in w]

    def plan(self, encoder_outputs: List[CacheGenGPUEncoderOutput], out: torch.Tensor = None,
             peer_out: bool = False, workspace: dict = None) -> DecodePlan:
        """The launch plan decode_many would run, for callers that decode the same chunks repeatedly.
        peer_out: `out` lives on another GPU of the box (see DecodePlan).  Plans built on one workspace
        (default: this object's) share its offset buffer: `run` recomputes the offsets every time, but
        `run_decode` alone is only valid while no other plan of the workspace has run in between."""
        return DecodePlan(encoder_outputs, self._bins_on(_device_of(encoder_outputs[0])), self.fmt, self.out_dtype,
                          out=out, workspace=self._workspace if workspace is None else workspace, peer_out=peer_out,
                          delta=self.delta)

    def _bins_on(self, dev) -> torch.Tensor:
        if not dev.type == "cuda":
            dev = torch.device("cuda", torch.cuda.current_device())
        if self._bins.device != dev:
            self._bins = self._bins.to(dev)
        return self._bins

    def check_status(self) -> None:
        """Synchronises and raises if a decode since the last check met malformed stream lengths."""
        words = ([self._workspace["status"]] if "status" in self._workspace else []) + self.group_status_words()
        for status in words:
            bits = int(status.item())
            if bits:
                status.zero_()
                raise RuntimeError("cachegen decode: " + _lib.status_text(bits))

    def from_bytes_many(self, blobs: List[bytes], out: torch.Tensor = None) -> torch.Tensor:
        """from_bytes for the blobs of consecutive chunks of one KV cache: one result tensor, as
        decode_many builds it; each blob is loaded while the copies of the one before are still on
        their way to the GPU."""
        dev = torch.device("cuda", torch.cuda.current_device())
        chunks = [flat_format.from_bytes(b, device=dev) if flat_format.is_flat(b) else CacheGenGPUEncoderOutput.from_bytes(b)
                  for b in blobs]
        return self.decode_many(chunks, out=out)

    @_lmcache_nvtx_annotate
    def from_bytes(self, bs: bytes) -> torch.Tensor:
        if flat_format.is_flat(bs):
            # a CGB2 container: one copy to the GPU, decoded in place
            return self.decode(flat_format.from_bytes(bs, device=torch.device("cuda", torch.cuda.current_device())))
        # tensors pickled on a GPU come back on that GPU; anything else is staged by the decode plan
        return self.decode(CacheGenGPUEncoderOutput.from_bytes(bs))
