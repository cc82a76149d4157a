"""Sharding of the codec's independent units across the GPUs of one box, one process per GPU.

Every (row, channel, sub-chunk) stream is independent, tables are per chunk and scales per (row,
token), so the codec has no exchange step: work is split by request, by token chunk or by layer and
each rank runs the single-GPU path on its share.  The only communication is the optional delivery of
decoded KV to the GPU that consumes it (`gather_layers`, NCCL over NVLink; gloo on CPU in the tests).
"""
from typing import List, Optional

import torch
import torch.distributed as dist


def partition(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced share of `n_units` for `rank` (the first n_units % world ranks get one more)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def max_over_ranks(value: float, device="cpu", group=None) -> float:
    """The slowest rank's time: what a whole-job throughput must be computed from."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def all_agree_ok(ok: bool, device="cpu", group=None) -> bool:
    """True when every rank reports success (a rank that met a malformed blob says so before any
    collective on the data path is entered)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(ok)
    t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item()) == 0


def gather_layers(local: torch.Tensor, total_layers: int, root: int = 0, out: Optional[torch.Tensor] = None,
                  group=None) -> Optional[torch.Tensor]:
    """Delivers layer-sharded decoded KV to `root`.

    local: this rank's layers, [L_r, 2, T, H, D] ("vllm") or [L_r, 2, H, T, D], L_r = len(partition(
    total_layers, world, rank)), contiguous.  On `root` returns the full blob [total_layers, ...]
    (`out` when given); elsewhere returns None.  Layer-major layout makes every rank's share one
    contiguous slab of the result, so each transfer is a single send / receive.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    mine = partition(total_layers, world, rank)
    if local.shape[0] != len(mine) or not local.is_contiguous():
        raise RuntimeError("local slab must be contiguous and hold exactly this rank's layers")
    if world == 1:
        if out is not None:
            out.copy_(local)
            return out
        return local
    if rank == root:
        if out is None:
            out = torch.empty((total_layers,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        ops: List[dist.P2POp] = []
        for r in range(world):
            part = partition(total_layers, world, r)
            if len(part) == 0:
                continue
            if r == root:
                out[part.start:part.stop].copy_(local)
            else:
                ops.append(dist.P2POp(dist.irecv, out[part.start:part.stop], r, group))
        for req in (dist.batch_isend_irecv(ops) if ops else []):
            req.wait()
        return out
    if len(mine):
        for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, local, root, group)]):
            req.wait()
    return None


_DTYPE_STR = {torch.float16: "<f2", torch.bfloat16: "<u2", torch.uint8: "|u1", torch.float32: "<f4"}
_ipc_mappings = []  # device pointers opened or allocated here; they live until the process exits


class _DevicePointer:
    """A raw device pointer dressed up for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _cuda_check(err, what):
    from cuda.bindings import runtime as cudart
    if err != cudart.cudaError_t.cudaSuccess:
        raise RuntimeError(f"{what}: {cudart.cudaGetErrorString(err)[1].decode()}")


def buffer_on_root(shape, dtype: torch.dtype, root: int = 0, group=None) -> torch.Tensor:
    """Allocates one buffer of `shape` on `root`'s GPU and returns, on every rank of the box, a tensor
    that addresses it from that rank's own GPU.

    On the other ranks the memory is mapped with CUDA IPC *with their own device current*, which is
    what makes it addressable by kernels running there (a mapping opened under the owner's device
    index is not: kernels of another device fault on it), and peer access is enabled by the same call.
    A decode whose output is such a tensor stores its KV straight into the consuming GPU's memory with
    ordinary stores over NVLink, so the delivery overlaps the decode instead of following it.  Ranks
    must synchronise (barrier) before the consumer reads.  The buffer lives until the processes exit."""
    from cuda.bindings import runtime as cudart
    rank = dist.get_rank(group)
    here = torch.cuda.current_device()
    nbytes = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
    payload = [None]
    if rank == root:
        err, ptr = cudart.cudaMalloc(nbytes)
        _cuda_check(err, "cudaMalloc")
        err, handle = cudart.cudaIpcGetMemHandle(ptr)
        _cuda_check(err, "cudaIpcGetMemHandle")
        payload[0] = bytes(handle.reserved)
    dist.broadcast_object_list(payload, src=root, group=group)
    if rank != root:
        handle = cudart.cudaIpcMemHandle_t()
        handle.reserved = payload[0]
        err, ptr = cudart.cudaIpcOpenMemHandle(handle, cudart.cudaIpcMemLazyEnablePeerAccess)
        _cuda_check(err, "cudaIpcOpenMemHandle")
    _ipc_mappings.append(int(ptr))
    flat = torch.as_tensor(_DevicePointer(int(ptr), nbytes), device=torch.device("cuda", here))
    return flat.view(dtype).view(shape)


def copy_token_range_async(dst: torch.Tensor, src: torch.Tensor, stream: torch.cuda.Stream) -> None:
    """Copies a token range of a KV slab, `src` = slab[:, :, t0:t1] of a contiguous [L, 2, T, H, D] tensor,
    to the same range of another such tensor (`dst`, possibly memory of another GPU obtained from
    buffer_on_root) with one two-dimensional asynchronous copy on `stream`: 2L rows of (t1 - t0)*H*D
    elements, T*H*D elements apart.  The copy engines move it, no kernel runs."""
    if src.shape != dst.shape or src.dtype != dst.dtype or src.dim() != 5 or src.shape[1] != 2:
        raise RuntimeError("expected two [L, 2, t, H, D] views of the same shape and type")
    L, _, t, H, D = src.shape
    for x in (src, dst):
        if x.stride(4) != 1 or x.stride(3) != D or x.stride(2) != H * D or x.stride(0) != 2 * x.stride(1):
            raise RuntimeError("views must be token ranges of contiguous [L, 2, T, H, D] tensors")
    from cuda.bindings import runtime as cudart
    esz = src.element_size()
    err, = cudart.cudaMemcpy2DAsync(dst.data_ptr(), dst.stride(1) * esz, src.data_ptr(), src.stride(1) * esz,
                                    t * H * D * esz, 2 * L, cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice,
                                    stream.cuda_stream)
    _cuda_check(err, "cudaMemcpy2DAsync")


class PipelinedDelivery:
    """Decode a rank's chunks of one KV cache and deliver the result into a blob on another GPU of the
    box, overlapped: the chunks are decoded in `parts` parts into the rank's own slab `local`
    ([L_rank, 2, T, H, D]); as soon as a part is decoded its token range is copied into `target` (the
    rank's layers of the consumer's blob, from buffer_on_root) on a second stream while the next part
    is decoded.  When `target` is this GPU's own memory the parts decode straight into it.

    `deserializer`: a CacheGenDeserializer in "vllm" layout; `chunks`: its encoded chunks, in token
    order.  `run()` enqueues everything; the caller's current stream waits for the copies at the end."""

    def __init__(self, deserializer, chunks: list, local: torch.Tensor, target: torch.Tensor, parts: int = 8,
                 target_is_local: bool = False):
        self.dev = local.device
        self.local, self.target, self.direct = local, target, target_is_local
        self.copy_stream = torch.cuda.Stream(device=self.dev)
        self.workspace = {}
        nparts = max(1, min(parts, len(chunks)))
        per = (len(chunks) + nparts - 1) // nparts
        self.parts, t0 = [], 0
        for i in range(0, len(chunks), per):
            group = chunks[i:i + per]
            tn = sum(c.num_tokens if hasattr(c, "num_tokens") else c.max_tensors_key.shape[1] for c in group)
            dst = (target if target_is_local else local)[:, :, t0:t0 + tn]
            self.parts.append((deserializer.plan(group, out=dst, workspace=self.workspace), t0, tn))
            t0 += tn

    def run(self) -> None:
        cur = torch.cuda.current_stream(self.dev)
        for plan, a, n in self.parts:
            plan.run()
            if not self.direct:
                done = torch.cuda.Event()
                done.record(cur)
                self.copy_stream.wait_event(done)
                copy_token_range_async(self.target[:, :, a:a + n], self.local[:, :, a:a + n], self.copy_stream)
        cur.wait_stream(self.copy_stream)

    def status(self) -> int:
        """The parts' status word (synchronises); 0 = nothing reported."""
        return int(self.workspace["status"].item()) if "status" in self.workspace else 0
