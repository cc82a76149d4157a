"""Benchmark of the codec's decode path: decoded KV GB/s and context tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one full decode of the workload's encoded KV cache (every chunk of the context) into the
16-bit KV blob.  Default workload: Llama-7B shape (32 layers x 32 heads x 128, fp16), 8,192 tokens,
seed 1, 7B-default bins, one serializer call per 256 tokens -- synthetic AR(1) KV (cachegen_b200.synth)
standing in for real model KV.

  value        whole-job decoded-KV throughput with the encoded chunks resident in HBM (CUDA events)
  e2e          the same through CacheGenDeserializer.decode_many_host with the encoded chunks (CGB2
               containers) in pinned host memory: host->device copies of every step's inputs and a
               device->host read of the status word inside the timed region; e2e_reference_blob_tensors is
               the same call on the tensors of the reference's own blob layout
  roofline     the dominant kernel (fused decode + dequantise + KV store) timed alone, algorithmic bytes
               over its duration against the measured HBM copy bandwidth
  cpu_baseline the CPU oracle's decode + dequantise on a bounded sample of the same chunks, all host cores

With N > 1 (under torchrun) every rank decodes its own request of the same shape (weak scaling, no
data-path collective); the time is the max over ranks and the value the sum of all ranks' bytes.
`--impl reference` times the CPU restatement of the reference's decode path on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CHUNK_TOKENS = 256
HBM_FALLBACK_GBS = 6650.0
# DRAM bytes (read + write) of one decode_dequant_kernel launch per decoded token, Llama-7B shape,
# 256-token chunks: 1260 MB measured by ncu on a 2,048-token launch
# (profiles/launch_list_llama7b_2k_tokens.md); traffic grows in proportion to the tokens of a launch.
NCU_TRAFFIC_BYTES_PER_TOKEN = {(32, 32, 128): 1259.6e6 / 2048}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b-8k")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's token count")
    ap.add_argument("--shard", default="requests", choices=["requests", "layers"],
                    help="N > 1: one request per GPU (weak scaling, default) or the layers of ONE request "
                         "split across the GPUs and the decoded KV gathered to GPU 0 over NCCL (strong scaling)")
    ap.add_argument("--deliver", default="copy", choices=["copy", "nccl", "peer"],
                    help="--shard layers: decode in --parts parts and copy each to GPU 0's blob while the next is "
                         "decoded (default), gather the decoded slabs with NCCL after the decode, or let every "
                         "decode kernel store straight into GPU 0's blob over NVLink (CUDA IPC mapping)")
    ap.add_argument("--parts", type=int, default=8, help="--deliver copy: parts a rank's chunks are decoded in")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the baseline sample")
    return ap.parse_args()


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


# ------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, reasons, smax = [], set(), None
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------------- workload
def workload_spec(args):
    from cachegen_b200.synth import WORKLOADS
    spec = dict(WORKLOADS[args.workload])
    if args.tokens:
        spec["num_tokens"] = args.tokens
    return spec


def describe(spec, args):
    return {"workload": args.workload, "layers": spec["num_layers"], "kv_heads": spec["num_heads"],
            "head_size": spec["head_size"], "tokens": spec["num_tokens"], "seed": spec["seed"],
            "chunk_tokens": CHUNK_TOKENS, "bins": spec["model_name"], "kv_dtype": "fp16", "fmt": "vllm",
            "cache": "per-step inputs + outputs exceed the 126 MB L2"}


# ------------------------------------------------------------------------------------------- CPU legs
def cpu_sample_chunks(spec, nchunks, seed_offset=0):
    """Encodes `nchunks` chunks of the workload with the CPU oracle (no GPU, no product code)."""
    import numpy as np
    import torch

    from cachegen_b200.serde.cachegen_basics import CacheGenConfig, make_key_bins, make_value_bins
    from cachegen_b200.synth import generate_kv
    from oracle import cg_oracle as oracle
    L, H, D = spec["num_layers"], spec["num_heads"], spec["head_size"]
    T = nchunks * CHUNK_TOKENS
    kv = generate_kv(L, H, D, T, spec["seed"] + seed_offset, key_rho=spec["key_rho"], device="cpu", dtype=torch.float16)
    cfg = CacheGenConfig.from_model_name(spec["model_name"])
    bins = torch.cat((make_key_bins(cfg, "cpu"), make_value_bins(cfg, "cpu"))).numpy()
    rows = kv.reshape(L, 2, T, H * D).transpose(0, 1).reshape(2 * L, T, H * D)
    chunks = []
    for i in range(nchunks):
        x = rows[:, i * CHUNK_TOKENS:(i + 1) * CHUNK_TOKENS].contiguous().view(torch.int16).numpy().view(np.uint16)
        sym, mx = oracle.quantize(x, bins)
        cdf = oracle.calculate_cdf(sym, int(bins.max()))
        stream_bytes, lengths = oracle.encode_chunk(cdf, sym)
        chunks.append((cdf, stream_bytes, lengths, mx))
    return chunks, bins


def cpu_decode_pass(spec, chunks, bins, threads):
    """Decode + dequantise of the sample chunks into a [L,2,T,H,D] fp16 blob; returns seconds."""
    import numpy as np

    from oracle import cg_oracle as oracle
    L, H, D = spec["num_layers"], spec["num_heads"], spec["head_size"]
    C = H * D
    T = len(chunks) * CHUNK_TOKENS
    out = np.empty((L, 2, T, C), dtype=np.uint16)
    rows_view = out.reshape(-1)
    t0 = time.perf_counter()
    for i, (cdf, stream_bytes, lengths, mx) in enumerate(chunks):
        # row r = (kv, layer): element offset of (row, token, channel) in the vllm blob
        # layer*2*T*C + kv*T*C + token*C + channel; the oracle takes one stride per row, so K and V halves
        # are decoded by two calls
        for kvi in range(2):
            sl = slice(kvi * L, (kvi + 1) * L)
            base = rows_view[(kvi * T + i * CHUNK_TOKENS) * C:]
            oracle.decode_dequant_chunk(cdf[sl], stream_bytes_slice(stream_bytes, lengths, sl), lengths[sl],
                                        CHUNK_TOKENS, bins[sl], mx[sl], base, [2 * T * C, C, 1], threads=threads)
    return time.perf_counter() - t0, out


def stream_bytes_slice(stream_bytes, lengths, sl):
    import numpy as np
    flat = lengths.reshape(lengths.shape[0], -1).sum(axis=1)
    offs = np.concatenate(([0], np.cumsum(flat)))
    return stream_bytes[offs[sl.start]:offs[sl.stop]]


def run_cpu_baseline(spec, seconds_budget):
    from oracle import cg_oracle as oracle
    threads = oracle.host_threads()
    chunks, bins = cpu_sample_chunks(spec, 1)
    dt, _ = cpu_decode_pass(spec, chunks, bins, threads)  # also warms the library
    dt, _ = cpu_decode_pass(spec, chunks, bins, threads)
    reps = max(1, min(64, int(seconds_budget / max(dt, 1e-3))))
    t = 0.0
    for _ in range(reps):
        d, _ = cpu_decode_pass(spec, chunks, bins, threads)
        t += d
    kv_bytes = 2 * spec["num_layers"] * spec["num_heads"] * spec["head_size"] * CHUNK_TOKENS * 2
    return {"value": kv_bytes * reps / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "tokens_per_s": CHUNK_TOKENS * reps / t,
            "sample": f"{reps} passes over one {CHUNK_TOKENS}-token chunk of the workload "
                      f"({kv_bytes / 2**20:.0f} MiB of KV each), {t:.1f} s of wall time on {threads} threads"}


def run_reference_arm(args, spec):
    """The reference's decode path restated on the CPU (the reference itself has no CPU coder: its
    torchac_cuda kernels are GPU-only and the `torchac` package it imports is never called), all host
    threads, each step a bounded sample: two 256-token chunks of the workload."""
    from oracle import cg_oracle as oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = oracle.host_threads()
    nchunks = 2
    chunks, bins = cpu_sample_chunks(spec, nchunks)
    for _ in range(max(1, args.warmup)):
        cpu_decode_pass(spec, chunks[:1], bins, threads)
    times = []
    for _ in range(args.steps):
        dt, _ = cpu_decode_pass(spec, chunks, bins, threads)
        times.append(dt)
    total = sum(times)
    kv_bytes = 2 * spec["num_layers"] * spec["num_heads"] * spec["head_size"] * CHUNK_TOKENS * nchunks * 2
    value = kv_bytes * args.steps / total / 1e9
    sample = f"{nchunks} chunks of {CHUNK_TOKENS} tokens per step ({kv_bytes / 2**20:.0f} MiB of KV), {threads} threads"
    line = {"impl": "reference", "metric": "decoded_kv_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": describe(spec, args), "tokens_per_s": CHUNK_TOKENS * nchunks * args.steps / total,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- GPU arm
def run_ours(args, spec):
    import torch
    import torch.distributed as dist

    from cachegen_b200 import _lib
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    from cachegen_b200.serde.cachegen_basics import CacheGenGPUBytestream, CacheGenGPUEncoderOutput
    from cachegen_b200.parallel import PipelinedDelivery, buffer_on_root, gather_layers, max_over_ranks, partition
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import generate_kv

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU fallback); use --impl reference for the CPU arm")
    _lib.lib()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    L_total, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    C = H * D
    config = LMCacheEngineConfig.from_defaults(chunk_size=CHUNK_TOKENS)
    meta = LMCacheEngineMetadata(model_name=spec["model_name"], world_size=world, worker_id=rank, fmt="vllm")
    by_layers = args.shard == "layers" and world > 1
    full_cfg = CacheGenConfig.from_model_name(spec["model_name"])
    if by_layers:
        mine = partition(L_total, world, rank)
        if len(mine) == 0:
            raise SystemExit("more GPUs than layers")
        cfg, L, first_layer, seed = full_cfg.layer_slice(mine.start, mine.stop), len(mine), mine.start, spec["seed"]
    else:
        cfg, L, first_layer, seed = full_cfg, L_total, 0, spec["seed"] + 1000 * rank
    ser = CacheGenSerializer(config, meta, cachegen_config=cfg, table_max_bins=full_cfg.max_bins)
    de = CacheGenDeserializer(config, meta, cachegen_config=cfg, out_dtype=torch.float16)

    # ---- set-up (untimed): this rank's share, encoded chunk by chunk as LMCacheEngine.store would
    kv = generate_kv(L, H, D, T, seed, key_rho=spec["key_rho"], device=dev, dtype=torch.float16, first_layer=first_layer)
    ms_encode = None
    for attempt in range(2):  # the first pass warms the allocator, the second is timed
        chunks = None
        torch.cuda.synchronize()
        enc0, enc1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        enc0.record()
        chunks = ser.encode_many(kv, CHUNK_TOKENS, batch=16)
        enc1.record()
        torch.cuda.synchronize()
        ms_encode = enc0.elapsed_time(enc1)
    out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=dev)
    plan = de.plan(chunks, out=out)
    kv_bytes = 2 * L * C * T * 2
    payload = plan.payload_bytes
    per_token = {"payload": payload / T, "tables": plan.table_bytes / T, "lengths": plan.length_bytes / T,
                 "scales": plan.scale_bytes / T}
    per_token["total"] = sum(per_token.values())
    algorithmic = plan.output_bytes + payload + plan.table_bytes + plan.length_bytes + plan.scale_bytes

    # correctness gate before timing: decoded values within the quantiser's error bound
    plan.run()
    de.check_status()
    step = torch.cat((chunks[0].max_tensors_key, chunks[0].max_tensors_value)).float().reshape(2 * L, -1, 1)
    cq = torch.cat((ser.key_bins, ser.value_bins)).div(2, rounding_mode="floor") - 1
    got = out[:, :, :CHUNK_TOKENS].reshape(L, 2, -1, C).transpose(0, 1).reshape(2 * L, -1, C).float()
    ref = kv[:, :, :CHUNK_TOKENS].reshape(L, 2, -1, C).transpose(0, 1).reshape(2 * L, -1, C).float()
    bound = 0.5 * step / cq[:, None, None] * 1.001 + step * 2.0 ** -10 + 1e-6
    assert bool(((got - ref).abs() <= bound).all()), "decoded KV violates the quantiser's error bound"
    del got, ref

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1), device=dev) / steps

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # ---- the headline: full decode, inputs resident in HBM
    full_out = None
    delivery = "none"
    if by_layers:
        if args.deliver == "peer":
            # every rank's kernel writes its layers straight into GPU 0's blob
            shared = buffer_on_root((L_total, 2, T, H, D), torch.float16, root=0)
            full_out = shared if rank == 0 else None
            peer_plan = de.plan(chunks, out=shared[mine.start:mine.stop], peer_out=True)
            delivery = "decode kernels store into GPU 0's blob over NVLink (peer mapping), no separate transfer"

            def step():
                peer_plan.run()
            # check once against the NCCL path
            step()
            barrier()
            check = gather_layers(out, L_total, root=0)
            if rank == 0:
                assert torch.equal(check, full_out), "peer-stored KV differs from the gathered KV"
            del check
        elif args.deliver == "copy":
            # decode in parts of a few chunks; each part's token range goes to GPU 0's blob by an asynchronous
            # copy on a second stream while the next part is decoded
            shared = buffer_on_root((L_total, 2, T, H, D), torch.float16, root=0)
            full_out = shared if rank == 0 else None
            target = shared[mine.start:mine.stop]
            pipe = PipelinedDelivery(de, chunks, out, target, parts=args.parts, target_is_local=(rank == 0))
            delivery = (f"decode in {len(pipe.parts)} parts; each part's token range is copied to GPU 0's blob over NVLink "
                        "(cudaMemcpy2DAsync on a second stream) while the next part is decoded")
            step = pipe.run
            step()
            barrier()
            assert pipe.status() == 0, "a part's decode reported a problem"
            check = gather_layers(out if rank != 0 else target.contiguous(), L_total, root=0)
            if rank == 0:
                assert torch.equal(check, full_out), "copied KV differs from the gathered KV"
            del check
        else:
            if rank == 0:
                full_out = torch.empty((L_total, 2, T, H, D), dtype=torch.float16, device=dev)
            delivery = "NCCL send/recv of each rank's layer slab to GPU 0, inside the step"

            def step():
                plan.run()
                gather_layers(out, L_total, root=0, out=full_out)
    else:
        step = plan.run
    ms_step = timed(step, args.steps, max(3, args.warmup))
    # ---- the dominant kernel alone (offsets already in place)
    ms_kernel = timed(plan.run_decode, args.steps, 1)
    ms_offsets = timed(plan.run_offsets, args.steps, 1)
    clocks = sampler.stop() if rank == 0 else None
    de.check_status()

    # ---- end to end: encoded chunks in pinned host memory, copied in every step
    e2e = None
    extra = {}
    if not args.no_e2e and not by_layers:
        def pin(t):
            return t.detach().cpu().pin_memory()
        status_host = torch.zeros(1, dtype=torch.int32).pin_memory()

        def measure_host(host_chunks, nbytes, what):
            def e2e_step():
                de.decode_many_host(host_chunks, out=out, groups=16)
                status_host.copy_(de.group_status_words()[-1], non_blocking=True)
            ms = timed(e2e_step, max(2, args.steps // 2), 2)
            torch.cuda.synchronize()
            assert int(status_host.item()) == 0
            de.check_status()
            return {"value": world * kv_bytes / ms / 1e6, "unit": "GB/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": 4, "ms_per_step": ms, "tokens_per_s": world * T / ms * 1e3, "api": what}

        # (1) the library's own container (CGB2: one buffer per chunk, tables as byte counts)
        flat_gpu = [ser.encode_flat(kv[:, :, s:s + CHUNK_TOKENS]) for s in range(0, T, CHUNK_TOKENS)]
        flat_plan = de.plan(flat_gpu, out=out)
        ms_flat = timed(flat_plan.run, args.steps, 2)
        extra["value_flat_container"] = {"value": world * kv_bytes / ms_flat / 1e6, "unit": "GB/s", "ms_per_step": ms_flat,
                                         "what": "as `value`, chunks held as CGB2 containers in HBM"}
        extra["bytes_per_token_flat_container"] = {
            "payload": flat_plan.payload_bytes / T, "tables": flat_plan.table_bytes / T,
            "lengths": flat_plan.length_bytes / T, "scales": flat_plan.scale_bytes / T,
            "container": sum(c.header.total for c in flat_gpu) / T}
        flat_host = [c.pin_memory() for c in flat_gpu]
        kv_chunk0 = kv[:, :, :CHUNK_TOKENS].clone()
        del flat_plan, flat_gpu, kv
        e2e = measure_host(flat_host, sum(c.header.total for c in flat_host),
                           "CacheGenDeserializer.decode_many_host on CGB2 containers (CacheGenSerializer.encode_flat) "
                           "held in pinned host memory; 16 groups, copies of one group overlap the decode of the previous")
        del flat_host
        # (2) the reference's blob layout (tensors of CacheGenGPUEncoderOutput), same call
        host_chunks = [CacheGenGPUEncoderOutput(
            [CacheGenGPUBytestream(pin(dc.bytestream), pin(dc.bytestream_lengths), dc.ntokens) for dc in eo.data_chunks],
            pin(eo.cdf), pin(eo.max_tensors_key), pin(eo.max_tensors_value), eo.num_heads, eo.head_size) for eo in chunks]
        h2d = sum(t.numel() * t.element_size() for eo in host_chunks
                  for t in [eo.cdf, eo.max_tensors_key, eo.max_tensors_value] +
                  [x for dc in eo.data_chunks for x in (dc.bytestream, dc.bytestream_lengths)])
        extra["e2e_reference_blob_tensors"] = measure_host(
            host_chunks, h2d, "the same call on the tensors of the reference's blob (int16 tables, int32 lengths) in pinned host memory")
        del host_chunks
        # (3) the reference's wire format itself: pickled blobs through from_bytes, a few chunks
        nb = min(8, len(chunks))
        blobs = [eo.to_bytes() for eo in chunks[:nb]]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for blob in blobs:
            de.from_bytes(blob)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        extra["from_bytes_pickle"] = {"ms_per_chunk": 1e3 * dt / nb, "blob_bytes_per_chunk": sum(map(len, blobs)) / nb,
                                      "value": nb * kv_bytes / len(chunks) / dt / 1e9, "unit": "GB/s",
                                      "what": "CacheGenDeserializer.from_bytes on the reference-format pickle, chunk by "
                                              "chunk, wall clock: the load of the blob (30 MB per chunk through pinned staging) dominates"}
        de.from_bytes_many(blobs)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        de.from_bytes_many(blobs)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        extra["from_bytes_many_pickle"] = {"ms_per_chunk": 1e3 * dt / nb, "value": nb * kv_bytes / len(chunks) / dt / 1e9,
                                           "unit": "GB/s", "what": f"CacheGenDeserializer.from_bytes_many on {nb} such blobs"}
        del blobs
        ser.to_bytes(kv_chunk0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(3):
            blob_len = len(ser.to_bytes(kv_chunk0))
        dt = (time.perf_counter() - t0) / 3
        extra["to_bytes_pickle"] = {"ms_per_chunk": 1e3 * dt, "blob_bytes_per_chunk": blob_len,
                                    "value": kv_chunk0.numel() * 2 / dt / 1e9, "unit": "GB/s",
                                    "what": "CacheGenSerializer.to_bytes of one chunk (KV on the GPU) to the "
                                            "reference-format pickle, wall clock"}
        # (4) the two decoder layouts on one chunk's first sub-chunk: symbols only, same inputs and output
        from cachegen_b200 import torchac_cuda as tcu
        eo, dc = chunks[0], chunks[0].data_chunks[0]
        if eo.cdf.shape[2] <= 33:
            pref = dc.bytestream_lengths.to(torch.int64).reshape(-1).cumsum(0).reshape(dc.bytestream_lengths.shape)
            sym = torch.empty((eo.cdf.shape[0], dc.ntokens, eo.cdf.shape[1]), dtype=torch.uint8, device=dev)
            extra["decoder_layouts"] = {
                "thread_per_stream_ms": timed(lambda: tcu.decode_fast_prefsum(eo.cdf, dc.bytestream, pref, sym), 10, 3),
                "warp_per_stream_ms": timed(lambda: tcu.decode_fast_prefsum_warp(eo.cdf, dc.bytestream, pref, sym), 10, 3),
                "what": f"decode_fast_prefsum of one {dc.ntokens}-token sub-chunk ({pref.numel()} streams) on the "
                        "thread-per-stream kernel and on the warp-per-stream (ballot search) kernel"}
            tcu.check_status(dev)

        # (5) one chunk at the three quality levels of the reference's adaptation runs: together and one by one
        from cachegen_b200.serde.cachegen_basics import CacheGenConfig
        if L == 32:
            lv = [CacheGenConfig(10, 20, 32, 16, 16, 12, 2, 16, 12), CacheGenConfig(10, 20, 32, 32, 16, 16, 2, 32, 16),
                  CacheGenConfig(10, 20, 32, 32, 32, 32, 2, 32, 32)]
            sers = [CacheGenSerializer(config, meta, cachegen_config=c) for c in lv]
            one = kv_chunk0
            extra["encode_levels"] = {
                "together_ms": timed(lambda: ser.encode_levels(one, lv), 5, 2),
                "one_by_one_ms": timed(lambda: [s_.encode(one) for s_ in sers], 5, 2),
                "what": f"one {one.shape[2]}-token chunk at QUANT_LEVEL 1, 2 and 3: CacheGenSerializer.encode_levels "
                        "against three CacheGenSerializer.encode calls"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_hbm_peak()
    achieved = algorithmic / ms_kernel / 1e6
    total_kv_bytes = 2 * L_total * C * T * 2 if by_layers else world * kv_bytes
    line = {
        "metric": "decoded_kv_gbps", "value": total_kv_bytes / ms_step / 1e6, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if by_layers else "weak", "vs_baseline": None, "dtype": "u32",
        "data": "synthetic", "config": dict(describe(spec, args), shard=args.shard if world > 1 else "none",
                                             delivery=delivery),
        "tokens_per_s": (T if by_layers else world * T) / ms_step * 1e3,
        "bytes_per_token": per_token,
        "kv_bytes_per_token": kv_bytes / T,
        "gpu_launches": plan.launches * args.steps,
        "launches_per_step": plan.launches,
        "kernel_ms": {"decode_dequant": ms_kernel, "offsets": ms_offsets},
        "encode": {"value": kv_bytes / ms_encode / 1e6, "unit": "GB/s", "ms": ms_encode,
                   "what": "CacheGenSerializer.encode_many: every chunk of the cache, one host sync per 16 chunks, "
                           "KV resident in HBM, second pass of set-up"},
        "roofline": {"bound": "hbm", "kernel": "decode_dequant_kernel", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (NCU_TRAFFIC_BYTES_PER_TOKEN[(L, H, D)] * T
                                 if (L, H, D) in NCU_TRAFFIC_BYTES_PER_TOKEN else None),
                     "traffic_source": "ncu capture of a 2,048-token launch scaled by tokens",
                     "algorithmic_bytes_per_launch": algorithmic},
        "clocks": clocks,
    }
    if e2e:
        line["e2e"] = e2e
    line.update(extra)
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = run_cpu_baseline(spec, args.cpu_seconds)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    spec = workload_spec(args)
    if args.impl == "reference":
        run_reference_arm(args, spec)
    else:
        run_ours(args, spec)


if __name__ == "__main__":
    main()
