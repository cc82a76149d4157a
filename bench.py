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
               (and the same on one thread)
  reference_cuda_ext  the reference's own CUDA extension (oracle/_ref, built unmodified) and the torch chain
               around it, on one 256-token chunk of the workload on this GPU, beside this package's kernels
  config3 / config5   the long-context GQA decode and a shortened three-quality-level encode + decode sweep
  whole_context_call  the workload through one serializer call over all its tokens

With N > 1 (under torchrun) every rank decodes its own request of the same shape (weak scaling, no
data-path collective); the time is the max over ranks and the value the sum of all ranks' bytes.  The
same run then measures, in the same process group, `h2d_only_ms` (the end-to-end leg's host-to-device
copies alone) and `delivered_kv`: the Llama-70B-shape cache sharded by layers, every rank decoding its
layers and the decoded KV delivered to GPU 0 over NVLink (pipelined copies, and NCCL after the decode),
and `token_sharded`: one long-context request of the Mistral-7B GQA shape sharded by token chunks.
`--impl reference` times the CPU restatement of the reference's decode path on the host cores.
"""
import argparse
import glob
import importlib.util
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
# Counters of the dominant kernel (decode_dequant_multi_kernel<2, fp16>) from ncu captures of this
# kernel on the Llama-7B shape with 256-token chunks; they belong to the kernel as committed with this
# file and have to be re-captured when the kernel changes.  DRAM bytes (read + write) come from a
# 2,048-token launch and grow in proportion to the tokens of a launch; the issue figures come from a
# 512-token launch (`--set full`, and sass__inst_executed_per_opcode).
NCU_CAPTURE = {
    (32, 32, 128): {"traffic_bytes_per_token": 1255.9e6 / 2048, "issue_active_pct": 64.8, "alu_pipe_pct": 59.8,
                    "warp_instr_per_32_symbols": 56.2,
                    "source": "ncu on bench.py --tokens 2048 (dram__bytes_read.sum + dram__bytes_write.sum) and "
                              "--tokens 512 (--set full; sass__inst_executed_per_opcode), B200, kernel "
                              "decode_dequant_multi_kernel<2,0>"},
}


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
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the legs beside the headline: reference CUDA extension, configs 3 and 5 (N = 1), "
                         "delivery of decoded KV to GPU 0 (N > 1)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the baseline sample")
    return ap.parse_args()


def ncu_counters(L, H, D, tokens):
    """The committed ncu figures of the dominant kernel for this shape (None when there is no capture)."""
    cap = NCU_CAPTURE.get((L, H, D))
    if cap is None:
        return {}
    return {"traffic": cap["traffic_bytes_per_token"] * tokens, "issue_active_pct": cap["issue_active_pct"],
            "alu_pipe_pct": cap["alu_pipe_pct"], "warp_instr_per_32_symbols": cap["warp_instr_per_32_symbols"],
            "traffic_source": cap["source"]}


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
    one, _ = cpu_decode_pass(spec, chunks, bins, 1)  # the same chunk on a single thread
    return {"value": kv_bytes * reps / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "one_thread": {"value": kv_bytes / one / 1e9, "unit": "GB/s", "cores": 1, "sample": "one pass over the same chunk"},
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
            "config": dict(describe(spec, args), shard=args.shard if args.gpus > 1 else "none", delivery="none"),
            "tokens_per_s": CHUNK_TOKENS * nchunks * args.steps / total,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- GPU arm
class Harness:
    """Timing plumbing shared by the legs: barrier + synchronise on both sides of K steps, CUDA events on
    the current stream, max over ranks."""

    def __init__(self, dev, rank, world):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.dev, self.rank, self.world = torch, dist, dev, rank, world

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps, warmup, local=False):
        """ms per step.  local=True: this rank alone (no barrier, no reduction): legs only rank 0 runs."""
        from cachegen_b200.parallel import max_over_ranks
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize() if local else self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize() if local else self.barrier()
        ms = e0.elapsed_time(e1) / steps
        return ms if local else max_over_ranks(ms, device=self.dev)


def make_serde(spec, world, rank, cachegen_config=None, table_max_bins=None, chunk_size=None):
    import torch

    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    config = LMCacheEngineConfig.from_defaults(chunk_size=chunk_size or CHUNK_TOKENS)
    meta = LMCacheEngineMetadata(model_name=spec["model_name"], world_size=world, worker_id=rank, fmt="vllm")
    kw = {} if cachegen_config is None else {"cachegen_config": cachegen_config}
    ser = CacheGenSerializer(config, meta, table_max_bins=table_max_bins, **kw)
    de = CacheGenDeserializer(config, meta, out_dtype=torch.float16, **kw)
    return ser, de, config, meta


def load_reference_extension():
    """The reference's torchac_cuda, compiled unmodified into oracle/_ref by oracle/build_ref.py."""
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "torchac_cuda*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("torchac_cuda", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def leg_reference_cuda_ext(h, ser, de, kv_chunk, eo):
    """One 256-token chunk of the workload through the reference's own kernels and the torch chain the
    reference wraps around them (cachegen_decoder.py:24-34,78-112,159-173 and cachegen_encoder.py:42-59,
    210-292 of the reference, re-typed here as the baseline), beside this package's kernels and fused
    calls on the same inputs, same GPU, same clocks.  Inputs are valid by construction (this package's
    encoder made them and the reference's decoder reads them back identically in the tests); the
    reference encoder is only called when every stream fits its 256-byte shared-memory row."""
    torch = h.torch
    ref = load_reference_extension()
    if ref is None:
        return {"unavailable": "oracle/_ref/torchac_cuda*.so is not built (python oracle/build_ref.py)"}
    import cachegen_b200.torchac_cuda as mine
    from cachegen_b200.serde.cachegen_encoder import quantize_and_tables

    L, _, T, H, D = kv_chunk.shape
    C, NL = H * D, 2 * L
    dc = eo.data_chunks[0]
    cdf, lengths, payload = eo.cdf, dc.bytestream_lengths, dc.bytestream
    key_bins, value_bins = de.key_bins.to(h.dev), de.value_bins.to(h.dev)
    max_bins = cdf.shape[2] - 1
    reps, warm = 10, 3
    out = {"what": f"one {T}-token chunk ({NL * C} streams): the reference's torchac_cuda kernels, recompiled for "
                   "sm_100, and the torch chain of its serializer classes against this package on the same inputs"}

    # ---- decode: kernel against kernel
    pref = lengths.flatten().cumsum(0).reshape(lengths.shape)
    buf_r = torch.zeros((T, NL * C), dtype=torch.uint8, device=h.dev).reshape(NL, T, C)
    buf_m = torch.zeros_like(buf_r)
    k_ref = h.timed(lambda: ref.decode_fast_prefsum(cdf, payload, pref, buf_r), reps, warm, local=True)
    k_our = h.timed(lambda: mine.decode_fast_prefsum(cdf, payload, pref, buf_m), reps, warm, local=True)
    mine.check_status(h.dev)
    same_symbols = bool(torch.equal(buf_r, buf_m))

    # ---- decode: the reference's from_bytes after unpickling against the fused call
    def dequantize(t, bins, maxes):
        c = (bins // 2 - 1)[:, None, None]
        return (t - c) / c * maxes

    def ref_decode_chain():
        ps = lengths.flatten().cumsum(0).reshape(lengths.shape)
        ref.decode_fast_prefsum(cdf, payload, ps, buf_r)
        key, value = buf_r.reshape(2, L, T, C).float()
        key = dequantize(key, key_bins, eo.max_tensors_key)
        value = dequantize(value, value_bins, eo.max_tensors_value)
        blob = torch.stack([key, value]).reshape(2, L, T, H, D)
        return blob.permute(1, 0, 2, 3, 4).to(torch.float16)  # the reference casts to bf16 here; fp16 to compare

    out1 = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
    plan1 = de.plan([eo], out=out1, workspace={})
    c_ref = h.timed(ref_decode_chain, reps, warm, local=True)
    c_our = h.timed(plan1.run, reps, warm, local=True)
    same_kv = bool(torch.equal(ref_decode_chain().contiguous(), out1))
    kv_bytes = NL * T * C * 2
    out["decode"] = {
        "kernel_ms": {"reference_decode_fast_prefsum": k_ref, "ours_decode_fast_prefsum": k_our, "speedup": k_ref / k_our},
        "chain_ms": {"reference_kernel_plus_torch_chain": c_ref, "ours_fused": c_our, "speedup": c_ref / c_our},
        "decoded_kv_gbps": {"reference": kv_bytes / c_ref / 1e6, "ours": kv_bytes / c_our / 1e6},
        "same_symbols": same_symbols, "same_kv_bits": same_kv}

    # ---- encode: kernels, then the chains
    sym, _, cdf_m = quantize_and_tables(kv_chunk, key_bins, value_bins, max_bins)
    fits = int(lengths.max()) <= 256
    t_cdf_ref = h.timed(lambda: (ref.calculate_cdf(sym[:L], max_bins), ref.calculate_cdf(sym[L:], max_bins)), reps, warm, local=True)
    t_cdf_our = h.timed(lambda: (mine.calculate_cdf(sym[:L], max_bins), mine.calculate_cdf(sym[L:], max_bins)), reps, warm, local=True)
    enc = {"calculate_cdf_ms": {"reference": t_cdf_ref, "ours": t_cdf_our, "speedup": t_cdf_ref / t_cdf_our}}
    sbuf_r = torch.zeros((NL, C, 256), dtype=torch.uint8, device=h.dev)
    slen_r = torch.zeros((NL, C), dtype=torch.int32, device=h.dev)
    sbuf_m, slen_m = torch.zeros_like(sbuf_r), torch.zeros_like(slen_r)

    def collect_bytes(output_buffer, output_lengths):
        size = output_buffer.shape[-1]
        fl, fb = output_lengths.flatten(), output_buffer.flatten()
        summed = (size - fl).cumsum(0).roll(1)
        summed[0] = 0
        idx = summed.repeat_interleave(fl)
        return fb[idx + torch.arange(len(idx), device=idx.device)]

    def quant(bins, x):
        mx = (bins // 2 - 1)[:, None, None]
        m1 = torch.amax(torch.abs(x), dim=-1, keepdim=True)
        return torch.round(x * (mx / m1) + mx).to(torch.int8), m1

    def ref_encode_chain():
        k, v = torch.unbind(kv_chunk.reshape(L, 2, T, C), dim=1)
        nk, mk = quant(key_bins, k)
        nv, mv = quant(value_bins, v)
        enc_in = torch.cat((nk, nv), dim=0).reshape(NL, T, C)
        tables = torch.cat([ref.calculate_cdf(nk, max_bins), ref.calculate_cdf(nv, max_bins)])
        ob = torch.zeros((NL, C, 256), dtype=torch.uint8, device=h.dev)
        ol = torch.zeros((NL, C), dtype=torch.int32, device=h.dev)
        ref.encode_fast_new(tables, enc_in, ob, ol)
        return collect_bytes(ob, ol), ol, tables

    if fits:
        t_enc_ref = h.timed(lambda: ref.encode_fast_new(cdf_m, sym, sbuf_r, slen_r), reps, warm, local=True)
        t_enc_our = h.timed(lambda: mine.encode_fast_new(cdf_m, sym, sbuf_m, slen_m), reps, warm, local=True)
        mine.check_status(h.dev)
        keep = torch.arange(256, device=h.dev)[None, None, :] < slen_r[:, :, None]
        enc["encode_fast_new_ms"] = {"reference": t_enc_ref, "ours": t_enc_our, "speedup": t_enc_ref / t_enc_our}
        enc["same_lengths"] = bool(torch.equal(slen_r, slen_m))
        enc["same_bytes"] = bool(torch.equal(sbuf_r[keep], sbuf_m[keep]))
        c_enc_ref = h.timed(ref_encode_chain, 5, 2, local=True)
        c_enc_our = h.timed(lambda: ser.encode(kv_chunk), 5, 2, local=True)
        got_bytes, got_len, got_cdf = ref_encode_chain()
        enc["chain_ms"] = {"reference_torch_quant_cdf_encode_collect": c_enc_ref, "ours_serializer_encode": c_enc_our,
                           "speedup": c_enc_ref / c_enc_our}
        enc["chain_same_payload"] = bool(torch.equal(got_bytes, payload) and torch.equal(got_len, lengths) and
                                         torch.equal(got_cdf, cdf))
        enc["kv_consumed_gbps"] = {"reference": kv_bytes / c_enc_ref / 1e6, "ours": kv_bytes / c_enc_our / 1e6}
    else:
        enc["skipped"] = "a stream of this chunk is longer than the reference encoder's 256-byte row"
    out["encode"] = enc
    return out


def leg_config3(h, args):
    """BASELINE config 3: the Mistral-7B GQA shape (32 layers x 8 KV heads x 128), 32,768 tokens, key
    rho 0.95, decode only from pre-encoded streams on this GPU."""
    torch = h.torch
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = dict(WORKLOADS["mistral7b-gqa-32k"])
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    ser, de, _, _ = make_serde(spec, 1, 0)
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device=h.dev, dtype=torch.float16)
    chunks = ser.encode_many(kv, CHUNK_TOKENS, batch=16)
    del kv
    out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
    plan = de.plan(chunks, out=out, workspace={})
    ms = h.timed(plan.run, max(3, args.steps // 2), 3, local=True)
    ms_kernel = h.timed(plan.run_decode, max(3, args.steps // 2), 1, local=True)
    de.check_status()
    kv_bytes = 2 * L * H * D * T * 2
    algorithmic = plan.output_bytes + plan.payload_bytes + plan.table_bytes + plan.length_bytes + plan.scale_bytes
    peak, kind = measured_hbm_peak()
    return {"workload": "mistral7b-gqa-32k", "tokens": T, "value": kv_bytes / ms / 1e6, "unit": "GB/s",
            "ms_per_step": ms, "tokens_per_s": T / ms * 1e3, "launches_per_step": plan.launches,
            "bytes_per_token": (plan.payload_bytes + plan.table_bytes + plan.length_bytes + plan.scale_bytes) / T,
            "roofline_frac": algorithmic / ms_kernel / 1e6 / peak, "peak_kind": kind}


def leg_whole_context(h, spec, args):
    """The workload through ONE serializer call over all its tokens, as the reference's evaluation scripts
    do (run_cachegen.py:53 there: chunk_size = the context length): one table per (row, channel) built over
    the whole context, one stream per 256-token sub-chunk.  Encode and decode of that one object."""
    torch = h.torch
    from cachegen_b200.synth import generate_kv
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    ser, de, _, _ = make_serde(spec, 1, 0, chunk_size=T)
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device=h.dev, dtype=torch.float16)
    box = {}

    def encode():
        box["enc"] = ser.encode(kv)
    encode()
    ms_enc = h.timed(encode, 2, 1, local=True)
    del kv
    out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
    plan = de.plan([box["enc"]], out=out, workspace={})
    ms = h.timed(plan.run, max(3, args.steps // 2), 3, local=True)
    de.check_status()
    kv_bytes = 2 * L * H * D * T * 2
    wire = plan.payload_bytes + plan.table_bytes + plan.length_bytes + plan.scale_bytes
    return {"tokens": T, "serializer_calls": 1, "sub_chunks": len(box["enc"].data_chunks),
            "value": kv_bytes / ms / 1e6, "unit": "GB/s", "ms_per_step": ms, "launches_per_step": plan.launches,
            "encode_gbps": kv_bytes / ms_enc / 1e6, "encode_ms": ms_enc,
            "bytes_per_token": wire / T,
            "bytes_per_token_parts": {"payload": plan.payload_bytes / T, "tables": plan.table_bytes / T,
                                      "lengths": plan.length_bytes / T, "scales": plan.scale_bytes / T}}


def leg_config5(h, args):
    """BASELINE config 5, shortened: requests of the Llama-7B shape, 4,096 tokens each (seeds 100..), split
    evenly over three quality levels (default bins, half, quarter with a minimum of 4); every request is
    encoded and decoded on this GPU.  Six requests instead of 64: the per-request work is identical."""
    torch = h.torch
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = dict(WORKLOADS["llama7b-4k"])
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    base = CacheGenConfig.from_model_name(spec["model_name"])
    levels = [("default", base), ("half", base.with_bins_divided(2)), ("quarter", base.with_bins_divided(4))]
    nreq = 6
    kv_bytes = 2 * L * H * D * T * 2
    out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
    per_level = {}
    enc_ms_total = dec_ms_total = 0.0
    for i in range(nreq):
        name, cfg = levels[i % 3]
        ser, de, _, _ = make_serde(spec, 1, 0, cachegen_config=cfg)
        kv = generate_kv(L, H, D, T, 100 + i, key_rho=spec["key_rho"], device=h.dev, dtype=torch.float16)
        ser.encode_many(kv, CHUNK_TOKENS, batch=16)  # warms the allocator for this level's sizes
        box = {}

        def encode():
            box["chunks"] = ser.encode_many(kv, CHUNK_TOKENS, batch=16)
        ms_enc = h.timed(encode, 1, 0, local=True)
        plan = de.plan(box["chunks"], out=out, workspace={})
        ms_dec = h.timed(plan.run, 2, 1, local=True)
        de.check_status()
        wire = plan.payload_bytes + plan.table_bytes + plan.length_bytes + plan.scale_bytes
        lv = per_level.setdefault(name, {"requests": 0, "encode_ms": 0.0, "decode_ms": 0.0, "wire_bytes": 0,
                                         "bins": [cfg.key_first_bins, cfg.key_second_bins, cfg.key_third_bins,
                                                  cfg.value_first_bins, cfg.value_second_bins]})
        lv["requests"] += 1
        lv["encode_ms"] += ms_enc
        lv["decode_ms"] += ms_dec
        lv["wire_bytes"] += wire
        enc_ms_total += ms_enc
        dec_ms_total += ms_dec
        del kv, plan, box
    for lv in per_level.values():
        n = lv["requests"]
        lv["encode_gbps"] = n * kv_bytes / lv.pop("encode_ms") / 1e6
        lv["decode_gbps"] = n * kv_bytes / lv.pop("decode_ms") / 1e6
        lv["bytes_per_token"] = lv.pop("wire_bytes") / (n * T)
    return {"workload": "llama7b-4k x %d requests, seeds 100..%d, levels default / half / quarter" % (nreq, 99 + nreq),
            "requests": nreq, "tokens_per_request": T,
            "encode_gbps": nreq * kv_bytes / enc_ms_total / 1e6, "decode_gbps": nreq * kv_bytes / dec_ms_total / 1e6,
            "encode_plus_decode_gbps": nreq * kv_bytes / (enc_ms_total + dec_ms_total) / 1e6,
            "levels": per_level,
            "what": "reference-layout chunks (int16 tables) held in HBM; bytes_per_token counts payload, tables, "
                    "lengths and scales"}


def leg_anchor_delta(h, spec, kv_part):
    """Anchor-token delta coding (no counterpart in the reference) on the first tokens of the workload:
    key rows in groups of 4 with half the bins on the residual tokens, against the plain codec."""
    torch = h.torch
    from cachegen_b200.serde import DeltaCoding
    L, _, T, H, D = kv_part.shape
    res = {"tokens": T, "settings": "groups of 4, residual bins = bins // 2, key rows only"}
    for name, delta in (("plain", None), ("delta", DeltaCoding(4, 2, "keys"))):
        import cachegen_b200.serde as S
        from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
        config = LMCacheEngineConfig.from_defaults(chunk_size=CHUNK_TOKENS)
        meta = LMCacheEngineMetadata(model_name=spec["model_name"], world_size=1, worker_id=0, fmt="vllm")
        ser = S.CacheGenSerializer(config, meta, delta=delta)
        de = S.CacheGenDeserializer(config, meta, out_dtype=torch.float16, delta=delta)
        box = {}

        def encode():
            box["chunks"] = ser.encode_many(kv_part, CHUNK_TOKENS, batch=16)
        encode()
        ms_enc = h.timed(encode, 3, 1, local=True)
        out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
        plan = de.plan(box["chunks"], out=out, workspace={})
        ms_dec = h.timed(plan.run, 5, 2, local=True)
        de.check_status()
        kv_bytes = kv_part.numel() * 2
        err = (out.float() - kv_part.float())
        res[name] = {"payload_bytes_per_token": plan.payload_bytes / T, "encode_gbps": kv_bytes / ms_enc / 1e6,
                     "decode_gbps": kv_bytes / ms_dec / 1e6,
                     "key_mse": float((err[:, 0] ** 2).mean()), "value_mse": float((err[:, 1] ** 2).mean())}
        del out, plan, box
    res["payload_ratio"] = res["delta"]["payload_bytes_per_token"] / res["plain"]["payload_bytes_per_token"]
    return res


def leg_delivered_kv(h, args):
    """BASELINE config 4 in the process group of the --gpus N run: the Llama-70B-shape cache (80 layers x 8
    KV heads x 128, 16,384 tokens) sharded by layers, every rank decodes its layers and the decoded KV is
    delivered into one blob on GPU 0 -- by pipelined peer copies while the decode runs, and by NCCL
    send/recv after it.  Plain peer copies and NCCL only."""
    torch = h.torch
    from cachegen_b200.parallel import PipelinedDelivery, buffer_on_root, gather_layers, partition
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = dict(WORKLOADS["llama70b-gqa-16k"])
    L_total, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    mine = partition(L_total, h.world, h.rank)
    full_cfg = CacheGenConfig.from_model_name(spec["model_name"])
    cfg = full_cfg.layer_slice(mine.start, mine.stop)
    ser, de, _, _ = make_serde(spec, h.world, h.rank, cachegen_config=cfg, table_max_bins=full_cfg.max_bins)
    L = len(mine)
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device=h.dev, dtype=torch.float16,
                     first_layer=mine.start)
    chunks = ser.encode_many(kv, CHUNK_TOKENS, batch=16)
    del kv
    local = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=h.dev)
    plan = de.plan(chunks, out=local, workspace={})
    steps, warm = max(3, args.steps // 2), 2
    total_bytes = 2 * L_total * H * D * T * 2
    res = {"workload": "llama70b-gqa-16k", "tokens": T, "layers_per_gpu": L, "kv_bytes": total_bytes}

    ms_decode = h.timed(plan.run, steps, warm)
    res["decode_only_ms"] = ms_decode
    # (1) NCCL after the decode
    full_nccl = torch.empty((L_total, 2, T, H, D), dtype=torch.float16, device=h.dev) if h.rank == 0 else None

    def step_nccl():
        plan.run()
        gather_layers(local, L_total, root=0, out=full_nccl)
    ms_nccl = h.timed(step_nccl, steps, warm)
    # (2) pipelined peer copies into GPU 0's blob
    shared = buffer_on_root((L_total, 2, T, H, D), torch.float16, root=0)
    pipe = PipelinedDelivery(de, chunks, local, shared[mine.start:mine.stop], parts=args.parts,
                             target_is_local=(h.rank == 0))
    ms_copy = h.timed(pipe.run, steps, warm)
    ok_status = pipe.status() == 0
    h.barrier()
    same = bool(torch.equal(shared, full_nccl)) if h.rank == 0 else True
    de.check_status()
    res["nccl_after_decode"] = {"ms_per_step": ms_nccl, "gbps_into_gpu0": total_bytes / ms_nccl / 1e6,
                                "what": "decode, then NCCL send/recv of every rank's layer slab to GPU 0"}
    res["pipelined_copy"] = {"ms_per_step": ms_copy, "gbps_into_gpu0": total_bytes / ms_copy / 1e6, "parts": len(pipe.parts),
                             "what": "decode in parts; each part's token range is copied into GPU 0's blob "
                                     "(cudaMemcpy2DAsync over NVLink, second stream) while the next part is decoded"}
    res["delivered_bits_equal"] = same and ok_status
    res["tokens_per_s"] = T / min(ms_copy, ms_nccl) * 1e3
    return res


def leg_token_sharded(h, args):
    """BASELINE config 3 on the GPUs of the --gpus N run: ONE request of the Mistral-7B GQA shape (32 layers
    x 8 KV heads x 128, 32,768 tokens = 128 chunks) sharded by token chunks -- every rank decodes a
    contiguous run of the chunks -- with the decoded KV delivered into that token range of one blob on GPU 0
    by pipelined peer copies.  Rank 0 also decodes the whole request alone and compares the delivered blob
    bit for bit."""
    torch = h.torch
    from cachegen_b200.parallel import PipelinedDelivery, buffer_on_root, partition
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = dict(WORKLOADS["mistral7b-gqa-32k"])
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    nchunks = (T + CHUNK_TOKENS - 1) // CHUNK_TOKENS
    mine = partition(nchunks, h.world, h.rank)
    t0, t1 = mine.start * CHUNK_TOKENS, min(mine.stop * CHUNK_TOKENS, T)
    ser, de, _, _ = make_serde(spec, h.world, h.rank)
    # the generator's recurrence runs along the tokens: every rank makes the request and keeps its range
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device=h.dev, dtype=torch.float16)
    chunks = ser.encode_many(kv[:, :, t0:t1], CHUNK_TOKENS, batch=16)
    want = None
    if h.rank == 0:
        want = de.decode_many(ser.encode_many(kv, CHUNK_TOKENS, batch=16))
        de.check_status()
    del kv
    local = torch.empty((L, 2, t1 - t0, H, D), dtype=torch.float16, device=h.dev)
    plan = de.plan(chunks, out=local, workspace={})
    steps, warm = max(3, args.steps // 2), 2
    total_bytes = 2 * L * H * D * T * 2
    ms_decode = h.timed(plan.run, steps, warm)
    shared = buffer_on_root((L, 2, T, H, D), torch.float16, root=0)
    pipe = PipelinedDelivery(de, chunks, local, shared[:, :, t0:t1], parts=args.parts, target_is_local=(h.rank == 0))
    ms_copy = h.timed(pipe.run, steps, warm)
    ok_status = pipe.status() == 0
    h.barrier()
    same = bool(torch.equal(shared, want)) if h.rank == 0 else True
    de.check_status()
    return {"workload": "mistral7b-gqa-32k", "tokens": T, "chunks_per_gpu": len(mine), "kv_bytes": total_bytes,
            "decode_only": {"ms_per_step": ms_decode, "value": total_bytes / ms_decode / 1e6, "unit": "GB/s",
                            "tokens_per_s": T / ms_decode * 1e3,
                            "what": "every rank decodes its run of chunks into its own memory; slowest rank"},
            "pipelined_copy": {"ms_per_step": ms_copy, "gbps_into_gpu0": total_bytes / ms_copy / 1e6,
                               "tokens_per_s": T / ms_copy * 1e3, "parts": len(pipe.parts),
                               "what": "decode in parts; each part's token range goes into GPU 0's blob by peer "
                                       "copies on a second stream while the next part is decoded"},
            "delivered_bits_equal": same and ok_status, "scaling": "strong"}


def run_ours(args, spec):
    import torch
    import torch.distributed as dist

    from cachegen_b200 import _lib
    from cachegen_b200.serde import CacheGenSerializer
    from cachegen_b200.serde.cachegen_basics import CacheGenGPUBytestream, CacheGenGPUEncoderOutput
    from cachegen_b200.parallel import PipelinedDelivery, buffer_on_root, gather_layers, partition
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
        # torchrun sets OMP_NUM_THREADS=1; the blob legs' host copies are torch's multi-threaded copies,
        # so every rank gets its share of the host's cores, as a single process gets all of them
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    h = Harness(dev, rank, world)
    barrier, timed = h.barrier, h.timed

    L_total, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    C = H * D
    by_layers = args.shard == "layers" and world > 1
    full_cfg = CacheGenConfig.from_model_name(spec["model_name"])
    if by_layers:
        mine = partition(L_total, world, rank)
        if len(mine) == 0:
            raise SystemExit("more GPUs than layers")
        cfg, L, first_layer, seed = full_cfg.layer_slice(mine.start, mine.stop), len(mine), mine.start, spec["seed"]
    else:
        cfg, L, first_layer, seed = full_cfg, L_total, 0, spec["seed"] + 1000 * rank
    ser, de, config, meta = make_serde(spec, world, rank, cachegen_config=cfg, table_max_bins=full_cfg.max_bins)

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
    kv_chunk0 = kv[:, :, :CHUNK_TOKENS].clone()
    out = torch.empty((L, 2, T, H, D), dtype=torch.float16, device=dev)
    plan = de.plan(chunks, out=out)
    launches_per_step = plan.launches
    kv_bytes = 2 * L * C * T * 2
    payload = plan.payload_bytes
    per_token = {"payload": payload / T, "tables": plan.table_bytes / T, "lengths": plan.length_bytes / T,
                 "scales": plan.scale_bytes / T}
    per_token["total"] = sum(per_token.values())
    algorithmic = plan.output_bytes + payload + plan.table_bytes + plan.length_bytes + plan.scale_bytes

    # sanity gate before timing: decoded values within the quantiser's error bound (bit equality with the
    # reference's results is what the GPU tests check, not this)
    plan.run()
    de.check_status()
    step = torch.cat((chunks[0].max_tensors_key, chunks[0].max_tensors_value)).float().reshape(2 * L, -1, 1)
    cq = torch.cat((ser.key_bins, ser.value_bins)).div(2, rounding_mode="floor") - 1
    got = out[:, :, :CHUNK_TOKENS].reshape(L, 2, -1, C).transpose(0, 1).reshape(2 * L, -1, C).float()
    ref = kv[:, :, :CHUNK_TOKENS].reshape(L, 2, -1, C).transpose(0, 1).reshape(2 * L, -1, C).float()
    bound = 0.5 * step / cq[:, None, None] * 1.001 + step * 2.0 ** -10 + 1e-6
    assert bool(((got - ref).abs() <= bound).all()), "decoded KV violates the quantiser's error bound"
    del got, ref

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
                de.decode_many_host(host_chunks, out=out, groups=32)
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
        del flat_plan, flat_gpu
        kv = None
        e2e = measure_host(flat_host, sum(c.header.total for c in flat_host),
                           "CacheGenDeserializer.decode_many_host on CGB2 containers (CacheGenSerializer.encode_flat) "
                           "held in pinned host memory; 32 groups, copies of one group overlap the decode of the previous")
        # the same copies with no decode: what the bus alone takes (every rank copies at once)
        dev_flat = [torch.empty_like(c.blob, device=dev) for c in flat_host]

        def copy_only():
            for d_, c in zip(dev_flat, flat_host):
                d_.copy_(c.blob, non_blocking=True)
        extra["h2d_only_ms"] = timed(copy_only, max(2, args.steps // 2), 2)
        extra["h2d_only_gbps_per_gpu"] = sum(c.header.total for c in flat_host) / extra["h2d_only_ms"] / 1e6
        del dev_flat
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

    # ---- legs beside the headline
    if not args.no_extra and not by_layers:
        chunk0 = chunks[0]
        kv = plan = out = None
        if world == 1:
            extra["reference_cuda_ext"] = leg_reference_cuda_ext(h, ser, de, kv_chunk0, chunk0)
            del chunks
            torch.cuda.empty_cache()
            extra["anchor_delta"] = leg_anchor_delta(h, spec, generate_kv(L, H, D, 4 * CHUNK_TOKENS, spec["seed"],
                                                                       key_rho=spec["key_rho"], device=dev,
                                                                       dtype=torch.float16))
            torch.cuda.empty_cache()
            extra["whole_context_call"] = leg_whole_context(h, spec, args)
            torch.cuda.empty_cache()
            extra["config3"] = leg_config3(h, args)
            torch.cuda.empty_cache()
            extra["config5"] = leg_config5(h, args)
        else:
            del chunks
            torch.cuda.empty_cache()
            extra["delivered_kv"] = leg_delivered_kv(h, args)
            torch.cuda.empty_cache()
            extra["token_sharded"] = leg_token_sharded(h, args)

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
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "kernel_ms": {"decode_dequant": ms_kernel, "offsets": ms_offsets},
        "encode": {"value": kv_bytes / ms_encode / 1e6, "unit": "GB/s", "ms": ms_encode,
                   "what": "CacheGenSerializer.encode_many: every chunk of the cache, up to 16 chunks in flight on 3 streams, "
                           "KV resident in HBM, second pass of set-up"},
        "roofline": dict({"bound": "hbm", "kernel": "decode_dequant_multi_kernel", "achieved": achieved, "peak": peak,
                          "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                          "frac_of_write_roofline": total_kv_bytes / world / ms_kernel / 1e6 / peak if not by_layers else None,
                          "algorithmic_bytes_per_launch": algorithmic, "traffic": None}, **ncu_counters(L, H, D, T)),
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
