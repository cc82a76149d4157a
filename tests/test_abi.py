"""The C-ABI library loads without a GPU and exports every function include/cachegen_b200.h declares;
argument errors are rejected before anything touches CUDA."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cachegen_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "cachegen_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cg_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from cachegen_b200 import _lib
    names = declared_functions()
    assert len(names) >= 12
    assert sorted(_lib.EXPORTS) == names
    for n in names:
        assert hasattr(lib, n), n


def test_version_and_status_strings(lib):
    assert b"sm_100a" in lib.cg_version()
    assert lib.cg_status_string(0) == b"ok"
    for code in range(-9, 0):
        assert lib.cg_status_string(code) != b"unknown status"


def test_argument_errors_need_no_gpu(lib):
    from cachegen_b200 import _lib
    s3 = (ctypes.c_int64 * 3)(1, 1, 1)
    one = ctypes.c_void_p(16)  # never dereferenced: every call below is rejected before launching
    assert lib.cg_calculate_cdf(None, s3, 1, 1, 1, 4, one, None) == -1
    assert lib.cg_calculate_cdf(one, s3, 1, 1, 1, 64, one, None) == -4
    assert lib.cg_calculate_cdf(one, s3, 1, 65536, 1, 4, one, None) == -9
    assert lib.cg_calculate_cdf(one, s3, 0, 1, 1, 4, one, None) == -2
    assert lib.cg_encode_padded(one, one, s3, 1, 257, 1, 33, one, 256, one, None, None) == -3
    assert lib.cg_encode_padded(one, one, s3, 1, 256, 1, 65, one, 256, one, None, None) == -4
    assert lib.cg_encode_padded(one, one, s3, 1, 256, 1, 33, one, 255, one, None, None) == -5
    assert lib.cg_decode_prefsum(one, one, 8, None, one, s3, 1, 1, 1, 33, None, None) == -1
    assert lib.cg_decode_prefsum(one, one, 8, one, one, s3, 1, 300, 1, 33, None, None) == -3
    assert lib.cg_decode_padded(one, one, 0, one, one, s3, 1, 1, 1, 33, None, None) == -2
    assert lib.cg_quantize_cdf(one, 7, 1, 1, 1, 1, 1, 1, 1, 1, one, 32, one, one, one, None, None, None, None) == -7
    assert lib.cg_quantize_cdf(one, 0, 1, 1, 1, 1, 1, 70000, 1, 1, one, 32, one, one, one, None, None, None, None) == -9
    assert lib.cg_quantize_cdf(one, 0, 1, 1, 1, 1, 1, 16, 1, 1, one, 32, one, one, one, one, None, None, None) == -1
    assert lib.cg_encode_chunk(one, one, 1, 1, 1, 33, one, 10, one, one, one, None, None) == -5
    assert lib.cg_compact_streams(one, 8, one, one, one, 0, 1, 1, one, None) == -2
    jobs = (_lib.DecodeJob * 1)()
    assert lib.cg_decode_offsets(jobs, 41, 1, 1, one, None, None) == -6
    assert lib.cg_decode_offsets(jobs, 1, 1, 1, one, None, None) == -1   # job.lengths is NULL
    assert lib.cg_decode_dequant(jobs, 1, 1, 1, 1, 33, one, 0, 5, 1, 1, 1, 1, None, None) == -7
    assert lib.cg_decode_dequant(jobs, 1, 1, 1, 1, 33, one, 0, 0, 1, 1, 1, 1, None, None) == -1


def test_product_has_no_oracle_dependency():
    """Nothing under cachegen_b200/ may import or load the oracle."""
    for dirpath, _, files in os.walk(os.path.join(ROOT, "cachegen_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "cg_oracle" not in text and "libcg_oracle" not in text, f
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f


def test_config_lookup(monkeypatch, golden_cpu):
    import torch
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig, make_key_bins, make_value_bins
    monkeypatch.setenv("QUANT_LEVEL", "2")
    for name in ("lmsys/longchat-7b-16k", "Yukang/LongAlpaca-70B-16k", "mistralai/Mistral-7B-Instruct-v0.2"):
        cfg = CacheGenConfig.from_model_name(name)
        key = name.split("/")[1]
        assert (make_key_bins(cfg, "cpu").numpy() == golden_cpu[f"bins_{key}_k"]).all()
        assert (make_value_bins(cfg, "cpu").numpy() == golden_cpu[f"bins_{key}_v"]).all()
    monkeypatch.setenv("QUANT_LEVEL", "1")
    assert CacheGenConfig.from_model_name("x/Mistral-7B-y").key_third_bins == 12
    monkeypatch.delenv("QUANT_LEVEL")
    with pytest.raises(KeyError):
        CacheGenConfig.from_model_name("mistralai/Mistral-7B-Instruct-v0.2")
    with pytest.raises(ValueError):
        CacheGenConfig.from_model_name("gpt2")
    half = CacheGenConfig.from_model_name("lmsys/longchat-7b-16k").with_bins_divided(2)
    assert (half.key_first_bins, half.key_second_bins, half.value_second_bins) == (16, 8, 8)
    quarter = CacheGenConfig.from_model_name("lmsys/longchat-7b-16k").with_bins_divided(4)
    assert (quarter.key_first_bins, quarter.key_third_bins) == (8, 4)
    assert isinstance(make_key_bins(half, "cpu"), torch.Tensor)


def test_wire_classes_pickle_under_the_reference_path():
    import torch
    from cachegen_b200.serde.cachegen_basics import CacheGenGPUBytestream, CacheGenGPUEncoderOutput, CacheGenEncoderOutput
    o = CacheGenGPUEncoderOutput([CacheGenGPUBytestream(torch.zeros(3, dtype=torch.uint8),
                                                        torch.ones(2, 2, dtype=torch.int32), 5)],
                                 torch.zeros(2, 2, 3, dtype=torch.int16), torch.zeros(1, 5, 1), torch.ones(1, 5, 1), 1, 2)
    blob = o.to_bytes()
    import sys
    if getattr(sys.modules.get("lmcache"), "__cachegen_b200_alias__", False):  # no real lmcache installed
        assert b"lmcache.storage_backend.serde.cachegen_basics" in blob
    back = CacheGenEncoderOutput.from_bytes(blob)
    assert back.num_heads == 1 and back.head_size == 2 and back.data_chunks[0].ntokens == 5
    assert back["cdf"].shape == (2, 2, 3) and back.data_chunks[0]["bytestream_lengths"].sum() == 4


def test_blob_loader_reads_storages_in_one_copy_and_like_torch():
    """from_bytes replaces torch's storage loader with one that views the data inside the pickle; the
    result must equal what plain pickle.load gives, views and odd dtypes included."""
    import io
    import pickle
    import torch
    from cachegen_b200.serde import cachegen_basics as B
    base = torch.randn(6, 40, 1).to(torch.bfloat16)
    o = B.CacheGenGPUEncoderOutput(
        [B.CacheGenGPUBytestream(torch.arange(1000, dtype=torch.int64).to(torch.uint8), torch.ones(4, 8, dtype=torch.int32), 7),
         B.CacheGenGPUBytestream(torch.zeros(0, dtype=torch.uint8), torch.zeros(4, 8, dtype=torch.int32), 3)],
        torch.randint(-5, 5, (4, 8, 9), dtype=torch.int16), base[:3], base[3:, 5:15], 2, 4)
    with io.BytesIO() as f:
        pickle.dump(o, f)          # torch's own pickling, as the reference writes a blob
        blob = f.getvalue()
    calls = []
    orig = torch.storage._load_from_bytes
    torch.storage._load_from_bytes = lambda b: (calls.append(1), orig(b))[1]
    try:
        got = B.CacheGenGPUEncoderOutput.from_bytes(blob)
    finally:
        torch.storage._load_from_bytes = orig
    assert not calls  # torch's loader was never needed
    want = pickle.load(io.BytesIO(blob))
    for a, b in ((got.cdf, want.cdf), (got.max_tensors_key, want.max_tensors_key),
                 (got.max_tensors_value, want.max_tensors_value),
                 (got.data_chunks[0].bytestream, want.data_chunks[0].bytestream),
                 (got.data_chunks[1].bytestream, want.data_chunks[1].bytestream)):
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    got.cdf[0, 0, 0] = 7  # loaded tensors own writable memory


def test_blob_loader_views_large_storages_instead_of_copying_them():
    """Byte strings of 64 KB and more (the pickled storages of tables and streams) must reach the
    storage loader as views of the blob, and a blob the view reader cannot parse must still load."""
    import torch
    from cachegen_b200.serde import cachegen_basics as B
    big = torch.arange(300_000, dtype=torch.int32).to(torch.uint8)
    o = B.CacheGenGPUEncoderOutput([B.CacheGenGPUBytestream(big, torch.ones(4, 8, dtype=torch.int32), 7)],
                                   torch.arange(4 * 8 * 33, dtype=torch.int16).reshape(4, 8, 33),
                                   torch.ones(2, 7, 1, dtype=torch.float16), torch.ones(2, 7, 1, dtype=torch.float16), 2, 4)
    blob = o.to_bytes()
    kinds = []
    orig = B._load_storage_fast
    B._load_storage_fast = lambda b: (kinds.append((type(b).__name__, len(b))), orig(b))[1]
    try:
        got = B.CacheGenGPUEncoderOutput.from_bytes(blob)
    finally:
        B._load_storage_fast = orig
    assert torch.equal(got.data_chunks[0].bytestream, big) and torch.equal(got.cdf, o.cdf)
    assert any(k == "memoryview" and n > 300_000 for k, n in kinds)
    # the reader: small reads are bytes (the unpickler indexes them), large ones views, lines end at \n
    r = B._ViewReader(b"ab\ncd" + bytes(70_000))
    assert r.readline() == b"ab\n" and r.read(2) == b"cd" and isinstance(r.read(65_536), memoryview)
    assert len(r.read()) == 70_000 - 65_536 and r.read(5) == b""
    # fallback: a failure inside the view unpickler leaves the standard one to load the blob
    orig_cls = B._ViewUnpickler
    B._ViewUnpickler = lambda data: (_ for _ in ()).throw(RuntimeError("no"))
    try:
        again = B.load_blob(blob)
    finally:
        B._ViewUnpickler = orig_cls
    assert torch.equal(again.data_chunks[0].bytestream, big)


def test_blob_writer_gives_the_bytes_of_pickle_dump():
    """to_bytes builds each tensor's legacy torch.save stream itself (one copy through pinned memory on
    the GPU); the result must be pickle.dump's, byte for byte, also for tensors it leaves to torch
    (views that do not own their storage) and for empty ones."""
    import io
    import pickle
    import warnings
    import torch
    from cachegen_b200.serde import cachegen_basics as B
    warnings.simplefilter("ignore")
    base = torch.randn(6, 40, 1).to(torch.bfloat16)
    o = B.CacheGenGPUEncoderOutput(
        [B.CacheGenGPUBytestream(torch.arange(400_000, dtype=torch.int64).to(torch.uint8), torch.ones(4, 8, dtype=torch.int32), 7),
         B.CacheGenGPUBytestream(torch.zeros(0, dtype=torch.uint8), torch.zeros(4, 8, dtype=torch.int32), 3)],
        torch.randint(-5, 5, (40, 80, 33), dtype=torch.int16), base[:3].clone().to(torch.float16), base[3:, 5:15], 2, 4)
    f = io.BytesIO()
    pickle.dump(o, f)
    made = []
    orig = B._legacy_stream_head
    B._legacy_stream_head = lambda *a: (made.append(a[0]), orig(*a))[1]
    try:
        assert o.to_bytes() == f.getvalue()
    finally:
        B._legacy_stream_head = orig
    # every tensor but the view took the fast path
    assert sorted(map(str, made)) == sorted(map(str, [torch.uint8, torch.int32, torch.uint8, torch.int32, torch.int16, torch.float16]))
    for dt in (torch.uint8, torch.int16, torch.int32, torch.float16, torch.bfloat16):
        t = torch.arange(1000).to(dt)
        want = t._typed_storage().__reduce__()[1][0]   # torch's own stream of this storage
        head = B._legacy_stream_head(dt, str(t.untyped_storage()._cdata), "cpu", t.numel())
        assert head + bytes(memoryview(t.view(torch.uint8).numpy())) == want


def test_a_c_program_links_against_the_header_and_the_library(tmp_path):
    """gcc compiles tests/abi_link/c_client.c against include/cachegen_b200.h, links it with the
    library and runs it: no Python, no torch between a caller and the ABI."""
    import os
    import shutil
    import subprocess
    from cachegen_b200 import _lib
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    _lib.lib()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.dirname(_lib.LIB_PATH)
    exe = str(tmp_path / "c_client")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(root, "include"),
                    os.path.join(root, "tests", "abi_link", "c_client.c"), "-o", exe,
                    "-L", libdir, "-l:" + os.path.basename(_lib.LIB_PATH), "-Wl,-rpath," + libdir], check=True)
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all checks passed" in run.stdout
    assert ctypes.sizeof(_lib.DecodeJob) == 96   # the ctypes mirror has the size the C program checked


def test_workspace_sizes_match_what_the_encoder_allocates():
    """cg_workspace_bytes against the sizes the Python host side works out for itself."""
    from cachegen_b200 import _lib
    ws = _lib.workspace_sizes(64, 700, 4096)
    assert ws.nsub == 3 and ws.scratch_stride == _lib.stream_capacity(256)
    assert ws.encode_scratch == 3 * 64 * 4096 * 520 and ws.encode_lengths == 3 * 64 * 4096 * 4
    assert ws.encode_group_off == 3 * 64 * 32 * 8 and ws.encode_sub_off == 4 * 8
    assert ws.decode_group_off == 64 * 32 * 8 and ws.symbols == 64 * 700 * 4096
    short = _lib.workspace_sizes(2, 10, 130)
    assert short.scratch_stride == 28 and short.decode_group_off == 2 * 2 * 8
    import pytest
    with pytest.raises(RuntimeError):
        _lib.workspace_sizes(0, 10, 130)


def test_nvtx_decorator_is_a_no_op_without_the_package(monkeypatch):
    import builtins
    import sys
    from cachegen_b200.utils import _get_color_for_nvtx, _lmcache_nvtx_annotate
    real_import = builtins.__import__

    def no_nvtx(name, *a, **k):
        if name == "nvtx":
            raise ImportError(name)
        return real_import(name, *a, **k)
    monkeypatch.delitem(sys.modules, "nvtx", raising=False)
    monkeypatch.setattr(builtins, "__import__", no_nvtx)

    def f(x):
        return x + 1
    assert _lmcache_nvtx_annotate(f) is f and f(1) == 2
    assert _get_color_for_nvtx("decode_chunk") in ("green", "blue", "purple", "rapids")


def test_blob_writer_falls_back_to_plain_pickle(monkeypatch):
    """to_bytes must still give the reference's blob when the hand-built storage streams cannot be
    made (a torch release that changes the legacy format)."""
    import io
    import pickle
    import torch
    from cachegen_b200.serde import cachegen_basics as B
    o = B.CacheGenGPUEncoderOutput(
        [B.CacheGenGPUBytestream(torch.arange(100).to(torch.uint8), torch.ones(2, 4, dtype=torch.int32), 5)],
        torch.zeros((2, 4, 9), dtype=torch.int16), torch.ones(1, 5, 1).half(), torch.ones(1, 5, 1).half(), 1, 4)
    f = io.BytesIO()
    pickle.dump(o, f)

    def broken(*a, **k):
        raise AttributeError("storage stream layout changed")
    monkeypatch.setattr(B, "dump_blob", broken)
    blob = o.to_bytes()
    assert blob == f.getvalue()
    back = B.CacheGenGPUEncoderOutput.from_bytes(blob)
    assert torch.equal(back.cdf, o.cdf) and back.data_chunks[0].ntokens == 5
