"""Mirrors of the two config dataclasses the codec reads (reference: LMCache/lmcache/config.py:6-87).

The codec only looks at `chunk_size`, `model_name` and `fmt`; the other fields are carried so that
code written against the reference constructs these objects unchanged.
"""
import re
from dataclasses import dataclass
from typing import Optional


@dataclass
class LMCacheEngineMetadata:
    model_name: str   # name of the LLM; selects the CacheGenConfig
    world_size: int   # carried in cache keys only
    worker_id: int    # carried in cache keys only
    fmt: str          # "vllm" ([L,2,T,H,D]) or "huggingface" ([L,2,H,T,D])


@dataclass
class LMCacheEngineConfig:
    chunk_size: int
    local_device: Optional[str]
    remote_url: Optional[str]
    remote_serde: str  # "torch" or "cachegen"
    pipelined_backend: bool

    @staticmethod
    def from_defaults(chunk_size: int = 256, local_device: str = "cuda",
                      remote_url: str = "redis://localhost:6379", remote_serde: str = "torch",
                      pipelined_backend: bool = False) -> "LMCacheEngineConfig":
        return LMCacheEngineConfig(chunk_size, local_device, remote_url, remote_serde, pipelined_backend)

    @staticmethod
    def from_legacy(chunk_size: int = 256, backend: str = "cuda", persist_path: str = None,
                    remote_serde: str = "torch", pipelined_backend: bool = False) -> "LMCacheEngineConfig":
        if backend in ("cpu", "cuda"):
            local_device, remote_url = backend, None
        elif re.match(r"(.*)://(.*):(\d+)", backend):
            local_device, remote_url = None, backend
        else:
            raise ValueError(f"Invalid backend: {backend}")
        return LMCacheEngineConfig(chunk_size, local_device, remote_url, remote_serde, pipelined_backend)

    @staticmethod
    def from_file(file_path: str) -> "LMCacheEngineConfig":
        import yaml
        with open(file_path, "r") as fin:
            config = yaml.safe_load(fin)
        return LMCacheEngineConfig(config.get("chunk_size", 256), config.get("local_device", None),
                                   config.get("remote_url", None), config.get("remote_serde", "torch"),
                                   config.get("pipelined_backend", False))


class GlobalConfig:
    enable_debug: bool = True

    @classmethod
    def set_debug(cls, enable: bool):
        cls.enable_debug = enable

    @classmethod
    def is_debug(cls) -> bool:
        return cls.enable_debug
