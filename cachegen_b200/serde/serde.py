"""Serializer / Deserializer interfaces (reference: LMCache/lmcache/storage_backend/serde/serde.py:9-63)."""
import abc
import logging
import time

import torch

logger = logging.getLogger(__name__)


class Serializer(metaclass=abc.ABCMeta):
    @abc.abstractmethod
    def to_bytes(self, t: torch.Tensor) -> bytes:
        """Serialises a KV blob tensor to bytes."""
        raise NotImplementedError


class Deserializer(metaclass=abc.ABCMeta):
    @abc.abstractmethod
    def from_bytes(self, bs: bytes) -> torch.Tensor:
        """Rebuilds the KV blob tensor from bytes."""
        raise NotImplementedError


class SerializerDebugWrapper(Serializer):
    def __init__(self, s: Serializer):
        self.s = s

    def to_bytes(self, t: torch.Tensor) -> bytes:
        start = time.perf_counter()
        bs = self.s.to_bytes(t)
        logger.debug(f"Serialization took {time.perf_counter() - start:.2f} seconds")
        return bs


class DeserializerDebugWrapper(Deserializer):
    def __init__(self, d: Deserializer):
        self.d = d

    def from_bytes(self, bs: bytes) -> torch.Tensor:
        start = time.perf_counter()
        ret = self.d.from_bytes(bs)
        logger.debug(f"Deserialization took {(time.perf_counter() - start) * 1000:.2f} ms")
        return ret
