"""Drop-in for lmcache.storage_backend.serde, cachegen codec only
(reference: LMCache/lmcache/storage_backend/serde/__init__.py:7-28)."""
from ..config import GlobalConfig, LMCacheEngineConfig, LMCacheEngineMetadata
from .cachegen_basics import DeltaCoding  # noqa: F401
from .cachegen_basics import CacheGenConfig, CacheGenGPUBytestream, CacheGenGPUEncoderOutput
from .cachegen_decoder import CacheGenDeserializer
from .cachegen_encoder import CacheGenSerializer
from .serde import Deserializer, DeserializerDebugWrapper, Serializer, SerializerDebugWrapper


def CreateSerde(serde_type: str, config: LMCacheEngineConfig, metadata: LMCacheEngineMetadata):
    """("cachegen", config, metadata) -> (serializer, deserializer), wrapped in the timing wrappers when
    GlobalConfig.is_debug().  The reference's other serde type, "torch" (plain torch.save), is not part
    of the codec and is not provided here."""
    if serde_type == "cachegen":
        s, d = CacheGenSerializer(config, metadata), CacheGenDeserializer(config, metadata)
    elif serde_type == "torch":
        raise ValueError("serde type 'torch' is outside this package: only the cachegen codec is provided")
    else:
        raise ValueError(f"Invalid serde type: {serde_type}")
    if GlobalConfig.is_debug():
        return SerializerDebugWrapper(s), DeserializerDebugWrapper(d)
    return s, d


__all__ = ["Serializer", "Deserializer", "CacheGenDeserializer", "CacheGenSerializer", "CacheGenConfig",
           "CacheGenGPUBytestream", "CacheGenGPUEncoderOutput", "CreateSerde", "DeltaCoding"]
