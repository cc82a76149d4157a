"""cachegen_b200: the CacheGen KV-cache codec (quantise -> CDF tables -> arithmetic coding) for B200.

The package is a thin Python host over one C-ABI CUDA library (libcachegen_b200.so, sm_100a):

    cachegen_b200.torchac_cuda      drop-in for the reference's `torchac_cuda` extension module
    cachegen_b200.serde             drop-in for lmcache.storage_backend.serde (cachegen serializer,
                                    deserializer, CacheGenConfig, wire dataclasses, CreateSerde)
    cachegen_b200.config            LMCacheEngineConfig / LMCacheEngineMetadata mirrors
    cachegen_b200.synth             the synthetic KV generator used by the benchmark and the tests

There is no CPU or pure-PyTorch fallback: every codec call needs the CUDA library and a GPU.
"""
__version__ = "0.1.0"
