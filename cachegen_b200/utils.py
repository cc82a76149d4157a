"""Small helpers shared by the package (reference: LMCache/lmcache/utils.py:28-48, the NVTX part)."""
import hashlib

_NVTX_COLORS = ["green", "blue", "purple", "rapids"]


def _get_color_for_nvtx(name: str) -> str:
    digest = int(hashlib.sha256(name.encode()).hexdigest(), 16)
    return _NVTX_COLORS[digest % len(_NVTX_COLORS)]


def _lmcache_nvtx_annotate(func, domain: str = "lmcache"):
    """Decorator that wraps `func` in an NVTX range named after it, in the reference's domain and
    colour scheme (utils.py:42-48), so that a timeline of an engine that mixes both packages reads
    the same.  Without the optional `nvtx` package the function is returned as it is."""
    try:
        from nvtx import annotate
    except ImportError:
        return func
    return annotate(message=func.__qualname__, color=_get_color_for_nvtx(func.__qualname__), domain=domain)(func)
