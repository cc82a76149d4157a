"""Makes this package answer to the reference's import names.

  install()               `import torchac_cuda` and `import lmcache.storage_backend.serde...` resolve
                          to cachegen_b200 (only names that are not already importable are claimed)
  install_wire_aliases()  the minimum needed for pickle wire compatibility: the module path
                          `lmcache.storage_backend.serde.cachegen_basics`
"""
import importlib
import importlib.util
import sys
import types


def _have_real(name: str) -> bool:
    mod = sys.modules.get(name)
    if mod is not None:
        return not getattr(mod, "__cachegen_b200_alias__", False)
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def _ensure_package(name: str) -> types.ModuleType:
    mod = sys.modules.get(name)
    if mod is None:
        mod = types.ModuleType(name)
        mod.__path__ = []
        mod.__cachegen_b200_alias__ = True
        sys.modules[name] = mod
        if "." in name:
            parent, _, child = name.rpartition(".")
            setattr(_ensure_package(parent), child, mod)
    return mod


def _alias(name: str, target: types.ModuleType) -> None:
    parent, _, child = name.rpartition(".")
    if parent:
        setattr(_ensure_package(parent), child, target)
    sys.modules[name] = target


def install_wire_aliases(basics_module_name: str) -> bool:
    """Registers `lmcache.storage_backend.serde.cachegen_basics` -> our module unless a real
    `lmcache` is importable.  Returns True when the alias is in place."""
    if _have_real("lmcache"):
        return False
    _alias("lmcache.storage_backend.serde.cachegen_basics", sys.modules[basics_module_name])
    return True


def install() -> None:
    """Claims `torchac_cuda` and the `lmcache` serde / config import paths for this package."""
    if not _have_real("torchac_cuda"):
        sys.modules["torchac_cuda"] = importlib.import_module("cachegen_b200.torchac_cuda")
    if _have_real("lmcache"):
        return
    serde = importlib.import_module("cachegen_b200.serde")
    _alias("lmcache.config", importlib.import_module("cachegen_b200.config"))
    _alias("lmcache.storage_backend.serde", serde)
    for sub in ("serde", "cachegen_basics", "cachegen_encoder", "cachegen_decoder"):
        _alias(f"lmcache.storage_backend.serde.{sub}", importlib.import_module(f"cachegen_b200.serde.{sub}"))
