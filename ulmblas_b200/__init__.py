"""ulmblas_b200 -- B200-native Level-3 GEMM path behind ulmBLAS's BLAS entry points.

``ulmblas_b200.api`` holds the bindings; it loads ``libulmblas_b200.so`` on import and
raises ``LibraryMissing`` if the library has not been built (there is no CPU fallback).
The package itself imports lazily so that ``python -m ulmblas_b200.build`` can run
before the library exists: any attribute access (``ulmblas_b200.dgemm`` ...) loads the
bindings.
"""
import importlib

__all__ = ["api", "build", "sharded"]


def __getattr__(name):
    if name in ("api", "build", "sharded"):
        return importlib.import_module(f"{__name__}.{name}")
    api = importlib.import_module(f"{__name__}.api")
    try:
        return getattr(api, name)
    except AttributeError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
