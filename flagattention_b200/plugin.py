"""Registers this implementation as the reference's ``flash_attention``,
``flash_attention_split_kv``, ``paged_attention`` and ``piecewise_attention`` through the reference's
own operator registry.

The reference resolves every public operator by name: ``flag_attn.__getattr__``
(``src/flag_attn/__init__.py:123-135``) calls ``runtime.backend.resolve_operator``
(``runtime/backend/op_registry.py:44-60``), which looks the name up in the detected vendor
package's ``_OPERATOR_EXPORTS`` table (``op_registry.py:19-35``) and falls back to the generic
Triton implementation. ``install()`` adds one row per operator to the NVIDIA vendor package's
table, drops the registry's caches and the facade's cached callables, after which
``flag_attn.flash_attention``, ``flag_attn.flash_attention_split_kv`` and
``flag_attn.paged_attention`` are this package's functions. A declared override that fails to import is an error there, not a
fallback, which matches this package having no fallback either.
"""
from __future__ import annotations

import importlib
import sys

OPERATOR = "flash_attention"
TARGET = ("flagattention_b200.flash", "flash_attention")
OPERATORS = {
    OPERATOR: TARGET,
    "flash_attention_split_kv": ("flagattention_b200.flash", "flash_attention_split_kv"),
    "paged_attention": ("flagattention_b200.paged", "paged_attention"),
    "piecewise_attention": ("flagattention_b200.piecewise", "piecewise_attention"),
}


def _vendor_package(vendor: str):
    return importlib.import_module(f"flag_attn.runtime.backend._{vendor}")


def _drop_caches():
    registry = importlib.import_module("flag_attn.runtime.backend.op_registry")
    for fn_name in ("_backend_exports", "_resolve_operator"):
        fn = getattr(registry, fn_name, None)
        if fn is not None and hasattr(fn, "cache_clear"):
            fn.cache_clear()
    facade = sys.modules.get("flag_attn")
    if facade is not None:
        for name in OPERATORS:
            facade.__dict__.pop(name, None)


def install(vendor: str = "nvidia") -> None:
    """Make ``flag_attn.flash_attention``, ``flag_attn.flash_attention_split_kv`` and
    ``flag_attn.paged_attention`` resolve to this package's functions."""
    pkg = _vendor_package(vendor)
    exports = dict(vars(pkg).get("_OPERATOR_EXPORTS", {}))
    exports.update(OPERATORS)
    pkg._OPERATOR_EXPORTS = exports
    generic_only = tuple(n for n in vars(pkg).get("_GENERIC_ONLY_OPS", ()) if n not in OPERATORS)
    pkg._GENERIC_ONLY_OPS = generic_only
    _drop_caches()


def uninstall(vendor: str = "nvidia") -> None:
    """Undo ``install()``: the reference's generic implementation is selected again."""
    pkg = _vendor_package(vendor)
    exports = dict(vars(pkg).get("_OPERATOR_EXPORTS", {}))
    for name in OPERATORS:
        exports.pop(name, None)
    pkg._OPERATOR_EXPORTS = exports
    _drop_caches()
