"""install() against a stand-in that has the reference registry's shape (a package `flag_attn`
with `runtime.backend.op_registry` and a vendor package), built in a temp dir so the test needs
no reference checkout."""
import importlib
import sys
import textwrap

import pytest


@pytest.fixture
def fake_flag_attn(tmp_path, monkeypatch):
    root = tmp_path / "flag_attn"
    (root / "runtime" / "backend" / "_nvidia").mkdir(parents=True)
    (root / "__init__.py").write_text(textwrap.dedent('''
        import importlib
        from . import runtime
        _OPERATOR_EXPORTS = {"flash_attention": ("flag_attn.flash", "attention"),
                             "flash_attention_split_kv": ("flag_attn.split_kv", "attention"),
                             "paged_attention": ("flag_attn.paged", "attention"),
                             "piecewise_attention": ("flag_attn.piecewise", "attention")}
        def __getattr__(name):
            module_name, attribute_name = _OPERATOR_EXPORTS[name]
            value = runtime.backend.resolve_operator(name, module_name, attribute_name)
            globals()[name] = value
            return value
    '''))
    (root / "flash.py").write_text("def attention(*a, **k):\n    return 'generic'\n")
    (root / "split_kv.py").write_text("def attention(*a, **k):\n    return 'generic-split'\n")
    (root / "paged.py").write_text("def attention(*a, **k):\n    return 'generic-paged'\n")
    (root / "piecewise.py").write_text("def attention(*a, **k):\n    return 'generic-piecewise'\n")
    (root / "runtime" / "__init__.py").write_text(textwrap.dedent('''
        from . import backend
        class _Dev:
            vendor_name = "nvidia"
        device = _Dev()
    '''))
    (root / "runtime" / "backend" / "__init__.py").write_text("from .op_registry import resolve_operator\n")
    (root / "runtime" / "backend" / "_nvidia" / "__init__.py").write_text("")
    (root / "runtime" / "backend" / "op_registry.py").write_text(textwrap.dedent('''
        from functools import lru_cache
        from importlib import import_module
        @lru_cache(maxsize=None)
        def _backend_exports(vendor):
            backend = import_module(f"flag_attn.runtime.backend._{vendor}")
            exports = vars(backend).get("_OPERATOR_EXPORTS", {})
            generic_only = vars(backend).get("_GENERIC_ONLY_OPS", ())
            return {n: v for n, v in exports.items() if n not in generic_only}
        @lru_cache(maxsize=None)
        def _resolve_operator(name, generic_module, generic_name, vendor):
            module_name, symbol = _backend_exports(vendor).get(name, (generic_module, generic_name))
            return getattr(import_module(module_name), symbol)
        def resolve_operator(name, generic_module, generic_name=None, *, vendor=None):
            if vendor is None:
                vendor = import_module("flag_attn.runtime").device.vendor_name
            return _resolve_operator(name, generic_module, generic_name or name, vendor)
    '''))
    monkeypatch.syspath_prepend(str(tmp_path))
    for mod in [m for m in sys.modules if m == "flag_attn" or m.startswith("flag_attn.")]:
        monkeypatch.delitem(sys.modules, mod)
    yield importlib.import_module("flag_attn")
    for mod in [m for m in sys.modules if m == "flag_attn" or m.startswith("flag_attn.")]:
        sys.modules.pop(mod, None)


def test_install_and_uninstall(fake_flag_attn):
    from flagattention_b200 import flash_attention, flash_attention_split_kv, paged_attention, plugin
    fa = fake_flag_attn
    assert fa.flash_attention() == "generic"
    assert fa.flash_attention_split_kv() == "generic-split"
    plugin.install()
    assert fa.flash_attention is flash_attention
    assert fa.flash_attention_split_kv is flash_attention_split_kv
    assert fa.paged_attention is paged_attention
    assert fa.piecewise_attention.__module__ == "flagattention_b200.piecewise"
    plugin.uninstall()
    assert fa.piecewise_attention() == "generic-piecewise"
    assert fa.paged_attention() == "generic-paged"
    assert fa.flash_attention() == "generic"
    assert fa.flash_attention_split_kv() == "generic-split"


def _real_reference_root():
    """Directory holding the unmodified reference package: $FLAG_ATTN_REF (a checkout's `src`) or the
    install under baseline/_ref."""
    import os
    from conftest import REFERENCE_INSTALL
    env = os.environ.get("FLAG_ATTN_REF")
    for cand in ([env] if env else []) + [str(REFERENCE_INSTALL)]:
        if cand and os.path.isdir(os.path.join(cand, "flag_attn", "runtime", "backend")):
            return cand
    return None


@pytest.mark.skipif(_real_reference_root() is None,
                    reason="no reference package: set FLAG_ATTN_REF or pip install the reference with --target baseline/_ref")
def test_install_into_the_reference_registry_itself(monkeypatch):
    """The same round trip through the reference's real facade and registry
    (`src/flag_attn/__init__.py:123-135`, `runtime/backend/op_registry.py:18-60`). No kernel runs: the
    registry only resolves callables. The detected vendor of a machine without a GPU is "cpu", so the
    test pins the vendor name the way `resolve_operator(..., vendor=...)` allows."""
    root = _real_reference_root()
    for mod in [m for m in sys.modules if m == "flag_attn" or m.startswith("flag_attn.")]:
        monkeypatch.delitem(sys.modules, mod)
    monkeypatch.syspath_prepend(root)
    monkeypatch.setattr(sys, "dont_write_bytecode", True)
    fa = importlib.import_module("flag_attn")
    runtime = importlib.import_module("flag_attn.runtime")
    import types
    monkeypatch.setattr(runtime, "device", types.SimpleNamespace(vendor_name="nvidia", name="cuda"))
    from flagattention_b200 import (flash_attention, flash_attention_split_kv, paged_attention,
                                    piecewise_attention, plugin)
    plugin.uninstall()
    generic = fa.flash_attention
    assert generic.__module__.startswith("flag_attn")
    plugin.install()
    try:
        assert fa.flash_attention is flash_attention
        assert fa.flash_attention_split_kv is flash_attention_split_kv
        assert fa.paged_attention is paged_attention
        assert fa.piecewise_attention is piecewise_attention
    finally:
        plugin.uninstall()
    assert fa.flash_attention is generic
    for mod in [m for m in sys.modules if m == "flag_attn" or m.startswith("flag_attn.")]:
        sys.modules.pop(mod, None)
