"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(b200ait_[a-z0-9_]+|AITemplate[A-Za-z]+)\s*\(", text))
    # macro-declared families
    for macro, fam in re.findall(r"B200AIT_DECL_GEMM_BIAS(?:_D0(?:_D1)?)?\((\w+)\)()", text):
        if macro != "NAME":
            names.add("b200ait_" + macro)
    names.discard("b200ait_")
    return {n for n in names if not n.startswith("AITemplateParamShape") and n not in (
        "AITemplateAllocator", "AITemplateError", "AITemplateDtype", "AITemplateAllocatorType",
        "AITemplateMemcpyKind", "AITemplateModelOpaque", "AITemplateStreamOpaque", "AITemplateModelHandle",
        "AITemplateStreamHandle")}


def test_library_exports_every_declared_symbol():
    from aitemplate_b200 import _lib

    lib = _lib.load()
    per_op = _declared_functions("b200ait.h")
    container = _declared_functions("model_interface.h")
    assert len(per_op) >= 30 and len(container) >= 32, (len(per_op), len(container))
    missing = [n for n in sorted(per_op | container) if not hasattr(lib, n)]
    assert not missing, missing
    assert set(_lib.exported_symbols()) <= per_op
    assert lib.b200ait_version() == 1


def test_container_reports_errors_without_a_gpu():
    from aitemplate_b200 import _lib

    lib = _lib.load()
    handle = ctypes.c_void_p()
    lib.AITemplateModelContainerCreateFromPlan.restype = ctypes.c_int
    rc = lib.AITemplateModelContainerCreateFromPlan(ctypes.byref(handle), b"/nonexistent/plan", ctypes.c_size_t(1), None)
    assert rc == 1 and "cannot open plan file" in _lib.last_error()
    n = ctypes.c_size_t()
    lib.AITemplateModelContainerGetNumInputs.restype = ctypes.c_int
    assert lib.AITemplateModelContainerGetNumInputs(None, ctypes.byref(n)) == 1
    assert "handle is null" in _lib.last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from aitemplate_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libb200ait.so")
    try:
        import pytest

        with pytest.raises(RuntimeError, match="no CPU fallback"):
            _lib.load()
    finally:
        monkeypatch.undo()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "aitemplate_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, fn)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b|oracle/|reference_ops", src, flags=re.M), \
                    os.path.join(dirpath, fn)
