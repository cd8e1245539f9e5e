"""CPU-only checks of the drop-in boundary: the shared library builds, loads, exports every
symbol the header declares, and refuses to run without a device (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

from helpers import PKG, ROOT


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("ab_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    from alice_train import _ffi
    return _ffi.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "alice_b200.h")).read()
    return sorted(set(re.findall(r"AB_API\s+[\w\s\*]+?\b(ab_\w+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/alice_b200.h but not exported"


def test_binding_covers_header(lib):
    from alice_train import _ffi
    assert sorted(_ffi.SIGNATURES) == _declared_symbols()


def test_header_cites_reference_for_every_entry_point():
    text = open(os.path.join(ROOT, "include", "alice_b200.h")).read()
    assert text.count("src/") >= 30  # file:line citations into the reference crate


def test_no_device_means_no_context(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.ab_device_count() == 0
    assert lib.ab_ctx_create(0, None, C.byref(h)) == 7  # AB_ERR_NO_DEVICE
    import alice_train
    assert alice_train.GpuContext.new_blocking() is None  # Option::None, src/gpu.rs:37
    with pytest.raises(RuntimeError):
        alice_train.default_context()
    with pytest.raises(RuntimeError):
        alice_train.quantize_and_pack([0.5, -0.3])


def test_status_strings(lib):
    assert lib.ab_status_str(0) == b"ok"
    assert b"shape" in lib.ab_status_str(2)
    assert lib.ab_ctx_sync(None) == 1  # AB_ERR_NULL, never a crash


def test_product_code_does_not_touch_the_oracle():
    # the oracle is a checker only; nothing under the package may import, link or run it
    bad = []
    for dirpath, _, files in os.walk(PKG):
        if os.path.basename(dirpath) in ("build", "__pycache__"):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                if "oracle" in open(os.path.join(dirpath, f), errors="ignore").read().lower():
                    bad.append(os.path.join(dirpath, f))
    assert not bad, bad


def test_host_state_logic_matches_reference_rules():
    # pieces of the QAT API that are host arithmetic in the reference too (src/qat.rs:22-110,224-229)
    from alice_train import QatConfig, QuantBits
    assert QuantBits.Ternary.levels() == 3 and abs(QuantBits.Ternary.effective_bits() - 1.585) < 0.01
    assert QuantBits.Int4.levels() == 16 and QuantBits.Int8.levels() == 256
    c = QatConfig()
    assert c.bits == QuantBits.Ternary and c.learn_scale and c.temperature == 1.0
    assert QatConfig.int4().grad_clip == 1.0 and not QatConfig.int8().learn_scale


def test_integration_doc_binds_every_entry_point():
    """The Rust `extern "C"` block shown to the reference's maintainers names every symbol of the header."""
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    missing = [n for n in _declared_symbols() if f"fn {n}(" not in doc]
    assert not missing, missing


def test_python_constants_match_header():
    """Enumerators the Python binding repeats (status codes, options, exchange ops, guards) carry the header's values."""
    from alice_train import _ffi
    text = open(os.path.join(ROOT, "include", "alice_b200.h")).read()
    values = {}
    for body in re.findall(r"typedef enum \w+ \{(.*?)\}", text, flags=re.S):
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        nxt = 0
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            name, _, val = item.partition("=")
            nxt = int(val.strip(), 0) if val.strip() else nxt
            values[name.strip()] = nxt
            nxt += 1
    checked = 0
    for name, val in values.items():
        if hasattr(_ffi, name):
            assert getattr(_ffi, name) == val, name
            checked += 1
    assert checked >= 12
