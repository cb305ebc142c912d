"""The C-ABI library loads and exports exactly what include/hashattn.h declares; host-only
entry points and argument validation (which return before any CUDA call) behave."""
import ctypes
import os
import re

import pytest

from hashattention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hashattn.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ha_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_functions() == sorted(_lib.PROTOTYPES)


def test_constants_of_the_binding_are_the_header_s():
    """Every integer #define of the header that the Python binding mirrors (status codes, options, modes, the ABI
    version) has the header's value there."""
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    defines = {k: int(v, 0) for k, v in re.findall(r"^#define\s+(HA_[A-Z_0-9]+)\s+\(?(-?(?:0x)?[0-9a-fA-F]+)\)?\s*$", text, flags=re.M)}
    assert {"HA_OK", "HA_ERR_TIMEOUT", "HA_OPT_PLAN_HANDOVER", "HA_ABI_VERSION"} <= set(defines)
    mirrored = [k for k in defines if hasattr(_lib, k)]
    assert len(mirrored) >= 12
    for k in mirrored:
        assert getattr(_lib, k) == defines[k], k


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in hashattn.h but not exported"


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.ha_abi_version() == _lib.HA_ABI_VERSION
    seen = set()
    for code in range(0, 9):
        s = _lib.status_str(code)
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 9
    assert _lib.status_str(12345) == "unknown status"


def good_shape(**kw):
    d = dict(batch=1, num_kv_heads=8, gqa_group=4, head_dim=128, page_size=256, max_pages=128, num_pages=128,
             sel_stride=1024)
    d.update(kw)
    return _lib.HaShape(**d)


def test_workspace_bytes():
    lib = _lib.load()
    bud = _lib.HaBudget(128, 128, 1.0 / 32)
    n = lib.ha_workspace_bytes(good_shape(), bud)
    assert n > 0 and n % 256 == 0
    assert lib.ha_workspace_bytes(good_shape(batch=4), bud) > n
    # invalid shapes / budgets give 0
    assert lib.ha_workspace_bytes(good_shape(head_dim=64), bud) == 0
    assert lib.ha_workspace_bytes(good_shape(gqa_group=8), bud) == 0
    assert lib.ha_workspace_bytes(good_shape(page_size=128), bud) == 0
    assert lib.ha_workspace_bytes(good_shape(batch=0), bud) == 0
    assert lib.ha_workspace_bytes(good_shape(), _lib.HaBudget(-1, 128, 0.5)) == 0
    assert lib.ha_workspace_bytes(good_shape(), _lib.HaBudget(1, 128, float("nan"))) == 0
    assert lib.ha_workspace_bytes(None, bud) == 0


@pytest.mark.parametrize("shape_kw,expected", [
    (dict(head_dim=64), _lib.HA_ERR_UNSUPPORTED_DIM),
    (dict(gqa_group=1), _lib.HA_ERR_UNSUPPORTED_DIM),
    (dict(page_size=16), _lib.HA_ERR_UNSUPPORTED_DIM),
    (dict(batch=-3), _lib.HA_ERR_BAD_ARG),
    (dict(), _lib.HA_ERR_BAD_ARG),  # good shape, but every pointer is NULL
])
def test_entry_points_reject_bad_arguments_before_launching(shape_kw, expected):
    lib = _lib.load()
    shape, bud, w = good_shape(**shape_kw), _lib.HaBudget(128, 128, 1.0 / 32), _lib.HaHashWeights(None, None, None, None, 0)
    N = None
    assert lib.ha_hash_decode(shape, w, N, N, N, N, N, N, N, N, N, N, N, N) == expected
    assert lib.ha_hash_prefill(shape, w, N, N, N, N, N, N, N) == expected
    assert lib.ha_score_select(shape, bud, N, N, N, N, N, N, N, N, 0, N, N) == expected
    assert lib.ha_sparse_decode(shape, bud, N, N, N, N, N, N, N, 0.1, N, N, 0, N, N) == expected
    assert lib.ha_decode_step(shape, bud, w, N, N, N, N, N, N, N, N, N, N, N, 0.1, N, N, 0, N, N) == expected
    assert lib.ha_decode_step_host(shape, bud, w, N, N, N, N, N, N, N, N, N, N, N, N, N, N, N, N, N, 0.1, N, 0, N, N,
                                   1) == expected
    assert lib.ha_workspace_init(shape, bud, N, 0, N) == (expected if shape_kw else _lib.HA_ERR_WORKSPACE)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libhashattn.so"))
    with pytest.raises(_lib.HashAttnLibraryError, match="no CPU or PyTorch fallback"):
        _lib.load()
