"""The C-ABI library loads and exports every symbol include/tempest_b200.h
declares; status texts; argument validation that needs no GPU."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def built():
    entry.build()
    return entry.load_package()


def declared_symbols():
    header = open(os.path.join(entry.ROOT, "include", "tempest_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", header)))


def test_header_declares_symbols():
    names = declared_symbols()
    assert "tb200_softmax_fwd" in names and "tb200_layernorm_bwd" in names


def test_library_exports_every_declared_symbol(built):
    handle = ctypes.CDLL(built.lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol(built):
    assert set(declared_symbols()) == set(built.lib.SIGNATURES), \
        set(declared_symbols()) ^ set(built.lib.SIGNATURES)


def test_version_and_status_texts(built):
    lib = built.lib.load()
    assert lib.tb200_version() >= 100
    assert lib.tb200_strerror(0) == b"ok"
    seen = {lib.tb200_strerror(-k) for k in range(1, 9)}
    assert len(seen) == 8 and b"unknown status" not in seen
    assert lib.tb200_strerror(-99) == b"unknown status"


def test_argument_validation_needs_no_device(built):
    L = built.lib
    with pytest.raises(L.TB200Error) as e:
        L.softmax_fwd(16, 16, 0, 4, 2, 4, 7)  # unknown dtype
    assert e.value.status == -3
    with pytest.raises(L.TB200Error) as e:
        L.softmax_fwd(16, 16, 0, 8, 2, 4, L.F32)  # ld < n
    assert e.value.status == -2
    with pytest.raises(L.TB200Error) as e:
        L.softmax_fwd(16, 16, 0, -1, 2, 4, L.F32)
    assert e.value.status == -2
    # nothing to do: no pointer is looked at, no device is needed
    L.softmax_fwd(0, 0, 0, 4, 0, 4, L.F32)
    L.softmax_bwd(0, 0, 0, 0, 0, 5, 0, L.BF16)
    with pytest.raises(L.TB200Error) as e:
        L.softmax_fwd(0, 16, 0, 4, 2, 4, L.F32)  # null x
    assert e.value.status == -1
    with pytest.raises(L.TB200Error) as e:
        L.softmax_fwd(18, 16, 0, 4, 2, 4, L.F32)  # x not aligned to Float32
    assert e.value.status == -4


def test_missing_library_fails_loudly(built, tmp_path):
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        built.lib.load(str(tmp_path / "libtempest_b200.so"))
