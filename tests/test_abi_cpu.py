"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the header declares, and the
argument validation that needs no GPU behaves like the header says."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from customnetworklayers_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "cnl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cnl_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from customnetworklayers_b200 import _lib
    declared = _declared_symbols()
    assert "cnl_tv_forward" in declared and "cnl_tv_backward" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/cnl_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared


def test_version_and_scratch_size(lib):
    assert b"sm_100a" in lib.cnl_version()
    assert lib.cnl_dot_scratch_floats() > 0


def test_argument_validation_needs_no_gpu(lib):
    from customnetworklayers_b200 import _lib
    # a bad id is rejected before anything touches the device, with the reference's return code 1
    assert lib.cnl_tv_forward(1, 1, 1, 1, 1, 1, 1, 2, 8, 8, 20, 10, None) == 1
    assert "outside 0..9" in _lib.last_error()
    assert lib.cnl_tv_forward(1, 1, 1, 1, 1, 1, 1, 2, 8, 8, 20, -1, None) == 1
    assert lib.cnl_tv_forward(1, 1, 1, 1, 1, 1, 0, 2, 8, 8, 20, 0, None) == 2      # bad shape
    assert lib.cnl_tv_forward(1, 1, 1, 1, 1, 1, 1, 2, 8, 8, 1, 0, None) == 3       # its < 2
    assert lib.cnl_tv_forward(None, 1, 1, 1, 1, 1, 1, 2, 8, 8, 20, 0, None) == 7   # null pointer
    assert lib.cnl_tv_backward(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 2, 8, 8, 20, 12, None) == 1
    assert lib.cnl_tv_release(10) == 1
    assert lib.cnl_tv_set_option(0, 99, 1) == 8      # unknown option: rejected before the device is touched
    assert "unknown option 99" in _lib.last_error()
    assert lib.cnl_tv_set_option(10, 1, 1) == 1


def test_python_layer_refuses_cpu_tensors():
    import torch
    from customnetworklayers_b200 import tvInpaint_cuda_ext as ext
    t = torch.zeros(1, 1, 4, 4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.forward(t, t, t, t, t, 4, 0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from customnetworklayers_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_median_bin_limit_is_the_documented_one(lib):
    from customnetworklayers_b200 import _lib
    # validation precedes any device work: 454 bins do not fit the staging rows of a block, 0 bins is no problem at all
    assert lib.cnl_median_forward(1, 1, None, 1, 4, 4, 454, None) == 2
    assert "at most 453 bins" in _lib.last_error()
    assert lib.cnl_median_backward(1, 1, 1, 1, 4, 4, 454, None) == 2
    assert lib.cnl_median_forward(1, 1, None, 1, 4, 4, 0, None) == 2


def test_hierarchy_rejects_id_ranges_outside_the_ten_slots():
    from customnetworklayers_b200.hierarchical import HierarchicalTV
    for first_id, levels in ((8, 3), (-1, 2), (10, 1), (0, 11), (0, 0)):
        with pytest.raises(ValueError):
            HierarchicalTV(levels=levels, first_id=first_id)
    assert HierarchicalTV(levels=3, first_id=7).first_id == 7
