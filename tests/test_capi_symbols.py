"""The C-ABI library loads and exports every function include/omt_b200.h declares (no compute calls: runs without a GPU)."""
import ctypes
import pathlib
import re

from conftest import ROOT


def declared_functions():
    text = (ROOT / "include" / "omt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(omt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from omarchy_mac_torch_b200 import build, capi
    build.build_lib()
    lib = ctypes.CDLL(str(capi.LIB_PATH))
    names = declared_functions()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_signatures_cover_the_header():
    from omarchy_mac_torch_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_functions()


def test_header_cites_the_reference_for_every_entry_point_group():
    text = (ROOT / "include" / "omt_b200.h").read_text()
    for cite in ("csrc/conv.cpp", "csrc/nn.cpp", "csrc/optim.cpp", "csrc/runtime.cpp", "csrc/device.cpp", "gemm.py"):
        assert cite in text


def test_argument_errors_are_reported_without_a_device():
    """Argument validation happens before any CUDA call, so it can be exercised here."""
    from omarchy_mac_torch_b200 import capi
    g = capi.geo(1, 3, 4, 8, 8, 3, 1, 1)
    g.groups = 2
    try:
        capi.call("omt_conv_fwd", g, capi.null_act(), None, None, capi.null_act(), None, 0, None, 0, None)
        raise AssertionError("expected OmtError")
    except capi.OmtError as e:
        assert e.code == -1 and "groups" in str(e)
    g = capi.geo(1, 3, 4, 8, 8, 13, 1, 1)
    try:
        capi.call("omt_conv_dgrad", g, capi.null_act(), None, capi.null_act(), 0, None, 0, None)
        raise AssertionError("expected OmtError")
    except capi.OmtError as e:
        assert "ks<=11" in str(e)
