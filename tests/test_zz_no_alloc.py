"""The allocation-free weight-gradient entry point against the regular one, through the C ABI.

omt_conv_wgrad_noalloc serves hosts that cannot allocate device memory while they run (a fixed launch sequence inside a
real-time loop; a process whose device memory was handed out in full at start-up): its split-K scratch is a fixed array
inside the library. The file name keeps this test last in collection order. Run with -m gpu."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _wgrad_pair(capi, n, ci, co, hw, ks, s, p, scale):
    x = torch.randn(n, ci, hw, hw, device="cuda")
    g = capi.geo(n, ci, co, hw, hw, ks, s, p)
    gy = torch.randn(n, co, g.oh, g.ow, device="cuda")
    ref = capi.conv_wgrad(x, gy, ks, s, p, flags=capi.FORCE_SIMT, scale=scale)
    out = torch.full((co, ci, ks, ks), float("nan"), device="cuda")
    capi.call("omt_conv_wgrad_noalloc", g, capi.act(x), capi.act(gy), capi.ptr(out), scale, capi.stream_handle())
    torch.cuda.synchronize()
    return out, ref


def test_noalloc_wgrad_matches_regular_entry_point_twice_in_a_row():
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    from omarchy_mac_torch_b200 import capi
    capi.lib()
    torch.manual_seed(0)
    cap = capi.lib().omt_conv_wgrad_noalloc_capacity()
    assert cap == 16 << 20
    # two calls in a row with different geometries: the second reuses the same built-in scratch (left dirty by the first)
    for shape in ((8, 16, 32, 20, 3, 1, 1, 1.0), (4, 3, 64, 63, 11, 4, 2, 0.5)):
        out, ref = _wgrad_pair(capi, *shape)
        err = ((out - ref).abs().max() / ref.abs().max()).item()
        assert err <= 1e-4, (shape, err)
    # a geometry whose split-K slabs exceed the built-in scratch is refused with a clear error, before anything is launched
    g = capi.geo(64, 512, 512, 14, 14, 3, 1, 1)
    need = capi.lib().omt_conv_workspace_bytes(2, g, capi.FORCE_SIMT)
    assert need > cap
    dummy = torch.zeros(8, device="cuda")
    with pytest.raises(capi.OmtError) as e:
        capi.call("omt_conv_wgrad_noalloc", g, capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.ptr(dummy), 1.0,
                  capi.stream_handle())
    assert e.value.code == -5 and "scratch" in str(e.value)
