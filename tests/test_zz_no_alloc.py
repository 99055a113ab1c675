"""The allocation-free weight-gradient entry point against the regular one, through the C ABI.

omt_conv_wgrad_noalloc serves hosts that cannot allocate device memory while they run (a fixed launch sequence inside a
real-time loop; a process whose device memory was handed out in full at start-up): its split-K scratch is a fixed array
inside the library. The file name keeps this test last in collection order. Run with -m gpu."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _wgrad_pair(capi, n, ci, co, hw, ks, s, p, scale):
    x = torch.randn(n, ci, hw, hw, device="cuda")
    g = capi.geo(n, ci, co, hw, hw, ks, s, p)
    gy = torch.randn(n, co, g.oh, g.ow, device="cuda")
    ref = capi.conv_wgrad(x, gy, ks, s, p, flags=capi.FORCE_SIMT, scale=scale)
    out = torch.full((co, ci, ks, ks), float("nan"), device="cuda")
    torch.cuda.synchronize()
    # nothing may be allocated by the call: neither from the library's caching allocator nor from torch's
    lib_before, torch_before = capi.lib().omt_memory_reserved(), torch.cuda.memory_reserved()
    lib_live, torch_live = capi.lib().omt_memory_allocated(), torch.cuda.memory_allocated()
    capi.call("omt_conv_wgrad_noalloc", g, capi.act(x), capi.act(gy), capi.ptr(out), scale, capi.stream_handle())
    torch.cuda.synchronize()
    assert capi.lib().omt_memory_reserved() == lib_before and capi.lib().omt_memory_allocated() == lib_live
    assert torch.cuda.memory_reserved() == torch_before and torch.cuda.memory_allocated() == torch_live
    return out, ref, x, gy


def test_noalloc_wgrad_matches_regular_entry_point_twice_in_a_row():
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    from omarchy_mac_torch_b200 import capi
    capi.lib()
    torch.manual_seed(0)
    cap = capi.lib().omt_conv_wgrad_noalloc_capacity()
    assert cap == 16 << 20
    # two calls in a row with different geometries: the second reuses the same built-in scratch (left dirty by the first)
    for shape in ((8, 16, 32, 20, 3, 1, 1, 1.0), (4, 3, 64, 63, 11, 4, 2, 0.5)):
        out, ref, x, gy = _wgrad_pair(capi, *shape)
        err = ((out - ref).abs().max() / ref.abs().max()).item()
        assert err <= 1e-4, (shape, err)
        # and against implementations that share no code with it: the CPU oracle's plain loops, and aten in float64
        n, ci, co, hw, ks, s, p, scale = shape
        want = scale * oracle.c.conv_wgrad(x.cpu().numpy(), gy.cpu().numpy(), ks, s, p)
        assert oracle.rel_err(out.cpu().numpy(), want) <= 1e-4, shape
        _, _, dw64, _ = oracle.aten_conv(x.cpu().double(), torch.zeros(co, ci, ks, ks, dtype=torch.float64), None, s, p, gy.cpu().double())
        assert oracle.rel_err(out.cpu().numpy(), (scale * dw64).float().numpy()) <= 1e-4, shape
    # A geometry whose split-K slabs exceed the built-in scratch is refused with a clear error before anything is launched.
    # Found by growing the channel counts until the library's own scratch figure passes the capacity (the slab count depends
    # on the device's SM count, so no fixed geometry is assumed).
    g, c = None, 64
    while c <= 4096:
        g = capi.geo(64, c, c, 14, 14, 3, 1, 1)
        if capi.lib().omt_conv_workspace_bytes(2, g, capi.FORCE_SIMT) > cap:
            break
        c *= 2
    assert capi.lib().omt_conv_workspace_bytes(2, g, capi.FORCE_SIMT) > cap
    dummy = torch.zeros(8, device="cuda")
    before = capi.lib().omt_launch_count()
    with pytest.raises(capi.OmtError) as e:
        capi.call("omt_conv_wgrad_noalloc", g, capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.ptr(dummy), 1.0,
                  capi.stream_handle())
    assert e.value.code == -5 and "scratch" in str(e.value)
    assert capi.lib().omt_launch_count() == before
    # extents the kernels' 32-bit indices cannot hold are refused like omt_conv_wgrad refuses them
    huge = capi.geo(1 << 20, 3, 8, 64, 64, 3, 1, 1)
    with pytest.raises(capi.OmtError) as e:
        capi.call("omt_conv_wgrad_noalloc", huge, capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.Act(dummy.data_ptr(), 1, 1, 1, 1), capi.ptr(dummy), 1.0,
                  capi.stream_handle())
    assert e.value.code == -1 and "2^31" in str(e.value)
