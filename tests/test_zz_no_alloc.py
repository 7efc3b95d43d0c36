"""The allocation-free prefill entry point (rn_gsu_fwd_static) against rn_gsu_fwd.

Callers that run where device allocation is off limits (allocator callbacks, pre-sized serving
loops, plugins whose host owns the memory) use rn_gsu_fwd_static: it keeps the event schedule in
an array built into the library instead of a caller workspace.  This test drives both entry points
through the C ABI with the same inputs, twice in a row (the built-in array is shared between calls
and keeps stale contents), and expects identical outputs.  torch is used only to hold device memory.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import ramnet_ops._C as C
    lib = C.lib
    i64, i32, f64, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_void_p
    i64p = ctypes.POINTER(ctypes.c_int64)
    lib.rn_gsu_static_scratch_bytes.restype = ctypes.c_int64
    lib.rn_gsu_fwd_static.restype = ctypes.c_int
    lib.rn_gsu_fwd_static.argtypes = [vp, vp, i64p, vp, i64p, vp, i64p, i32, vp, i64p, vp, vp, vp, vp, vp, i64p,
                                      i64, i64, i64, i64, i64, i64, i64, i32, f64, i32, vp]
    return C, lib


def _case(seed, B, H, T, A, C, Kw, Kr, dev, dtype=torch.float32):
    g = torch.Generator(device=dev).manual_seed(seed)
    KT = Kw + Kr
    # distinct slots per token and head, as a Top-K decode produces them; token-major storage
    scores = torch.rand(B, T, H, A, device=dev, generator=g)
    w_idx = scores.topk(Kw, dim=-1).indices
    r_idx = torch.rand(B, T, H, A, device=dev, generator=g).topk(Kr, dim=-1).indices
    idx = torch.cat([w_idx, r_idx], dim=-1).to(torch.int32)
    val = torch.rand(B, T, H, KT, device=dev, generator=g) * 0.5 + 0.01
    val[..., Kw:] *= -1  # reads are stored negated
    val[:, 3, :, 1] = 0.0  # a few no-op events
    x = torch.randn(B, T, H, C, device=dev, generator=g).to(dtype)
    gamma = (torch.randn(B, T, H, device=dev, generator=g) * 0.3).to(dtype)
    slot = torch.randn(B, H, A, C, device=dev, generator=g)
    mass = torch.rand(B, H, A, device=dev, generator=g) + 0.1
    mask = torch.ones(B, T, dtype=torch.uint8, device=dev)
    mask[:, 5:9] = 0
    return idx.permute(0, 2, 3, 1), val.permute(0, 2, 3, 1), x.permute(0, 2, 1, 3), gamma.permute(0, 2, 1), slot, mass, mask


def _run(C, lib, static, tensors, dims, mass_aware):
    idx, val, x, gamma, slot, mass, mask = tensors
    B, H, T, A, Cc, Kw, Kr = dims
    slot_out, mass_out = torch.empty_like(slot), torch.empty_like(mass)
    y = torch.empty(B, T, H, Cc, device=x.device, dtype=x.dtype).permute(0, 2, 1, 3)
    common = [C.ptr(idx), C.ptr(val), C.strides(idx), C.ptr(x), C.strides(x), C.ptr(gamma), C.strides(gamma), C.dtype_code(x),
              C.ptr(mask), C.strides(mask), C.ptr(slot), C.ptr(mass), C.ptr(slot_out), C.ptr(mass_out), C.ptr(y),
              C.strides(y)]
    tail = [B, H, T, A, Cc, Kw, Kr, int(mass_aware), 1e-6, x.device.index, C.stream_of(x)]
    if static:
        rc = lib.rn_gsu_fwd_static(*common, *tail)
    else:
        n = lib.rn_gsu_workspace_bytes(B, H, T, A, Cc, Kw, Kr, x.device.index)
        ws = torch.empty(n, dtype=torch.uint8, device=x.device)
        rc = lib.rn_gsu_fwd(*common, C.ptr(ws), n, *tail)
    assert rc == 0, lib.rn_last_error().decode()
    torch.cuda.synchronize()
    return y, slot_out, mass_out


def test_static_scratch_entry_point_matches_workspace_entry_point():
    C, lib = _lib()
    dev = torch.device("cuda", 0)
    assert lib.rn_gsu_static_scratch_bytes() == 32 << 20
    # two different calls in a row: the second one finds the first one's schedule in the array
    for seed, dims, mass_aware, dtype in ((1, (2, 3, 150, 64, 20, 4, 6), False, torch.float32),
                                          (2, (1, 4, 70, 256, 8, 8, 3), True, torch.float32),
                                          (3, (2, 2, 130, 4096, 128, 16, 16), False, torch.bfloat16)):
        tensors = _case(seed, *dims, dev, dtype)
        want = _run(C, lib, False, tensors, dims, mass_aware)
        got = _run(C, lib, True, tensors, dims, mass_aware)
        for name, a, b in zip(("y", "slot", "mass"), got, want):
            # same kernels, same schedule contents: the results are identical, not merely close
            torch.testing.assert_close(a, b, atol=0, rtol=0, msg=lambda m, n=name: f"{n}: {m}")
        assert float(want[0].abs().max()) > 0


def test_static_scratch_entry_point_rejects_oversized_shapes():
    C, lib = _lib()
    dev = torch.device("cuda", 0)
    dims = (4, 16, 8192, 64, 8, 16, 16)  # schedule of ~200 MB: beyond the built-in array
    assert lib.rn_gsu_workspace_bytes(*dims, 0) > lib.rn_gsu_static_scratch_bytes()
    B, H, T, A, Cc, Kw, Kr = dims
    tiny = torch.zeros(16, device=dev)
    st = (ctypes.c_int64 * 4)(0, 0, 0, 1)
    st3 = (ctypes.c_int64 * 3)(0, 0, 0)
    rc = lib.rn_gsu_fwd_static(C.ptr(tiny), C.ptr(tiny), st, C.ptr(tiny), st, C.ptr(tiny), st3, 0, None, None,
                               C.ptr(tiny), C.ptr(tiny), C.ptr(tiny), C.ptr(tiny), C.ptr(tiny), st,
                               B, H, T, A, Cc, Kw, Kr, 0, 1e-6, 0, None)
    assert rc != 0
    assert "built-in array" in lib.rn_last_error().decode()
