"""CPU checks: the C-ABI library loads and exports every symbol declared in include/ramnet_b200.h,
argument validation of the entry points (no GPU needed: validation happens before any CUDA call),
and the public API's option handling (the contract of the reference's
tests/ops/test_ram_attention_api.py)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _lib():
    import ramnet_ops._C as C
    return C


def test_library_exports_every_declared_symbol():
    C = _lib()
    header = (ROOT / "include" / "ramnet_b200.h").read_text()
    names = set(re.findall(r"\b(rn_[a-z0-9_]+)\s*\(", header))
    assert {"rn_addr_fwd", "rn_addr_bwd", "rn_decode_step", "rn_gsu_fwd", "rn_gsu_bwd", "rn_gsu_fwd_static",
            "rn_gsu_workspace_bytes", "rn_last_error", "rn_int_bits"} <= names
    for name in sorted(names):
        assert hasattr(C.lib, name), f"{name} is declared in the header but missing from the library"
    assert C.INT_BITS == 32
    assert b"sm_100a" in C.lib.rn_version()


def test_entry_points_reject_bad_arguments_without_a_gpu():
    C = _lib()
    lib = C.lib
    st5 = (ctypes.c_int64 * 5)(1, 1, 1, 1, 1)
    st4 = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    st2 = (ctypes.c_int64 * 2)(1, 1)
    rc = lib.rn_addr_fwd(None, None, 0, st5, None, st2, None, None, st4, 1, 1, 2, 200, 4, 0, 4, 0, 0.0, 0.0, 0, 0, 1, 0, None)
    assert rc != 0 and b"P <= 128" in lib.rn_last_error()
    rc = lib.rn_addr_fwd(None, None, 0, st5, None, st2, None, None, st4, 1, 1, 2, 4, 4, 0, 4, 0, 1.5, 0.0, 0, 0, 1, 0, None)
    assert rc != 0 and b"re_norm" in lib.rn_last_error()
    rc = lib.rn_addr_fwd(None, None, 0, st5, None, st2, None, None, st4, 1, 1, 2, 4, 4, 0, 40, 0, 0.0, 0.0, 0, 0, 1, 0, None)
    assert rc != 0 and b"w_top_k" in lib.rn_last_error()
    rc = lib.rn_addr_fwd(None, None, 7, st5, None, st2, None, None, st4, 1, 1, 2, 4, 4, 0, 4, 0, 0.0, 0.0, 0, 0, 1, 0, None)
    assert rc != 0 and b"dtype" in lib.rn_last_error()
    rc = lib.rn_addr_fwd(None, None, 0, st5, None, st2, None, None, st4, 1, 1, 2, 4, 4, 0, 4, 0, 0.0, 0.0, 0, 0, 1, 0, None)
    assert rc != 0 and b"null pointer" in lib.rn_last_error()
    assert lib.rn_gsu_workspace_bytes(1, 1, 8, 16, 4, 300, 2, 0) == -1 and b"top_k" in lib.rn_last_error()
    n = lib.rn_gsu_workspace_bytes(2, 4, 100, 256, 64, 4, 4, 0)
    assert n > 0 and n % 256 == 0
    assert lib.rn_gsu_bwd_workspace_bytes(2, 4, 100, 256, 64, 4, 4, 0) > n


def test_status_and_plan_entry_points_validate_before_touching_cuda():
    C = _lib()
    lib = C.lib
    assert lib.rn_device_status(0, None, 0, None) != 0 and b"null pointer" in lib.rn_last_error()
    assert lib.rn_selftest_wait_timeout(8, 16, 0, None) != 0 and b"multiple of 16" in lib.rn_last_error()
    assert lib.rn_selftest_wait_timeout(16, 40, 0, None) != 0 and b"limit_log2" in lib.rn_last_error()
    info = C.gsu_plan_info(8, 16, 16384, 4096, 128, 16, 16)
    assert info["L"] == 64 and info["cs"] * info["nslices"] >= 128
    assert lib.rn_gsu_plan_info(1, 1, 8, 16, 4, 2, 2, 0, 0, None, 8) != 0


def test_cuda_backend_refuses_cpu_tensors():
    import ramnet_ops
    q = torch.randn(1, 4, 2, 2, 4)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ramnet_ops.random_access_memory_attention(q, q, torch.randn(1, 4, 2, 8), top_k=2, impl_backend="cuda")


def _ram(**kw):
    import ramnet_ops
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 6, 3, 2, 4, generator=g)
    args = dict(w_addr=q, r_addr=q.flip(1), values=torch.randn(2, 6, 3, 5, generator=g), impl_backend="torch")
    args.update(kw)
    return ramnet_ops.random_access_memory_attention(**args)


def test_public_api_option_normalisation_and_errors():
    y, (slot, mass) = _ram(top_k=3)
    assert y.shape == (2, 6, 3, 5) and slot.shape == (2, 3, 16, 5) and mass.shape == (2, 3, 16)
    y2, _ = _ram(top_k=(3, 3), top_k_re_norm=[0.0, 0.0])
    torch.testing.assert_close(y, y2)
    for bad in ("3", (1, 2, 3), (1.0, 2)):
        with pytest.raises(TypeError):
            _ram(top_k=bad)
    for bad in ("x", (0.1,), (0.1, "y")):
        with pytest.raises(TypeError):
            _ram(top_k_re_norm=bad)
    with pytest.raises(ValueError):
        _ram(top_k_re_norm=1.5)
    with pytest.raises(ValueError):
        _ram(impl_backend="metal")
    with pytest.raises(TypeError):
        _ram(init_ram=[None, None])
    with pytest.raises(AssertionError):
        _ram(top_k=99)
    with pytest.raises(AssertionError):
        _ram(embed_num=9)
    with pytest.raises(AssertionError):
        _ram(inplace=True)
    with pytest.raises(AssertionError):
        _ram(eps=0.0)


def test_public_api_time_axis_defaults_and_state_carry():
    import ramnet_ops
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(2, 9, 3, 2, 4, generator=g), torch.randn(2, 9, 3, 2, 4, generator=g)
    v, gm = torch.randn(2, 9, 3, 5, generator=g), 0.3 * torch.randn(2, 9, 3, generator=g)
    full, (s_full, m_full) = ramnet_ops.random_access_memory_attention(k, q, v, gm, embed_num=2, top_k=3, impl_backend="torch")
    # time axis first + scalar mass + explicit positions
    tf, (s2, m2) = ramnet_ops.random_access_memory_attention(
        k.transpose(0, 1), q.transpose(0, 1), v.transpose(0, 1), gm.transpose(0, 1), (None, 1.0 / 16), embed_num=2,
        position_ids=torch.arange(9).view(9, 1).expand(9, 2), top_k=3, t_dim=0, impl_backend="torch")
    torch.testing.assert_close(tf.transpose(0, 1), full)
    torch.testing.assert_close(s2, s_full)
    # chunked calls with state carry and continued positions
    y1, st = ramnet_ops.random_access_memory_attention(k[:, :4], q[:, :4], v[:, :4], gm[:, :4], embed_num=2, top_k=3,
                                                       impl_backend="torch")
    y2, (s3, m3) = ramnet_ops.random_access_memory_attention(k[:, 4:], q[:, 4:], v[:, 4:], gm[:, 4:], st, embed_num=2,
                                                             position_ids=torch.arange(4, 9).view(1, 5), top_k=3,
                                                             impl_backend="torch")
    torch.testing.assert_close(torch.cat([y1, y2], 1), full, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(s3, s_full, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(m3, m_full, atol=1e-6, rtol=1e-5)


def test_topk_addr_public_wrapper_matches_oracle_on_cpu():
    import ramnet_ops
    from oracle import ramnet_oracle as orc
    addr = torch.randn(2, 3, 2, 5, 7)
    pos = torch.arange(7).view(1, 7).expand(2, 7) * 2 + 1
    idx, val = ramnet_ops.topk_addr(addr, 2, pos, 4, 0.5, True, False, impl_backend="torch")
    ridx, rval = orc.topk_addr(addr, 2, pos, 4, 0.5, True, False)
    assert torch.equal(idx.sort(dim=2).values, ridx.sort(dim=2).values)
    torch.testing.assert_close(val.sort(dim=2).values, rval.sort(dim=2).values, atol=1e-6, rtol=1e-5)
    with pytest.raises(ValueError):
        ramnet_ops.topk_addr(addr, 2, pos, 4, 2.0)
    with pytest.raises(TypeError):
        ramnet_ops.topk_addr(addr, 2, pos, 4, "a")
