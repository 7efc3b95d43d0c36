"""Pin the CPU oracle against outputs of the unmodified reference PyTorch backend
(fixtures under tests/golden, produced by tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.helpers import FP32_TOL, assert_close_stats, load, t

ADDR_CASES = ["addr_u2p16k4_f32.npz", "addr_u3p8k8_f32_renorm.npz", "addr_u2p64k16_bf16.npz",
              "addr_u3p32k8_bf16.npz", "addr_u4p4k16_special.npz", "addr_u2p3kall_f32.npz"]


@pytest.mark.parametrize("name", ADDR_CASES)
def test_addr_oracle_matches_reference(name):
    z = load(name)
    B, H, U, P, T, K, E, neg, enc = (int(v) for v in z["meta"])
    A = P ** U
    addr, pos = t(z["addr"]), t(z["pos"])
    idx, val = orc.topk_addr(addr, E, pos, K, float(z["renorm"]), bool(neg), bool(enc))
    ref_idx, ref_val = t(z["idx"]), t(z["val"])
    assert idx.dtype == torch.int32 and idx.shape == ref_idx.shape == (B, H, K, T)
    # weights: the sorted selected weights agree everywhere (ties may pick other members)
    torch.testing.assert_close(val.abs().sort(dim=2).values, ref_val.abs().sort(dim=2).values, atol=1e-6, rtol=1e-5)
    assert (val <= 0).all() if neg else (val >= 0).all()
    # indices: on rows whose K / K+1 boundary gap is clear the selected SET equals the reference's
    clear = t(z["gap"]) > 1e-5  # (B,H,T)
    same = (idx.sort(dim=2).values == ref_idx.sort(dim=2).values).all(dim=2)
    assert bool(same[clear].all()), f"{int((~same[clear]).sum())} clear rows differ"
    assert int(clear.sum()) > 0 or "special" in name or "kall" in name
    # range and CAPE/offset encoding
    nb = B if enc else 1
    offs = (torch.arange(nb * H).view(nb, H, 1, 1) * A).to(torch.int32)
    local = idx - offs
    assert bool(((local >= 0) & (local < A)).all())
    # canonical order: scores non-increasing along K, index ascending inside ties (content space)
    caped = (torch.arange(H).view(1, H, 1, 1) < E).long()
    content = (local.long() + caped * pos[:, None, None, :]) % A
    x = addr.permute(0, 1, 4, 2, 3)
    inactive = torch.isneginf(x).all(-1).any(-1)
    x = x.masked_fill(inactive[..., None, None], 0)
    dense = t(orc.dense_scores(x.numpy()))  # (B,H,T,A)
    sel = dense.gather(-1, content.permute(0, 1, 3, 2))
    d = sel[..., 1:] - sel[..., :-1]
    assert bool((d <= 0).all())
    ties = d == 0
    ci = content.permute(0, 1, 3, 2)
    assert bool((ci[..., 1:] > ci[..., :-1])[ties].all())


@pytest.mark.parametrize("name", ADDR_CASES)
def test_beam_search_equals_dense_selection(name):
    z = load(name)
    B, H, U, P, T, K, E, neg, enc = (int(v) for v in z["meta"])
    addr, pos = t(z["addr"]), t(z["pos"])
    a = orc.topk_addr(addr, E, pos, K, float(z["renorm"]), bool(neg), bool(enc))
    b = orc.topk_addr(addr, E, pos, K, float(z["renorm"]), bool(neg), bool(enc), use_beam=True)
    assert torch.equal(a[0], b[0])
    torch.testing.assert_close(a[1], b[1], atol=0, rtol=0)


def _ram_inputs(z):
    B, H, U, P, T, Kw, Kr, C, E, ma = (int(v) for v in z["meta"])
    mask = t(z["mask"]) if z["mask"].size else None
    w = t(z["w_addr"]).permute(0, 2, 3, 4, 1)  # (B,T,H,U,P) -> (B,H,U,P,T)
    r = t(z["r_addr"]).permute(0, 2, 3, 4, 1)
    x = t(z["values"]).permute(0, 2, 1, 3)
    g = t(z["gamma"]).permute(0, 2, 1)
    return dict(w=w, r=r, x=x, g=g, slot=t(z["init_slot"]), mass=t(z["init_mass"]), mask=mask, pos=t(z["pos"]),
                E=E, K=(Kw, Kr), renorm=tuple(float(v) for v in z["renorm"]), ma=bool(ma), eps=float(z["eps"]))


def _valid(y_bhtc, mask):
    if mask is None:
        return y_bhtc
    return y_bhtc.permute(0, 2, 1, 3)[mask]


RAM_FWD = ["ram_config1.npz", "ram_grads_masked.npz", "ram_grads_massaware.npz", "ram_grads_plain.npz",
           "ram_bf16_u2p16.npz", "ram_decode_t1.npz", "ram_decode_t1_massaware.npz"]


@pytest.mark.parametrize("name", RAM_FWD)
def test_ram_forward_oracle_matches_reference(name):
    z = load(name)
    a = _ram_inputs(z)
    y, slot, mass = orc.ram_attn(a["w"], a["r"], a["x"], a["g"], a["slot"], a["mass"], a["mask"], a["E"], a["pos"],
                                 a["K"], a["renorm"], a["ma"], a["eps"])
    ref_y = t(z["out_y"]).permute(0, 2, 1, 3)
    tol = dict(FP32_TOL)
    if "bf16" in name:  # reference rounds y to bf16; compare against the rounded oracle output
        y = y.to(torch.bfloat16).float()
        tol = dict(atol=2e-2, rtol=2e-2, max_err_rate=0.01, max_q99=1.5)
    assert_close_stats("y", _valid(y, a["mask"]), _valid(ref_y, a["mask"]), **tol)
    assert_close_stats("slot", slot, t(z["out_slot"]), **FP32_TOL)
    assert_close_stats("mass", mass, t(z["out_mass"]), **FP32_TOL)
    if a["mask"] is not None:
        assert float(y.permute(0, 2, 1, 3)[~a["mask"]].abs().max()) == 0.0


@pytest.mark.parametrize("name", ["ram_grads_masked.npz", "ram_grads_massaware.npz", "ram_grads_plain.npz"])
def test_ram_gradients_oracle_matches_reference(name):
    z = load(name)
    a = _ram_inputs(z)
    d_y = t(z["d_y"]).permute(0, 2, 1, 3)
    if a["mask"] is not None:
        d_y = d_y * a["mask"][:, None, :, None]
    (_, _, _), grads = orc.ram_attn_grads(a["w"], a["r"], a["x"], a["g"], a["slot"], a["mass"], a["mask"], a["E"],
                                         a["pos"], a["K"], a["renorm"], a["ma"], a["eps"], d_y, t(z["d_slot"]),
                                         t(z["d_mass"]))
    D_w, D_r, D_x, D_g, D_s, D_m = grads
    tol = dict(atol=1e-7, rtol=1e-6, max_err_rate=0.0, max_q99=1.0)
    mask = a["mask"]

    def tv(g, tdim):  # restrict to valid tokens (reference reads at masked tokens, the op does not)
        if mask is None:
            return g
        g = g.movedim(tdim, 1)  # (B,T,...)
        return g[mask]

    assert_close_stats("D_w", tv(D_w, -1), tv(t(z["out64_D_w"]).permute(0, 2, 3, 4, 1), -1), **tol)
    assert_close_stats("D_r", tv(D_r, -1), tv(t(z["out64_D_r"]).permute(0, 2, 3, 4, 1), -1), **tol)
    assert_close_stats("D_x", tv(D_x, 2), tv(t(z["out64_D_x"]).permute(0, 2, 1, 3), 2), **tol)
    assert_close_stats("D_gamma", tv(D_g, -1), tv(t(z["out64_D_gamma"]).permute(0, 2, 1), -1), **tol)
    assert_close_stats("D_slot", D_s, t(z["out64_D_slot"]), **tol)
    assert_close_stats("D_mass", D_m, t(z["out64_D_mass"]), **tol)


def test_epilogue_restatement_equals_torch_rmsnorm_and_sigmoid():
    """head_rmsnorm_gate restates the layer epilogue of the reference
    (packages/ramnet/src/ramnet/layers/ram_attn_block.py:142-143,342-348): torch.nn.RMSNorm over the C channels
    of every head with eps=None, times Sigmoid(gate logits).  Pinned against those modules, with small inputs so
    that the epsilon matters: eps=None means the epsilon of the type torch computes the norm in, float32 for
    bfloat16 inputs too (not finfo(bfloat16).eps)."""
    g = torch.Generator().manual_seed(0)
    for dtype in (torch.float32, torch.bfloat16):
        for scale in (1.0, 1e-3):
            B, T, H, C = 2, 3, 4, 32
            y = (torch.randn(B, T, H, C, generator=g) * scale).to(dtype)
            gate_logits = torch.randn(B, T, H, C, generator=g).to(dtype)
            norm = torch.nn.RMSNorm(C, eps=None, dtype=dtype)
            with torch.no_grad():
                norm.weight.copy_((torch.randn(C, generator=g) * 0.1 + 1.0).to(dtype))
                want = norm(y) * torch.nn.Sigmoid()(gate_logits)
            got = orc.head_rmsnorm_gate(y.float(), norm.weight.float(), gate_logits.float(), float(torch.finfo(torch.float32).eps))
            tol = 1e-5 if dtype == torch.float32 else 3e-2
            torch.testing.assert_close(got, want.float(), atol=tol, rtol=tol)
