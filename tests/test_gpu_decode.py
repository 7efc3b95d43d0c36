"""GPU parity of the fused decode step against the CPU oracle and the reference golden vectors."""
import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.gpu_common import ops, randn
from tests.helpers import BF16_TOL, FP32_TOL, assert_close_stats, load, t

pytestmark = pytest.mark.gpu


def _inputs(B, H, U, P, C, dtype, seed):
    A = P ** U
    w = randn((B, H, U, P), seed, dtype)
    r = randn((B, H, U, P), seed + 1, dtype)
    x = randn((B, H, C), seed + 2, dtype)
    g = torch.sigmoid(randn((B, H), seed + 3)).to(dtype)
    slot = randn((B, H, A, C), seed + 4) * 0.1
    mass = torch.rand(B, H, A, generator=torch.Generator().manual_seed(seed + 5)) + 0.1
    pos = torch.arange(B) * 7 + 3
    return w, r, x, g, slot, mass, pos


@pytest.mark.parametrize("B,H,U,P,C,K,dtype", [
    (3, 4, 2, 8, 12, (4, 4), torch.float32),
    (2, 4, 2, 16, 64, (4, 6), torch.float32),
    (2, 2, 2, 64, 128, (16, 16), torch.bfloat16),
    (2, 3, 3, 8, 29, (8, 3), torch.float16),
    (1, 2, 4, 4, 7, (40, 33), torch.float32),
    (1, 2, 2, 64, 256, (16, 16), torch.bfloat16),
    (3, 7, 2, 64, 128, (16, 16), torch.bfloat16),   # 21 pairs: a full and a partial CTA of the specialised kernel
    (2, 4, 2, 16, 128, (4, 4), torch.float32),
    (2, 2, 3, 32, 128, (8, 8), torch.float16),
])
@pytest.mark.parametrize("mass_aware", [False, True])
def test_decode_step_matches_oracle(B, H, U, P, C, K, dtype, mass_aware):
    ops()
    w, r, x, g, slot, mass, pos = _inputs(B, H, U, P, C, dtype, 0)
    mask = torch.ones(B, dtype=torch.bool)
    if B > 1:
        mask[1] = False
    renorm = (0.25, 0.75)
    eps = 1e-6
    E = H // 2
    ref_y, ref_slot, ref_mass = orc.decode_step(w.float(), r.float(), x.float(), g.float(), slot.clone(), mass.clone(),
                                                mask, E, pos, K, renorm, mass_aware, eps)
    d_slot, d_mass = slot.clone().cuda(), mass.clone().cuda()
    y = torch.ops.ramnet_ops.topk_autoregressive_(w.cuda(), r.cuda(), x.cuda(), g.cuda(), d_slot, d_mass, mask.cuda(), E,
                                                  pos.cuda().int(), K[0], K[1], renorm[0], renorm[1], mass_aware, eps)
    assert y.dtype == dtype and y.shape == (B, H, C)
    tol = FP32_TOL if dtype == torch.float32 else (BF16_TOL if dtype == torch.bfloat16 else dict(atol=1e-2, rtol=1e-2, max_err_rate=0.01, max_q99=1.5))
    assert_close_stats("y", y.float().cpu(), ref_y, **tol)
    assert_close_stats("slot", d_slot.cpu(), ref_slot, **FP32_TOL)
    assert_close_stats("mass", d_mass.cpu(), ref_mass, **FP32_TOL)
    if B > 1:  # masked batch row: state untouched bit-for-bit, y exactly zero
        assert torch.equal(d_slot[1].cpu(), slot[1]) and torch.equal(d_mass[1].cpu(), mass[1])
        assert float(y[1].float().abs().max()) == 0.0


@pytest.mark.parametrize("name", ["ram_decode_t1.npz", "ram_decode_t1_massaware.npz"])
def test_decode_step_matches_reference_golden(name):
    ops()
    z = load(name)
    B, H, U, P, T, Kw, Kr, C, E, ma = (int(v) for v in z["meta"])
    w, r = t(z["w_addr"])[:, 0], t(z["r_addr"])[:, 0]          # (B,H,U,P)
    x, g = t(z["values"])[:, 0], t(z["gamma"])[:, 0]
    slot, mass = t(z["init_slot"]).cuda(), t(z["init_mass"]).cuda()
    rn = [float(v) for v in z["renorm"]]
    y = torch.ops.ramnet_ops.topk_autoregressive_(w.cuda(), r.cuda(), x.cuda(), g.cuda(), slot, mass,
                                                  torch.empty(0, dtype=torch.bool, device="cuda"), E,
                                                  t(z["pos"])[:, 0].cuda().int(), Kw, Kr, rn[0], rn[1], bool(ma), float(z["eps"]))
    assert_close_stats("y", y.cpu(), t(z["out_y"])[:, 0], **FP32_TOL)
    assert_close_stats("slot", slot.cpu(), t(z["out_slot"]), **FP32_TOL)
    assert_close_stats("mass", mass.cpu(), t(z["out_mass"]), **FP32_TOL)


def test_fused_epilogue_matches_oracle():
    ops()
    for (B, H, U, P, C, K), dtype in (((2, 4, 2, 16, 64, (4, 4)), torch.float32), ((2, 4, 2, 16, 64, (4, 4)), torch.bfloat16),
                                     ((2, 4, 2, 64, 128, (16, 16)), torch.bfloat16), ((1, 3, 2, 16, 128, (4, 4)), torch.float32)):
        w, r, x, g, slot, mass, pos = _inputs(B, H, U, P, C, dtype, 10)
        nw = randn((C,), 20) * 0.1 + 1.0
        gate = randn((B, H, C), 21, dtype)
        eps_n = float(torch.finfo(dtype).eps)
        ref_y, ref_slot, _ = orc.decode_step(w.float(), r.float(), x.float(), g.float(), slot.clone(), mass.clone(), None,
                                             2, pos, K, (0.0, 0.0), False, 1e-12)
        ref = orc.head_rmsnorm_gate(ref_y, nw, gate.float(), eps_n)
        d_slot, d_mass = slot.clone().cuda(), mass.clone().cuda()
        y = torch.ops.ramnet_ops.decode_fused_(w.cuda(), r.cuda(), x.cuda(), g.cuda(), d_slot, d_mass,
                                               torch.empty(0, dtype=torch.bool, device="cuda"), 2, pos.cuda().int(),
                                               K[0], K[1], 0.0, 0.0, False, 1e-12, nw.cuda(), gate.cuda(), eps_n)
        tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
        assert_close_stats("y", y.float().cpu(), ref, **tol)
        assert_close_stats("slot", d_slot.cpu(), ref_slot, **FP32_TOL)


def test_state_beyond_int32_offsets_is_rejected_or_supported_by_shape_checks():
    ops()
    x = torch.zeros(1, 1, 8, device="cuda")
    with pytest.raises(RuntimeError, match="state shape mismatch"):
        torch.ops.ramnet_ops.topk_autoregressive_(torch.zeros(1, 1, 2, 4, device="cuda"), torch.zeros(1, 1, 2, 4, device="cuda"),
                                                  x, torch.zeros(1, 1, device="cuda"), torch.zeros(1, 1, 15, 8, device="cuda"),
                                                  torch.zeros(1, 1, 15, device="cuda"), torch.empty(0, dtype=torch.bool, device="cuda"),
                                                  0, torch.zeros(1, dtype=torch.int32, device="cuda"), 2, 2, 0.0, 0.0, False, 1e-6)


@pytest.mark.parametrize("B,H,U,P,C,K,dtype", [
    (3, 7, 2, 64, 128, (16, 16), torch.bfloat16),   # scales applied inside the one-warp-per-pair kernel
    (2, 4, 2, 64, 256, (16, 16), torch.float16),
    (2, 4, 3, 8, 32, (8, 8), torch.bfloat16),        # no kernel support for this shape: the operator multiplies first
    (2, 4, 2, 16, 64, (4, 4), torch.float32),
])
def test_logit_scales_equal_a_multiply_beforehand(B, H, U, P, C, K, dtype):
    """decode_fused_ with (H,U) logit scales == the same step on logits multiplied beforehand in the logits'
    dtype (what the attention layer does with its learned scale over the temperature): same bits."""
    ops()
    w, r, x, g, slot, mass, pos = _inputs(B, H, U, P, C, dtype, 40)
    ws = (torch.rand(H, U, generator=torch.Generator().manual_seed(50)) * 1.5 + 0.25).to(dtype)
    rs = (torch.rand(H, U, generator=torch.Generator().manual_seed(51)) * 1.5 + 0.25).to(dtype)
    nomask = torch.empty(0, dtype=torch.bool, device="cuda")
    results = []
    for fold in (True, False):
        s, m = slot.clone().cuda(), mass.clone().cuda()
        wl, rl = w.cuda(), r.cuda()
        if not fold:
            wl, rl = ws.cuda().unsqueeze(-1) * wl, rs.cuda().unsqueeze(-1) * rl
        y = torch.ops.ramnet_ops.decode_fused_(wl, rl, x.cuda(), g.cuda(), s, m, nomask, H // 2, pos.cuda(), K[0], K[1],
                                               0.0, 0.5, False, 1e-6, None, None, 0.0,
                                               ws.cuda() if fold else None, rs.cuda().unsqueeze(-1) if fold else None)
        results.append((y.cpu(), s.cpu(), m.cpu()))
    for name, a, b in zip(("y", "slot", "mass"), results[0], results[1]):
        assert torch.equal(a, b), f"{name}: {int((a != b).sum())} elements differ"


@pytest.mark.parametrize("B,H,U,P,C,K,dtype", [
    (3, 7, 2, 64, 128, (16, 16), torch.bfloat16),   # one warp per pair
    (2, 4, 3, 32, 128, (8, 8), torch.float16),       # sixteen pairs per CTA
    (2, 3, 2, 6, 10, (3, 5), torch.float32),         # general kernel
])
def test_inputs_may_be_column_slices_of_one_projection_output(B, H, U, P, C, K, dtype):
    """The logits, values, gamma and gate logits of a step taken as column slices of ONE (B, N) matrix (the layer's
    projections merged into one GEMM) give the same bits as contiguous copies of them."""
    ops()
    w, r, x, g, slot, mass, pos = _inputs(B, H, U, P, C, dtype, 60)
    gate = randn((B, H, C), 66, dtype)
    n = H * U * P
    width = 8 + 2 * n + 2 * H * C + H
    width += (-width) % 8 + 8              # rows a multiple of 16 bytes apart, so that the same kernel takes both forms
    wide = torch.zeros(B, width, dtype=dtype)
    cols = [(w, n), (r, n), (x, H * C), (gate, H * C), (g, H)]
    off, views = 8, []                      # a leading pad: the slices do not start at the matrix's first column
    for tns, width in cols:
        wide[:, off:off + width] = tns.reshape(B, width)
        views.append((off, width))
        off += width
    wide = wide.cuda()
    shapes = [(B, H, U, P), (B, H, U, P), (B, H, C), (B, H, C), (B, H)]
    nomask = torch.empty(0, dtype=torch.bool, device="cuda")
    norm_w = (torch.rand(C, generator=torch.Generator().manual_seed(67)) + 0.5).cuda()
    results = []
    for sliced in (True, False):
        ins = [wide[:, o:o + wd].view(shp) for (o, wd), shp in zip(views, shapes)]
        if not sliced:
            ins = [v.contiguous() for v in ins]
        else:
            assert not ins[0].is_contiguous()
        s, m = slot.clone().cuda(), mass.clone().cuda()
        y = torch.ops.ramnet_ops.decode_fused_(ins[0], ins[1], ins[2], ins[4], s, m, nomask, H // 2, pos.cuda(), K[0], K[1],
                                               0.0, 0.0, False, 1e-6, norm_w, ins[3], 1e-6)
        results.append((y.cpu(), s.cpu(), m.cpu()))
    for name, a, b in zip(("y", "slot", "mass"), results[0], results[1]):
        assert torch.equal(a, b), f"{name}: {int((a != b).sum())} elements differ"
