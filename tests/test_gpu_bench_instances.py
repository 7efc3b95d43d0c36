"""GPU parity on the kernel instances the benchmark times.

The launch plan of the prefill path depends on B*H*C (how many channel slices fill the GPU), not on T,
and the decode kernel's warps only take a second and third (b,h) pair when there are more pairs than
resident warps.  The small cases of the other test files therefore run other template instances than
the benchmark shapes.  Here the shapes keep the benchmark's B, H, U, P, K, C (so the plan is the same,
which is asserted) with a short T, and the oracle checks seeded (b,h) slices: every (b,h) is independent.
"""
import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.gpu_common import ops, randn
from tests.helpers import BF16_TOL, FP32_TOL, assert_close_stats

pytestmark = pytest.mark.gpu

GRAD_TOL_BF16 = dict(atol=7.5e-2, rtol=7.5e-2, max_err_rate=0.02, max_q99=2.0)
BENCH_PREFILL = dict(B=8, H=16, T=16384, U=2, P=64, K=16, C=128, E=8)
PAIRS = [(0, 0), (3, 7), (5, 8), (7, 15)]  # (b, h): CAPE heads (h < 8) and content-only heads


def test_prefill_forward_and_backward_on_the_benchmarked_plan():
    C_ = ops()
    import ramnet_ops
    s = BENCH_PREFILL
    B, H, U, P, K, C, E = s["B"], s["H"], s["U"], s["P"], s["K"], s["C"], s["E"]
    T, A = 256, P ** U
    for reverse in (False, True):
        assert C_.gsu_plan_info(B, H, T, A, C, K, K, reverse) == C_.gsu_plan_info(B, H, s["T"], A, C, K, K, reverse), \
            "the test shape must select the kernels the benchmark shape selects"
    dt = torch.bfloat16
    w, r = randn((B, T, H, U, P), 11, dt), randn((B, T, H, U, P), 12, dt)
    x = randn((B, T, H, C), 13, dt)
    g = torch.sigmoid(randn((B, T, H), 14) + 1.0).to(dt)
    slot = randn((B, H, A, C), 15) * 0.1
    mass = torch.rand(B, H, A, generator=torch.Generator().manual_seed(16)) + 0.1
    d_y, d_slot, d_mass = randn((B, T, H, C), 17, dt), randn((B, H, A, C), 18), randn((B, H, A), 19)
    pos = torch.arange(T).view(1, T).expand(B, T).contiguous()

    leaves = [v.cuda().requires_grad_(True) for v in (w, r, x, g, slot, mass)]
    y, (s1, m1) = ramnet_ops.random_access_memory_attention(leaves[0], leaves[1], leaves[2], leaves[3], (leaves[4], leaves[5]),
                                                            embed_num=E, position_ids=pos.cuda(), top_k=K, impl_backend="cuda")
    grads = torch.autograd.grad((y, s1, m1), leaves, (d_y.cuda(), d_slot.cuda(), d_mass.cuda()))
    # run-to-run reproducibility of the forward (fixed reduction orders)
    y2, (s2, m2) = ramnet_ops.random_access_memory_attention(leaves[0], leaves[1], leaves[2], leaves[3], (leaves[4], leaves[5]),
                                                             embed_num=E, position_ids=pos.cuda(), top_k=K, impl_backend="cuda")
    assert torch.equal(y, y2) and torch.equal(s1, s2) and torch.equal(m1, m2)
    y, s1, m1 = y.detach().cpu(), s1.detach().cpu(), m1.detach().cpu()
    grads = [gr.float().cpu() for gr in grads]

    # the oracle runs the sampled pairs as batch rows of a one-head call: CAPE heads and content-only heads apart
    for e1, pairs in ((1, [q_ for q_ in PAIRS if q_[1] < E]), (0, [q_ for q_ in PAIRS if q_[1] >= E])):
        def take(tn):  # (B,T,H,...) or (B,H,...) -> rows of the sampled pairs, one head
            return torch.cat([tn[b:b + 1, :, h:h + 1] if tn.shape[1] == T else tn[b:b + 1, h:h + 1] for b, h in pairs])
        (ry, rs, rm), ref = orc.ram_attn_grads(
            take(w).float().permute(0, 2, 3, 4, 1), take(r).float().permute(0, 2, 3, 4, 1), take(x).float().permute(0, 2, 1, 3),
            take(g).float().permute(0, 2, 1), take(slot), take(mass), None, e1, pos[:len(pairs)], (K, K), (0.0, 0.0), False,
            1e-12, take(d_y).float().permute(0, 2, 1, 3), take(d_slot), take(d_mass))
        tag = f"(pairs {pairs})"
        assert_close_stats("y" + tag, take(y).float(), ry.permute(0, 2, 1, 3), **BF16_TOL)
        assert_close_stats("slot" + tag, take(s1), rs, **FP32_TOL)
        assert_close_stats("mass" + tag, take(m1), rm, **FP32_TOL)
        want = [ref[0].permute(0, 4, 1, 2, 3), ref[1].permute(0, 4, 1, 2, 3), ref[2].permute(0, 2, 1, 3),
                ref[3].permute(0, 2, 1), ref[4], ref[5]]
        for n, a_, b_ in zip(("D_w", "D_r", "D_x", "D_gamma", "D_slot", "D_mass"), [take(gr) for gr in grads], want):
            assert_close_stats(n + tag, a_, b_, **GRAD_TOL_BF16)


def test_address_decode_config2_slice_is_bit_exact():
    """B8 H16 U3 P32 K8 bf16 with CAPE on half the heads (the address-only benchmark shape) on a T-slice:
    indices bit-exact against the dense canonical Top-K on seeded (b,h) pairs."""
    ops()
    B, H, U, P, T, K, E = 8, 16, 3, 32, 64, 8, 8
    A = P ** U
    q, k = randn((B, T, H, U, P), 31, torch.bfloat16, 1.5), randn((B, T, H, U, P), 32, torch.bfloat16, 1.5)
    pos = (torch.arange(T).view(1, T) + 8128).expand(B, T).contiguous()   # late positions of a T=8192 sequence
    wv, rv = k.permute(0, 2, 3, 4, 1), q.permute(0, 2, 3, 4, 1)
    idx, val = torch.ops.ramnet_ops.topk_addr_forward(wv.cuda(), rv.cuda(), E, A, pos.cuda().int(), K, K, 0.0, 0.0)
    idx, val = idx.cpu(), val.cpu()
    for b, h in PAIRS:
        e1 = 1 if h < E else 0
        for view, lo, sign in ((wv, 0, 1.0), (rv, K, -1.0)):
            ri, rv_ = orc.topk_addr(view[b:b + 1, h:h + 1].float(), e1, pos[b:b + 1], K, 0.0, False, False)
            got = idx[b, h, lo:lo + K] - (b * H + h) * A
            assert torch.equal(got, ri[0, 0]), f"(b={b},h={h}) {int((got != ri[0, 0]).sum())} indices differ"
            assert_close_stats("val", sign * val[b, h, lo:lo + K], rv_[0, 0], atol=1e-6, rtol=2e-5, max_err_rate=0.0)


def test_decode_when_warps_take_several_pairs():
    """More (b,h) pairs than resident warps of the pair kernel (2 CTAs x 8 warps per SM): every warp draws a
    second pair from its CTA's counter, reuses its row buffer, flips its barrier's parity and consumes the
    logits it requested one pair ahead.  Two consecutive steps on a 5.4 GB state, oracle on sampled batch rows
    (one of them masked)."""
    ops()
    props = torch.cuda.get_device_properties(0)
    B, H, U, P, K, C, E = 160, 16, 2, 64, 16, 128, 8
    A = P ** U
    assert B * H > 2 * props.multi_processor_count * 8, "not enough pairs for a second pair per warp on this GPU"
    if props.total_memory < 12 * 2 ** 30:
        pytest.skip("needs 6 GB of device memory for the state")
    gen = torch.Generator(device="cuda").manual_seed(5)
    slot = torch.empty(B, H, A, C, device="cuda")
    for b0 in range(0, B, 16):
        slot[b0:b0 + 16] = torch.randn(16, H, A, C, device="cuda", generator=gen) * 0.1
    mass = torch.rand(B, H, A, device="cuda", generator=gen) + 0.1
    rows = [0, 1, 77, 158, 159]
    mask = torch.ones(B, dtype=torch.bool)
    mask[1] = False
    ref_slot, ref_mass = slot[rows].cpu(), mass[rows].cpu()
    for step in range(2):
        w, r = randn((B, H, U, P), 40 + step, torch.bfloat16), randn((B, H, U, P), 50 + step, torch.bfloat16)
        x = randn((B, H, C), 60 + step, torch.bfloat16)
        g = torch.sigmoid(randn((B, H), 70 + step)).to(torch.bfloat16)
        pos = torch.arange(B) * 7 + 3 + step
        y = torch.ops.ramnet_ops.topk_autoregressive_(w.cuda(), r.cuda(), x.cuda(), g.cuda(), slot, mass, mask.cuda(), E,
                                                      pos.cuda().int(), K, K, 0.0, 0.0, False, 1e-12)
        ry, ref_slot, ref_mass = orc.decode_step(w[rows].float(), r[rows].float(), x[rows].float(), g[rows].float(), ref_slot,
                                                 ref_mass, mask[rows], E, pos[rows], (K, K), (0.0, 0.0), False, 1e-12)
        assert_close_stats(f"y step {step}", y[rows].float().cpu(), ry, **BF16_TOL)
        assert float(y[1].float().abs().max()) == 0.0
    assert_close_stats("slot", slot[rows].cpu(), ref_slot, **FP32_TOL)
    assert_close_stats("mass", mass[rows].cpu(), ref_mass, **FP32_TOL)
    del slot, mass
    torch.cuda.empty_cache()
