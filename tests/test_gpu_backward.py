"""GPU parity of the backward pass (address backward + prefill backward) through the public API,
against the reference's fp64 gradients (golden fixtures) and the CPU oracle's autograd."""
import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.gpu_common import ops, randn
from tests.helpers import FP32_TOL, assert_close_stats, load, t

pytestmark = pytest.mark.gpu

GRAD_TOL_BF16 = dict(atol=7.5e-2, rtol=7.5e-2, max_err_rate=0.02, max_q99=2.0)


def run_api(w, r, x, g, slot, mass, mask, pos, E, K, renorm, eps, d_y, d_slot, d_mass, dtype, mass_aware=False):
    """Public API on GPU with autograd; inputs in (B,T,H,...) layout on CPU."""
    import ramnet_ops
    leaves = [v.to(dtype).cuda().requires_grad_(True) for v in (w, r, x, g)] + \
             [v.float().cuda().requires_grad_(True) for v in (slot, mass)]
    y, (s1, m1) = ramnet_ops.random_access_memory_attention(
        leaves[0], leaves[1], leaves[2], leaves[3], (leaves[4], leaves[5]),
        mask=None if mask is None else mask.cuda(), embed_num=E, position_ids=pos.cuda(), top_k=K, top_k_re_norm=renorm,
        mass_aware=mass_aware, eps=eps, impl_backend="cuda")
    up = d_y.to(dtype).cuda()
    if mask is not None:
        up = up * mask.cuda()[:, :, None, None]
    grads = torch.autograd.grad((y, s1, m1), leaves, (up, d_slot.cuda(), d_mass.cuda()))
    return (y, s1, m1), [gr.float().cpu() for gr in grads]


def valid(gr, mask):
    return gr if mask is None else gr[mask]


@pytest.mark.parametrize("name", ["ram_grads_masked.npz", "ram_grads_plain.npz", "ram_grads_massaware.npz"])
def test_gradients_match_reference_golden(name):
    ops()
    z = load(name)
    B, H, U, P, T, Kw, Kr, C, E, ma = (int(v) for v in z["meta"])
    mask = t(z["mask"]) if z["mask"].size else None
    rn = tuple(float(v) for v in z["renorm"])
    _, grads = run_api(t(z["w_addr"]), t(z["r_addr"]), t(z["values"]), t(z["gamma"]), t(z["init_slot"]), t(z["init_mass"]),
                       mask, t(z["pos"]), E, (Kw, Kr), rn, float(z["eps"]), t(z["d_y"]), t(z["d_slot"]), t(z["d_mass"]),
                       torch.float32, mass_aware=bool(ma))
    names = ("D_w", "D_r", "D_x", "D_gamma", "D_slot", "D_mass")
    for n, got in zip(names, grads):
        ref = t(z["out64_" + n])
        if n in ("D_w", "D_r", "D_x", "D_gamma"):
            got, ref = valid(got, mask), valid(ref, mask)
        assert_close_stats(n, got, ref, **FP32_TOL)


@pytest.mark.parametrize("B,H,U,P,T,C,K,dtype,masked,ma", [
    (2, 4, 2, 16, 130, 32, (4, 4), torch.float32, False, False),
    (1, 2, 2, 64, 96, 128, (16, 16), torch.bfloat16, False, False),
    (2, 2, 3, 4, 70, 29, (8, 3), torch.float32, True, False),       # C not a multiple of 4: padded internally
    (1, 2, 2, 2, 90, 8, (2, 3), torch.float32, False, False),       # 4 slots: long chains inside a chunk
    (1, 2, 4, 4, 40, 16, (40, 24), torch.float32, True, False),
    (2, 4, 2, 16, 130, 32, (4, 4), torch.float32, True, True),
    (1, 2, 2, 2, 90, 8, (2, 3), torch.float32, False, True),
    (1, 2, 2, 64, 96, 128, (16, 16), torch.bfloat16, False, True),
])
def test_gradients_match_oracle_autograd(B, H, U, P, T, C, K, dtype, masked, ma):
    ops()
    A = P ** U
    w = randn((B, T, H, U, P), 1, dtype)
    r = randn((B, T, H, U, P), 2, dtype)
    x = randn((B, T, H, C), 3, dtype)
    g = (0.5 * randn((B, T, H), 4)).to(dtype)
    slot = randn((B, H, A, C), 5)
    mass = torch.rand(B, H, A, generator=torch.Generator().manual_seed(6)) + 0.1
    d_y, d_slot, d_mass = randn((B, T, H, C), 7), randn((B, H, A, C), 8), randn((B, H, A), 9)
    if masked:
        mask = torch.ones(B, T, dtype=torch.bool)
        mask[:, :5] = False
        mask[0, T // 2: T // 2 + 7] = False
        pos = ((mask.long().cumsum(-1) - 1) * 3 + 11).masked_fill(~mask, 0)
    else:
        mask, pos = None, torch.arange(T).view(1, T).expand(B, T).contiguous()
    E, renorm, eps = H // 2, (0.25, 0.75), 1e-6
    _, grads = run_api(w, r, x, g, slot, mass, mask, pos, E, K, renorm, eps, d_y, d_slot, d_mass, dtype, mass_aware=ma)
    up = d_y.to(dtype).float()
    if mask is not None:
        up = up * mask[:, :, None, None]
    _, ref = orc.ram_attn_grads(
        w.float().permute(0, 2, 3, 4, 1), r.float().permute(0, 2, 3, 4, 1), x.float().permute(0, 2, 1, 3),
        g.float().permute(0, 2, 1), slot, mass, mask, E, pos, K, renorm, ma, eps, up.permute(0, 2, 1, 3), d_slot, d_mass)
    ref = [ref[0].permute(0, 4, 1, 2, 3), ref[1].permute(0, 4, 1, 2, 3), ref[2].permute(0, 2, 1, 3), ref[3].permute(0, 2, 1),
           ref[4], ref[5]]
    tol = FP32_TOL if dtype == torch.float32 else GRAD_TOL_BF16
    for n, got, want in zip(("D_w", "D_r", "D_x", "D_gamma", "D_slot", "D_mass"), grads, ref):
        if n in ("D_w", "D_r", "D_x", "D_gamma"):
            got, want = valid(got, mask), valid(want, mask)
        assert_close_stats(n, got, want, **(FP32_TOL if n in ("D_slot", "D_mass") and dtype == torch.float32 else tol))


def test_all_masked_gradients_are_identity():
    """No token takes part: state copied bit-exact, y zero, input gradients zero, state gradients pass through
    (the contract of the reference's tests/ops/test_cuda_registration.py:107-135)."""
    ops()
    import ramnet_ops
    B, T, H, U, P, C = 2, 32, 2, 2, 4, 7
    g = torch.Generator().manual_seed(3)
    leaves = [torch.randn(B, T, H, U, P, generator=g).cuda().requires_grad_(True) for _ in range(2)]
    leaves += [torch.randn(B, T, H, C, generator=g).cuda().requires_grad_(True), (0.2 * torch.randn(B, T, H, generator=g)).cuda().requires_grad_(True)]
    leaves += [torch.randn(B, H, 16, C, generator=g).cuda().requires_grad_(True), (torch.rand(B, H, 16, generator=g) + 0.1).cuda().requires_grad_(True)]
    mask = torch.zeros(B, T, dtype=torch.bool, device="cuda")
    y, (s1, m1) = ramnet_ops.random_access_memory_attention(leaves[0], leaves[1], leaves[2], leaves[3], (leaves[4], leaves[5]),
                                                            mask=mask, embed_num=1, top_k=(2, 3), top_k_re_norm=(0.25, 0.75),
                                                            mass_aware=True, eps=1e-6, impl_backend="cuda")
    assert float(y.abs().max()) == 0.0
    assert torch.equal(s1, leaves[4]) and torch.equal(m1, leaves[5]) and s1.data_ptr() != leaves[4].data_ptr()
    grads = torch.autograd.grad(s1.sum() + m1.sum(), leaves)
    for gr in grads[:4]:
        assert float(gr.abs().max()) == 0.0
    for gr in grads[4:]:
        assert torch.equal(gr, torch.ones_like(gr))


def test_gradients_are_bitwise_reproducible():
    """No float atomics on the backward path: two runs on the same inputs give the same bits (the model shape in
    bf16, chunks with chains, two batch rows, CAPE on half of the heads)."""
    ops()
    B, H, U, P, T, C, K = 2, 4, 2, 64, 200, 128, (16, 16)
    w = randn((B, T, H, U, P), 21, torch.float32, 1.5)
    r = randn((B, T, H, U, P), 22, torch.float32, 1.5)
    x = randn((B, T, H, C), 23)
    g = torch.sigmoid(randn((B, T, H), 24))
    A = P ** U
    slot, mass = randn((B, H, A, C), 25) * 0.1, torch.rand(B, H, A, generator=torch.Generator().manual_seed(26)) * 0.5
    pos = torch.arange(T).view(1, T).expand(B, T).contiguous()
    d_y, d_slot, d_mass = randn((B, T, H, C), 27), randn((B, H, A, C), 28) * 0.1, randn((B, H, A), 29) * 0.1
    runs = [run_api(w, r, x, g, slot, mass, None, pos, H // 2, K, (0.0, 0.0), 1e-6, d_y, d_slot, d_mass, torch.bfloat16)
            for _ in range(2)]
    for a, b in zip(runs[0][0], runs[1][0]):
        assert torch.equal(a, b)
    for name, a, b in zip(("D_w", "D_r", "D_x", "D_gamma", "D_slot", "D_mass"), runs[0][1], runs[1][1]):
        assert torch.equal(a, b), f"{name}: {int((a != b).sum())} elements differ between two runs"
