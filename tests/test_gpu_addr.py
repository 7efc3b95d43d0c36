"""GPU parity of the address decoder (forward bit-exact on indices, weights and gradients within
the fp32 budget) against the CPU oracle, through torch.ops.ramnet_ops -> C ABI."""
import itertools

import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.gpu_common import ops, randn
from tests.helpers import FP32_TOL, assert_close_stats, load, t

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, H, U, P, T, K, E, dtype, std
    (2, 4, 2, 16, 33, 4, 2, torch.float32, 1.0),
    (1, 4, 3, 8, 20, 8, 2, torch.float32, 1.0),
    (1, 2, 2, 64, 24, 16, 1, torch.bfloat16, 1.0),
    (1, 2, 3, 32, 12, 8, 1, torch.bfloat16, 1.5),
    (2, 2, 4, 4, 9, 16, 1, torch.float16, 1.0),
    (1, 3, 5, 4, 7, 32, 2, torch.float32, 1.0),
    (1, 2, 4, 7, 5, 128, 1, torch.float32, 1.0),
    (1, 2, 2, 3, 6, 9, 1, torch.float32, 1.0),
    (1, 2, 1, 40, 6, 5, 1, torch.float32, 1.0),
    (1, 1, 2, 100, 4, 64, 0, torch.bfloat16, 2.0),
    (2, 4, 5, 8, 40, 8, 2, torch.bfloat16, 1.5),     # 32768 slots at radix 8: thread-per-row kernel
    (1, 2, 5, 8, 20, 8, 1, torch.float32, 1.0),
    (2, 4, 4, 8, 40, 16, 2, torch.bfloat16, 1.5),    # K above the radix: 8 logits per digit, beam of 16
    (1, 2, 4, 8, 20, 16, 1, torch.float32, 1.0),
    (1, 2, 4, 8, 20, 16, 1, torch.float16, 3.0),
]


def _case(B, H, U, P, T, K, E, dtype, std, seed=0):
    addr = randn((B, T, H, U, P), seed, dtype, std)  # native layout
    pos = (torch.arange(T).view(1, T) * 3 + 11 + torch.arange(B).view(B, 1)).to(torch.int64)
    return addr, pos


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("renorm,neg,enc", [(0.0, False, True), (0.5, True, False), (1.0, False, True)])
def test_single_decode_matches_oracle(shape, renorm, neg, enc):
    ops()
    B, H, U, P, T, K, E, dtype, std = shape
    addr, pos = _case(*shape)
    view = addr.permute(0, 2, 3, 4, 1)  # (B,H,U,P,T), non-contiguous like the public API hands over
    idx, val = torch.ops.ramnet_ops.topk_addr_single_forward(view.cuda(), E, P ** U, pos.cuda(), K, renorm, neg, enc)
    ref_idx, ref_val = orc.topk_addr(view.float(), E, pos, K, renorm, neg, enc)
    assert idx.shape == (B, H, K, T) and idx.dtype == torch.int32 and val.dtype == torch.float32
    assert torch.equal(idx.cpu(), ref_idx), f"{int((idx.cpu() != ref_idx).sum())} indices differ"
    assert_close_stats("val", val.cpu(), ref_val, atol=1e-6, rtol=2e-5, max_err_rate=0.0)


@pytest.mark.parametrize("name", ["addr_u2p16k4_f32.npz", "addr_u3p8k8_f32_renorm.npz", "addr_u2p64k16_bf16.npz",
                                  "addr_u3p32k8_bf16.npz", "addr_u4p4k16_special.npz", "addr_u2p3kall_f32.npz"])
def test_single_decode_matches_reference_golden(name):
    ops()
    z = load(name)
    B, H, U, P, T, K, E, neg, enc = (int(v) for v in z["meta"])
    addr, pos = t(z["addr"]), t(z["pos"])
    idx, val = torch.ops.ramnet_ops.topk_addr_single_forward(addr.cuda(), E, P ** U, pos.cuda(), K, float(z["renorm"]),
                                                             bool(neg), bool(enc))
    idx, val = idx.cpu(), val.cpu()
    ref_idx, ref_val = t(z["idx"]), t(z["val"])
    torch.testing.assert_close(val.abs().sort(dim=2).values, ref_val.abs().sort(dim=2).values, atol=1e-6, rtol=2e-5)
    clear = t(z["gap"]) > 1e-5
    same = (idx.sort(dim=2).values == ref_idx.sort(dim=2).values).all(dim=2)
    assert bool(same[clear].all())
    o_idx, o_val = orc.topk_addr(addr, E, pos, K, float(z["renorm"]), bool(neg), bool(enc))
    assert torch.equal(idx, o_idx)


def test_joined_decode_layout_sign_and_ties():
    ops()
    B, H, U, P, T, Kw, Kr, E = 2, 4, 2, 16, 40, 4, 6, 2
    # bf16-representable logits on a coarse grid: many exact ties inside and at the Top-K boundary
    g = torch.Generator().manual_seed(3)
    q = (torch.randint(-4, 5, (B, T, H, U, P), generator=g).float() * 0.5)
    k = (torch.randint(-2, 3, (B, T, H, U, P), generator=g).float() * 0.25)
    pos = torch.arange(T).view(1, T).expand(B, T).contiguous()
    wv, rv = k.permute(0, 2, 3, 4, 1), q.permute(0, 2, 3, 4, 1)
    idx, val = torch.ops.ramnet_ops.topk_addr_forward(wv.cuda().bfloat16(), rv.cuda().bfloat16(), E, P ** U,
                                                      pos.cuda().int(), Kw, Kr, 0.0, 1.0)
    assert idx.shape == (B, H, Kw + Kr, T)
    wi, ww = orc.topk_addr(wv, E, pos, Kw, 0.0)
    ri, rw = orc.topk_addr(rv, E, pos, Kr, 1.0, addr_val_neg=True)
    assert torch.equal(idx[:, :, :Kw].cpu(), wi) and torch.equal(idx[:, :, Kw:].cpu(), ri)
    assert_close_stats("w", val[:, :, :Kw].cpu(), ww, atol=1e-6, rtol=2e-5, max_err_rate=0.0)
    assert_close_stats("r", val[:, :, Kw:].cpu(), rw, atol=1e-6, rtol=2e-5, max_err_rate=0.0)
    assert bool((val[:, :, Kw:] <= 0).all()) and bool((val[:, :, :Kw] >= 0).all())


def test_inactive_and_extreme_logits():
    ops()
    B, H, U, P, T, K = 2, 2, 2, 4, 6, 5
    addr = randn((B, H, U, P, T), 5)
    addr[..., 0] = -torch.inf
    addr[:, :, 0, :, 1] = -torch.inf
    addr[..., 2] = torch.tensor([-1000.0, 998.0, 999.0, 1000.0]).view(1, 1, 1, 4)
    addr[:, :, :, :2, 3] = -torch.inf
    pos = torch.arange(T).view(1, T).expand(B, T).contiguous()
    for renorm in (0.0, 0.5, 1.0):
        idx, val = torch.ops.ramnet_ops.topk_addr_single_forward(addr.cuda(), 1, P ** U, pos.cuda(), K, renorm)
        ref_idx, ref_val = orc.topk_addr(addr, 1, pos, K, renorm)
        assert torch.isfinite(val).all()
        assert float(val[..., :2].abs().max()) == 0.0
        assert torch.equal(idx.cpu(), ref_idx)
        # logits of magnitude 1000 cancel against their log-sum-exp: fp32 budget of the reference tests
        assert_close_stats("val", val.cpu(), ref_val, **FP32_TOL)


@pytest.mark.parametrize("shape", SHAPES[:6] + SHAPES[10:])
@pytest.mark.parametrize("renorm", [0.0, 0.5, 1.0])
@pytest.mark.parametrize("token_major", [False, True])
def test_backward_matches_oracle_autograd(shape, renorm, token_major):
    """token_major: the gradient of the weights laid out like the weights themselves (K entries of a
    token-head contiguous), which is what the prefill backward hands over and what the specialised
    backward kernel takes; otherwise (B,H,K,T)-contiguous, which only the general kernel takes."""
    ops()
    B, H, U, P, T, K, E, dtype, std = shape
    addr, pos = _case(*shape, seed=1)
    if token_major:
        addr[0, 1] = float("-inf")           # an inactive token: zero gradient
    view = addr.permute(0, 2, 3, 4, 1)
    dev = view.cuda()
    idx, val = torch.ops.ramnet_ops.topk_addr_single_forward(dev, E, P ** U, pos.cuda(), K, renorm, False, True)
    d_val = randn((B, T, H, K), 2).permute(0, 2, 3, 1) if token_major else randn((B, H, K, T), 2)
    got = torch.ops.ramnet_ops.topk_addr_single_backward(idx, val, dev, d_val.cuda(), E, pos.cuda(), K, renorm, False,
                                                         [B, H, U, P, P ** U, T], dtype)
    assert got.shape == view.shape and got.dtype == dtype
    # oracle: autograd through the weights at the selected content addresses
    A = P ** U
    caped = (torch.arange(H).view(1, H, 1, 1) < E).long()
    local = idx.cpu().long() % A
    content = ((local + caped * pos[:, None, None, :]) % A).permute(0, 1, 3, 2)
    leaf = view.float().double().requires_grad_(True)
    w = orc._weights_from_logits(leaf, content, renorm)
    ref, = torch.autograd.grad(w, leaf, d_val.double())
    tol = FP32_TOL if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2, max_err_rate=0.01, max_q99=1.5)
    assert_close_stats("D_addr", got.float().cpu(), ref, **tol)


def test_errors_are_runtime_errors():
    ops()
    addr = torch.zeros(1, 1, 2, 200, 4, device="cuda")
    pos = torch.zeros(1, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="P <= 128"):
        torch.ops.ramnet_ops.topk_addr_single_forward(addr, 0, 40000, pos, 4, 0.0)
    with pytest.raises(RuntimeError, match="re_norm"):
        torch.ops.ramnet_ops.topk_addr_single_forward(addr[:, :, :, :4], 0, 16, pos, 4, 1.5)


@pytest.mark.parametrize("U,P,K,dtype", [(2, 64, 16, torch.bfloat16), (3, 32, 8, torch.bfloat16), (2, 16, 4, torch.float32),
                                         (2, 64, 16, torch.float16), (3, 32, 8, torch.float32), (2, 64, 16, torch.float32),
                                         (5, 8, 8, torch.bfloat16), (4, 8, 16, torch.bfloat16), (4, 8, 16, torch.float32)])
def test_specialised_and_general_kernels_agree(U, P, K, dtype):
    """The thread-per-row kernel (contiguous U*P blocks) and the warp-cooperative kernel (any
    strides) implement the same total order: identical indices, weights equal to rounding.
    Coarse logits force many exact ties, inside the Top-K and at its boundary."""
    ops()
    B, T, H, E = 2, 257, 4, 2
    g = torch.Generator().manual_seed(11)
    fine = torch.randn(B, T, H, U, P, generator=g)
    coarse = torch.randint(-6, 7, (B, T, H, U, P), generator=g).float() * 0.25
    pos = (torch.arange(T).view(1, T) * 5 + 3).expand(B, T).contiguous()
    for logits, renorm in ((fine, 0.0), (coarse, 0.5)):
        logits = logits.to(dtype)
        logits[0, 3] = float("-inf")                      # inactive token
        logits[1, 5, :, :, : P - 2] = float("-inf")      # fewer finite addresses than K
        dense = logits.cuda()
        padded = torch.zeros(B, T, H, U, P + 8, dtype=dtype, device="cuda")
        padded[..., :P] = dense
        strided = padded[..., :P]                          # digit stride P + 8: not the specialised layout
        a = torch.ops.ramnet_ops.topk_addr_forward(dense.permute(0, 2, 3, 4, 1), dense.flip(1).permute(0, 2, 3, 4, 1),
                                                   E, P ** U, pos.cuda().int(), K, K, renorm, renorm)
        b = torch.ops.ramnet_ops.topk_addr_forward(
            strided.permute(0, 2, 3, 4, 1), torch.flip(padded, dims=[1])[..., :P].permute(0, 2, 3, 4, 1),
            E, P ** U, pos.cuda().int(), K, K, renorm, renorm)
        assert torch.equal(a[0], b[0]), f"{int((a[0] != b[0]).sum())} indices differ"
        assert_close_stats("val", a[1].cpu(), b[1].cpu(), atol=1e-6, rtol=2e-5, max_err_rate=0.0)
        ref_idx, ref_val = orc.topk_addr(logits.float().permute(0, 2, 3, 4, 1), E, pos, K, renorm)
        assert torch.equal(a[0][:, :, :K].cpu(), ref_idx)
        assert_close_stats("val", a[1][:, :, :K].cpu(), ref_val, atol=1e-6, rtol=2e-5, max_err_rate=0.0)
