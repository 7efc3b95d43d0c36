"""GPU parity of the prefill path (address decode -> schedule -> apply) against the CPU oracle and
the reference golden vectors, through torch.ops.ramnet_ops -> C ABI."""
import pytest
import torch

from oracle import ramnet_oracle as orc
from tests.gpu_common import ops, randn
from tests.helpers import BF16_TOL, FP16_TOL, FP32_TOL, assert_close_stats, load, t

pytestmark = pytest.mark.gpu


def run_gpu(w, r, x, g, slot, mass, mask, E, pos, K, renorm, mass_aware, eps, inplace=False):
    """w/r (B,H,U,P,T), x (B,H,T,C), g (B,H,T) on CPU -> GPU forward; returns CPU tensors."""
    ops()
    P, U = w.shape[3], w.shape[2]
    dev = "cuda"
    idx, val = torch.ops.ramnet_ops.topk_addr_forward(w.to(dev), r.to(dev), E, P ** U, pos.to(dev).int(), K[0], K[1],
                                                      renorm[0], renorm[1])
    m = None if mask is None else mask.to(dev)
    if inplace:
        s, ms = slot.clone().to(dev), mass.clone().to(dev)
        y = torch.ops.ramnet_ops.gsu_forward_(idx, val, x.to(dev), g.to(dev), s, ms, m, K[0], K[1], mass_aware, eps)
    else:
        y, s, ms = torch.ops.ramnet_ops.gsu_forward(idx, val, x.to(dev), g.to(dev), slot.to(dev), mass.to(dev), m,
                                                    K[0], K[1], mass_aware, eps)
    torch.cuda.synchronize()
    return y.cpu(), s.cpu(), ms.cpu()


def make_case(B, H, U, P, T, C, dtype, seed, zero_state=False, masked=False):
    A = P ** U
    w = randn((B, T, H, U, P), seed, dtype).permute(0, 2, 3, 4, 1)
    r = randn((B, T, H, U, P), seed + 1, dtype).permute(0, 2, 3, 4, 1)
    x = randn((B, T, H, C), seed + 2, dtype).permute(0, 2, 1, 3)
    g = (0.5 * randn((B, T, H), seed + 3)).to(dtype).permute(0, 2, 1)
    if zero_state:
        slot, mass = torch.zeros(B, H, A, C), torch.full((B, H, A), 1.0 / A)
    else:
        slot = randn((B, H, A, C), seed + 4)
        mass = torch.rand(B, H, A, generator=torch.Generator().manual_seed(seed + 5)) + 0.1
    if masked:
        mask = torch.ones(B, T, dtype=torch.bool)
        mask[:, : max(1, T // 8)] = False
        mask[0, T // 2: T // 2 + 3] = False
        mask[:, -2:] = False
        pos = ((mask.long().cumsum(-1) - 1) * 3 + 11).masked_fill(~mask, 0)
    else:
        mask, pos = None, torch.arange(T).view(1, T).expand(B, T).contiguous()
    return w, r, x, g, slot, mass, mask, pos


def check(name, got, ref, mask, dtype):
    y, s, m = got
    ry, rs, rm = ref
    tol = {torch.float32: FP32_TOL, torch.bfloat16: BF16_TOL, torch.float16: FP16_TOL}[dtype]
    if mask is not None:
        assert float(y.float().permute(0, 2, 1, 3)[~mask].abs().max()) == 0.0
        y, ry = y.permute(0, 2, 1, 3)[mask], ry.permute(0, 2, 1, 3)[mask]
    assert_close_stats(name + ".y", y.float(), ry.float(), **tol)
    assert_close_stats(name + ".slot", s, rs, **FP32_TOL)
    assert_close_stats(name + ".mass", m, rm, **FP32_TOL)


CASES = [
    # B, H, U, P, T, C, K, dtype, masked, mass_aware
    (1, 4, 2, 16, 130, 64, (4, 4), torch.float32, False, False),
    (2, 3, 2, 6, 40, 10, (3, 5), torch.float32, True, False),
    (2, 3, 2, 6, 40, 10, (3, 5), torch.float32, True, True),
    (1, 2, 3, 4, 33, 7, (8, 8), torch.float32, False, False),
    (2, 2, 2, 64, 96, 128, (16, 16), torch.bfloat16, False, False),
    (1, 2, 2, 2, 150, 5, (2, 3), torch.float32, False, True),      # 4 slots: long same-slot chains
    (1, 2, 2, 2, 150, 8, (2, 3), torch.float32, False, True),      # the same through the specialised apply kernel
    (2, 2, 2, 4, 200, 16, (4, 4), torch.float32, True, False),     # 16 slots, masked tokens inside the chains
    (1, 2, 4, 3, 65, 29, (4, 12), torch.float16, True, False),
    (1, 2, 5, 4, 70, 32, (128, 128), torch.float32, False, False),  # chunk length 16
    (1, 2, 3, 32, 40, 16, (8, 8), torch.bfloat16, False, True),     # A = 32768: slot state stays in global memory
    (1, 1, 2, 128, 20, 8, (5, 7), torch.float32, False, False),     # A = 16384
    (1, 2, 4, 7, 64, 65, (8, 8), torch.float32, True, True),
    (1, 2, 2, 128, 20, 48, (4, 4), torch.float32, False, False),    # A = 16384, state in global memory, last channel slice partial
    (1, 1, 2, 128, 20, 24, (4, 4), torch.float32, True, False),
    (1, 1, 2, 128, 20, 12, (4, 4), torch.float32, False, True),
    (1, 2, 3, 48, 40, 4, (4, 4), torch.float32, False, False),      # A = 110592 > 65536: wide records (separate slot array)
    (1, 1, 2, 300 // 3, 30, 8, (3, 5), torch.bfloat16, True, False),
]


@pytest.mark.parametrize("case", CASES)
def test_prefill_matches_oracle(case):
    B, H, U, P, T, C, K, dtype, masked, ma = case
    w, r, x, g, slot, mass, mask, pos = make_case(B, H, U, P, T, C, dtype, 3, masked=masked)
    renorm, eps, E = (0.25, 0.75), 1e-6, H // 2
    got = run_gpu(w, r, x, g, slot, mass, mask, E, pos, K, renorm, ma, eps)
    ref = orc.ram_attn(w.float(), r.float(), x.float(), g.float(), slot, mass, mask, E, pos, K, renorm, ma, eps)
    check("prefill", got, ref, mask, dtype)
    assert got[0].dtype == dtype


# shapes the slot-owner cluster kernel takes (C = 128, A a multiple of 16 up to 4096, 16-bit values)
OWNER_CASES = [
    # B, H, U, P, T, K, dtype, masked, mass_aware
    (2, 3, 2, 64, 200, (16, 16), torch.bfloat16, False, False),
    (1, 2, 2, 64, 130, (16, 16), torch.bfloat16, True, True),
    (2, 2, 2, 32, 100, (8, 8), torch.float16, True, False),      # A = 1024: 64 rows per CTA
    (1, 4, 2, 16, 300, (4, 6), torch.bfloat16, False, True),     # A = 256: 16 rows per CTA, one per worker warp
    (1, 2, 4, 4, 70, (16, 16), torch.bfloat16, True, False),
    (1, 1, 2, 64, 64, (3, 16), torch.bfloat16, False, False),    # exactly one chunk
    (1, 2, 3, 16, 90, (12, 5), torch.float16, False, True),
    (1, 2, 2, 4, 150, (4, 8), torch.bfloat16, False, True),      # A = 16: one row per CTA, > 32 events per warp and chunk
    (1, 2, 2, 4, 150, (2, 3), torch.bfloat16, True, False),      # A = 16, long same-row chains inside the fast path
    (3, 5, 2, 64, 1, (16, 16), torch.bfloat16, False, False),    # a single token with gradients-style entry (T = 1)
]


@pytest.fixture
def owner_kernel():
    """Switch the slot-owner forward kernel on for one test (it is off by default)."""
    C_ = ops()
    C_.lib.rn_gsu_owner_enable(1)
    yield C_
    C_.lib.rn_gsu_owner_enable(0)


@pytest.mark.parametrize("case", OWNER_CASES)
def test_owner_kernel_matches_oracle_and_the_channel_slice_kernels(case, owner_kernel):
    C_ = owner_kernel
    B, H, U, P, T, K, dtype, masked, ma = case
    C, A = 128, P ** U
    assert C_.gsu_plan_info(B, H, T, A, C, K[0], K[1])["owner_16bit"], "the device must keep a 16-CTA cluster resident"
    w, r, x, g, slot, mass, mask, pos = make_case(B, H, U, P, T, C, dtype, 23, masked=masked)
    slot = slot * 0.1
    renorm, eps, E = (0.25, 0.75), 1e-6, H // 2
    got = run_gpu(w, r, x, g, slot, mass, mask, E, pos, K, renorm, ma, eps)
    ref = orc.ram_attn(w.float(), r.float(), x.float(), g.float(), slot, mass, mask, E, pos, K, renorm, ma, eps)
    check("owner", got, ref, mask, dtype)
    assert got[0].dtype == dtype
    # the same 16-bit values handed over as fp32 run on the channel-slice kernels; the address decode sees the
    # same numbers, every slot sees the same operations in the same order: the state is equal bit for bit
    dev = "cuda"
    idx, val = torch.ops.ramnet_ops.topk_addr_forward(w.to(dev), r.to(dev), E, A, pos.to(dev).int(), K[0], K[1], *renorm)
    m_dev = None if mask is None else mask.to(dev)
    new = torch.ops.ramnet_ops.gsu_forward(idx, val, x.to(dev), g.to(dev), slot.to(dev), mass.to(dev), m_dev, K[0], K[1], ma, eps)
    old = torch.ops.ramnet_ops.gsu_forward(idx, val, x.float().to(dev), g.float().to(dev), slot.to(dev), mass.to(dev), m_dev,
                                           K[0], K[1], ma, eps)
    new, old = [v.cpu() for v in new], [v.cpu() for v in old]
    assert torch.equal(new[0], got[0]) and torch.equal(new[1], got[1])
    assert torch.equal(new[1], old[1]) and torch.equal(new[2], old[2])
    tol = BF16_TOL if dtype == torch.bfloat16 else FP16_TOL
    yv, ov = (got[0], old[0]) if mask is None else (got[0].permute(0, 2, 1, 3)[mask], old[0].permute(0, 2, 1, 3)[mask])
    assert_close_stats("y vs channel-slice", yv.float(), ov, **tol)
    # in place on the same inputs: identical results
    inpl = run_gpu(w, r, x, g, slot, mass, mask, E, pos, K, renorm, ma, eps, inplace=True)
    for a, b in zip(got, inpl):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name", ["ram_config1.npz", "ram_grads_masked.npz", "ram_grads_massaware.npz",
                                  "ram_grads_plain.npz", "ram_bf16_u2p16.npz"])
def test_prefill_matches_reference_golden(name):
    z = load(name)
    B, H, U, P, T, Kw, Kr, C, E, ma = (int(v) for v in z["meta"])
    dtype = torch.bfloat16 if "bfloat16" in str(z["in_dtype"]) else torch.float32
    mask = t(z["mask"]) if z["mask"].size else None
    w = t(z["w_addr"]).to(dtype).permute(0, 2, 3, 4, 1)
    r = t(z["r_addr"]).to(dtype).permute(0, 2, 3, 4, 1)
    x = t(z["values"]).to(dtype).permute(0, 2, 1, 3)
    g = t(z["gamma"]).to(dtype).permute(0, 2, 1)
    rn = tuple(float(v) for v in z["renorm"])
    got = run_gpu(w, r, x, g, t(z["init_slot"]), t(z["init_mass"]), mask, E, t(z["pos"]), (Kw, Kr), rn, bool(ma),
                  float(z["eps"]))
    ref = (t(z["out_y"]).permute(0, 2, 1, 3), t(z["out_slot"]), t(z["out_mass"]))
    check(name, got, ref, mask, dtype)


@pytest.mark.parametrize("C", [12, 24, 48])
def test_untouched_slots_keep_their_bits_when_the_state_stays_in_global_memory(C):
    """A >= 16384 keeps the slot state in global memory and C need not be a multiple of the channel slice: no
    thread may touch the channels of a neighbouring slot or run past the last slot."""
    B, H, U, P, T, K = 1, 2, 2, 128, 12, (4, 4)
    A = P ** U
    w, r, x, g, slot, mass, _, pos = make_case(B, H, U, P, T, C, torch.float32, 17)
    E = 1
    y, s, m = run_gpu(w, r, x, g, slot, mass, None, E, pos, K, (0.0, 0.0), False, 1e-6)
    wi, _ = orc.topk_addr(w.float(), E, pos, K[0])
    touched = torch.zeros(B * H * A, dtype=torch.bool)
    touched[wi.reshape(-1).long()] = True
    touched = touched.view(B, H, A)
    assert torch.equal(s[~touched], slot[~touched]) and torch.equal(m[~touched], mass[~touched])
    ref = orc.ram_attn(w.float(), r.float(), x.float(), g.float(), slot, mass, None, E, pos, K, (0.0, 0.0), False, 1e-6)
    check("global-state", (y, s, m), ref, None, torch.float32)


def test_inplace_equals_functional_and_chunked_calls_carry_state():
    B, H, U, P, T, C, K = 2, 2, 2, 8, 100, 12, (4, 6)
    w, r, x, g, slot, mass, mask, pos = make_case(B, H, U, P, T, C, torch.float32, 9, masked=True)
    args = dict(E=1, K=K, renorm=(0.0, 0.5), mass_aware=False, eps=1e-6)
    full = run_gpu(w, r, x, g, slot, mass, mask, args["E"], pos, K, args["renorm"], False, 1e-6)
    inpl = run_gpu(w, r, x, g, slot, mass, mask, args["E"], pos, K, args["renorm"], False, 1e-6, inplace=True)
    for a, b in zip(full, inpl):
        assert torch.equal(a, b)
    ys, s, m = [], slot, mass
    for lo in range(0, T, 33):
        hi = min(T, lo + 33)
        y, s, m = run_gpu(w[..., lo:hi], r[..., lo:hi], x[:, :, lo:hi], g[..., lo:hi], s, m, mask[:, lo:hi], args["E"],
                          pos[:, lo:hi], K, args["renorm"], False, 1e-6)
        ys.append(y)
    # the state follows the same per-slot operation sequence however the calls are cut: bit-exact;
    # y sums a token's K reads in an order that depends on the chunk boundaries: rounding only
    assert torch.equal(s, full[1]) and torch.equal(m, full[2])
    assert_close_stats("y", torch.cat(ys, dim=2), full[0], atol=1e-5, rtol=1e-5, max_err_rate=0.0)


def test_all_masked_leaves_state_bit_exact():
    B, H, U, P, T, C, K = 1, 2, 2, 4, 20, 8, (2, 2)
    w, r, x, g, slot, mass, _, pos = make_case(B, H, U, P, T, C, torch.float32, 4)
    mask = torch.zeros(B, T, dtype=torch.bool)
    y, s, m = run_gpu(w, r, x, g, slot, mass, mask, 1, pos, K, (0.0, 0.0), False, 1e-6)
    assert torch.equal(s, slot) and torch.equal(m, mass) and float(y.abs().max()) == 0.0


def test_prefill_equals_token_by_token_decode():
    B, H, U, P, T, C, K = 2, 4, 2, 8, 24, 16, (4, 4)
    w, r, x, g, slot, mass, _, pos = make_case(B, H, U, P, T, C, torch.float32, 6)
    full = run_gpu(w, r, x, g, slot, mass, None, 2, pos, K, (0.5, 0.5), True, 1e-6)
    ops()
    s, m = slot.clone().cuda(), mass.clone().cuda()
    ys = []
    for i in range(T):
        y = torch.ops.ramnet_ops.topk_autoregressive_(
            w[..., i].contiguous().cuda(), r[..., i].contiguous().cuda(), x[:, :, i].contiguous().cuda(),
            g[..., i].contiguous().cuda(), s, m, torch.empty(0, dtype=torch.bool, device="cuda"), 2,
            pos[:, i].cuda().int(), K[0], K[1], 0.5, 0.5, True, 1e-6)
        ys.append(y.cpu())
    tol = dict(atol=1e-4, rtol=1e-4, max_err_rate=0.01, max_q99=1.5)
    assert_close_stats("y", torch.stack(ys, dim=2), full[0], **tol)
    assert_close_stats("slot", s.cpu(), full[1], **tol)
    assert_close_stats("mass", m.cpu(), full[2], **tol)


def test_segment_formulation_ops_match_the_direct_path():
    """gather_segment + torch.ops.ramnet_ops.topk_segment_forward[_] / backward (the reference's event
    and segment schemas) give the results of the time-chunked operators."""
    ops()
    from ramnet_ops.impl.cuda_impl import gather_segment
    B, H, U, P, T, C, K = 2, 3, 2, 8, 70, 12, (3, 5)
    A = P ** U
    w, r, x, g, slot, mass, mask, pos = make_case(B, H, U, P, T, C, torch.float32, 21, masked=True)
    dev = "cuda"
    idx, val = torch.ops.ramnet_ops.topk_addr_forward(w.to(dev), r.to(dev), 1, A, pos.to(dev).int(), K[0], K[1], 0.0, 0.5)
    for m in (None, mask.to(dev)):
        meta = gather_segment(idx, m, A)
        assert meta.seg_idx.numel() == B * H * A and meta.event_i.numel() == B * H * T * sum(K)
        xs, gs = x.to(dev).requires_grad_(True), g.to(dev)
        s0, m0 = slot.to(dev).requires_grad_(True), mass.to(dev)
        y, s1, m1, ev = torch.ops.ramnet_ops.topk_segment_forward(val, meta.seg_idx, meta.seg_off, meta.seg_len, meta.event_i,
                                                                  xs, gs, s0, m0, K[0], K[1], False, 1e-6)
        ry, rs, rm = torch.ops.ramnet_ops.gsu_forward(idx, val, x.to(dev), gs, slot.to(dev), m0, m, K[0], K[1], False, 1e-6)
        assert y.dtype == torch.float32 and ev.shape == meta.event_i.shape
        assert torch.equal(y, ry.float()) and torch.equal(s1, rs) and torch.equal(m1, rm)
        gx, gs0 = torch.autograd.grad(y.sum() + s1.square().sum(), (xs, s0))
        xs2, s02 = x.to(dev).requires_grad_(True), slot.to(dev).requires_grad_(True)
        ry2, rs2, _ = torch.ops.ramnet_ops.gsu_forward(idx, val, xs2, gs, s02, m0, m, K[0], K[1], False, 1e-6)
        hx, hs0 = torch.autograd.grad(ry2.sum() + rs2.square().sum(), (xs2, s02))
        assert_close_stats("D_x", gx, hx, atol=1e-5, rtol=1e-5, max_err_rate=0.0)
        assert_close_stats("D_slot", gs0, hs0, atol=1e-5, rtol=1e-5, max_err_rate=0.0)
        s_in, m_in = slot.clone().to(dev), mass.clone().to(dev)
        y2 = torch.ops.ramnet_ops.topk_segment_forward_(val, meta.seg_idx, meta.seg_off, meta.seg_len, meta.event_i,
                                                        x.to(dev), gs, s_in, m_in, K[0], K[1], False, 1e-6)
        assert torch.equal(y2, y) and torch.equal(s_in, s1) and torch.equal(m_in, m1)
