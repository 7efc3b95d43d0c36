"""Generate the golden fixtures in this folder from the UNMODIFIED reference PyTorch backend.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py <path to a checkout of the reference project>

It imports ``ramnet_ops`` from ``<ref>/packages/ramnet-ops/src`` (the CUDA extension is absent
there, so only ``impl_backend='torch'`` is exercised), feeds it seeded inputs and stores inputs
and outputs as ``.npz``.  The fixtures travel with the repository; this script does not.
"""
import sys
import warnings
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _np(t):
    return t.detach().to(torch.float64 if t.dtype == torch.float64 else torch.float32).numpy() if t.is_floating_point() else t.detach().numpy()


def addr_case(ref, name, B, H, U, P, T, K, E, dtype, std, renorm, neg, encode, seed, special=False):
    from ramnet_ops.impl.torch_impl import kronecker_sum, circular_shift_embed
    g = torch.Generator().manual_seed(seed)
    addr = (torch.randn(B, H, U, P, T, generator=g) * std).to(dtype).float()
    if special:
        addr[..., 0] = -torch.inf                 # token 0: every digit inactive
        addr[:, :, 0, :, 1] = -torch.inf          # token 1: digit 0 inactive
        addr[..., 2] = torch.linspace(-1000, 1000, P).view(1, 1, 1, P)
        addr[:, :, :, : P // 2, 3] = -torch.inf   # token 3: half of each digit -inf (still active)
        addr[..., 4] = 0.25                        # token 4: all logits tie
    pos = (torch.arange(T).view(1, T) * 3 + 5 + torch.arange(B).view(B, 1)).long()
    idx, val = ref.topk_addr(addr, E, pos, K, renorm, neg, encode, impl_backend="torch")
    # dense reference scores (content space) for the boundary gap K / K+1
    x = addr.permute(4, 0, 1, 2, 3)
    inactive = torch.isneginf(x).all(-1).any(-1)
    x = x.masked_fill(inactive[..., None, None], 0)
    dense = kronecker_sum(x.log_softmax(-1))  # (T,B,H,A)
    srt = dense.sort(dim=-1, descending=True).values
    A = P ** U
    gap = (srt[..., K - 1] - srt[..., K]) if K < A else torch.full(srt.shape[:-1], float("inf"))
    gap = torch.nan_to_num(gap, nan=0.0, posinf=1e30)
    np.savez(HERE / f"addr_{name}.npz", addr=_np(addr), pos=pos.numpy(), idx=idx.numpy(), val=_np(val),
             gap=_np(gap.permute(1, 2, 0)), ref_topk_scores=_np(srt[..., :K].permute(1, 2, 3, 0)),
             meta=np.array([B, H, U, P, T, K, E, int(neg), int(encode)]), renorm=np.float64(renorm),
             in_dtype=str(dtype))


def ram_case(ref, name, B, H, U, P, T, K, C, E, dtype, renorm, mass_aware, eps, seed, masked, zero_state,
             grads, gamma_kind="randn"):
    A = P ** U
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, U, P, generator=g).to(dtype)
    k = torch.randn(B, T, H, U, P, generator=g).to(dtype)
    v = torch.randn(B, T, H, C, generator=g).to(dtype)
    gm = torch.randn(B, T, H, generator=g)
    gamma = (torch.sigmoid(gm) if gamma_kind == "sigmoid" else 0.2 * gm).to(dtype)
    if zero_state:
        slot, mass = torch.zeros(B, H, A, C), torch.full((B, H, A), 1.0 / A)
    else:
        slot, mass = torch.randn(B, H, A, C, generator=g), torch.rand(B, H, A, generator=g) + 0.1
    if masked:
        mask = torch.ones(B, T, dtype=torch.bool)
        mask[:, : max(1, T // 8)] = False
        mask[0, T // 2: T // 2 + 3] = False
        mask[:, -2:] = False
        pos = ((mask.long().cumsum(-1) - 1) * 3 + 11).masked_fill(~mask, 0)
    else:
        mask, pos = None, torch.arange(T).view(1, T).expand(B, T).contiguous()
    d_y = torch.randn(B, T, H, C, generator=g)
    d_slot = torch.randn(B, H, A, C, generator=g)
    d_mass = torch.randn(B, H, A, generator=g)

    def run(cast):
        leaves = [t.to(cast).detach().requires_grad_(grads) for t in (k, q, v, gamma, slot, mass)]
        wk, rq, vv, gg, s0, m0 = leaves
        y, (s1, m1) = ref.random_access_memory_attention(
            wk, rq, vv, gg, (s0, m0), mask=mask, embed_num=E, position_ids=pos, top_k=K,
            top_k_re_norm=renorm, mass_aware=mass_aware, eps=eps, impl_backend="torch")
        out = dict(y=_np(y), slot=_np(s1), mass=_np(m1))
        if grads:
            up = d_y.to(cast)
            if mask is not None:
                up = up * mask[:, :, None, None].to(cast)
            gr = torch.autograd.grad((y, s1, m1), leaves, (up.to(y.dtype), d_slot.to(s1.dtype), d_mass.to(m1.dtype)))
            out.update({n: _np(t) for n, t in zip(("D_w", "D_r", "D_x", "D_gamma", "D_slot", "D_mass"), gr)})
        return out

    fwd = run(dtype if dtype != torch.float32 else torch.float32)
    save = dict(w_addr=_np(k), r_addr=_np(q), values=_np(v), gamma=_np(gamma), init_slot=_np(slot), init_mass=_np(mass),
                pos=pos.numpy(), mask=(mask.numpy() if mask is not None else np.zeros((0,), dtype=bool)),
                d_y=_np(d_y), d_slot=_np(d_slot), d_mass=_np(d_mass),
                meta=np.array([B, H, U, P, T, K[0], K[1], C, E, int(mass_aware)]),
                renorm=np.array(renorm, dtype=np.float64), eps=np.float64(eps), in_dtype=str(dtype))
    save.update({f"out_{n}": a for n, a in fwd.items()})
    if grads:
        f64 = run(torch.float64)
        save.update({f"out64_{n}": a for n, a in f64.items()})
    np.savez(HERE / f"ram_{name}.npz", **save)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    root = Path(sys.argv[1])
    sys.path.insert(0, str(root / "packages" / "ramnet-ops" / "src"))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import ramnet_ops as ref
    f32, bf16 = torch.float32, torch.bfloat16
    addr_case(ref, "u2p16k4_f32", 2, 4, 2, 16, 24, 4, 2, f32, 1.0, 0.0, False, True, 1)
    addr_case(ref, "u3p8k8_f32_renorm", 1, 4, 3, 8, 16, 8, 2, f32, 1.0, 0.5, True, False, 2)
    addr_case(ref, "u2p64k16_bf16", 1, 2, 2, 64, 8, 16, 1, bf16, 1.0, 0.0, False, True, 3)
    addr_case(ref, "u3p32k8_bf16", 1, 2, 3, 32, 4, 8, 1, bf16, 1.5, 0.0, False, True, 4)
    addr_case(ref, "u4p4k16_special", 2, 2, 4, 4, 6, 16, 1, f32, 1.0, 1.0, False, True, 5, special=True)
    addr_case(ref, "u2p3kall_f32", 1, 2, 2, 3, 5, 9, 1, f32, 1.0, 0.25, False, True, 6)
    # BASELINE config 1: B1 T512 H4 U2 P16 K4 C64 fp32, CAPE on heads 0-1, zero slot state
    ram_case(ref, "config1", 1, 4, 2, 16, 512, (4, 4), 64, 2, f32, (0.0, 0.0), False, 1e-12, 0, False, True, False,
             gamma_kind="sigmoid")
    ram_case(ref, "grads_masked", 2, 3, 2, 6, 40, (3, 5), 10, 2, f32, (0.25, 0.75), False, 1e-6, 7, True, False, True)
    ram_case(ref, "grads_massaware", 2, 3, 2, 6, 40, (3, 5), 10, 2, f32, (0.25, 0.75), True, 1e-6, 8, True, False, True)
    ram_case(ref, "grads_plain", 1, 2, 3, 4, 33, (8, 8), 7, 1, f32, (0.0, 0.0), False, 1e-12, 9, False, False, True)
    ram_case(ref, "bf16_u2p16", 2, 4, 2, 16, 64, (4, 4), 16, 2, bf16, (0.0, 0.0), False, 1e-12, 10, False, True, False,
             gamma_kind="sigmoid")
    ram_case(ref, "decode_t1", 3, 4, 2, 8, 1, (4, 4), 12, 2, f32, (0.0, 1.0), False, 1e-12, 11, False, False, False)
    ram_case(ref, "decode_t1_massaware", 3, 4, 2, 8, 1, (4, 6), 12, 2, f32, (0.5, 0.5), True, 1e-6, 12, False, False, False)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
