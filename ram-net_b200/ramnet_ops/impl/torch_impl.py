"""Dense PyTorch formulation of RAM attention (``impl_backend='torch'``).

Same contract as the reference's ``packages/ramnet-ops/src/ramnet_ops/impl/torch_impl.py``: every one
of the P ** U address scores is materialised per token, so it is meant for small shapes, CPU
tensors and as a differentiable cross-check.  It is never selected silently for CUDA tensors
that the CUDA backend supports.
"""
from __future__ import annotations

import torch


def kronecker_sum(xs: torch.Tensor) -> torch.Tensor:
    """(..., U, P) per-digit log-values -> (..., P ** U) sums; digit 0 is the least significant."""
    assert isinstance(xs, torch.Tensor), f"Expected xs to be Tensor, got {type(xs).__name__}."
    assert xs.ndim >= 2 and xs.size(-2) > 0 and xs.size(-1) > 0, f"Expected a non-empty (..., U, P) tensor, but got shape {tuple(xs.shape)}."
    total = xs[..., 0, :]
    for u in range(1, xs.size(-2)):
        total = (total.unsqueeze(-2) + xs[..., u, :].unsqueeze(-1)).flatten(-2)
    return total


def circular_shift_embed(xs: torch.Tensor, position_ids: torch.Tensor, embed_num: int = 0) -> torch.Tensor:
    """CAPE on dense weights (T, B, H, A): heads below ``embed_num`` read slot (a + pos) mod A."""
    assert isinstance(xs, torch.Tensor) and isinstance(position_ids, torch.Tensor), f"Expected xs/position_ids tensors, got {type(xs).__name__}/{type(position_ids).__name__}."
    assert isinstance(embed_num, int) and embed_num >= 0, f"Expected embed_num >= 0, got {embed_num!r}."
    if embed_num == 0:
        return xs
    assert xs.ndim == 4, f"Expected xs in (T, B, H, A), but got shape {tuple(xs.shape)}."
    T, B, H, A = xs.shape
    assert embed_num <= H, f"embed_num must not exceed H={H}, but got {embed_num}."
    assert position_ids.shape == (B, T), f"Expected position_ids.shape={(B, T)}, got {tuple(position_ids.shape)}."
    pos = position_ids.to(device=xs.device, dtype=torch.long).t().reshape(T, B, 1, 1)
    shifted_head = (torch.arange(H, device=xs.device) < embed_num).reshape(1, 1, H, 1)
    source = (torch.arange(A, device=xs.device).reshape(1, 1, 1, A) + pos * shifted_head) % A
    return xs.gather(-1, source.expand(T, B, H, A))


def mask_top_k(val: torch.Tensor, top_k: int | None = None, top_k_re_norm: float = 1.0) -> torch.Tensor:
    """Keep the ``top_k`` largest log-values (others -> -inf) and subtract rho * logsumexp of the kept ones."""
    assert isinstance(val, torch.Tensor), f"Expected val to be Tensor, got {type(val).__name__}."
    assert val.ndim > 0 and val.size(-1) > 0, f"Expected val with non-empty final dimension, got shape={tuple(val.shape)}."
    assert top_k is None or isinstance(top_k, int), f"Expected top_k to be int or None, got {type(top_k).__name__}."
    assert top_k is None or 0 < top_k <= val.size(-1), f"top_k must be in [1, {val.size(-1)}], but got {top_k}."
    assert isinstance(top_k_re_norm, (int, float)) and 0 <= top_k_re_norm <= 1, f"Expected top_k_re_norm in [0, 1], got {top_k_re_norm!r}."
    if top_k is not None and top_k < val.size(-1):
        keep = torch.zeros_like(val, dtype=torch.bool).scatter_(-1, val.topk(top_k, dim=-1).indices, True)
        val = torch.where(keep, val, val.new_tensor(float("-inf")))
    if top_k_re_norm != 0:
        val = val - float(top_k_re_norm) * torch.logsumexp(val, dim=-1, keepdim=True)
    return val


def addr_decode(addr: torch.Tensor, position_ids: torch.Tensor, embed_num: int = 0, top_k: int | None = None,
                top_k_re_norm: float = 0.0) -> torch.Tensor:
    """Per-digit log-probabilities (T, B, H, U, P) -> dense weights (T, B, H, P ** U)."""
    assert isinstance(addr, torch.Tensor) and isinstance(position_ids, torch.Tensor), f"Expected addr/position_ids tensors, got {type(addr).__name__}/{type(position_ids).__name__}."
    assert addr.ndim == 5, f"Expected addr in (T, B, H, U, P), but got shape {tuple(addr.shape)}."
    dense = circular_shift_embed(kronecker_sum(addr), position_ids=position_ids, embed_num=embed_num)
    return mask_top_k(dense, top_k=top_k, top_k_re_norm=top_k_re_norm).exp()


def _torch_topk_addr(addr, embed_num, position_ids, top_k, top_k_re_norm, addr_val_neg=False, encode_batch_idx=True):
    """Dense Top-K address decode: addr (B, H, U, P, T) -> (idx int32, val) both (B, H, K, T).

    Weights are float32 (float64 for float64 input) and differentiable; a token with an all -inf
    digit gets zero weights (and zero gradients)."""
    assert addr.ndim == 5, "Expected address shape (B, H, U, P, T)."
    B, H, U, P, T = addr.shape
    A = P ** U
    assert 0 < top_k <= A, f"Expected top_k in [1, A={A}], got {top_k!r}."
    assert isinstance(top_k_re_norm, (int, float)) and 0 <= top_k_re_norm <= 1, f"Expected top_k_re_norm in [0, 1], got {top_k_re_norm!r}."
    assert position_ids.shape == (B, T), f"Expected position_ids.shape={(B, T)}."
    acc = torch.float64 if addr.dtype == torch.float64 else torch.float32
    x = addr.to(acc).permute(4, 0, 1, 2, 3)  # (T,B,H,U,P)
    dead = torch.isneginf(x).all(dim=-1).any(dim=-1)  # (T,B,H)
    x = x.masked_fill(dead[..., None, None], 0)
    dense = circular_shift_embed(kronecker_sum(x.log_softmax(dim=-1)), position_ids, embed_num)  # (T,B,H,A)
    val, idx = dense.topk(top_k, dim=-1)
    if top_k_re_norm != 0:
        val = val - float(top_k_re_norm) * val.logsumexp(dim=-1, keepdim=True)
    val = val.exp().masked_fill(dead.unsqueeze(-1), 0)
    heads = torch.arange((B if encode_batch_idx else 1) * H, device=addr.device).view(-1, H, 1, 1) * A
    idx = (idx.permute(1, 2, 3, 0) + heads).to(torch.int32)
    val = val.permute(1, 2, 3, 0)
    return idx, (-val if addr_val_neg else val)


def _torch_impl_gsu(ws, rs, xs, gamma, slot, mass, mass_aware=False, eps=1e-12, inplace=False):
    """Dense recurrence over T.  ws/rs (T, ..., A), xs (T, ..., C), gamma (T, ...), slot (..., A, C), mass (..., A).

        alpha = (1 - w) / ((1 - w) + e^gamma w);  mass <- alpha mass + w;  gain = w / (mass + eps)
        slot  <- slot + gain (x - slot);           y = sum_a r[a] slot[a]   (after the write)
    """
    dt = slot.dtype
    outs = []
    for step in range(xs.size(0)):
        w = ws[step].to(dt)
        r = rs[step].to(dt)
        x = xs[step].to(dt).unsqueeze(-2)
        g = gamma[step].to(dt).unsqueeze(-1)
        keep = 1 - w
        alpha = keep / (keep + torch.exp(g) * w)
        if inplace:
            mass.mul_(alpha).add_(w)
        else:
            mass = alpha * mass + w
        gain = (w / (mass + eps)).unsqueeze(-1)
        if inplace:
            slot.add_(gain * (x - slot))
        else:
            slot = slot + gain * (x - slot)
        if mass_aware:
            rm = mass * r
            r = r.sum(dim=-1, keepdim=True) * rm / (rm.sum(dim=-1, keepdim=True) + eps)
        outs.append(torch.einsum('...ac,...a->...c', slot, r))
    return torch.stack(outs, dim=0), slot, mass


def _torch_ram_attn(w_addr, r_addr, xs, gamma, init_slot, init_mass, mask, embed_num, position_ids, top_k,
                    top_k_re_norm, mass_aware, eps, inplace):
    """Backend entry with the flattened layout: w/r (B,H,U,P,T), xs (B,H,T,C), gamma (B,H,T), state (B,H,A,C)/(B,H,A)."""
    acc = torch.float32 if xs.dtype in (torch.float16, torch.bfloat16) else xs.dtype
    if inplace:
        assert not any(t.requires_grad for t in (w_addr, r_addr, xs, gamma, init_slot, init_mass)), "inplace=True does not support backward."
        assert init_slot.dtype == init_mass.dtype == acc, f"Expected inplace state dtype={acc}, got slot={init_slot.dtype}, mass={init_mass.dtype}."
    assert isinstance(top_k_re_norm, tuple) and len(top_k_re_norm) == 2 and all(isinstance(v, (int, float)) and 0 <= v <= 1 for v in top_k_re_norm), \
        f"Expected top_k_re_norm=(write, read) in [0, 1], got {top_k_re_norm!r}."
    w_k, r_k = top_k or (None, None)
    B, _, T, _ = xs.shape
    assert position_ids.shape == (B, T), f"Expected position_ids.shape={(B, T)}, got {tuple(position_ids.shape)}."
    position_ids = position_ids.to(device=xs.device, dtype=torch.long)

    def dense_weights(logits, k, rho):
        logp = torch.log_softmax(logits, dim=-2, dtype=acc).permute(4, 0, 1, 2, 3)
        return addr_decode(logp, position_ids, embed_num, k, float(rho))  # (T,B,H,A)

    ws = dense_weights(w_addr, w_k, top_k_re_norm[0])
    rs = dense_weights(r_addr, r_k, top_k_re_norm[1])
    if mask is not None:
        ws = ws * mask.to(device=xs.device, dtype=ws.dtype).t().reshape(T, B, 1, 1)  # invalid tokens do not write
    if not inplace:
        init_slot, init_mass = init_slot.to(acc), init_mass.to(acc)
    ys, slot, mass = _torch_impl_gsu(ws, rs, xs.permute(2, 0, 1, 3), gamma.permute(2, 0, 1), init_slot, init_mass,
                                     mass_aware, eps, inplace)
    return ys.permute(1, 2, 0, 3).to(xs.dtype), slot, mass
