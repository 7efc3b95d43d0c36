"""CUDA backend of ramnet_ops on sm_100a (B200).

Mirrors the callables of the reference's ``packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py``
(``_cuda_ram_attn``, ``_cuda_topk_addr``) with the same argument layout and checks, on top of
this package's own kernels:

* ``T == 1`` without autograd: one fused decode-step kernel (``topk_autoregressive_``);
* otherwise: joined address decode (``topk_addr_forward``) followed by the time-chunked gated
  sparse update (``gsu_forward`` / ``gsu_forward_``).  No padding of T, no sort of the events and
  no transposed copies of the logits are needed.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

import ramnet_ops._C  # noqa: F401  loads the C-ABI library and defines torch.ops.ramnet_ops.*
from . import _cuda_autograd  # noqa: F401  fake kernels and autograd formulas
from ._cuda_config import ADDRESS_LIMIT, check_int_capacity


@dataclass(slots=True)
class SegmentMeta:
    """Grouped-event tables of the reference's segment formulation (fixed capacities: S = B*H*A segments,
    N = B*H*T*(Kw+Kr) events).  This package's own path does not need them; they are provided so code written
    against ``gather_segment`` + ``torch.ops.ramnet_ops.topk_segment_forward`` keeps working."""
    seg_idx: torch.Tensor  # (S)
    seg_off: torch.Tensor  # (S)
    seg_len: torch.Tensor  # (S)
    event_i: torch.Tensor  # (N)
    event_v: torch.Tensor | None = None


def gather_segment(addr_idx: torch.Tensor, mask: torch.Tensor | None, address_size: int) -> SegmentMeta:
    """Group the events of ``addr_idx`` (B,H,Kw+Kr,T) by slot, time order kept inside a slot (same contract as
    packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py:72-102; no data-dependent shapes, no host sync)."""
    B, H, K, T = addr_idx.shape
    n_slots = B * H * address_size
    keys = addr_idx.permute(0, 1, 3, 2).reshape(-1)  # event id = ((b*H + h)*T + t)*K + k
    if mask is not None:
        live = mask.to(torch.bool)[:, None, :, None].expand(B, H, T, K).reshape(-1)
        keys = torch.where(live, keys, torch.full_like(keys, n_slots))  # masked events sort behind every slot
    ordered, event_i = torch.sort(keys, stable=True)  # stable: time order, writes before reads of a token
    edges = torch.searchsorted(ordered, torch.arange(n_slots + 1, device=keys.device, dtype=torch.int32), out_int32=True)
    seg_len, order = torch.sort(edges[1:] - edges[:-1], descending=True)
    seg_idx = torch.arange(n_slots, device=keys.device, dtype=torch.int32)[order]
    return SegmentMeta(seg_idx, edges[:-1][order], seg_len, event_i.to(torch.int32))


def _cuda_topk_autoregressive_(w_addr, r_addr, x, gamma, slot_, mass_, mask, embed_num, position_ids, w_top_k, r_top_k,
                               w_re_norm, r_re_norm, mass_aware, eps) -> torch.Tensor:
    """One decode step, state updated in place.  w/r_addr (B,H,U,P), x (B,H,C), gamma (B,H), mask (B) or None."""
    assert slot_.is_contiguous() and mass_.is_contiguous(), f"Expected contiguous state, got slot={slot_.is_contiguous()}, mass={mass_.is_contiguous()}."
    if mask is None:
        mask = torch.empty(0, dtype=torch.bool, device=x.device)
    else:
        mask = mask.to(device=x.device, dtype=torch.bool)
    return torch.ops.ramnet_ops.topk_autoregressive_(w_addr, r_addr, x, gamma, slot_, mass_, mask, embed_num,
                                                     position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm, mass_aware, eps)


def _cuda_ram_attn(w_addr, r_addr, xs, gamma, init_slot, init_mass, mask, embed_num, position_ids, top_k,
                   top_k_re_norm, mass_aware, eps, inplace):
    """w/r_addr (B,H,U,P,T), xs (B,H,T,C), gamma (B,H,T), state (B,H,A,C)/(B,H,A), mask (B,T)|None,
    position_ids (B,T) -> (y (B,H,T,C) in xs.dtype, slot, mass).  Tensors may be arbitrary-stride views."""
    assert xs.ndim == 4 and w_addr.ndim == 5 and r_addr.ndim == 5, \
        f"Expected xs (B, H, T, C), w/r (B, H, U, P, T); got {tuple(xs.shape)}, {tuple(w_addr.shape)}, {tuple(r_addr.shape)}."
    if top_k is None:
        raise ValueError("CUDA RAM attention only supports Top-K mode. Use top_k or impl_backend='torch' for dense mode.")
    assert isinstance(top_k, tuple) and len(top_k) == 2 and all(isinstance(k, int) and k > 0 for k in top_k), \
        f"Expected top_k=(positive write_k, positive read_k), got {top_k!r}."
    assert isinstance(top_k_re_norm, tuple) and len(top_k_re_norm) == 2 and all(isinstance(v, (int, float)) and 0 <= v <= 1 for v in top_k_re_norm), \
        f"Expected top_k_re_norm=(w, r) in [0, 1], got {top_k_re_norm!r}."
    (B, H, T, C), (_, _, U, P, _) = xs.shape, w_addr.shape
    A = P ** U
    w_k, r_k = top_k
    w_rho, r_rho = (float(v) for v in top_k_re_norm)
    assert all(k <= A for k in top_k), f"Expected top_k <= A={A}, got {top_k}."
    assert isinstance(embed_num, int) and 0 <= embed_num <= H, f"Expected embed_num in [0, {H}], got {embed_num!r}."
    assert A < ADDRESS_LIMIT, f"Address space overflow: A={A}, limit={ADDRESS_LIMIT}."
    requires_grad = any(t.requires_grad for t in (w_addr, r_addr, xs, gamma, init_slot, init_mass))
    # int32 quantities: per-call slot numbers and event counts (state element offsets are 64-bit).  T counts
    # rounded up to a multiple of 32 like the reference's padded length (cuda_impl.py:190-195), so that the
    # accepted range of T is the same although nothing is padded here.
    T32 = T if T == 1 and not requires_grad else (T + 31) // 32 * 32
    check_int_capacity(B, H, U, P, A, C, T32, embed_num, w_k, r_k, B * H * A, B * H * T32 * (w_k + r_k))

    position_ids = position_ids.to(device=xs.device, dtype=torch.int32)
    if mask is not None:
        mask = mask.to(device=xs.device, dtype=torch.bool)
    assert w_addr.dtype == r_addr.dtype == xs.dtype == gamma.dtype, \
        f"Expected matching dtypes, got w={w_addr.dtype}, r={r_addr.dtype}, x={xs.dtype}, gamma={gamma.dtype}."
    assert w_addr.device == r_addr.device == xs.device == gamma.device == init_slot.device == init_mass.device == position_ids.device, \
        f"Expected one device, got w={w_addr.device}, r={r_addr.device}, x={xs.device}, gamma={gamma.device}, slot={init_slot.device}, mass={init_mass.device}, position_ids={position_ids.device}."
    assert mask is None or mask.device == position_ids.device, f"Expected mask.device={position_ids.device}, got {mask.device}."
    for name, tensor, want in (("w_addr", w_addr, (B, H, U, P, T)), ("r_addr", r_addr, (B, H, U, P, T)), ("xs", xs, (B, H, T, C)),
                               ("gamma", gamma, (B, H, T)), ("position_ids", position_ids, (B, T)),
                               ("init_slot", init_slot, (B, H, A, C)), ("init_mass", init_mass, (B, H, A))):
        assert tuple(tensor.shape) == want, f"Expected {name}.shape == {want}, but got {tuple(tensor.shape)}."
    assert mask is None or tuple(mask.shape) == (B, T), f"Expected mask.shape={(B, T)}, got {tuple(mask.shape)}."

    acc = torch.float32 if xs.dtype in (torch.float16, torch.bfloat16) else xs.dtype
    if inplace:
        assert not requires_grad, "inplace=True does not support backward."
        assert init_slot.dtype == init_mass.dtype == acc, f"Expected inplace state dtype={acc}, got slot={init_slot.dtype}, mass={init_mass.dtype}."
        assert init_slot.is_contiguous() and init_mass.is_contiguous(), \
            f"Expected contiguous inplace state, got slot={init_slot.is_contiguous()}, mass={init_mass.is_contiguous()}."

    if T == 1 and not requires_grad:
        with torch.no_grad():
            slot = init_slot if inplace else init_slot.to(dtype=acc, memory_format=torch.contiguous_format, copy=True)
            mass = init_mass if inplace else init_mass.to(dtype=acc, memory_format=torch.contiguous_format, copy=True)
            y = _cuda_topk_autoregressive_(
                w_addr.squeeze(-1), r_addr.squeeze(-1), xs.squeeze(-2), gamma.squeeze(-1), slot, mass,
                None if mask is None else mask.squeeze(-1), embed_num, position_ids.squeeze(-1),
                w_k, r_k, w_rho, r_rho, mass_aware, eps)
        return y.unsqueeze(-2), slot, mass

    idx, val = torch.ops.ramnet_ops.topk_addr_forward(w_addr, r_addr, embed_num, A, position_ids, w_k, r_k, w_rho, r_rho)
    # The update / read runs under the reference's operator names (topk_segment_forward[_]) so that traced graphs
    # show the same operators, in their DIRECT form: the decoded indices themselves stand where the segment table
    # would be and the token mask where the event list would be; no sort, no event tables (see _ops.py).
    none = idx.new_empty(0)
    events = none if mask is None else mask.to(torch.uint8)
    if inplace:
        y = torch.ops.ramnet_ops.topk_segment_forward_(val, idx, none, none, events, xs, gamma, init_slot, init_mass,
                                                       w_k, r_k, mass_aware, eps)
        return y, init_slot, init_mass
    y, slot, mass, _ = torch.ops.ramnet_ops.topk_segment_forward(val, idx, none, none, events, xs, gamma, init_slot.to(acc),
                                                                 init_mass.to(acc), w_k, r_k, mass_aware, eps)
    return y, slot, mass


def _cuda_topk_addr(addr, embed_num, position_ids, top_k, top_k_re_norm, addr_val_neg=False, encode_batch_idx=True):
    """Decode one address tensor (B,H,U,P,T) -> (idx int32, val float32), both (B,H,K,T); gradients flow through val."""
    assert addr.ndim == 5, f"Expected address shape (B, H, U, P, T), got {tuple(addr.shape)}."
    assert addr.is_cuda, f"Expected CUDA addresses, got {addr.device}."
    B, H, U, P, T = addr.shape
    A = P ** U
    assert A < ADDRESS_LIMIT, f"Address space overflow: A={A}, limit={ADDRESS_LIMIT}."
    assert isinstance(top_k, int) and 0 < top_k <= A, f"Expected top_k in [1, A={A}], got {top_k!r}."
    assert isinstance(embed_num, int) and 0 <= embed_num <= H, f"Expected embed_num in [0, {H}], got {embed_num!r}."
    assert isinstance(top_k_re_norm, (int, float)) and 0 <= top_k_re_norm <= 1, f"Expected top_k_re_norm in [0, 1], got {top_k_re_norm!r}."
    assert isinstance(addr_val_neg, bool), f"Expected boolean addr_val_neg, got {addr_val_neg!r}."
    assert isinstance(encode_batch_idx, bool), f"Expected boolean encode_batch_idx, got {encode_batch_idx!r}."
    assert tuple(position_ids.shape) == (B, T), f"Expected position_ids.shape={(B, T)}, got {tuple(position_ids.shape)}."
    T32 = (T + 31) // 32 * 32  # same accepted range of T as the reference, which pads T to a multiple of 32
    check_int_capacity(B, H, U, P, A, T32, embed_num, top_k, B * H * U * P * T32, B * H * A, B * H * top_k * T32)
    position_ids = position_ids.to(device=addr.device, dtype=torch.int32)
    return torch.ops.ramnet_ops.topk_addr_single_forward(addr, embed_num, A, position_ids, top_k, float(top_k_re_norm),
                                                         addr_val_neg, encode_batch_idx)
