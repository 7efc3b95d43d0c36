"""Fake (meta) kernels and autograd formulas of the ``ramnet_ops`` operators.

Same conventions as the reference's ``packages/ramnet-ops/src/ramnet_ops/impl/_cuda_autograd.py``:
indices are non-differentiable, missing upstream gradients are not materialised, read-weight
gradients exchanged between the update operator and the address operator are w.r.t. the POSITIVE
weight although the joined decode stores reads negated.
"""
from __future__ import annotations

import torch


def _token_major(like, B, H, K, T, dtype):
    return like.new_empty((B, T, H, K), dtype=dtype).permute(0, 2, 3, 1)


# ---------------------------------------------------------------------------- address decode
@torch.library.register_fake("ramnet_ops::topk_addr_single_forward")
def _(addr, embed_num, A, position_ids, top_k, top_k_re_norm, addr_val_neg=False, encode_batch_idx=True):
    B, H, _, _, T = addr.shape
    return _token_major(addr, B, H, top_k, T, torch.int32), _token_major(addr, B, H, top_k, T, torch.float32)


@torch.library.register_fake("ramnet_ops::topk_addr_single_backward")
def _(idx, val, addr, D_val, embed_num, position_ids, top_k, top_k_re_norm, addr_val_neg, shape, dtype):
    B, H, U, P, _, T = shape
    return val.new_empty((B, T, H, U, P), dtype=dtype).permute(0, 2, 3, 4, 1)


def _single_setup(ctx, inputs, output):
    addr, embed_num, A, position_ids, top_k, top_k_re_norm, addr_val_neg, _ = inputs
    idx, val = output
    B, H, U, P, T = addr.shape
    ctx.opts = (embed_num, top_k, top_k_re_norm, addr_val_neg, (B, H, U, P, A, T), addr.dtype)
    ctx.save_for_backward(idx, val, position_ids, addr)
    ctx.mark_non_differentiable(idx)
    ctx.set_materialize_grads(False)


def _single_backward(ctx, D_idx, D_val):
    if D_val is None:
        return (None,) * 8
    idx, val, position_ids, addr = ctx.saved_tensors
    embed_num, top_k, rho, neg, shape, dtype = ctx.opts
    d_addr = torch.ops.ramnet_ops.topk_addr_single_backward(idx, val, addr, D_val, embed_num, position_ids, top_k, rho,
                                                            neg, shape, dtype)
    return (d_addr,) + (None,) * 7


torch.library.register_autograd("ramnet_ops::topk_addr_single_forward", _single_backward, setup_context=_single_setup)


@torch.library.register_fake("ramnet_ops::topk_addr_forward")
def _(w_addr, r_addr, embed_num, A, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm, encode_batch_idx=True):
    B, H, _, _, T = w_addr.shape
    K = w_top_k + r_top_k
    return _token_major(w_addr, B, H, K, T, torch.int32), _token_major(w_addr, B, H, K, T, torch.float32)


@torch.library.register_fake("ramnet_ops::topk_addr_backward")
def _(idx, val, w_addr, r_addr, D_val, embed_num, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm, shape, dtype):
    B, H, U, P, _, T = shape
    make = lambda: val.new_empty((B, T, H, U, P), dtype=dtype).permute(0, 2, 3, 4, 1)  # noqa: E731
    return make(), make()


def _joined_setup(ctx, inputs, output):
    w_addr, r_addr, embed_num, A, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm, _ = inputs
    idx, val = output
    B, H, U, P, T = w_addr.shape
    ctx.opts = (embed_num, w_top_k, r_top_k, w_re_norm, r_re_norm, (B, H, U, P, A, T), w_addr.dtype)
    ctx.save_for_backward(idx, val, position_ids, w_addr, r_addr)
    ctx.mark_non_differentiable(idx)
    ctx.set_materialize_grads(False)


def _joined_backward(ctx, D_idx, D_val):
    if D_val is None:
        return (None,) * 10
    idx, val, position_ids, w_addr, r_addr = ctx.saved_tensors
    embed_num, w_k, r_k, w_rho, r_rho, shape, dtype = ctx.opts
    d_w, d_r = torch.ops.ramnet_ops.topk_addr_backward(idx, val, w_addr, r_addr, D_val, embed_num, position_ids, w_k,
                                                       r_k, w_rho, r_rho, shape, dtype)
    return (d_w if ctx.needs_input_grad[0] else None, d_r if ctx.needs_input_grad[1] else None) + (None,) * 8


torch.library.register_autograd("ramnet_ops::topk_addr_forward", _joined_backward, setup_context=_joined_setup)


# ---------------------------------------------------------------------------- decode step
@torch.library.register_fake("ramnet_ops::topk_autoregressive_")
def _(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm,
      mass_aware, eps):
    return x.new_empty(x.shape)


@torch.library.register_fake("ramnet_ops::decode_fused_")
def _(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm,
      mass_aware, eps, norm_weight, gate_logits, norm_eps, w_scale=None, r_scale=None):
    return x.new_empty(x.shape)


# ---------------------------------------------------------------------------- prefill update / read
def _y_like(x):
    B, H, T, C = x.shape
    return x.new_empty((B, T, H, C)).permute(0, 2, 1, 3)


@torch.library.register_fake("ramnet_ops::gsu_forward")
def _(addr_idx, addr_val, x, gamma, init_slot, init_mass, mask, w_top_k, r_top_k, mass_aware, eps):
    return (_y_like(x), init_slot.new_empty(init_slot.shape, dtype=torch.float32),
            init_mass.new_empty(init_mass.shape, dtype=torch.float32))


@torch.library.register_fake("ramnet_ops::gsu_forward_")
def _(addr_idx, addr_val, x, gamma, slot, mass, mask, w_top_k, r_top_k, mass_aware, eps):
    return _y_like(x)


@torch.library.register_fake("ramnet_ops::gsu_backward")
def _(addr_idx, addr_val, x, gamma, init_slot, init_mass, mask, D_y, D_post_slot, D_post_mass, w_top_k, r_top_k,
      mass_aware, eps):
    B, H, T, C = x.shape
    return (_token_major(x, B, H, w_top_k + r_top_k, T, torch.float32), torch.empty_like(x),
            x.new_empty((B, H, T), dtype=torch.float32), init_slot.new_empty(init_slot.shape, dtype=torch.float32),
            init_mass.new_empty(init_mass.shape, dtype=torch.float32))


def _gsu_setup(ctx, inputs, output):
    addr_idx, addr_val, x, gamma, init_slot, init_mass, mask, w_top_k, r_top_k, mass_aware, eps = inputs
    ctx.opts = (w_top_k, r_top_k, mass_aware, eps, mask is not None)
    saved = [addr_idx, addr_val, x, gamma, init_slot, init_mass] + ([mask] if mask is not None else [])
    ctx.save_for_backward(*saved)
    ctx.set_materialize_grads(False)


def _gsu_backward(ctx, D_y, D_slot, D_mass):
    w_top_k, r_top_k, mass_aware, eps, has_mask = ctx.opts
    addr_idx, addr_val, x, gamma, slot, mass = ctx.saved_tensors[:6]
    mask = ctx.saved_tensors[6] if has_mask else None
    if D_y is None and D_slot is None and D_mass is None:
        return (None,) * 11
    d_val, d_x, d_gamma, d_slot, d_mass = torch.ops.ramnet_ops.gsu_backward(
        addr_idx, addr_val, x, gamma, slot, mass, mask,
        torch.zeros_like(x) if D_y is None else D_y,
        torch.zeros_like(slot, dtype=torch.float32) if D_slot is None else D_slot,
        torch.zeros_like(mass, dtype=torch.float32) if D_mass is None else D_mass,
        w_top_k, r_top_k, mass_aware, eps)
    need = ctx.needs_input_grad
    # d_val is w.r.t. the positive weight of each event; the joined decode stored reads negated and its
    # backward expects exactly this convention
    return (None, d_val if need[1] else None, d_x.to(x.dtype) if need[2] else None,
            d_gamma.to(gamma.dtype) if need[3] else None, d_slot.to(slot.dtype) if need[4] else None,
            d_mass.to(mass.dtype) if need[5] else None, None, None, None, None, None)


torch.library.register_autograd("ramnet_ops::gsu_forward", _gsu_backward, setup_context=_gsu_setup)


# ---------------------------------------------------------------------------- event / segment schemas
# Two calling conventions (see _ops.is_direct): the reference's segment tables, or the direct form in which
# seg_off is empty and seg_idx / event_i are the decoded indices and the token mask.
def _direct(seg_off):
    return seg_off.numel() == 0


@torch.library.register_fake("ramnet_ops::topk_segment_forward")
def _(addr_val, seg_idx, seg_off, seg_len, event_i, x, gamma, init_slot, init_mass, w_top_k, r_top_k, mass_aware, eps):
    slot = init_slot.new_empty(init_slot.shape, dtype=torch.float32)
    mass = init_mass.new_empty(init_mass.shape, dtype=torch.float32)
    if _direct(seg_off):
        return _y_like(x), slot, mass, addr_val.new_empty(0)
    return x.new_empty(x.shape, dtype=torch.float32), slot, mass, addr_val.new_empty(event_i.shape)


@torch.library.register_fake("ramnet_ops::topk_segment_forward_")
def _(addr_val, seg_idx, seg_off, seg_len, event_i, x, gamma, slot, mass, w_top_k, r_top_k, mass_aware, eps):
    return _y_like(x) if _direct(seg_off) else x.new_empty(x.shape, dtype=torch.float32)


@torch.library.register_fake("ramnet_ops::topk_segment_backward")
def _(seg_idx, seg_off, seg_len, event_i, event_v, x, gamma, init_slot, init_mass, D_y, D_post_slot, D_post_mass,
      w_top_k, r_top_k, mass_aware, eps):
    B, H, T, _ = x.shape
    K = w_top_k + r_top_k
    d_slot = init_slot.new_empty(init_slot.shape, dtype=torch.float32)
    d_mass = init_mass.new_empty(init_mass.shape, dtype=torch.float32)
    if _direct(seg_off):
        return (_token_major(x, B, H, K, T, torch.float32), torch.empty_like(x), x.new_empty((B, H, T), dtype=torch.float32),
                d_slot, d_mass)
    return (x.new_empty((B, H, K, T), dtype=torch.float32), x.new_empty(x.shape, dtype=torch.float32),
            gamma.new_empty(gamma.shape, dtype=torch.float32), d_slot, d_mass)


def _segment_setup(ctx, inputs, output):
    addr_val, seg_idx, seg_off, seg_len, event_i, x, gamma, init_slot, init_mass, w_top_k, r_top_k, mass_aware, eps = inputs
    ctx.opts = (w_top_k, r_top_k, mass_aware, eps)
    # the backward operator wants the weight of every event: the replay cache in the segment form, the decoded
    # weights themselves in the direct form
    values = addr_val if _direct(seg_off) else output[3]
    ctx.save_for_backward(seg_idx, seg_off, seg_len, event_i, values, x, gamma, init_slot, init_mass)
    ctx.mark_non_differentiable(output[3])
    ctx.set_materialize_grads(False)


def _segment_backward(ctx, D_y, D_slot, D_mass, D_event_v):
    seg_idx, seg_off, seg_len, event_i, event_v, x, gamma, slot, mass = ctx.saved_tensors
    w_top_k, r_top_k, mass_aware, eps = ctx.opts
    if D_y is None and D_slot is None and D_mass is None:
        return (None,) * 13
    d_addr, d_x, d_gamma, d_slot, d_mass = torch.ops.ramnet_ops.topk_segment_backward(
        seg_idx, seg_off, seg_len, event_i, event_v, x, gamma, slot, mass,
        torch.zeros_like(x) if D_y is None else D_y,
        torch.zeros_like(slot, dtype=torch.float32) if D_slot is None else D_slot,
        torch.zeros_like(mass, dtype=torch.float32) if D_mass is None else D_mass,
        w_top_k, r_top_k, mass_aware, eps)
    need = ctx.needs_input_grad
    # d_addr is w.r.t. the positive weight of each event; the joined decode stored reads negated and its backward
    # expects exactly this convention
    return (d_addr if need[0] else None,) + (None,) * 4 + (
        d_x.to(x.dtype) if need[5] else None, d_gamma.to(gamma.dtype) if need[6] else None,
        d_slot.to(slot.dtype) if need[7] else None, d_mass.to(mass.dtype) if need[8] else None) + (None,) * 4


torch.library.register_autograd("ramnet_ops::topk_segment_forward", _segment_backward, setup_context=_segment_setup)
