"""Operator schemas of the ``ramnet_ops`` namespace and their CUDA implementations.

The eight schemas are those of the reference dispatcher library
(packages/ramnet-ops/csrc/ram_attn_bind.cpp:27-101); the ``gsu_*`` and ``decode_fused_``
operators are additions used by this package's own call path.  Every implementation
allocates its outputs with PyTorch (caching allocator, CUDA-graph friendly) and hands raw
pointers, sizes and strides to the C ABI; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes

import torch

from . import _C
from ._C import check, check_device, dtype_code, lib, ptr, stream_of, strides

_lib = torch.library.Library("ramnet_ops", "DEF")

_lib.define(
    "topk_addr_single_forward(Tensor addr, int embed_num, int A, Tensor position_ids, int top_k, float top_k_re_norm, "
    "bool addr_val_neg=False, bool encode_batch_idx=True) -> (Tensor, Tensor)")
_lib.define(
    "topk_addr_single_backward(Tensor idx, Tensor val, Tensor addr, Tensor D_val, int embed_num, Tensor position_ids, "
    "int top_k, float top_k_re_norm, bool addr_val_neg, int[] shape, ScalarType dtype) -> Tensor")
_lib.define(
    "topk_addr_forward(Tensor w_addr, Tensor r_addr, int embed_num, int A, Tensor position_ids, int w_top_k, int r_top_k, "
    "float w_re_norm, float r_re_norm, bool encode_batch_idx=True) -> (Tensor, Tensor)")
_lib.define(
    "topk_addr_backward(Tensor idx, Tensor val, Tensor w_addr, Tensor r_addr, Tensor D_val, int embed_num, "
    "Tensor position_ids, int w_top_k, int r_top_k, float w_re_norm, float r_re_norm, int[] shape, ScalarType dtype) "
    "-> (Tensor, Tensor)")
_lib.define(
    "topk_autoregressive_(Tensor w_addr, Tensor r_addr, Tensor x, Tensor gamma, Tensor(a!) slot, Tensor(b!) mass, "
    "Tensor mask, int embed_num, Tensor position_ids, int w_top_k, int r_top_k, float w_re_norm, float r_re_norm, "
    "bool mass_aware, float eps) -> Tensor")
_lib.define(
    "decode_fused_(Tensor w_addr, Tensor r_addr, Tensor x, Tensor gamma, Tensor(a!) slot, Tensor(b!) mass, "
    "Tensor mask, int embed_num, Tensor position_ids, int w_top_k, int r_top_k, float w_re_norm, float r_re_norm, "
    "bool mass_aware, float eps, Tensor? norm_weight, Tensor? gate_logits, float norm_eps, "
    "Tensor? w_scale=None, Tensor? r_scale=None) -> Tensor")
_lib.define(
    "gsu_forward(Tensor addr_idx, Tensor addr_val, Tensor x, Tensor gamma, Tensor init_slot, Tensor init_mass, "
    "Tensor? mask, int w_top_k, int r_top_k, bool mass_aware, float eps) -> (Tensor, Tensor, Tensor)")
_lib.define(
    "gsu_forward_(Tensor addr_idx, Tensor addr_val, Tensor x, Tensor gamma, Tensor(a!) slot, Tensor(b!) mass, "
    "Tensor? mask, int w_top_k, int r_top_k, bool mass_aware, float eps) -> Tensor")
_lib.define(
    "gsu_backward(Tensor addr_idx, Tensor addr_val, Tensor x, Tensor gamma, Tensor init_slot, Tensor init_mass, "
    "Tensor? mask, Tensor D_y, Tensor D_post_slot, Tensor D_post_mass, int w_top_k, int r_top_k, bool mass_aware, "
    "float eps) -> (Tensor, Tensor, Tensor, Tensor, Tensor)")
# operators of the reference's event/segment formulation, kept for call compatibility: the slot of an
# event is recovered from the segment tables and the work is done by the time-chunked kernels
_lib.define(
    "topk_segment_forward(Tensor addr_val, Tensor seg_idx, Tensor seg_off, Tensor seg_len, Tensor event_i, Tensor x, "
    "Tensor gamma, Tensor init_slot, Tensor init_mass, int w_top_k, int r_top_k, bool mass_aware, float eps) "
    "-> (Tensor, Tensor, Tensor, Tensor)")
_lib.define(
    "topk_segment_backward(Tensor seg_idx, Tensor seg_off, Tensor seg_len, Tensor event_i, Tensor event_v, Tensor x, "
    "Tensor gamma, Tensor init_slot, Tensor init_mass, Tensor D_y, Tensor D_post_slot, Tensor D_post_mass, int w_top_k, "
    "int r_top_k, bool mass_aware, float eps) -> (Tensor, Tensor, Tensor, Tensor, Tensor)")
_lib.define(
    "topk_segment_forward_(Tensor addr_val, Tensor seg_idx, Tensor seg_off, Tensor seg_len, Tensor event_i, Tensor x, "
    "Tensor gamma, Tensor(a!) slot, Tensor(b!) mass, int w_top_k, int r_top_k, bool mass_aware, float eps) -> Tensor")


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("ramnet_ops CUDA operators need CUDA tensors")


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(like: torch.Tensor, nbytes: int) -> torch.Tensor:
    """Scratch for one kernel sequence on the current stream of ``like.device``.

    One buffer per (device, stream) is kept and grown on demand, so steady-state calls allocate nothing (a
    fresh gigabyte-sized block per call can make the caching allocator go back to the driver).  Calls on one
    stream are ordered, so they may share it; every call rewrites what it later reads.  During a stream
    capture the buffer comes from the capturing allocator instead and is not kept."""
    nbytes = max(int(nbytes), 256)
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=like.device)
    key = (like.device.index, torch.cuda.current_stream(like.device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        _WORKSPACES.pop(key, None)
        ws = None
        ws = torch.empty(nbytes, dtype=torch.uint8, device=like.device)
        _WORKSPACES[key] = ws
    return ws


def release_workspaces() -> None:
    """Drop the cached scratch buffers (they are re-created on the next call)."""
    _WORKSPACES.clear()


def _int32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


def _slots(addr: torch.Tensor, A: int) -> None:
    U, P = addr.shape[2], addr.shape[3]
    if A != P ** U:
        raise RuntimeError(f"A={A} does not equal P**U={P ** U}")


def _new_token_major(like: torch.Tensor, B: int, H: int, K: int, T: int, dtype: torch.dtype) -> torch.Tensor:
    """(B,H,K,T)-shaped tensor stored token-major (B,T,H,K): one token-head's K entries are contiguous."""
    return torch.empty((B, T, H, K), dtype=dtype, device=like.device).permute(0, 2, 3, 1)


def _new_logit_grad(like: torch.Tensor, B: int, H: int, U: int, P: int, T: int, dtype: torch.dtype) -> torch.Tensor:
    return torch.empty((B, T, H, U, P), dtype=dtype, device=like.device).permute(0, 2, 3, 4, 1)


# ----------------------------------------------------------------------------------------------
# address decode
# ----------------------------------------------------------------------------------------------
def addr_forward_impl(w_addr, r_addr, embed_num, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm,
                      w_neg, r_neg, encode_batch_idx):
    _require_cuda(w_addr, r_addr, position_ids)
    B, H, U, P, T = w_addr.shape
    if r_addr is not None and r_addr.stride() != w_addr.stride():
        w_addr, r_addr = w_addr.contiguous(), r_addr.contiguous()
    pos = _int32(position_ids)
    K = w_top_k + r_top_k
    idx = _new_token_major(w_addr, B, H, K, T, torch.int32)
    val = _new_token_major(w_addr, B, H, K, T, torch.float32)
    if idx.numel() == 0:
        return idx, val
    check(lib.rn_addr_fwd(ptr(w_addr), ptr(r_addr), dtype_code(w_addr), strides(w_addr), ptr(pos), strides(pos),
                          ptr(idx), ptr(val), strides(idx), B, H, U, P, T, embed_num, w_top_k, r_top_k,
                          float(w_re_norm), float(r_re_norm), int(w_neg), int(r_neg), int(encode_batch_idx),
                          w_addr.device.index, stream_of(w_addr)))
    return idx, val


def addr_backward_impl(idx, val, w_addr, r_addr, d_val, embed_num, position_ids, w_top_k, r_top_k, w_re_norm,
                       r_re_norm, w_neg, r_neg, dtype):
    _require_cuda(idx, val, w_addr, r_addr, d_val, position_ids)
    B, H, U, P, T = w_addr.shape
    if r_addr is not None and r_addr.stride() != w_addr.stride():
        w_addr, r_addr = w_addr.contiguous(), r_addr.contiguous()
    if w_addr.dtype != dtype:
        w_addr = w_addr.to(dtype)
        r_addr = None if r_addr is None else r_addr.to(dtype)
    if val.stride() != idx.stride():
        val = val.contiguous()
        idx = idx.contiguous()
    pos = _int32(position_ids)
    d_val = d_val.to(torch.float32)
    d_w = _new_logit_grad(w_addr, B, H, U, P, T, dtype)
    d_r = _new_logit_grad(w_addr, B, H, U, P, T, dtype) if r_addr is not None else None
    if d_w.numel() == 0:
        return d_w, d_r
    check(lib.rn_addr_bwd(ptr(idx), ptr(val), strides(idx), ptr(d_val), strides(d_val), ptr(w_addr), ptr(r_addr),
                          dtype_code(w_addr), strides(w_addr), ptr(pos), strides(pos), ptr(d_w), ptr(d_r), strides(d_w),
                          B, H, U, P, T, embed_num, w_top_k, r_top_k, float(w_re_norm), float(r_re_norm),
                          int(w_neg), int(r_neg), w_addr.device.index, stream_of(w_addr)))
    return d_w, d_r


@torch.library.impl(_lib, "topk_addr_single_forward", "CUDA")
def _topk_addr_single_forward(addr, embed_num, A, position_ids, top_k, top_k_re_norm, addr_val_neg=False,
                              encode_batch_idx=True):
    _slots(addr, A)
    return addr_forward_impl(addr, None, embed_num, position_ids, top_k, 0, top_k_re_norm, 0.0, addr_val_neg, False,
                             encode_batch_idx)


@torch.library.impl(_lib, "topk_addr_single_backward", "CUDA")
def _topk_addr_single_backward(idx, val, addr, D_val, embed_num, position_ids, top_k, top_k_re_norm, addr_val_neg,
                               shape, dtype):
    if len(shape) != 6:
        raise RuntimeError("Expected address dimensions (B, H, U, P, A, T).")
    if addr is None or idx is None or val is None or D_val is None:
        raise RuntimeError("topk_addr_single_backward needs idx, val, addr and D_val")
    # D_val is the gradient of the stored (signed) value; the kernel wants it w.r.t. the positive weight
    d_pos = -D_val if addr_val_neg else D_val
    d_w, _ = addr_backward_impl(idx, val, addr, None, d_pos, embed_num, position_ids, top_k, 0, top_k_re_norm, 0.0,
                                addr_val_neg, False, dtype)
    return d_w


@torch.library.impl(_lib, "topk_addr_forward", "CUDA")
def _topk_addr_forward(w_addr, r_addr, embed_num, A, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm,
                       encode_batch_idx=True):
    _slots(w_addr, A)
    # joined decode: writes keep a positive sign, reads are stored negated
    return addr_forward_impl(w_addr, r_addr, embed_num, position_ids, w_top_k, r_top_k, w_re_norm, r_re_norm, False,
                             True, encode_batch_idx)


@torch.library.impl(_lib, "topk_addr_backward", "CUDA")
def _topk_addr_backward(idx, val, w_addr, r_addr, D_val, embed_num, position_ids, w_top_k, r_top_k, w_re_norm,
                        r_re_norm, shape, dtype):
    if len(shape) != 6:
        raise RuntimeError("Expected address dimensions (B, H, U, P, A, T).")
    return addr_backward_impl(idx, val, w_addr, r_addr, D_val, embed_num, position_ids, w_top_k, r_top_k, w_re_norm,
                              r_re_norm, False, True, dtype)


# ----------------------------------------------------------------------------------------------
# fused decode step
# ----------------------------------------------------------------------------------------------
def _batch_rows(t: torch.Tensor) -> torch.Tensor:
    """A decode input as the kernels take it: every batch row one contiguous block (heads and what follows them
    contiguous), any stride between the batch rows: a column slice of a wider projection output needs no copy."""
    if t.is_contiguous():
        return t
    if t.dim() >= 2:
        inner, ok = 1, True
        for size, stride in zip(reversed(t.shape[1:]), reversed(t.stride()[1:])):
            ok = ok and (size == 1 or stride == inner)
            inner *= size
        if ok and t.stride(0) >= inner:
            return t
    return t.contiguous()


def decode_scales_supported(dtype, U, P, C, w_top_k, r_top_k) -> bool:
    from ._C import DTYPE_CODE
    code = DTYPE_CODE.get(dtype)
    return code is not None and bool(lib.rn_decode_scales_supported(code, U, P, C, w_top_k, r_top_k))


def decode_impl(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k, w_re_norm,
                r_re_norm, mass_aware, eps, norm_weight=None, gate_logits=None, norm_eps=0.0, w_scale=None, r_scale=None):
    """One decode step.  ``w_scale`` / ``r_scale`` (H,U) or (H,U,1): factors of the logits, applied inside the
    kernel where decode_scales_supported() says so, else by a multiply here (same rounding either way)."""
    _require_cuda(w_addr, r_addr, x, gamma, slot, mass, position_ids)
    B, H, U, P = w_addr.shape
    C = x.shape[-1]
    if slot.dtype != torch.float32 or mass.dtype != torch.float32:
        raise RuntimeError(f"slot/mass state must be float32, got {slot.dtype}/{mass.dtype}")
    if not (slot.is_contiguous() and mass.is_contiguous()):
        raise RuntimeError("Tensor slot/mass must be contiguous")
    if tuple(slot.shape) != (B, H, P ** U, C) or tuple(mass.shape) != (B, H, P ** U):
        raise RuntimeError(f"state shape mismatch: slot {tuple(slot.shape)}, mass {tuple(mass.shape)}")
    if (w_scale is None) != (r_scale is None):
        raise RuntimeError("give both logit scales or none")
    if w_scale is not None:
        w_scale = w_scale.to(w_addr.dtype).reshape(H, U).contiguous()
        r_scale = r_scale.to(r_addr.dtype).reshape(H, U).contiguous()
        if not decode_scales_supported(w_addr.dtype, U, P, C, w_top_k, r_top_k):
            w_addr, r_addr = w_scale.unsqueeze(-1) * w_addr, r_scale.unsqueeze(-1) * r_addr
            w_scale = r_scale = None
    w_addr, r_addr, x, gamma = (_batch_rows(t) for t in (w_addr, r_addr, x, gamma))
    if not (r_addr.dtype == x.dtype == gamma.dtype == w_addr.dtype):
        raise RuntimeError("w_addr, r_addr, x and gamma must share one dtype")
    pos = _int32(position_ids).contiguous()
    mask_u8 = None
    if mask is not None and mask.numel() > 0:
        mask_u8 = mask.to(torch.bool).contiguous().view(torch.uint8)
    if norm_weight is not None:
        norm_weight = norm_weight.to(torch.float32).contiguous()
    if gate_logits is not None:
        gate_logits = _batch_rows(gate_logits.to(x.dtype))
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if y.numel() == 0:
        return y
    batch_strides = (ctypes.c_int64 * 5)(w_addr.stride(0), r_addr.stride(0), x.stride(0), gamma.stride(0),
                                         H * C if gate_logits is None else gate_logits.stride(0))
    check(lib.rn_decode_step_scaled(ptr(w_addr), ptr(r_addr), ptr(x), ptr(gamma), dtype_code(x), ptr(slot), ptr(mass),
                                    ptr(mask_u8), ptr(pos), ptr(y), ptr(norm_weight), ptr(gate_logits), float(norm_eps),
                                    ptr(w_scale), ptr(r_scale), batch_strides, B, H, U, P, C, embed_num, w_top_k, r_top_k,
                                    float(w_re_norm), float(r_re_norm), int(mass_aware), float(eps), x.device.index,
                                    stream_of(x)))
    check_device(y)
    return y


@torch.library.impl(_lib, "topk_autoregressive_", "CUDA")
def _topk_autoregressive_(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k,
                          w_re_norm, r_re_norm, mass_aware, eps):
    return decode_impl(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k,
                       w_re_norm, r_re_norm, mass_aware, eps)


@torch.library.impl(_lib, "decode_fused_", "CUDA")
def _decode_fused_(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k, w_re_norm,
                   r_re_norm, mass_aware, eps, norm_weight, gate_logits, norm_eps, w_scale=None, r_scale=None):
    return decode_impl(w_addr, r_addr, x, gamma, slot, mass, mask, embed_num, position_ids, w_top_k, r_top_k,
                       w_re_norm, r_re_norm, mass_aware, eps, norm_weight, gate_logits, norm_eps, w_scale, r_scale)


# ----------------------------------------------------------------------------------------------
# prefill: gated sparse update + read over decoded addresses
# ----------------------------------------------------------------------------------------------
def gsu_forward_impl(addr_idx, addr_val, x, gamma, slot_in, mass_in, slot_out, mass_out, mask, w_top_k, r_top_k,
                     mass_aware, eps, y_dtype=None):
    """Launch the schedule + apply kernels.  ``slot_out``/``mass_out`` may alias the inputs."""
    _require_cuda(addr_idx, addr_val, x, gamma, slot_in, mass_in)
    B, H, T, C = x.shape
    A = slot_in.shape[2]
    if tuple(addr_idx.shape) != (B, H, w_top_k + r_top_k, T) or addr_val.shape != addr_idx.shape:
        raise RuntimeError(f"Tensor addr_idx/addr_val shape mismatch: expect {(B, H, w_top_k + r_top_k, T)}, "
                           f"but got {tuple(addr_idx.shape)} / {tuple(addr_val.shape)}")
    for name, s in (("slot", slot_in), ("mass", mass_in), ("slot", slot_out), ("mass", mass_out)):
        if s.dtype != torch.float32 or not s.is_contiguous():
            raise RuntimeError(f"Tensor {name} must be contiguous float32")
    if tuple(slot_in.shape) != (B, H, A, C) or tuple(mass_in.shape) != (B, H, A):
        raise RuntimeError(f"state shape mismatch: slot {tuple(slot_in.shape)}, mass {tuple(mass_in.shape)}")
    if addr_val.dtype != torch.float32 or addr_idx.dtype != torch.int32:
        raise RuntimeError("addr_idx must be int32 and addr_val float32")
    if addr_val.stride() != addr_idx.stride():
        addr_idx, addr_val = addr_idx.contiguous(), addr_val.contiguous()
    if x.stride(-1) != 1:
        x = x.contiguous()
    if gamma.dtype != x.dtype:
        raise RuntimeError(f"Tensor gamma type mismatch: expect {x.dtype}, but got {gamma.dtype}")
    y_dtype = x.dtype if y_dtype is None else y_dtype
    if y_dtype != x.dtype:
        raise RuntimeError("y is produced in the dtype of x")
    y = torch.empty((B, T, H, C), dtype=x.dtype, device=x.device).permute(0, 2, 1, 3)
    if y.numel() == 0:
        if slot_out.data_ptr() != slot_in.data_ptr():
            slot_out.copy_(slot_in)
            mass_out.copy_(mass_in)
        return y
    mask_u8 = None
    if mask is not None:
        mask_u8 = mask.to(torch.bool).view(torch.uint8)
    rows_aligned = x.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in x.stride()[:3])
    nbytes = lib.rn_gsu_fwd_workspace_bytes(dtype_code(x), int(rows_aligned), B, H, T, A, C, w_top_k, r_top_k, x.device.index)
    if nbytes < 0:
        check(1)
    ws = _workspace(x, nbytes)
    check(lib.rn_gsu_fwd(ptr(addr_idx), ptr(addr_val), strides(addr_idx), ptr(x), strides(x), ptr(gamma), strides(gamma),
                         dtype_code(x), ptr(mask_u8), None if mask_u8 is None else strides(mask_u8), ptr(slot_in),
                         ptr(mass_in), ptr(slot_out), ptr(mass_out), ptr(y), strides(y), ptr(ws), ws.numel(), B, H, T,
                         A, C, w_top_k, r_top_k, int(mass_aware), float(eps), x.device.index, stream_of(x)))
    check_device(y)
    return y


@torch.library.impl(_lib, "gsu_forward", "CUDA")
def _gsu_forward(addr_idx, addr_val, x, gamma, init_slot, init_mass, mask, w_top_k, r_top_k, mass_aware, eps):
    slot_in = init_slot.to(torch.float32).contiguous()
    mass_in = init_mass.to(torch.float32).contiguous()
    slot_out, mass_out = torch.empty_like(slot_in), torch.empty_like(mass_in)
    y = gsu_forward_impl(addr_idx, addr_val, x, gamma, slot_in, mass_in, slot_out, mass_out, mask, w_top_k, r_top_k,
                         mass_aware, eps)
    return y, slot_out, mass_out


@torch.library.impl(_lib, "gsu_forward_", "CUDA")
def _gsu_forward_(addr_idx, addr_val, x, gamma, slot, mass, mask, w_top_k, r_top_k, mass_aware, eps):
    return gsu_forward_impl(addr_idx, addr_val, x, gamma, slot, mass, slot, mass, mask, w_top_k, r_top_k, mass_aware, eps)


def _rows_as_given(t: torch.Tensor) -> torch.Tensor:
    """(B,H,T,C) tensor as the backward kernels take it: any batch / head / token strides (a token-major tensor
    seen head-major needs no copy), channels contiguous, rows aligned to four elements."""
    ok = t.stride(-1) == 1 and all(st % 4 == 0 for st in t.stride()[:3]) and t.data_ptr() % (4 * t.element_size()) == 0
    return t if ok else t.contiguous()


def _pad_channels(t: torch.Tensor, C4: int) -> torch.Tensor:
    C = t.shape[-1]
    return t if C == C4 else torch.nn.functional.pad(t, (0, C4 - C))


@torch.library.impl(_lib, "gsu_backward", "CUDA")
def _gsu_backward(addr_idx, addr_val, x, gamma, init_slot, init_mass, mask, D_y, D_post_slot, D_post_mass, w_top_k,
                  r_top_k, mass_aware, eps):
    """(D_val (B,H,Kw+Kr,T) w.r.t. positive weights, D_x in x.dtype, D_gamma fp32, D_slot, D_mass)."""
    _require_cuda(addr_idx, addr_val, x, gamma, init_slot, init_mass, D_y, D_post_slot, D_post_mass)
    B, H, T, C = x.shape
    A = init_slot.shape[2]
    K = w_top_k + r_top_k
    C4 = (C + 3) // 4 * 4  # the kernels move channels in groups of four
    if addr_val.stride() != addr_idx.stride():
        addr_idx, addr_val = addr_idx.contiguous(), addr_val.contiguous()
    xs = _rows_as_given(_pad_channels(x, C4))
    dy = _rows_as_given(_pad_channels(D_y.to(x.dtype), C4))
    slot_in = _pad_channels(init_slot.to(torch.float32), C4).contiguous()
    mass_in = init_mass.to(torch.float32).contiguous()
    d_slot_post = _pad_channels(D_post_slot.to(torch.float32), C4).contiguous()
    d_mass_post = D_post_mass.to(torch.float32).contiguous()
    d_val = torch.zeros((B, T, H, K), dtype=torch.float32, device=x.device).permute(0, 2, 3, 1)
    d_x = torch.empty_like(xs)  # in the layout of x: a token-major x gets a token-major gradient, which autograd can hand on as it is
    d_gamma = torch.empty((B, H, T), dtype=torch.float32, device=x.device)
    d_slot, d_mass = torch.empty_like(slot_in), torch.empty_like(mass_in)
    if x.numel() == 0:
        return d_val, torch.empty_like(x), d_gamma, d_slot_post[..., :C].clone(), d_mass_post.clone()
    mask_u8 = None if mask is None else mask.to(torch.bool).view(torch.uint8)
    nbytes = lib.rn_gsu_bwd_workspace_bytes(B, H, T, A, C4, w_top_k, r_top_k, x.device.index)
    if nbytes < 0:
        check(1)
    ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=x.device)
    check(lib.rn_gsu_bwd(ptr(addr_idx), ptr(addr_val), strides(addr_idx), ptr(xs), strides(xs), ptr(gamma), strides(gamma),
                         dtype_code(xs), ptr(mask_u8), None if mask_u8 is None else strides(mask_u8), ptr(slot_in),
                         ptr(mass_in), ptr(dy), strides(dy), ptr(d_slot_post), ptr(d_mass_post), ptr(d_val), strides(d_val),
                         ptr(d_x), strides(d_x), ptr(d_gamma), ptr(d_slot), ptr(d_mass), ptr(ws), int(nbytes), B, H, T, A,
                         C4, w_top_k, r_top_k, int(mass_aware), float(eps), x.device.index, stream_of(x)))
    check_device(d_val)
    if C4 != C:  # results of the padded run: hand back dense tensors, as the fake kernel promises
        return d_val, torch.empty_like(x).copy_(d_x[..., :C]), d_gamma, d_slot[..., :C].contiguous(), d_mass
    return d_val, d_x, d_gamma, d_slot, d_mass


# ----------------------------------------------------------------------------------------------
# event / segment formulation (reference schemas, packages/ramnet-ops/csrc/ram_attn_bind.cpp:69-91)
# ----------------------------------------------------------------------------------------------
def _events_to_token_major(seg_idx, seg_off, seg_len, event_i, event_v, B, H, T, K, A):
    """Rebuild (idx, val) of shape (B,H,K,T) from the grouped-event tables.

    Events sit in ``event_i`` grouped by segment: positions [seg_off[s], seg_off[s] + seg_len[s]) belong to
    slot ``seg_idx[s]``; positions covered by no segment are masked events (they become no-ops).  Event ids
    flatten (b, h, t, k) with k fastest, which is exactly the token-major storage the kernels read.
    Static shapes only, no host synchronisation."""
    N = event_i.numel()
    dev = event_i.device
    pos = torch.arange(N, device=dev, dtype=torch.int64)
    live_seg = seg_len > 0
    starts = torch.where(live_seg, seg_off.to(torch.int64), torch.full_like(seg_off, N, dtype=torch.int64))
    # tables indexed by sorted position: slot + 1 and end of the segment that starts there
    slot_at = torch.zeros(N + 1, dtype=torch.int64, device=dev).scatter_(0, starts, seg_idx.to(torch.int64) + 1)
    end_at = torch.zeros(N + 1, dtype=torch.int64, device=dev).scatter_(0, starts, (seg_off + seg_len).to(torch.int64))
    start_of = torch.where(slot_at[:N] > 0, pos, torch.zeros_like(pos)).cummax(dim=0).values
    slot = slot_at[start_of] - 1
    covered = (slot >= 0) & (pos < end_at[start_of])
    idx_flat = torch.zeros(N, dtype=torch.int32, device=dev)
    val_flat = torch.zeros(N, dtype=torch.float32, device=dev)
    where = event_i.to(torch.int64)
    idx_flat.scatter_(0, where, torch.where(covered, slot, torch.zeros_like(slot)).to(torch.int32))
    val_flat.scatter_(0, where, torch.where(covered, event_v.to(torch.float32), torch.zeros_like(val_flat)))
    shape = (B, H, T, K)
    return idx_flat.view(shape).permute(0, 1, 3, 2), val_flat.view(shape).permute(0, 1, 3, 2)


def _event_values(addr_val, event_i):
    return addr_val.transpose(-2, -1).reshape(-1).index_select(0, event_i.to(torch.int64))


def is_direct(seg_off: torch.Tensor) -> bool:
    """The update / read operators under the reference's names accept two calling conventions.  SEGMENT form
    (the reference's): seg_idx / seg_off / seg_len / event_i are the tables of ``gather_segment``.  DIRECT form
    (this package's own path): ``seg_off`` and ``seg_len`` are empty, ``seg_idx`` is the decoded index tensor
    (B,H,Kw+Kr,T) itself and ``event_i`` is the token mask (B,T) as uint8, or empty for no mask; y then comes
    back in the dtype of x, stored token-major, and the replay-cache output is empty."""
    return seg_off.numel() == 0


def _direct_mask(event_i: torch.Tensor):
    return None if event_i.numel() == 0 else event_i


@torch.library.impl(_lib, "topk_segment_forward", "CUDA")
def _topk_segment_forward(addr_val, seg_idx, seg_off, seg_len, event_i, x, gamma, init_slot, init_mass, w_top_k, r_top_k,
                          mass_aware, eps):
    if is_direct(seg_off):
        y, slot, mass = _gsu_forward(seg_idx, addr_val, x, gamma, init_slot, init_mass, _direct_mask(event_i), w_top_k,
                                     r_top_k, mass_aware, eps)
        return y, slot, mass, addr_val.new_empty(0)
    B, H, T, C = x.shape
    A = init_slot.shape[2]
    event_v = _event_values(addr_val, event_i)
    idx, val = _events_to_token_major(seg_idx, seg_off, seg_len, event_i, event_v, B, H, T, w_top_k + r_top_k, A)
    y, slot, mass = _gsu_forward(idx, val, x, gamma, init_slot, init_mass, None, w_top_k, r_top_k, mass_aware, eps)
    return y.to(torch.float32).contiguous(), slot, mass, event_v


@torch.library.impl(_lib, "topk_segment_forward_", "CUDA")
def _topk_segment_forward_(addr_val, seg_idx, seg_off, seg_len, event_i, x, gamma, slot, mass, w_top_k, r_top_k,
                           mass_aware, eps):
    if is_direct(seg_off):
        return gsu_forward_impl(seg_idx, addr_val, x, gamma, slot, mass, slot, mass, _direct_mask(event_i), w_top_k, r_top_k,
                                mass_aware, eps)
    B, H, T, C = x.shape
    event_v = _event_values(addr_val, event_i)
    idx, val = _events_to_token_major(seg_idx, seg_off, seg_len, event_i, event_v, B, H, T, w_top_k + r_top_k, slot.shape[2])
    y = gsu_forward_impl(idx, val, x, gamma, slot, mass, slot, mass, None, w_top_k, r_top_k, mass_aware, eps)
    return y.to(torch.float32).contiguous()


@torch.library.impl(_lib, "topk_segment_backward", "CUDA")
def _topk_segment_backward(seg_idx, seg_off, seg_len, event_i, event_v, x, gamma, init_slot, init_mass, D_y, D_post_slot,
                           D_post_mass, w_top_k, r_top_k, mass_aware, eps):
    if is_direct(seg_off):  # event_v carries the decoded weights (B,H,Kw+Kr,T)
        return _gsu_backward(seg_idx, event_v, x, gamma, init_slot, init_mass, _direct_mask(event_i), D_y.to(x.dtype),
                             D_post_slot, D_post_mass, w_top_k, r_top_k, mass_aware, eps)
    B, H, T, C = x.shape
    idx, val = _events_to_token_major(seg_idx, seg_off, seg_len, event_i, event_v, B, H, T, w_top_k + r_top_k,
                                      init_slot.shape[2])
    d_val, d_x, d_gamma, d_slot, d_mass = _gsu_backward(idx, val, x, gamma, init_slot, init_mass, None, D_y.to(x.dtype),
                                                        D_post_slot, D_post_mass, w_top_k, r_top_k, mass_aware, eps)
    return d_val.contiguous(), d_x.to(torch.float32).contiguous(), d_gamma, d_slot, d_mass
