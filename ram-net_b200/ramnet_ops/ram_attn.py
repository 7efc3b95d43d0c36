"""Public operator API of ramnet_ops (call-compatible with the reference package's
``packages/ramnet-ops/src/ramnet_ops/ram_attn.py``): ``random_access_memory_attention`` and
``topk_addr``.

CUDA tensors go to the sm_100a kernels behind ``torch.ops.ramnet_ops`` (there is no silent
fallback: an unavailable CUDA backend raises); ``impl_backend='torch'`` selects the dense PyTorch
formulation in ``impl/torch_impl.py`` explicitly.
"""
from __future__ import annotations

import warnings
from typing import Callable, Literal

import torch

from .impl.torch_impl import _torch_ram_attn, _torch_topk_addr

_triton_ram_attn = None
_cuda_load_error: Exception | None = None
try:
    from .impl.cuda_impl import _cuda_ram_attn, _cuda_topk_addr
except Exception as exc:  # pragma: no cover - exercised only without the built library
    _cuda_load_error = exc
    warnings.warn(f"Failed to load the CUDA implementation: {exc}. Build it with `python ram-net_b200/build.py`.")
    _cuda_ram_attn = None
    _cuda_topk_addr = None

ImplCallableType = Callable[..., tuple[torch.Tensor, torch.Tensor, torch.Tensor]]

_CUDA_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def get_broadcast(*vals: int) -> int:
    """The one non-singleton size among broadcast-compatible sizes (1 if all are 1)."""
    sizes = {v for v in vals if v != 1}
    assert len(sizes) <= 1, f"Cannot broadcast {vals}"
    return sizes.pop() if sizes else 1


def topk_addr(
        addr: torch.Tensor,
        embed_num: int,
        position_ids: torch.Tensor,
        top_k: int,
        top_k_re_norm: float,
        addr_val_neg: bool = False,
        encode_batch_idx: bool = True,
        impl_backend: Literal['torch', 'cuda'] | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-K address decoding.

    :param addr: address logits (B, H, U, P, T); A = P ** U slots per head.
    :param embed_num: number of leading heads that get the CAPE cyclic shift, in ``[0, H]``.
    :param position_ids: token positions (B, T).
    :param top_k: addresses kept per token and head, in ``[1, A]``.
    :param top_k_re_norm: rho in [0, 1]; kept probabilities q become q / sum(q) ** rho.
    :param addr_val_neg: return the weights negated.
    :param encode_batch_idx: indices are ``(b * H + h) * A + a`` (True) or ``h * A + a`` (False).
    :param impl_backend: 'torch', 'cuda' or None (CUDA tensors of a supported dtype use 'cuda').
    :return: ``(idx, val)``, both (B, H, K, T); int32 indices and float32 weights.  Entry k is
        the k-th address under (score descending, content index ascending).
    """
    assert isinstance(addr, torch.Tensor), f"Expected addr to be Tensor, got {type(addr).__name__}."
    if not isinstance(top_k_re_norm, (int, float)):
        raise TypeError("`top_k_re_norm` must be a number in [0, 1].")
    if not 0 <= top_k_re_norm <= 1:
        raise ValueError("`top_k_re_norm` must be in [0, 1].")
    if impl_backend not in (None, 'torch', 'cuda'):
        raise ValueError(f"Unsupported impl_backend: {impl_backend!r}.")

    if impl_backend is None:
        impl_backend = 'torch'
        if addr.is_cuda:
            if _cuda_topk_addr is not None and addr.dtype in _CUDA_DTYPES:
                impl_backend = 'cuda'
            else:
                warnings.warn("CUDA address decoder is unavailable for this input; falling back to Torch, "
                              "which materializes all P ** U address scores.")
    if impl_backend == 'cuda' and _cuda_topk_addr is None:
        raise RuntimeError("CUDA address decoder is unavailable.") from _cuda_load_error

    func = _cuda_topk_addr if impl_backend == 'cuda' else _torch_topk_addr
    return func(addr, embed_num, position_ids, top_k, float(top_k_re_norm), addr_val_neg, encode_batch_idx)


def _pair(value, kind, name):
    """Normalise a scalar-or-pair option to a 2-tuple; TypeError on anything else."""
    message = {
        "top_k": "`top_k` must be int, a two-item tuple/list of ints, or None.",
        "top_k_re_norm": "`top_k_re_norm` must be a number or a two-item tuple/list of numbers in [0, 1].",
    }[name]
    if isinstance(value, kind):
        return (value, value)
    if isinstance(value, (tuple, list)) and len(value) == 2 and all(isinstance(v, kind) for v in value):
        return tuple(value)
    raise TypeError(message)


def random_access_memory_attention(
        w_addr: torch.Tensor,
        r_addr: torch.Tensor,
        values: torch.Tensor,
        gamma: torch.Tensor | float = 0.0,
        init_ram: tuple[torch.Tensor | None, torch.Tensor | float | None] | None = None,
        mask: torch.Tensor | None = None,
        embed_num: int = 0,
        position_ids: torch.Tensor | None = None,
        top_k: tuple[int, int] | list[int] | int | None = 8,
        top_k_re_norm: float | tuple[float, float] | list[float] = 0.0,
        mass_aware: bool = False,
        eps: float = 1e-12,
        t_dim: int = 1,
        inplace: bool = False,
        impl_backend: Literal['torch', 'triton', 'cuda'] | None = None,
) -> tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor]]:
    """Random-access memory attention.

    :param w_addr: write address logits (..., T, ..., H, U, P).
    :param r_addr: read address logits (..., T, ..., H, U, P).
    :param values: values to write (..., T, ..., H, C).
    :param gamma: forget-rate control (..., T, ..., H) or a scalar; > 0 forgets faster.
    :param init_ram: previous ``(slot, mass)``; slot may be None, mass a tensor, scalar or None.
    :param mask: valid-token mask broadcastable to position_ids; False tokens leave the state alone.
    :param embed_num: number of leading heads with the CAPE cyclic shift, in ``[0, H]``.
    :param position_ids: token positions broadcastable to (..., T, ...); default ``arange(T)``.
    :param top_k: Top-K for write and read (int, or ``(write_k, read_k)``); None = dense (torch only).
    :param top_k_re_norm: rho in [0, 1] (number, or ``(write, read)``): q -> q / sum(q) ** rho.
    :param mass_aware: weight reads by the updated slot mass.
    :param eps: strictly positive stabiliser.
    :param t_dim: index of the time axis.
    :param inplace: update ``init_ram`` tensors in place (no autograd).
    :param impl_backend: 'torch', 'cuda' ('triton' is accepted for API parity but not provided) or None.
    :return: ``(output, (slot, mass))`` shaped like values, (..., H, P**U, C) and (..., H, P**U).
    """
    assert all(isinstance(v, torch.Tensor) for v in (r_addr, w_addr, values)), \
        f"Expected r_addr/w_addr/values to be tensors, got {type(r_addr).__name__}, {type(w_addr).__name__}, {type(values).__name__}."
    if init_ram is None:
        init_slot = init_mass = None
    elif isinstance(init_ram, tuple) and len(init_ram) == 2:
        init_slot, init_mass = init_ram
    else:
        raise TypeError("init_ram must be a (slot, mass) tuple or None.")

    T_ = torch.Tensor
    assert init_slot is None or isinstance(init_slot, T_), f"Expected init_slot to be Tensor or None, got {type(init_slot).__name__}."
    assert init_mass is None or isinstance(init_mass, (T_, int, float)), f"Expected init_mass to be Tensor, scalar, or None, got {type(init_mass).__name__}."
    assert isinstance(gamma, (T_, int, float)), f"Expected gamma to be Tensor or scalar, got {type(gamma).__name__}."
    assert position_ids is None or isinstance(position_ids, T_), f"Expected position_ids to be Tensor or None, got {type(position_ids).__name__}."
    assert mask is None or isinstance(mask, T_), f"Expected mask to be Tensor or None, got {type(mask).__name__}."
    assert isinstance(t_dim, int), f"Expected t_dim to be int, got {type(t_dim).__name__}."
    assert isinstance(embed_num, int) and embed_num >= 0, f"Expected embed_num >= 0, got {embed_num!r}."
    assert isinstance(eps, (int, float)) and eps > 0, f"Expected eps > 0, got {eps!r}."
    assert isinstance(mass_aware, bool), f"Expected mass_aware to be bool, got {type(mass_aware).__name__}."
    assert not inplace or (isinstance(init_slot, T_) and isinstance(init_mass, T_)), \
        f"inplace=True requires Tensor state, got slot={type(init_slot).__name__}, mass={type(init_mass).__name__}."

    # (name, tensor, trailing non-time dims, minimal ndim)
    timed = [("w_addr", w_addr, 3, 4), ("r_addr", r_addr, 3, 4), ("values", values, 2, 3)]
    if isinstance(gamma, T_):
        timed.append(("gamma", gamma, 1, 2))
    if isinstance(position_ids, T_):
        timed.append(("position_ids", position_ids, 0, 1))
    if isinstance(mask, T_):
        timed.append(("mask", mask, 0, 1))
    for name, tensor, _, min_ndim in timed:
        assert tensor.ndim >= min_ndim, f"Expected {name}.ndim >= {min_ndim}, got shape={tuple(tensor.shape)}."
    assert not isinstance(init_slot, T_) or init_slot.ndim >= 3, f"Expected init_slot.ndim >= 3, got shape={tuple(init_slot.shape)}."
    assert not isinstance(init_mass, T_) or init_mass.ndim >= 2, f"Expected init_mass.ndim >= 2, got shape={tuple(init_mass.shape)}."
    for name, tensor, trailing, _ in timed:
        assert -tensor.ndim <= t_dim < tensor.ndim and t_dim % tensor.ndim < tensor.ndim - trailing, \
            f"t_dim={t_dim} does not select the time dimension of {name} with shape {tuple(tensor.shape)}."

    assert w_addr.is_floating_point() and r_addr.is_floating_point() and values.is_floating_point(), \
        f"Expected floating-point addresses/values, got {w_addr.dtype=}, {r_addr.dtype=}, {values.dtype=}."
    assert w_addr.dtype == r_addr.dtype == values.dtype, f"Expected matching dtypes, got {w_addr.dtype=}, {r_addr.dtype=}, {values.dtype=}."
    assert not isinstance(gamma, T_) or gamma.dtype == values.dtype, f"Expected gamma.dtype={values.dtype}, got {gamma.dtype}."

    # backend layout: time last for logits / gamma / positions / mask, second to last for values
    w_addr = w_addr.movedim(t_dim, -1)
    r_addr = r_addr.movedim(t_dim, -1)
    values = values.movedim(t_dim, -2)
    if isinstance(gamma, T_):
        gamma = gamma.movedim(t_dim, -1)
    if isinstance(position_ids, T_):
        position_ids = position_ids.movedim(t_dim, -1)
    if isinstance(mask, T_):
        mask = mask.movedim(t_dim, -1)

    slot_shape = tuple(init_slot.shape) if isinstance(init_slot, T_) else (1, 1, 1)
    mass_shape = tuple(init_mass.shape) if isinstance(init_mass, T_) else (1, 1)
    gamma_shape = tuple(gamma.shape) if isinstance(gamma, T_) else (1, 1)
    pos_shape = tuple(position_ids.shape) if isinstance(position_ids, T_) else (1,)
    mask_shape = tuple(mask.shape) if isinstance(mask, T_) else (1,)
    batch_shape = torch.broadcast_shapes(w_addr.shape[:-4], r_addr.shape[:-4], values.shape[:-3], gamma_shape[:-2],
                                         slot_shape[:-3], mass_shape[:-2], pos_shape[:-1], mask_shape[:-1])
    H = get_broadcast(w_addr.size(-4), r_addr.size(-4), values.size(-3), gamma_shape[-2], slot_shape[-3], mass_shape[-2])
    U = get_broadcast(w_addr.size(-3), r_addr.size(-3))
    P = get_broadcast(w_addr.size(-2), r_addr.size(-2))
    A = get_broadcast(slot_shape[-2], mass_shape[-1], P ** U)
    C = get_broadcast(values.size(-1), slot_shape[-1])
    T = get_broadcast(w_addr.size(-1), r_addr.size(-1), values.size(-2), gamma_shape[-1], pos_shape[-1], mask_shape[-1])
    assert all(size > 0 for size in (H, U, P, A, C, T)), f"RAM dimensions must be positive, got {H=}, {U=}, {P=}, {A=}, {C=}, {T=}."
    assert embed_num <= H, f"embed_num must not exceed H={H}, but got {embed_num}."
    if inplace:
        want_slot, want_mass = (*batch_shape, H, A, C), (*batch_shape, H, A)
        assert tuple(init_slot.shape) == want_slot and tuple(init_mass.shape) == want_mass, \
            f"inplace=True expects slot.shape={want_slot}, mass.shape={want_mass}; got {tuple(init_slot.shape)} and {tuple(init_mass.shape)}."
        assert init_slot.is_contiguous() and init_mass.is_contiguous(), \
            f"inplace=True requires contiguous init_ram tensors, got slot{init_slot.is_contiguous()=} and mass{init_mass.is_contiguous()=}."

    # defaults
    if not isinstance(gamma, T_):
        gamma = values.new_full((*batch_shape, H, 1), gamma).expand(*batch_shape, H, T)
    # A default state is created in the dtype the CUDA backend keeps state in (float32 for 16-bit values), so that
    # the backend does not convert a fresh 16-bit tensor of A*C zeros per head first
    state_dtype = values.dtype
    if impl_backend in (None, 'cuda') and values.is_cuda and values.dtype in (torch.float16, torch.bfloat16):
        state_dtype = torch.float32
    if not isinstance(init_slot, T_):
        init_slot = values.new_zeros(*batch_shape, H, A, C, dtype=state_dtype)
    if not isinstance(init_mass, T_):
        init_mass = values.new_full((*batch_shape, H, A), 1.0 / (P ** U) if init_mass is None else init_mass, dtype=state_dtype)
    if not isinstance(position_ids, T_):
        position_ids = torch.arange(T, device=values.device, dtype=torch.long).view(*([1] * len(batch_shape)), T)
    else:
        position_ids = position_ids.to(device=values.device)
    if isinstance(mask, T_):
        mask = mask.to(device=values.device, dtype=torch.bool)

    w_addr = w_addr.broadcast_to([*batch_shape, H, U, P, T])
    r_addr = r_addr.broadcast_to([*batch_shape, H, U, P, T])
    values = values.broadcast_to([*batch_shape, H, T, C])
    gamma = gamma.broadcast_to([*batch_shape, H, T])
    init_slot = init_slot.broadcast_to([*batch_shape, H, A, C])
    init_mass = init_mass.broadcast_to([*batch_shape, H, A])
    position_ids = position_ids.broadcast_to([*batch_shape, T])
    if isinstance(mask, T_):
        mask = mask.broadcast_to([*batch_shape, T])

    devices = {t.device for t in (w_addr, r_addr, values, gamma, init_slot, init_mass, position_ids)}
    assert len(devices) == 1, \
        f"Expected one device, got w={w_addr.device}, r={r_addr.device}, values={values.device}, gamma={gamma.device}, slot={init_slot.device}, mass={init_mass.device}, position_ids={position_ids.device}."
    assert mask is None or mask.device == position_ids.device, f"Expected mask.device={position_ids.device}, got {mask.device}."

    # one flat batch axis for the backends
    w_addr = w_addr.reshape(-1, H, U, P, T)
    r_addr = r_addr.reshape(-1, H, U, P, T)
    values = values.reshape(-1, H, T, C)
    gamma = gamma.reshape(-1, H, T)
    init_slot = init_slot.reshape(-1, H, A, C)
    init_mass = init_mass.reshape(-1, H, A)
    position_ids = position_ids.reshape(-1, T)
    if isinstance(mask, T_):
        mask = mask.reshape(-1, T)

    if top_k is not None:
        top_k = _pair(top_k, int, "top_k")
        assert all(0 < k <= P ** U for k in top_k), f"top_k values must be in the range (0, {P ** U}], but got {top_k}"
    top_k_re_norm = _pair(top_k_re_norm, (int, float), "top_k_re_norm")
    if not all(0 <= v <= 1 for v in top_k_re_norm):
        raise ValueError("`top_k_re_norm` exponents must be in [0, 1].")
    top_k_re_norm = tuple(float(v) for v in top_k_re_norm)

    if impl_backend not in (None, 'torch', 'triton', 'cuda'):
        raise ValueError(f"Unsupported impl_backend: {impl_backend!r}.")
    if impl_backend is None:
        impl_backend = 'torch'
        if values.is_cuda:
            if _cuda_ram_attn is not None and top_k is not None and values.dtype in _CUDA_DTYPES:
                impl_backend = 'cuda'
            elif _triton_ram_attn is not None and top_k is None:
                impl_backend = 'triton'
            if impl_backend != 'cuda':
                warnings.warn(
                    f"CUDA backend is unavailable for this input/configuration; falling back to {impl_backend}. "
                    "Input is a CUDA tensor, so this may significantly reduce performance and increase GPU memory usage. "
                    "Check your ramnet-ops installation, or manually set 'impl_backend' to suppress this warning.")
    if inplace and impl_backend not in ('torch', 'cuda'):
        raise ValueError("inplace=True is only supported by the Torch backend and CUDA top-k backend.")
    if impl_backend == 'cuda' and _cuda_ram_attn is None:
        raise RuntimeError("CUDA RAM attention backend is unavailable.") from _cuda_load_error
    if impl_backend == 'triton' and _triton_ram_attn is None:
        raise RuntimeError("This build has no Triton backend; use impl_backend='cuda' or 'torch'.")
    func: ImplCallableType = {'torch': _torch_ram_attn, 'cuda': _cuda_ram_attn, 'triton': _triton_ram_attn}[impl_backend]

    y, slot, mass = func(w_addr, r_addr, values, gamma, init_slot, init_mass, mask, embed_num, position_ids,
                         top_k, top_k_re_norm, mass_aware, eps, inplace)

    y = y.reshape(*batch_shape, H, T, C).movedim(-2, t_dim)
    return y, (slot.reshape(*batch_shape, H, A, C), mass.reshape(*batch_shape, H, A))
