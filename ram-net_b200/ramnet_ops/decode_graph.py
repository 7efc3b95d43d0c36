"""Decode loop under a CUDA graph.

One autoregressive step of the slot memory is a single small kernel (tens of microseconds); launched
from Python the host cost of a step is of the same size, so a generation loop is host bound.  This
module captures ``n`` consecutive steps -- the fused decode operator on static input buffers plus the
on-device increment of the position counter -- into one CUDA graph that is replayed with one launch.

It plays the role of the static-state decode loop of the reference's cache
(packages/ramnet/src/ramnet/layers/cache.py:33-50,123-130: ``RAMCache.update`` keeps ``slot``/``mass`` and a
``next_position`` counter per layer; packages/ramnet/src/ramnet/layers/ram_attn_block.py:324-350 calls the
in-place operator once per token and then the layer epilogue): the slot and mass tensors are updated in place,
the position lives on the device, and the caller only refreshes the input buffers between replays.  For a whole
model see ``ramnet_ops.layers.GreedyGraphDecoder``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _ops  # noqa: F401  (registers torch.ops.ramnet_ops.*)


class DecodeGraph:
    """``n`` decode steps of one RAM-Net layer as a replayable CUDA graph.

    Static buffers (the caller writes new values into them between replays):
      ``w_addr``, ``r_addr``  (n, B, H, U, P)   write / read address logits of each step
      ``x``                   (n, B, H, C)      values
      ``gamma``               (n, B, H)         forget gate values, as the operator takes them
      ``gate_logits``         (n, B, H, C)      optional: sigmoid gate of the fused epilogue
    State updated in place by every replay: ``slot`` (B, H, A, C) fp32, ``mass`` (B, H, A) fp32 and
    ``position_ids`` (B,) int32, which is advanced by one after every step.
    ``outputs[j]`` is the (B, H, C) result of step ``j`` of the latest replay.
    """

    def __init__(self, w_addr: torch.Tensor, r_addr: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor,
                 slot: torch.Tensor, mass: torch.Tensor, position_ids: torch.Tensor, *, embed_num: int, top_k: int,
                 read_top_k: Optional[int] = None, w_re_norm: float = 0.0, r_re_norm: float = 0.0,
                 mass_aware: bool = False, eps: float = 1e-12, mask: Optional[torch.Tensor] = None,
                 norm_weight: Optional[torch.Tensor] = None, gate_logits: Optional[torch.Tensor] = None,
                 norm_eps: float = 1e-6, warmup: int = 2):
        if not w_addr.is_cuda:
            raise RuntimeError("DecodeGraph needs CUDA tensors (there is no CPU path)")
        if w_addr.dim() != 5 or r_addr.shape != w_addr.shape:
            raise ValueError("w_addr / r_addr must be (n, B, H, U, P)")
        n = w_addr.shape[0]
        if x.shape[0] != n or gamma.shape[0] != n or (gate_logits is not None and gate_logits.shape[0] != n):
            raise ValueError("all per-step buffers must have the same leading length n")
        if position_ids.dtype != torch.int32:
            raise TypeError("position_ids must be int32")
        self.n = n
        self.w_addr, self.r_addr, self.x, self.gamma = w_addr, r_addr, x, gamma
        self.slot, self.mass, self.position_ids = slot, mass, position_ids
        self.gate_logits = gate_logits
        self.outputs: List[torch.Tensor] = []
        self._mask = mask if mask is not None else torch.empty(0, dtype=torch.bool, device=w_addr.device)
        rk = top_k if read_top_k is None else read_top_k
        fused = norm_weight is not None or gate_logits is not None
        ops = torch.ops.ramnet_ops

        def step(j: int, bsel=slice(None), state=None) -> torch.Tensor:
            sl, ms, pos = state if state is not None else (slot, mass, position_ids)
            msk = self._mask if self._mask.numel() == 0 else self._mask[bsel]
            if fused:
                y = ops.decode_fused_(w_addr[j][bsel], r_addr[j][bsel], x[j][bsel], gamma[j][bsel], sl, ms, msk,
                                      embed_num, pos, top_k, rk, w_re_norm, r_re_norm, mass_aware, eps, norm_weight,
                                      None if gate_logits is None else gate_logits[j][bsel], norm_eps)
            else:
                y = ops.topk_autoregressive_(w_addr[j][bsel], r_addr[j][bsel], x[j][bsel], gamma[j][bsel], sl, ms, msk,
                                             embed_num, pos, top_k, rk, w_re_norm, r_re_norm, mass_aware, eps)
            pos.add_(1)
            return y

        # Warm-up on a side stream (lazy initialisation must not happen under capture), on a copy of the
        # first batch row only, so constructing the graph leaves slot / mass / position as they were.
        if warmup > 0:
            one = slice(0, 1)
            scratch = (slot[one].clone(), mass[one].clone(), position_ids[one].clone())
            side = torch.cuda.Stream(device=w_addr.device)
            side.wait_stream(torch.cuda.current_stream(w_addr.device))
            with torch.cuda.stream(side):
                for j in range(min(warmup, n)):
                    step(j, one, scratch)
            torch.cuda.current_stream(w_addr.device).wait_stream(side)
            del scratch
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):  # records the launches; nothing runs until replay()
            self.outputs = [step(j) for j in range(n)]

    def replay(self) -> List[torch.Tensor]:
        """Run the ``n`` captured steps on the current contents of the static buffers."""
        self.graph.replay()
        return self.outputs
