"""Glue between the reference MODEL package (``ramnet``) and this package's fused decode entry.

The reference attention layer runs, per decode step and layer, the operator followed by three small
elementwise kernels (head-wise RMSNorm, sigmoid of the gate projection, multiply) and rebuilds the
position tensors of its cache on every call
(packages/ramnet/src/ramnet/layers/ram_attn_block.py:226-277,309-350,
 packages/ramnet/src/ramnet/layers/cache.py:33-50,123-130).  Here:

* ``fused_attention_class()`` returns a subclass of ``ramnet.layers.RAMNetAttention`` whose one-token
  step calls ``torch.ops.ramnet_ops.decode_fused_`` (address decode + gated update + read + RMSNorm +
  sigmoid gate in ONE kernel) and advances the cache's position tensor in place, so the step has
  fixed tensor addresses and can be replayed from a CUDA graph.  Everything else (prefill, training,
  masks, explicit positions) goes through the parent class unchanged.
* ``use_fused_attention(model)`` switches every ``RAMNetAttention`` of a model to that class
  (weights untouched).
* ``GreedyGraphDecoder`` captures one greedy decode step of a ``RAMNetForCausalLM`` (all layers, LM
  head, argmax) into a CUDA graph over the model's ``RAMCache`` and replays it per generated token.

The reference package is imported lazily: nothing here is needed by the operators themselves.
"""
from __future__ import annotations

import torch

_FUSED_CLASS = None


def _pair(top_k):
    if isinstance(top_k, int):
        return top_k, top_k
    if isinstance(top_k, (tuple, list)) and len(top_k) == 2 and all(isinstance(k, int) for k in top_k):
        return int(top_k[0]), int(top_k[1])
    return None


def fused_attention_class():
    """``ramnet.layers.RAMNetAttention`` with the fused one-token step (built on first use)."""
    global _FUSED_CLASS
    if _FUSED_CLASS is not None:
        return _FUSED_CLASS
    from ramnet.layers import RAMNetAttention, RAMState  # the reference model package

    import ramnet_ops  # noqa: F401  (registers torch.ops.ramnet_ops.*)

    class FusedRAMNetAttention(RAMNetAttention):
        """Drop-in for RAMNetAttention; same parameters, same state dict."""

        def _fused_step_ok(self, hidden_states, init_ram, t_dim, inplace) -> bool:
            if self.training or torch.is_grad_enabled() and any(p.requires_grad for p in (self.r_proj.weight, self.v_proj.weight)):
                return False
            if hidden_states.ndim != 3 or t_dim not in (1, -2) or hidden_states.size(1) != 1 or not hidden_states.is_cuda:
                return False
            if init_ram is None or inplace is False or _pair(self.top_k) is None:
                return False
            slot, mass = init_ram
            if not (isinstance(slot, torch.Tensor) and isinstance(mass, torch.Tensor)):
                return False
            if slot.dtype != torch.float32 or mass.dtype != torch.float32 or not (slot.is_contiguous() and mass.is_contiguous()):
                return False
            if slot.requires_grad or mass.requires_grad or hidden_states.requires_grad:
                return False
            if self.o_gate is not None and not isinstance(self.o_gate[1], torch.nn.Sigmoid):
                return False
            return hidden_states.dtype in (torch.float32, torch.float16, torch.bfloat16)

        def _step_constants(self, what, dtype, device, B):
            """Per-step tensors that depend on parameters only, computed as the parent class computes them and kept
            until a parameter changes (in-place updates bump ``_version``; a new tensor has a new ``data_ptr``):
            the learned address scales over the temperature, (H,U,1) each, and gamma expanded to (B,H).  One token
            step then multiplies and launches, instead of re-deriving them with half a dozen small kernels."""
            params = [p for p in (self.r_scale, self.w_scale, getattr(self, "gamma_modifier", None),
                                  getattr(getattr(self, "gamma_modifier", None), "bias", None)) if isinstance(p, torch.Tensor)]
            key = (what, dtype, device, B, float(self.addr_temperature), tuple((p.data_ptr(), p._version) for p in params))
            cache = self.__dict__.setdefault("_rn_step_cache", {})
            hit = cache.get(what)
            if hit is not None and hit[0] == key:
                return hit[1]
            with torch.no_grad():
                if what == "scales":
                    value = ((torch.exp(self.r_scale) / self.addr_temperature).to(dtype=dtype).unsqueeze(-1).contiguous(),
                             (torch.exp(self.w_scale) / self.addr_temperature).to(dtype=dtype).unsqueeze(-1).contiguous())
                elif what == "gamma_bias":
                    value = (self.gamma_modifier.bias + self.gamma).contiguous()
                elif self.gamma_mode == 'learnable':
                    value = (self.gamma_modifier + self.gamma).to(dtype=dtype).expand(B, self.n_heads).contiguous()
                else:
                    value = torch.full((B, self.n_heads), float(self.gamma), dtype=dtype, device=device)
            cache[what] = (key, value)
            return value

        def _merged_projection(self, h):
            """(r_addr (B,H,U,P), w_addr, values (B,H,C), gate logits or None, dynamic gamma (B,H) or None) from one
            GEMM over the concatenated projection weights, or None when the modules are not plain ``Linear``.  The
            concatenation is kept until a weight or bias changes."""
            H, U, P, C = self.n_heads, self.addr_order, self.addr_radix, self.value_chs
            mods = [self.r_proj, self.w_proj, self.v_proj]
            if self.o_gate is not None:
                mods.append(self.o_gate[0])
            dyn = self.gamma_mode == 'dynamic'
            if dyn:
                mods.append(self.gamma_modifier)
            if any(type(m) is not torch.nn.Linear for m in mods):
                return None
            tensors = [t for m in mods for t in (m.weight, m.bias) if t is not None]
            key = (h.dtype, h.device, float(self.gamma), tuple((t.data_ptr(), t._version) for t in tensors))
            cache = self.__dict__.setdefault("_rn_step_cache", {})
            hit = cache.get("merged")
            if hit is None or hit[0] != key:
                with torch.no_grad():
                    weight = torch.cat([m.weight for m in mods], dim=0).to(h.dtype)
                    # rows of the output a multiple of 16 bytes apart (zero rows appended), so that the column slices
                    # keep the alignment the vectorised decode kernels ask for
                    pad = (-weight.size(0)) % 8
                    if pad:
                        weight = torch.cat([weight, weight.new_zeros(pad, weight.size(1))], dim=0)
                    weight = weight.contiguous()
                    bias = None
                    if any(m.bias is not None for m in mods):
                        parts = [m.bias if m.bias is not None else m.weight.new_zeros(m.weight.shape[0]) for m in mods]
                        if dyn:  # the constant gamma rides on the bias of the gamma projection
                            parts[-1] = parts[-1] + self.gamma
                        if pad:
                            parts.append(parts[0].new_zeros(pad))
                        bias = torch.cat(parts).to(h.dtype).contiguous()
                    elif dyn and float(self.gamma) != 0.0:
                        return None
                hit = (key, (weight, bias))
                cache["merged"] = hit
            weight, bias = hit[1]
            z = torch.nn.functional.linear(h, weight, bias)
            B, n = h.size(0), H * U * P
            r_addr = z[:, :n].view(B, H, U, P)
            w_addr = z[:, n:2 * n].view(B, H, U, P)
            values = z[:, 2 * n:2 * n + H * C].view(B, H, C)
            off = 2 * n + H * C
            gate = None
            if self.o_gate is not None:
                gate = z[:, off:off + H * C].view(B, H, C)
                off += H * C
            gamma = z[:, off:off + H] if dyn else None
            return r_addr, w_addr, values, gate, gamma

        def forward_with_state(self, hidden_states, init_ram=None, mask=None, position_ids=None, t_dim=1, inplace=False):
            if not self._fused_step_ok(hidden_states, init_ram, t_dim, inplace):
                return super().forward_with_state(hidden_states, init_ram=init_ram, mask=mask, position_ids=position_ids,
                                                  t_dim=t_dim, inplace=inplace)
            slot, mass = init_ram
            B = hidden_states.size(0)
            H, U, P, C = self.n_heads, self.addr_order, self.addr_radix, self.value_chs
            h = hidden_states[:, 0]
            # The projections of the step (read / write logits, values, output gate, dynamic gamma) read the same
            # input: one GEMM over their concatenated weights instead of five small ones.  At one token per
            # sequence every GEMM is bound by reading its weights, and the small ones reach a fraction of the rate
            # of the merged one.
            merged = self._merged_projection(h)
            if merged is None:
                r_addr = self.r_proj(h).view(B, H, U, P)
                w_addr = self.w_proj(h).view(B, H, U, P)
                values = self.v_proj(h).view(B, H, C)
                gate_logits = None if self.o_gate is None else self.o_gate[0](h).view(B, H, C)
                gamma_dyn = None
            else:
                r_addr, w_addr, values, gate_logits, gamma_dyn = merged
            r_mul = w_mul = None
            if self.r_scale is not None:  # applied inside the kernel where it takes them, else by the operator
                r_mul, w_mul = self._step_constants("scales", r_addr.dtype, h.device, B)
            else:
                r_addr = r_addr / self.addr_temperature
                w_addr = w_addr / self.addr_temperature
            if self.gamma_mode == 'dynamic' and gamma_dyn is not None:
                gamma = gamma_dyn
            elif self.gamma_mode == 'dynamic':
                lin = self.gamma_modifier
                if lin.bias is None or type(lin) is not torch.nn.Linear:
                    gamma = lin(h) + self.gamma
                else:  # the constant is folded into the bias: one GEMM, no separate add
                    gamma = torch.nn.functional.linear(h, lin.weight, self._step_constants("gamma_bias", lin.bias.dtype, h.device, B))
            else:
                gamma = self._step_constants("gamma", values.dtype, h.device, B)
            if position_ids is None:
                position_ids = torch.zeros(B, 1, dtype=torch.long, device=h.device)
            pos = position_ids.reshape(B).to(torch.int32)
            step_mask = torch.empty(0, dtype=torch.bool, device=h.device) if mask is None else mask.reshape(B).to(torch.bool)
            norm_weight = None if self.o_norm is None else self.o_norm.weight
            norm_eps = 0.0
            if self.o_norm is not None:
                # torch.nn.RMSNorm(eps=None) takes the epsilon of the type it computes in, which is float32 for
                # 16-bit inputs (not the epsilon of the input dtype); y is small, so which of the two is used matters
                opmath = torch.float64 if values.dtype == torch.float64 else torch.float32
                norm_eps = float(self.o_norm.eps) if self.o_norm.eps is not None else float(torch.finfo(opmath).eps)
            w_k, r_k = _pair(self.top_k)
            y = torch.ops.ramnet_ops.decode_fused_(
                w_addr, r_addr, values, gamma.to(values.dtype), slot, mass,
                step_mask, self.embed_num, pos, w_k, r_k, float(self.top_k_re_norm[0]), float(self.top_k_re_norm[1]),
                bool(self.mass_aware), float(self.ram_attn_eps), norm_weight, gate_logits, norm_eps, w_mul, r_mul)
            return self.o_proj(y.reshape(B, 1, H * C)), RAMState(slot, mass)

        def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False,
                    output_attentions=False, position_ids=None):
            layer = None
            if (use_cache and past_key_values is not None and self.layer_idx is not None and not output_attentions
                    and attention_mask is None and position_ids is None and hidden_states.ndim == 3
                    and hidden_states.size(1) == 1 and len(past_key_values) > self.layer_idx):
                layer = past_key_values.get_layer(self.layer_idx)
            if (layer is None or layer.state is None or layer.next_position is None
                    or not self._fused_step_ok(hidden_states, layer.state, 1, None)):
                return super().forward(hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
                                       use_cache=use_cache, output_attentions=output_attentions, position_ids=position_ids)
            # one cached token: the state is updated in place and the cache's position tensor is advanced in
            # place too, so that every tensor of the step keeps its address from call to call
            output, _ = self.forward_with_state(hidden_states, init_ram=layer.state, position_ids=layer.next_position,
                                                inplace=True)
            layer.next_position.add_(1)
            layer.cache_length += 1
            return output, None, past_key_values

    FusedRAMNetAttention.__name__ = "FusedRAMNetAttention"
    _FUSED_CLASS = FusedRAMNetAttention
    return _FUSED_CLASS


def use_fused_attention(model: torch.nn.Module) -> int:
    """Switch every RAMNetAttention inside ``model`` to the fused class; returns how many were switched."""
    from ramnet.layers import RAMNetAttention
    fused = fused_attention_class()
    n = 0
    for module in model.modules():
        if type(module) is RAMNetAttention:
            module.__class__ = fused
            n += 1
    return n


class GreedyGraphDecoder:
    """Greedy generation of a ``RAMNetForCausalLM`` with one CUDA-graph replay per token.

    ``cache`` is the model's ``RAMCache`` after the prompt has been run (``use_cache=True``) and ``last_tokens``
    (B, 1) the first generated tokens (argmax of the prompt's last logits).  The graph holds the embedding, every
    block (fused one-token attention step, state and positions in place), the final norm, the LM head on the last
    position and the argmax, writing the next token back into the static input buffer.
    """

    def __init__(self, model, cache, last_tokens: torch.Tensor, warmup: int = 2):
        assert last_tokens.ndim == 2 and last_tokens.size(1) == 1 and last_tokens.is_cuda
        self.model, self.cache = model, cache
        self.tokens = last_tokens.clone()
        use_fused_attention(model)
        # snapshot what the warm-up steps change, so that capture starts from the caller's state
        layers = [cache.get_layer(i) for i in range(len(cache))]
        saved = [(l.state.slot.clone(), l.state.mass.clone(), l.next_position.clone(), l.cache_length) for l in layers]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for l, (slot, mass, pos, n) in zip(layers, saved):
            l.state.slot.copy_(slot)
            l.state.mass.copy_(mass)
            l.next_position.copy_(pos)
            l.cache_length = n
        self.tokens.copy_(last_tokens)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self._step()
        # the capture itself ran no kernel, but it did run the Python bookkeeping once
        for l, (_, _, _, n) in zip(layers, saved):
            l.cache_length = n
        self._layers = layers

    def _step(self):
        hidden = self.model.model(input_ids=self.tokens, past_key_values=self.cache, use_cache=True).last_hidden_state
        logits = self.model.lm_head(hidden[:, -1])
        self.tokens.copy_(logits.argmax(dim=-1, keepdim=True))

    def generate(self, n_tokens: int) -> torch.Tensor:
        """Generates ``n_tokens`` more tokens; returns (B, n_tokens).  The tokens given at construction are the
        input of the first step and are not part of the result."""
        out = torch.empty(self.tokens.size(0), n_tokens, dtype=self.tokens.dtype, device=self.tokens.device)
        for i in range(n_tokens):
            self.graph.replay()
            out[:, i:i + 1].copy_(self.tokens)
        for l in self._layers:
            l.cache_length += n_tokens
        return out
