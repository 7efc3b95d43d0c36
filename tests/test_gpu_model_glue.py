"""The fused one-token attention step and the graph-replayed greedy decoder against the reference model classes.

Needs the reference MODEL package ``ramnet`` (not part of this repository): it is looked for on the import path
and under ``baseline/_ref`` (where ``pip install --target baseline/_ref <reference>/packages/ramnet`` puts it);
without it these tests are skipped.  The reference classes run on this package's operators either way; what is
compared is the reference's own layer code (operator + RMSNorm + sigmoid gate as separate modules, cache positions
rebuilt per call) with the fused step (``decode_fused_`` + positions advanced in place).
"""
import copy
import sys
from pathlib import Path

import pytest
import torch

from tests.gpu_common import ops

pytestmark = pytest.mark.gpu

_REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
if _REF.exists() and str(_REF) not in sys.path:
    sys.path.append(str(_REF))


def _models(dtype, U, P, C, K, H=4, layers=2, hidden=64):
    ops()
    pytest.importorskip("ramnet", reason="reference model package not installed")
    from ramnet.models import RAMNetConfig, RAMNetForCausalLM
    from ramnet_ops.layers import use_fused_attention
    torch.manual_seed(0)
    cfg = RAMNetConfig(hidden_size=hidden, num_attention_heads=H, num_hidden_layers=layers, addr_order=U, addr_radix=P,
                       value_chs=C, embed_num=H // 2, addr_top_k=K, hidden_act="SwiGLU", intermediate_size=2 * hidden,
                       fuse_norm=False, fuse_cross_entropy=False, vocab_size=97)
    ref = RAMNetForCausalLM(cfg).to("cuda", dtype).eval()
    fused = copy.deepcopy(ref)
    assert use_fused_attention(fused) == layers
    return ref, fused


def _greedy(model, ids, steps, forced=None):
    """Prompt with use_cache, then `steps` one-token calls fed with the argmax of the previous call (or with the
    columns of `forced`); returns (logits per call, argmax tokens, cache)."""
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=True)
        cache = out.past_key_values
        logits = [out.logits[:, -1].float()]
        toks = [logits[-1].argmax(-1, keepdim=True)]
        for i in range(steps):
            tok = toks[-1] if forced is None else forced[:, i:i + 1]
            out = model(input_ids=tok, past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            toks.append(logits[-1].argmax(-1, keepdim=True))
    return logits, torch.cat(toks, dim=1), cache


@pytest.mark.parametrize("dtype,U,P,C,K", [
    (torch.float32, 2, 16, 32, 4),
    (torch.bfloat16, 2, 64, 128, 16),     # the model shape: the one-warp-per-pair decode kernel with the fused epilogue
    (torch.float32, 3, 4, 24, (3, 5)),
])
def test_fused_step_matches_the_reference_layer(dtype, U, P, C, K):
    ref, fused = _models(dtype, U, P, C, K)
    ids = torch.randint(3, 97, (3, 21), device="cuda")
    forced = torch.randint(3, 97, (3, 5), device="cuda")  # the same continuation for both models
    l_ref, t_ref, c_ref = _greedy(ref, ids, 5, forced)
    l_fus, t_fus, c_fus = _greedy(fused, ids, 5, forced)
    # bf16: the reference layer rounds y, the normalised y and the gate to bf16 one after the other, the fused
    # step rounds once; the logits of this small random model are O(0.1)
    tol = 2e-4 if dtype == torch.float32 else 6e-2
    for step, (a, b) in enumerate(zip(l_fus, l_ref)):
        torch.testing.assert_close(a, b, atol=tol, rtol=tol, msg=lambda m, s_=step: f"call {s_}: {m}")
    if dtype == torch.float32:
        assert torch.equal(t_fus, t_ref)
    for i in range(len(c_ref)):
        a, b = c_fus.get_layer(i), c_ref.get_layer(i)
        if dtype == torch.float32:
            torch.testing.assert_close(a.state.slot, b.state.slot, atol=1e-4, rtol=1e-2)
        else:
            # the two epilogues round differently, so the next layer's address logits differ in the last bit and a
            # Top-K choice between (nearly) tied slots can fall the other way: a handful of rows, not more
            differ = ((a.state.slot - b.state.slot).abs() > 5e-3).float().mean().item()
            assert differ < 1e-3, f"layer {i}: {differ:.2%} of the state differs"
        assert torch.equal(a.next_position, b.next_position) and a.get_seq_length() == b.get_seq_length()


def test_graph_replayed_greedy_decoding_gives_the_eager_tokens():
    from ramnet_ops.layers import GreedyGraphDecoder
    ref, fused = _models(torch.float32, 2, 16, 32, 4)
    ids = torch.randint(3, 97, (4, 17), device="cuda")
    n = 12
    _, t_eager, _ = _greedy(fused, ids, n)
    with torch.no_grad():
        out = fused(input_ids=ids, use_cache=True)
    first = out.logits[:, -1].argmax(-1, keepdim=True)
    dec = GreedyGraphDecoder(fused, out.past_key_values, first)
    got = dec.generate(n)
    torch.cuda.synchronize()
    assert torch.equal(first, t_eager[:, :1])
    assert torch.equal(got, t_eager[:, 1:]), "graph replay must generate the tokens of the step-by-step loop"
    assert out.past_key_values.get_layer(0).get_seq_length() == 17 + n
    _, t_ref, _ = _greedy(ref, ids, n)
    assert torch.equal(t_ref, t_eager)
