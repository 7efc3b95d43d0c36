"""The graphed decode loop replays exactly what the eager per-step calls compute."""
import pytest
import torch

from tests.gpu_common import ops, randn

pytestmark = pytest.mark.gpu


def _buffers(n, B, H, U, P, C, dtype, seed):
    A = P ** U
    dev = "cuda"
    w = randn((n, B, H, U, P), seed, dtype).to(dev)
    r = randn((n, B, H, U, P), seed + 1, dtype).to(dev)
    x = randn((n, B, H, C), seed + 2, dtype).to(dev)
    g = torch.sigmoid(randn((n, B, H), seed + 3)).to(dtype).to(dev)
    gate = randn((n, B, H, C), seed + 4, dtype).to(dev)
    slot = (randn((B, H, A, C), seed + 5) * 0.1).to(dev)
    mass = (torch.rand(B, H, A, generator=torch.Generator().manual_seed(seed + 6)) + 0.1).to(dev)
    pos = (torch.arange(B) * 5 + 2).int().to(dev)
    return w, r, x, g, gate, slot, mass, pos


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("B,H,U,P,C,K,dtype", [
    (3, 4, 2, 16, 64, 4, torch.float32),
    (2, 8, 2, 64, 128, 16, torch.bfloat16),
])
def test_graph_replay_equals_eager_steps(B, H, U, P, C, K, dtype, fused):
    ops()
    import ramnet_ops
    n = 4
    w, r, x, g, gate, slot, mass, pos = _buffers(n, B, H, U, P, C, dtype, 11)
    E = H // 2
    nw = torch.linspace(0.5, 1.5, C, device="cuda") if fused else None
    nomask = torch.empty(0, dtype=torch.bool, device="cuda")

    # eager: two rounds of n steps on a copy of the state
    e_slot, e_mass, e_pos = slot.clone(), mass.clone(), pos.clone()
    eager = []
    for rnd in range(2):
        for j in range(n):
            if fused:
                y = torch.ops.ramnet_ops.decode_fused_(w[j], r[j], x[j], g[j], e_slot, e_mass, nomask, E, e_pos, K, K, 0.0,
                                                       0.0, False, 1e-12, nw, gate[j], 1e-6)
            else:
                y = torch.ops.ramnet_ops.topk_autoregressive_(w[j], r[j], x[j], g[j], e_slot, e_mass, nomask, E, e_pos, K,
                                                              K, 0.0, 0.0, False, 1e-12)
            e_pos += 1
            eager.append(y.clone())

    slot0, mass0, pos0 = slot.clone(), mass.clone(), pos.clone()
    graph = ramnet_ops.DecodeGraph(w, r, x, g, slot, mass, pos, embed_num=E, top_k=K, norm_weight=nw,
                                   gate_logits=gate if fused else None)
    torch.cuda.synchronize()
    # building the graph leaves the state alone
    assert torch.equal(slot, slot0) and torch.equal(mass, mass0) and torch.equal(pos, pos0)
    for rnd in range(2):
        outs = graph.replay()
        torch.cuda.synchronize()
        for j in range(n):
            assert torch.equal(outs[j], eager[rnd * n + j]), (rnd, j)
    assert torch.equal(slot, e_slot) and torch.equal(mass, e_mass) and torch.equal(pos, e_pos)
