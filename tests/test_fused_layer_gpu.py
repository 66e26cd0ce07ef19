"""Fused hidden-layer epilogue and the fused layer node against the chain of stock PyTorch fp32
ops they replace (bias add, dropout by a given mask, LayerNorm, relu): forward and every
gradient within 1e-5 relative to the magnitude of the quantity."""
import pytest
import torch
import torch.nn.functional as F

from super_gnn_b200 import graphsage, supergnn_ops as ops, synthetic
from super_gnn_b200.data_manager import build_distributed_graph

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol=1e-5):
    scale = b.abs().max().item() + 1e-12
    return (a - b).abs().max().item() <= tol * scale * 8


@pytest.mark.parametrize("H", [256, 128, 64, 512, 100])
@pytest.mark.parametrize("mode", ["mask", "none", "seed"])
def test_epilogue_forward_backward_match_torch(H, mode):
    n, p = 3001, 0.5
    g = torch.Generator(device=DEV).manual_seed(H)
    h = torch.randn(n, H, generator=g, device=DEV) * 2 + 0.3
    bias = torch.randn(H, generator=g, device=DEV)
    gamma = torch.rand(H, generator=g, device=DEV) + 0.5
    beta = torch.randn(H, generator=g, device=DEV) * 0.1
    gy = torch.randn(n, H, generator=g, device=DEV)
    training = mode != "none"
    seed = 1234567
    if mode == "mask":
        mask = (torch.rand(n, H, generator=g, device=DEV) >= p).float() / (1 - p)
        kmask = mask
    elif mode == "seed":
        mask = ops.dropout_mask(seed, p, n, H, DEV)  # what the kernel will apply
        keep = (mask > 0).float().mean().item()
        assert abs(keep - (1 - p)) < 0.01 and torch.all((mask == 0) | (mask == 1 / (1 - p)))
        kmask = None
    else:
        mask, kmask = None, None
    # reference chain
    hr = h.clone().requires_grad_(True)
    br, gr, ber = (t.clone().requires_grad_(True) for t in (bias, gamma, beta))
    z = hr + br
    if mask is not None:
        z = z * mask
    yr = F.relu(F.layer_norm(z, (H,), gr, ber, 1e-5))
    yr.backward(gy)
    # fused
    hk = h.clone()
    y, stats = ops.sage_epilogue_forward(hk, bias, gamma, beta, p, training, seed, 1e-5, kmask)
    assert torch.equal(hk, h)  # the input is left alone: the backward recomputes from it
    assert close(y, yr.detach())
    zr = z.detach()
    assert close(stats[:, 0], zr.mean(1)) and close(stats[:, 1], (zr.var(1, unbiased=False) + 1e-5).rsqrt())
    gh, gb, gg, gbe = ops.sage_epilogue_backward(gy, hk, stats, bias, gamma, beta, p, training, seed, kmask)
    assert close(gh, hr.grad) and close(gb, br.grad) and close(gg, gr.grad) and close(gbe, ber.grad)
    # the relu mask the backward recomputes is the forward's: grad_beta is the column sum of grad_y where y > 0
    assert close(gbe, (gy * (y > 0)).sum(0))
    # deterministic reductions: a second run gives bit-identical parameter gradients
    gh2, gb2, gg2, gbe2 = ops.sage_epilogue_backward(gy, hk, stats, bias, gamma, beta, p, training, seed, kmask)
    assert torch.equal(gb, gb2) and torch.equal(gg, gg2) and torch.equal(gbe, gbe2) and torch.equal(gh, gh2)
    # rows given with a leading dimension (a column slice of a wider buffer)
    wide = torch.full((n, H + 8), float("nan"), device=DEV)
    wide[:, :H] = h
    y3, stats3 = ops.sage_epilogue_forward(wide[:, :H], bias, gamma, beta, p, training, seed, 1e-5, kmask)
    assert torch.equal(y3, y) and torch.equal(stats3, stats)


def test_fused_model_matches_unfused_model():
    """Whole 3-layer model, injected dropout masks: loss and all parameter gradients."""
    n, e, fin, hid, ncls = 6000, 60_000, 100, 256, 47
    dev = torch.device(DEV)
    s, t = synthetic.rmat_edges(n, e, 0.57, 0.19, 0.19, 0.05, seed=5, device=dev)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    graph = build_distributed_graph(torch.stack([s, t]), torch.zeros((2, 0), dtype=torch.int64, device=dev), [0, n],
                                    hid, 32, device=dev)
    torch.manual_seed(0)
    model, _ = graphsage.create_model_and_optimizer(
        dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=0.5), device=dev)
    x = torch.randn(n, fin, device=dev)
    labels = torch.randint(0, ncls, (n,), device=dev)
    masks = [(torch.rand(n, hid, device=dev) >= 0.5).float() * 2 for _ in range(2)]
    model.dropout_masks = masks
    model.train()
    grads = {}
    # "fold": mean normalisation inside the SpMM kernels; "*-ref-order": last layer aggregates before it projects
    for fused in (True, False, "fold", "fold-ref-order", "ref-order"):
        graph.set_fold_mean(str(fused).startswith("fold"))
        model.fused = bool(fused)
        model.project_first = not str(fused).endswith("ref-order")
        model.zero_grad()
        out = model(graph, x)
        loss = F.nll_loss(out, labels)
        loss.backward()
        grads[fused] = (loss.item(), {k: v.grad.clone() for k, v in model.named_parameters()})
    assert abs(grads[True][0] - grads[False][0]) <= 1e-5 * abs(grads[False][0])
    graph.set_fold_mean(False)
    assert abs(grads["fold"][0] - grads[False][0]) <= 1e-5 * abs(grads[False][0])
    for variant in (True, "fold", "fold-ref-order", "ref-order"):
        assert abs(grads[variant][0] - grads[False][0]) <= 1e-5 * abs(grads[False][0]), variant
        for k, gref in grads[False][1].items():
            assert close(grads[variant][1][k], gref, tol=2e-5), (variant, k)
    model.project_first = "auto"
    # inference path (no dropout)
    model.eval()
    with torch.no_grad():
        model.fused = True
        a = model(graph, x)
        model.project_first = False
        a_ref_order = model(graph, x)
        model.fused = False
        b = model(graph, x)
    assert close(a, b) and close(a_ref_order, b)
