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


@pytest.mark.parametrize("fin,hid", [(602, 256), (100, 130), (1024, 64), (6, 8)])
def test_layers_the_fused_path_cannot_take_fall_back_one_by_one(fin, hid):
    """Input widths that are not a multiple of 4 (reddit's 602), hidden widths the fused epilogue does not take (130)
    and widths above the vector kernels' range (1024): the default model still runs, layer by layer on whichever
    path takes the layer, and equals the unfused model."""
    n, e, ncls = 3000, 30_000, 10
    dev = torch.device(DEV)
    s, t = synthetic.rmat_edges(n, e, 0.57, 0.19, 0.19, 0.05, seed=6, device=dev)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    graph = build_distributed_graph(torch.stack([s, t]), torch.zeros((2, 0), dtype=torch.int64, device=dev), [0, n],
                                    max(fin, hid), 32, device=dev)
    torch.manual_seed(0)
    model, _ = graphsage.create_model_and_optimizer(
        dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=0.5), device=dev)
    x = torch.randn(n, fin, device=dev)
    labels = torch.randint(0, ncls, (n,), device=dev)
    model.dropout_masks = [(torch.rand(n, hid, device=dev) >= 0.5).float() * 2 for _ in range(2)]
    model.train()
    res = {}
    for fused in (True, False):
        model.fused = fused
        model.zero_grad()
        loss = F.nll_loss(model(graph, x), labels)
        loss.backward()
        res[fused] = (loss.item(), {k: v.grad.clone() for k, v in model.named_parameters()})
    assert abs(res[True][0] - res[False][0]) <= 1e-5 * abs(res[False][0])
    for k, gref in res[False][1].items():
        assert close(res[True][1][k], gref, tol=2e-5), k
    # and a whole training step through train_step (fused loss where the last layer allows it)
    model.fused = True
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    data = dict(graph=graph, nodes_features=x, nodes_labels=labels, nodes_train_masks=torch.rand(n, device=dev) < 0.5)
    assert torch.isfinite(graphsage.train_step(model, data, opt, float(data["nodes_train_masks"].sum())))


@pytest.mark.parametrize("C", [7, 47, 48, 100, 172, 256])
def test_softmax_nll_loss_matches_torch(C):
    n = 5003
    g = torch.Generator(device=DEV).manual_seed(C)
    logits = torch.randn(n, C, generator=g, device=DEV) * 3
    bias = torch.randn(C, generator=g, device=DEV)
    labels = torch.randint(0, C, (n,), generator=g, device=DEV)
    mask = torch.rand(n, generator=g, device=DEV) < 0.3
    inv = 1.0 / float(mask.sum())
    zr = logits.clone().requires_grad_(True)
    br = bias.clone().requires_grad_(True)
    ref = F.nll_loss(F.log_softmax(zr + br, 1)[mask], labels[mask], reduction="sum") * inv
    ref.backward()
    loss, grad = ops.softmax_nll_loss(logits, bias, labels, mask, inv)
    assert abs(loss.item() - ref.item()) <= 1e-5 * abs(ref.item())
    assert close(grad, zr.grad) and close(grad.sum(0), br.grad)
    assert torch.all(grad[~mask] == 0)
    # reproducible: a second run gives the same bits
    loss2, grad2 = ops.softmax_nll_loss(logits, bias, labels, mask, inv)
    assert torch.equal(loss, loss2) and torch.equal(grad, grad2)
    # logits and gradient as column slices of wider buffers, padded gradient width, no mask, no bias
    Cp = (C + 3) // 4 * 4
    wide = torch.full((n, 2 * Cp), float("nan"), device=DEV)
    wide[:, Cp:Cp + C] = logits
    G = torch.full((n, 2 * Cp), float("nan"), device=DEV)
    loss3, _ = ops.softmax_nll_loss(wide[:, Cp:Cp + C], None, labels, None, 1.0 / n, grad=G[:, Cp:])
    zr2 = logits.clone().requires_grad_(True)
    ref3 = F.nll_loss(F.log_softmax(zr2, 1), labels, reduction="sum") / n
    ref3.backward()
    assert abs(loss3.item() - ref3.item()) <= 1e-5 * abs(ref3.item())
    assert close(G[:, Cp:Cp + C], zr2.grad) and torch.all(G[:, Cp + C:] == 0) and torch.isnan(G[:, :Cp]).all()


def test_softmax_nll_loss_leaves_unlabelled_rows_out():
    """A label outside [0, C) — the -1 of an unlabelled node in the partition files, or F.nll_loss's ignore_index —
    takes the row out of the loss even when the mask lists it: no contribution, zero gradient."""
    n, C = 3001, 47
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = torch.randn(n, C, generator=g, device=DEV)
    labels = torch.randint(0, C, (n,), generator=g, device=DEV)
    mask = torch.rand(n, generator=g, device=DEV) < 0.5
    odd = torch.arange(n, device=DEV) % 7 == 0
    labels[odd] = -1
    labels[3] = -100
    labels[4] = C
    valid = mask & (labels >= 0) & (labels < C)
    zr = logits.clone().requires_grad_(True)
    ref = F.nll_loss(F.log_softmax(zr, 1)[valid], labels[valid], reduction="sum") * 0.01
    ref.backward()
    loss, grad = ops.softmax_nll_loss(logits, None, labels, mask, 0.01)
    assert abs(loss.item() - ref.item()) <= 1e-5 * abs(ref.item())
    assert close(grad, zr.grad) and torch.all(grad[~valid] == 0)


def test_loss_fused_with_the_last_layer_matches_the_separate_ops():
    n, e, fin, hid, ncls = 4000, 40_000, 100, 128, 47
    dev = torch.device(DEV)
    s, t = synthetic.rmat_edges(n, e, 0.57, 0.19, 0.19, 0.05, seed=9, device=dev)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    graph = build_distributed_graph(torch.stack([s, t]), torch.zeros((2, 0), dtype=torch.int64, device=dev), [0, n],
                                    hid, 32, device=dev)
    torch.manual_seed(1)
    model, opt = graphsage.create_model_and_optimizer(
        dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=0.5), device=dev)
    x = torch.randn(n, fin, device=dev)
    labels = torch.randint(0, ncls, (n,), device=dev)
    mask = torch.rand(n, device=dev) < 0.2
    model.dropout_masks = [(torch.rand(n, hid, device=dev) >= 0.5).float() * 2 for _ in range(2)]
    model.train()
    inv = 1.0 / float(mask.sum())
    res = {}
    for fold in (True, False):
        graph.set_fold_mean(fold)
        for fused_loss in (True, False):
            model.zero_grad()
            assert model.can_fuse_loss(x)
            if fused_loss:
                loss = model(graph, x, labels, None, loss_mask=mask, loss_inv_count=inv)
                (loss * 3.0).backward()  # a gradient other than 1 reaches the node
            else:
                out = model(graph, x, labels, None)
                loss = F.nll_loss(out[mask], labels[mask], reduction="sum") * inv
                (loss * 3.0).backward()
            res[(fold, fused_loss)] = (loss.item(), {k: v.grad.clone() for k, v in model.named_parameters()})
        a, b = res[(fold, True)], res[(fold, False)]
        assert abs(a[0] - b[0]) <= 1e-5 * abs(b[0])
        for k, want in b[1].items():
            assert close(a[1][k], want, tol=2e-5), (fold, k)
    graph.set_fold_mean(False)
    # train_step goes through the fused node (unit gradient) and still matches the separate ops
    data = dict(graph=graph, nodes_features=x, nodes_labels=labels, nodes_train_masks=mask)
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    losses = {}
    for flag in (True, False):
        model.load_state_dict(state)
        opt = torch.optim.Adam(model.parameters(), lr=0.01)
        graphsage.fuse_loss = flag
        losses[flag] = [graphsage.train_step(model, data, opt, float(mask.sum())).item() for _ in range(3)]
    graphsage.fuse_loss = True
    for u, v in zip(losses[True], losses[False]):
        assert abs(u - v) <= 1e-4 * abs(v)
