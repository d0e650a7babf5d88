"""The flat arena keeps channels-last weights in channels-last order, and reducers see memory-order views."""
import torch

from gradient_compression_b200 import make_reducer
from gradient_compression_b200.parallel.arena import FlatArena, FlatSGD
from gradient_compression_b200.reducers.base import physical


def _nets():
    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(8, 4, 1), torch.nn.Flatten(),
                            torch.nn.Linear(4 * 6 * 6, 5))
    b = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(8, 4, 1), torch.nn.Flatten(),
                            torch.nn.Linear(4 * 6 * 6, 5))
    b.load_state_dict(a.state_dict())
    return a, b.to(memory_format=torch.channels_last)


def test_channels_last_weights_keep_their_layout_and_train_identically():
    ref, net = _nets()
    arena = FlatArena(list(net.parameters()))
    w = net[0].weight
    assert w.is_contiguous(memory_format=torch.channels_last) and not w.is_contiguous()
    assert w.grad.stride() == w.stride()
    # the segment holds [Cout][kh][kw][Cin]
    assert torch.equal(arena.param_views[0], w.detach().permute(0, 2, 3, 1))
    assert arena.param_views[0].is_contiguous() and arena.param_views[0].data_ptr() == arena.flat_params.data_ptr()
    opt = FlatSGD(arena, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    x = torch.randn(4, 3, 6, 6)
    y = torch.randint(0, 5, (4,))
    for _ in range(3):
        arena.zero_grad()
        torch.nn.functional.cross_entropy(net(x.contiguous(memory_format=torch.channels_last)), y).backward()
        opt.step()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(x), y).backward()
        ref_opt.step()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-6)
    # detach / collect round trip keeps the logical gradient
    arena.detach_grads()
    torch.nn.functional.cross_entropy(net(x.contiguous(memory_format=torch.channels_last)), y).backward()
    g_logical = net[0].weight.grad.clone()
    arena.collect_grads()
    assert torch.equal(net[0].weight.grad, g_logical)
    assert torch.equal(arena.grad_views[0], g_logical.permute(0, 2, 3, 1))


def test_reducers_see_memory_order_views():
    _, net = _nets()
    arena = FlatArena(list(net.parameters()))
    for p in net.parameters():
        p.grad.copy_(torch.randn(p.shape))
    logical = [p.grad for p in net.parameters()]
    assert physical(logical[0]).is_contiguous() and physical(logical[0]).shape == (8, 3, 3, 3)
    assert physical(logical[4]) is logical[4]
    before = [g.clone() for g in logical]
    for name in ("NoneAllReducer", "QSGDMaxNormReducer", "RankKReducer", "TopKReducer"):
        for g, b in zip(logical, before):
            g.copy_(b)
        red = make_reducer(name, torch.device("cpu"), None, {"quantization_level": 8, "seed": 3, "K": 50, "rank": 2})
        red.reduce(logical, logical)                 # logical (permuted) views in, same views out
        assert all(torch.isfinite(g).all() for g in logical)
        if name == "NoneAllReducer":
            assert all(torch.equal(g, b) for g, b in zip(logical, before))
        if name == "QSGDMaxNormReducer":             # elementwise: within one quantisation step of the input
            norm = max(float(b.abs().max()) for b in before)
            assert all(float((g - b).abs().max()) <= norm / 255 + 1e-6 for g, b in zip(logical, before))
