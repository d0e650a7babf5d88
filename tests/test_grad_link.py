"""The gradient hand-over of ``ops.conv.GradLink`` (skip-connection gradient -> first convolution's backward), exercised on
the CPU with toy autograd functions that follow the protocol of the tensor-core convolution."""
import torch

from gradient_compression_b200.ops.bn import own_grad, take_owned_grad
from gradient_compression_b200.ops.conv import GradLink


class _ToyConv(torch.autograd.Function):
    """y = x w; the backward adds onto a stashed skip gradient the way the input-gradient GEMM does."""

    log = []

    @staticmethod
    def forward(ctx, x, w, link):
        ctx.save_for_backward(x, w)
        ctx.link = link
        return x @ w

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        link = ctx.link
        dx = g @ w.t()
        if link is not None and link.stash is not None:
            acc, link.stash = link.stash, None
            _ToyConv.log.append("in-place" if link.stash_owned else "copy")
            if not link.stash_owned:
                acc = acc.clone()
            acc += dx
            dx = acc
        if link is not None:
            link.conv_done = True
        return dx, x.t() @ g, None


class _ToyAddRelu(torch.autograd.Function):
    """relu(y + res) with a residual gradient this library allocates itself (``own_grad``)."""

    @staticmethod
    def forward(ctx, y, res):
        out = torch.relu(y + res)
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, g):
        (out,) = ctx.saved_tensors
        d = g * (out > 0)
        return d, own_grad(d.clone())


def _block(x, w1, w3, use_link, residual_first=False, owned=True):
    link = GradLink() if use_link else None
    if use_link:
        link.armed = True
    res = link.residual(x) if (use_link and residual_first) else None
    y = _ToyConv.apply(x, w1, link)
    y = _ToyConv.apply(torch.tanh(y), w3, None)
    if res is None:
        res = link.residual(x) if use_link else x
    return _ToyAddRelu.apply(y, res) if owned else torch.relu(y + res)


def _grads(**kw):
    torch.manual_seed(0)
    x0 = torch.randn(6, 5, dtype=torch.float64)
    w1 = torch.randn(5, 4, dtype=torch.float64, requires_grad=True)
    w3 = torch.randn(4, 5, dtype=torch.float64, requires_grad=True)
    x = (x0 * 1.0).requires_grad_(True)
    x.retain_grad()
    _block(x, w1, w3, **kw).pow(2).sum().backward()
    return x.grad, w1.grad, w3.grad


def test_link_matches_plain_autograd_in_every_order():
    ref = _grads(use_link=False)
    for kw, expect in ((dict(use_link=True), ["in-place"]),                         # owned gradient: accumulated in place
                       (dict(use_link=True, owned=False), ["copy"]),                # torch add shares its gradient: copied first
                       (dict(use_link=True, residual_first=True), [])):             # conv backward first: autograd sums as usual
        _ToyConv.log.clear()
        got = _grads(**kw)
        assert _ToyConv.log == expect, (kw, _ToyConv.log)
        for a, b in zip(got, ref):
            assert torch.allclose(a, b, atol=1e-12), kw


def test_unarmed_link_is_transparent_and_ownership_is_single_use():
    link = GradLink()
    x = torch.randn(3, requires_grad=True)
    assert link.residual(x) is x                      # the convolution did not take the GEMM path
    t = own_grad(torch.zeros(4))
    assert take_owned_grad(t) and not take_owned_grad(t)
    assert not take_owned_grad(torch.zeros(4))
