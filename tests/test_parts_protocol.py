"""The hand-over of a part's output to the part that follows, on the CPU: a deferred output is turned
into a tensor for every consumer that does not ask for it, and handed over as it is to one that does."""

import torch

from mini_infer_b200.parts import Deferred, FeedForward, Norm, apply_norm, resolve


class Twice(Deferred):
    def __init__(self, t):
        self.t, self.asked = t, 0

    def materialize(self):
        self.asked += 1
        return 2 * self.t


class PlainNorm(Norm):
    def apply(self, hidden, delta, rows=None):
        assert delta is None or isinstance(delta, torch.Tensor)
        return hidden if delta is None else hidden + delta


class FoldingNorm(Norm):
    accepts_deferred = True

    def apply(self, hidden, delta, rows=None):
        assert isinstance(delta, Twice)
        return hidden + 2 * delta.t                      # its own way of forming the sum


def test_resolve_and_apply_norm():
    t = torch.arange(6.0).view(2, 3)
    d = Twice(t)
    assert resolve(t) is t and resolve(None) is None
    assert torch.equal(resolve(d), 2 * t) and d.asked == 1
    h = torch.ones(2, 3)
    assert torch.equal(apply_norm(PlainNorm({}, ""), h, d), h + 2 * t) and d.asked == 2
    assert torch.equal(apply_norm(FoldingNorm({}, ""), h, d), h + 2 * t) and d.asked == 2   # not materialised
    assert torch.equal(apply_norm(PlainNorm({}, ""), h, None), h)
    assert PlainNorm({}, "").rms_parameters() is None


def test_feed_forward_defaults_fall_back_to_forward():
    class Half(FeedForward):
        def forward(self, x, ctx):
            return 0.5 * x

    ff = Half({}, "")
    x = torch.full((2, 3), 4.0)
    assert torch.equal(ff.forward_deferred(x, None), 0.5 * x)
    hidden, delta = torch.ones(2, 3), torch.full((2, 3), 3.0)
    assert torch.equal(ff.forward_from_residual(hidden, delta, PlainNorm({}, ""), None), 0.5 * (hidden + delta))
    assert torch.equal(ff.forward_from_residual(hidden, Twice(delta), PlainNorm({}, ""), None), 0.5 * (hidden + 2 * delta))
