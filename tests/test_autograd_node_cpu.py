"""CPU: the package's single autograd node (`hackaton_b200._autograd.call`) with a stand-in
operation: saved tensors and facts reach `grad`, gradients line up with the inputs, outputs
declared constant carry no graph."""

import torch

from hackaton_b200._autograd import call


class _ScaleAndCount:
    def __init__(self, factor):
        self.factor = factor

    def run(self, keep, x, w, idx):
        keep(x, w, rows=x.shape[0])
        count = torch.full((1,), float(idx.numel()))
        keep.constant(count)
        return x * w * self.factor, count

    def grad(self, kept, dy, _dcount):
        x, w = kept.tensors
        assert kept.rows == x.shape[0]
        assert kept.wants == (True, True, False)
        return dy * w * self.factor, (dy * x * self.factor).sum(0), None


def test_node_routes_gradients_and_facts():
    x = torch.randn(5, 3, requires_grad=True)
    w = torch.randn(3, requires_grad=True)
    idx = torch.arange(4)
    y, count = call(_ScaleAndCount(2.0), x, w, idx)
    assert not count.requires_grad and float(count) == 4.0
    y.sum().backward()
    torch.testing.assert_close(x.grad, (w * 2.0).expand(5, 3))
    torch.testing.assert_close(w.grad, (x.detach() * 2.0).sum(0))


def test_single_output_and_single_gradient():
    class Double:
        def run(self, keep, x):
            keep()
            return x * 2

        def grad(self, kept, dy):
            return dy * 2

    x = torch.ones(3, requires_grad=True)
    call(Double(), x).sum().backward()
    assert torch.equal(x.grad, torch.full((3,), 2.0))
