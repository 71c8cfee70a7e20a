"""One autograd node for every kernel-backed operation of the package.

An operation is a plain object with two methods and whatever per-call settings it needs as
attributes:

    run(keep, *tensors)   -> tensor or tuple of tensors; `keep(*tensors, **facts)` stores what the
                             gradient pass needs (tensors through autograd's own saved-tensor
                             mechanism, everything else as plain attributes)
    grad(kept, *grads)    -> one gradient (or None) per tensor given to `run`, in the same order;
                             `kept.tensors` are the stored tensors, `kept.<fact>` the stored facts,
                             `kept.wants[i]` says whether input i needs a gradient at all

`call(op, *tensors)` runs the operation under autograd. Tensors are the only things that travel
through `torch.autograd.Function.apply`; sizes, flags and dtypes live on the operation object, so
an operation's `grad` never returns placeholders for them.
"""

from __future__ import annotations

import torch


class _Kept:
    """What `run` asked to keep, as `grad` sees it."""

    def __init__(self, ctx):
        self._ctx = ctx

    @property
    def tensors(self):
        return self._ctx.saved_tensors

    @property
    def wants(self):
        return self._ctx.needs_input_grad[1:]

    def __getattr__(self, name):
        try:
            return self._ctx.facts[name]
        except KeyError:
            raise AttributeError(name) from None


class _Node(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, *tensors):
        ctx.op = op
        ctx.facts = {}

        def keep(*saved, **facts):
            ctx.save_for_backward(*saved)
            ctx.facts.update(facts)

        def constant(*outputs):
            ctx.mark_non_differentiable(*outputs)

        keep.constant = constant
        return op.run(keep, *tensors)

    @staticmethod
    def backward(ctx, *grads):
        result = ctx.op.grad(_Kept(ctx), *grads)
        if not isinstance(result, tuple):
            result = (result,)
        return (None,) + result


def call(op, *tensors):
    return _Node.apply(op, *tensors)
