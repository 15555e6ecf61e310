"""Autograd rule for the fused kernels: run the fused forward (no intermediate signal is written),
and in backward recompute the same values through the unfused chain - whose own autograd rules are
the reference's - and differentiate that.  This is activation recomputation restricted to one layer
boundary: the backward pass costs one extra unfused forward of that boundary, the forward pass keeps
the speed and, above all, the memory footprint of the fused kernel (the signal between two layers,
[batch, features, (2b)^3] floats, never exists).  It is opt-in (``module.fused_training = True``):
when time rather than memory is the constraint, storing the activations is faster."""
import torch


class FusedRecompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fused_fn, plain_fn, *tensors):
        ctx.plain_fn = plain_fn
        ctx.save_for_backward(*tensors)
        with torch.no_grad():
            return fused_fn(*tensors)

    @staticmethod
    def backward(ctx, grad_output):
        inputs = [t.detach().requires_grad_(need) for t, need in
                  zip(ctx.saved_tensors, ctx.needs_input_grad[2:])]
        with torch.enable_grad():
            out = ctx.plain_fn(*inputs)
        wanted = [t for t in inputs if t.requires_grad]
        grads = torch.autograd.grad(out, wanted, grad_output.contiguous(), allow_unused=True)
        it = iter(grads)
        return (None, None) + tuple(next(it) if t.requires_grad else None for t in inputs)


def fused_or_recompute(fused_fn, plain_fn, tensors, needs_grad, opt_in):
    """The fused kernel when no gradient is wanted, the fused kernel with the recompute rule when the
    module opted in, else the unfused chain (activations stored, the reference's behaviour)."""
    if not needs_grad:
        return fused_fn(*tensors)
    if opt_in:
        return FusedRecompute.apply(fused_fn, plain_fn, *tensors)
    return plain_fn(*tensors)
