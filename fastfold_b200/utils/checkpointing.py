"""Activation checkpointing over a list of blocks.

``checkpoint_blocks(blocks, args, blocks_per_ckpt)`` has the reference's
signature (fastfold/utils/checkpointing.py:31-84).  The checkpoint itself is a
small autograd Function of our own rather than ``torch.utils.checkpoint``: it
never saves or restores RNG state (the blocks receive their dropout masks as
inputs, so recomputation is deterministic by construction), which is what
allows a whole training step - forward, recomputation, backward, optimizer -
to be captured in one CUDA graph.
"""
import torch


def _flatten_tensors(args):
    return tuple(a for a in args if isinstance(a, torch.Tensor))


# Called with the checkpointed function right after its backward (recomputation + gradient kernels of its blocks) has
# been enqueued: the trainer uses it to start reducing that segment's weight gradients while backward continues.
POST_BACKWARD_HOOKS = []


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_args, *args):
        ctx.fn = fn
        ctx.n_args = n_args
        ctx.save_for_backward(*args[:n_args])
        with torch.no_grad():
            outs = fn(*args[:n_args])
        return outs if isinstance(outs, tuple) else (outs,)

    @staticmethod
    def backward(ctx, *grads):
        inputs = [t.detach().requires_grad_(t.requires_grad or t.is_floating_point()) for t in ctx.saved_tensors]
        with torch.enable_grad():
            outs = ctx.fn(*inputs)
        outs = outs if isinstance(outs, tuple) else (outs,)
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = tuple(t.grad if t.requires_grad else None for t in inputs)
        for hook in POST_BACKWARD_HOOKS:
            hook(ctx.fn)
        # trailing entries: parameters passed only so that autograd records a dependency
        return (None, None) + in_grads + (None,) * (len(ctx.needs_input_grad) - 2 - len(in_grads))


def checkpoint(fn, *args):
    """Runs ``fn(*args)`` without storing its intermediates; they are recomputed in backward."""
    params = []
    owner = getattr(fn, "func", fn)
    mod = getattr(owner, "__self__", owner)
    if isinstance(mod, torch.nn.Module):
        params = [p for p in mod.parameters() if p.requires_grad]
    if not (torch.is_grad_enabled() and (any(a.requires_grad for a in args if isinstance(a, torch.Tensor)) or params)):
        return fn(*args)
    # a dummy that requires grad makes the node part of the graph even when no input does
    outs = _Checkpoint.apply(fn, len(args), *args, *params)
    return outs


def checkpoint_blocks(blocks, args, blocks_per_ckpt):
    """Chains ``blocks`` over ``args``; every ``blocks_per_ckpt`` consecutive blocks form one checkpoint.

    ``blocks_per_ckpt=None`` (or grad disabled) runs the blocks plainly.
    """
    def wrap(a):
        return (a,) if not isinstance(a, tuple) else a

    def chunker(s, e):
        def run(*a):
            for b in blocks[s:e]:
                a = wrap(b(*a))
            return a
        run.__blocks__ = blocks[s:e]
        return run

    args = wrap(args)
    if blocks_per_ckpt is None or not torch.is_grad_enabled():
        for b in blocks:
            args = wrap(b(*args))
        return args
    if blocks_per_ckpt < 1 or blocks_per_ckpt > len(blocks):
        raise ValueError("blocks_per_ckpt must be between 1 and len(blocks)")
    for s in range(0, len(blocks), blocks_per_ckpt):
        e = s + blocks_per_ckpt
        run = chunker(s, e)
        params = []
        for b in blocks[s:e]:
            owner = getattr(b, "func", b)
            mod = getattr(owner, "__self__", owner)
            if isinstance(mod, torch.nn.Module):
                params += [p for p in mod.parameters() if p.requires_grad]
        if any(a.requires_grad for a in args if isinstance(a, torch.Tensor)) or params:
            args = _Checkpoint.apply(run, len(args), *args, *params)
        else:
            args = run(*args)
    return args


def get_checkpoint_fn():
    """``checkpoint(fn, *args)``: runs ``fn`` without saving its intermediates and recomputes it in backward (this
    package's own autograd function, the one ``checkpoint_blocks`` uses).  Returns what ``fn`` returns."""
    def checkpoint(fn, *args):
        single = []

        def block(*a):
            out = fn(*a)
            single.append(not isinstance(out, tuple))
            return out
        out = checkpoint_blocks([block], tuple(args), blocks_per_ckpt=1)
        return out[0] if single and single[-1] else out
    return checkpoint
