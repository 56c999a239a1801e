"""Small tensor helpers shared by the model code (role of fastfold/utils/tensor_utils.py)."""
from functools import partial

import torch


def permute_final_dims(tensor, inds):
    """Permutes the last ``len(inds)`` dims among themselves (``inds`` counts from the first of them); leading dims stay."""
    lead = tensor.dim() - len(inds)
    return tensor.permute(*range(lead), *(lead + i for i in inds))


def flatten_final_dims(t, no_dims):
    """Merges the last ``no_dims`` dims into one."""
    return t.reshape(*t.shape[:t.dim() - no_dims], -1)


def masked_mean(mask, value, dim, eps=1e-4):
    """Mean of ``value`` over ``dim`` counting only entries where ``mask`` (broadcast to ``value``) is set."""
    weight = mask.expand_as(value)
    return (weight * value).sum(dim=dim) / (weight.sum(dim=dim) + eps)


def pts_to_distogram(pts, min_bin=2.3125, max_bin=21.6875, no_bins=64):
    """Bin index of every pairwise distance of ``pts [*, N, 3]`` against ``no_bins - 1`` equally spaced boundaries."""
    edges = torch.linspace(min_bin, max_bin, no_bins - 1, device=pts.device)
    gaps = pts[..., :, None, :] - pts[..., None, :, :]
    return torch.bucketize(gaps.pow(2).sum(dim=-1).sqrt(), edges)


def one_hot(x, v_bins):
    """Nearest-bin one-hot of ``x`` against bin centres ``v_bins``."""
    nearest = (x.unsqueeze(-1) - v_bins).abs().argmin(dim=-1)
    return torch.nn.functional.one_hot(nearest, num_classes=v_bins.numel()).float()


def batched_gather(data, inds, dim=0, no_batch_dims=0):
    """``data`` indexed with ``inds`` along ``dim``, separately for every entry of the first ``no_batch_dims`` dims, which
    ``data`` and ``inds`` share: ``out[b, ..., j, ...] = data[b, ..., inds[b, j], ...]``."""
    batch_index = [torch.arange(n, device=inds.device).reshape((n,) + (1,) * (inds.dim() - i - 1))
                   for i, n in enumerate(data.shape[:no_batch_dims])]
    tail = [slice(None)] * (data.dim() - no_batch_dims)
    tail[dim - no_batch_dims if dim >= 0 else dim] = inds
    return data[tuple(batch_index + tail)]


def dict_multimap(fn, dicts):
    """``fn`` applied to the list of corresponding leaves of several equally nested dicts."""
    return {k: (dict_multimap(fn, [d[k] for d in dicts]) if isinstance(v, dict) else fn([d[k] for d in dicts])) for k, v in dicts[0].items()}


def dict_map(fn, dic, leaf_type):
    """``tree_map`` over the values of a (possibly nested) dict."""
    return {k: (dict_map(fn, v, leaf_type) if type(v) is dict else tree_map(fn, v, leaf_type)) for k, v in dic.items()}


def tree_map(fn, tree, leaf_type):
    if isinstance(tree, dict):
        return {k: tree_map(fn, v, leaf_type) for k, v in tree.items()}
    if isinstance(tree, list):
        return [tree_map(fn, x, leaf_type) for x in tree]
    if isinstance(tree, tuple):
        return tuple(tree_map(fn, x, leaf_type) for x in tree)
    if isinstance(tree, leaf_type):
        return fn(tree)
    raise ValueError("unsupported tree node %r" % type(tree))


tensor_tree_map = partial(tree_map, leaf_type=torch.Tensor)


def _leaves(tree):
    """Tensors of a nest of dicts / lists / tuples, depth first."""
    if isinstance(tree, torch.Tensor):
        return [tree]
    if isinstance(tree, dict):
        tree = tree.values()
    elif not isinstance(tree, (list, tuple)):
        raise ValueError("unsupported tree node %r" % type(tree))
    return [t for sub in tree for t in _leaves(sub)]


def _fetch_dims(tree):
    return [t.shape for t in _leaves(tree)]


def _store(dst, src, lo, hi):
    """Writes the leaves of ``src`` into rows ``lo:hi`` of the matching leaves of ``dst`` (same nesting)."""
    if isinstance(src, torch.Tensor):
        dst[lo:hi] = src
    elif isinstance(src, dict):
        for k, v in src.items():
            _store(dst[k], v, lo, hi)
    elif isinstance(src, (list, tuple)):
        for d, v in zip(dst, src):
            _store(d, v, lo, hi)
    else:
        raise ValueError("unsupported layer output %r" % type(src))


def chunk_layer(layer, inputs, chunk_size, no_batch_dims, low_mem=False):
    """Runs ``layer(**inputs)`` on ``chunk_size`` batch entries at a time and reassembles the result.

    The first ``no_batch_dims`` dims of every input tensor are batch-like and broadcast against each other; their product
    is the number of entries.  An input whose batch dims are all 1 (a bias shared by every entry) is handed to the layer
    whole.  Outputs (tensor, tuple / list or dict of tensors, nested) come back with the broadcast batch dims restored.
    By default every other input is expanded and flattened to one batch dim up front, which copies inputs that were
    broadcast; with ``low_mem`` only the entries of the current chunk are gathered from the un-flattened (expanded, not
    copied) input.  Contract of fastfold/utils/tensor_utils.py:298-415 (OpenFold's chunking, AlphaFold supplement 1.11.8).
    """
    shapes = _fetch_dims(inputs)
    if not shapes:
        raise ValueError("Must provide at least one input")
    batch = tuple(max(dims) for dims in zip(*[sh[:no_batch_dims] for sh in shapes]))
    total = 1
    for d in batch:
        total *= d

    def shared(t):
        return all(d == 1 for d in t.shape[:no_batch_dims])

    def flatten(t):
        rest = t.shape[no_batch_dims:]
        return t.reshape(1, *rest) if shared(t) else t.expand(batch + rest).reshape(total, *rest)

    staged = inputs if low_mem else tensor_tree_map(flatten, inputs)
    out = None
    for lo in range(0, total, chunk_size):
        hi = min(total, lo + chunk_size)
        if low_mem:
            where = torch.unravel_index(torch.arange(lo, hi), batch)

            def take(t):
                rest = t.shape[no_batch_dims:]
                if shared(t):
                    return t.reshape(1, *rest)
                return t.expand(batch + rest)[tuple(w.to(t.device) for w in where)]
        else:
            def take(t):
                return t if t.shape[0] == 1 else t[lo:hi]
        piece = layer(**tensor_tree_map(take, staged))
        if out is None:
            out = tensor_tree_map(lambda t: t.new_empty((total,) + t.shape[1:]), piece)
        _store(out, piece, lo, hi)
    return tensor_tree_map(lambda t: t.reshape(batch + t.shape[1:]), out)


_CONST_CACHE = {}


def const_like(ref, data, key):
    """``ref.new_tensor(data)``, cached per (key, device, dtype): small constant tables (bin edges, radii, one-hot
    indices) are uploaded once instead of on every call, which also keeps host-to-device copies out of CUDA-graph
    capture.  ``key`` names the constant (include any parameter the data depends on)."""
    k = (key, ref.device, ref.dtype)
    t = _CONST_CACHE.get(k)
    if t is None:
        t = ref.new_tensor(data)
        _CONST_CACHE[k] = t
    return t
