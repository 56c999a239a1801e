"""Small tensor helpers shared by the model code (role of fastfold/utils/tensor_utils.py)."""
from functools import partial

import torch


def permute_final_dims(tensor, inds):
    zero_index = -1 * len(inds)
    first = list(range(len(tensor.shape[:zero_index])))
    return tensor.permute(first + [zero_index + i for i in inds])


def flatten_final_dims(t, no_dims):
    return t.reshape(t.shape[:-no_dims] + (-1,))


def masked_mean(mask, value, dim, eps=1e-4):
    mask = mask.expand(*value.shape)
    return torch.sum(mask * value, dim=dim) / (eps + torch.sum(mask, dim=dim))


def pts_to_distogram(pts, min_bin=2.3125, max_bin=21.6875, no_bins=64):
    boundaries = torch.linspace(min_bin, max_bin, no_bins - 1, device=pts.device)
    dists = torch.sqrt(torch.sum((pts.unsqueeze(-2) - pts.unsqueeze(-3)) ** 2, dim=-1))
    return torch.bucketize(dists, boundaries)


def one_hot(x, v_bins):
    """Nearest-bin one-hot of ``x`` against bin centres ``v_bins``."""
    diffs = x[..., None] - v_bins.reshape((1,) * x.dim() + (len(v_bins),))
    am = torch.argmin(torch.abs(diffs), dim=-1)
    return torch.nn.functional.one_hot(am, num_classes=len(v_bins)).float()


def batched_gather(data, inds, dim=0, no_batch_dims=0):
    ranges = []
    for i, s in enumerate(data.shape[:no_batch_dims]):
        r = torch.arange(s, device=inds.device)
        r = r.view(*(*((1,) * i), -1, *((1,) * (len(inds.shape) - i - 1))))
        ranges.append(r)
    remaining = [slice(None) for _ in range(len(data.shape) - no_batch_dims)]
    remaining[dim - no_batch_dims if dim >= 0 else dim] = inds
    ranges.extend(remaining)
    return data[tuple(ranges)]


def dict_multimap(fn, dicts):
    first = dicts[0]
    out = {}
    for k, v in first.items():
        all_v = [d[k] for d in dicts]
        out[k] = dict_multimap(fn, all_v) if isinstance(v, dict) else fn(all_v)
    return out


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


def _fetch_dims(tree):
    shapes = []
    if isinstance(tree, dict):
        for v in tree.values():
            shapes.extend(_fetch_dims(v))
    elif isinstance(tree, (list, tuple)):
        for t in tree:
            shapes.extend(_fetch_dims(t))
    elif isinstance(tree, torch.Tensor):
        shapes.append(tree.shape)
    else:
        raise ValueError("unsupported tree node")
    return shapes


def chunk_layer(layer, inputs, chunk_size, no_batch_dims):
    """Applies ``layer(**inputs)`` over flattened leading (batch-like) dims in pieces of ``chunk_size``.

    Inputs are broadcast against each other over their first ``no_batch_dims`` dims, flattened to one
    batch dim, sliced, run, and the outputs (tensor / tuple / dict) reassembled - OpenFold's chunking
    technique (supplement 1.11.8), same contract as fastfold/utils/tensor_utils.py:298-415.
    """
    if not len(inputs) > 0:
        raise ValueError("Must provide at least one input")
    initial_dims = [shape[:no_batch_dims] for shape in _fetch_dims(inputs)]
    orig_batch_dims = tuple(max(s) for s in zip(*initial_dims))

    def prep(t):
        # inputs whose batch dims are all 1 (e.g. a bias shared by every row) stay un-expanded and are not sliced
        if not sum(t.shape[:no_batch_dims]) == no_batch_dims:
            t = t.expand(orig_batch_dims + t.shape[no_batch_dims:])
        return t.reshape(-1, *t.shape[no_batch_dims:])

    prepped = tensor_tree_map(prep, inputs)
    flat_batch_dim = 1
    for d in orig_batch_dims:
        flat_batch_dim *= d
    no_chunks = flat_batch_dim // chunk_size + (flat_batch_dim % chunk_size != 0)
    i = 0
    out = None
    for _ in range(no_chunks):
        def sel(t):
            return t[i:i + chunk_size] if t.shape[0] != 1 else t
        chunks = tensor_tree_map(sel, prepped)
        output_chunk = layer(**chunks)
        if out is None:
            alloc = lambda t: t.new_zeros((flat_batch_dim,) + t.shape[1:])
            out = tensor_tree_map(alloc, output_chunk)
        if isinstance(output_chunk, dict):
            def assign(d1, d2):
                for k, v in d1.items():
                    if isinstance(v, dict):
                        assign(v, d2[k])
                    else:
                        v[i:i + chunk_size] = d2[k]
            assign(out, output_chunk)
        elif isinstance(output_chunk, tuple):
            for x1, x2 in zip(out, output_chunk):
                x1[i:i + chunk_size] = x2
        elif isinstance(output_chunk, torch.Tensor):
            out[i:i + chunk_size] = output_chunk
        else:
            raise ValueError("unsupported layer output")
        i += chunk_size
    reshape = lambda t: t.view(orig_batch_dims + t.shape[1:])
    return tensor_tree_map(reshape, out)


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
