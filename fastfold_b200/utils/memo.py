"""Per-call memo for tensors that depend on the masks only.

Every block of a stack pads, scatters, transposes and converts the same two mask tensors, and combines them into the
same normalisers (48 blocks x forward and recomputation passes).  ``run_blocks`` creates one ``Memo`` per stack call
and each block runs under ``use(memo)``; ``cached(tag, sources, fn)`` then computes ``fn()`` once per distinct
``(tag, sources)`` and hands the same tensor to every later block.  Keys are the identities of the source tensors; the
memo keeps the sources alive, so an identity cannot be reused while the memo exists.  Tensors that require grad are
never memoised.  The results must be treated as read-only.

The reference recomputes these per block (fastfold/model/fastnn/evoformer.py:60-76, ops.py:137-160); the values are
the same, only the number of small kernels differs.
"""
import contextlib

_ACTIVE = None


class Memo:
    def __init__(self):
        self.values = {}
        self.keep = []


@contextlib.contextmanager
def use(memo):
    global _ACTIVE
    prev = _ACTIVE
    _ACTIVE = memo
    try:
        yield
    finally:
        _ACTIVE = prev


def cached(tag, sources, fn):
    m = _ACTIVE
    if m is None or any(t.requires_grad for t in sources):
        return fn()
    key = (tag,) + tuple(id(t) for t in sources)
    hit = m.values.get(key)
    if hit is None:
        m.keep.extend(sources)
        hit = fn()
        m.values[key] = hit
        if hasattr(hit, "requires_grad"):
            m.keep.append(hit)           # results are sources of later entries: keep their identities unique too
    return hit
