"""Tiny stand-in for dm-tree: only what the reference's constants module calls."""


def map_structure(fn, *structs):
    s0 = structs[0]
    if isinstance(s0, dict):
        return {k: map_structure(fn, *[s[k] for s in structs]) for k in s0}
    if isinstance(s0, (list, tuple)):
        out = [map_structure(fn, *xs) for xs in zip(*structs)]
        return type(s0)(out) if not hasattr(s0, "_fields") else type(s0)(*out)
    return fn(*structs)


def flatten(struct):
    if isinstance(struct, dict):
        return [x for k in sorted(struct) for x in flatten(struct[k])]
    if isinstance(struct, (list, tuple)):
        return [x for s in struct for x in flatten(s)]
    return [struct]
