"""Implementation registry: the reference's dispatch surface (src/moba_opt/api.py:14-27)."""

_IMPLS = {}


def register(name, fn):
    """Registers an implementation; a duplicate name is a KeyError (api.py:14-17)."""
    if name in _IMPLS:
        raise KeyError(f"impl already registered: {name}")
    _IMPLS[name] = fn


def available_impls():
    """Sorted implementation names (api.py:20-21)."""
    return sorted(_IMPLS)


def run_impl(name, q, k, v, cu_seqlens, max_seqlen, config):
    """Calls implementation `name` as fn(q, k, v, cu_seqlens, max_seqlen, config) (api.py:24-27)."""
    if name not in _IMPLS:
        raise KeyError(f"unknown impl {name!r}; available: {available_impls()}")
    return _IMPLS[name](q, k, v, cu_seqlens, max_seqlen, config)
