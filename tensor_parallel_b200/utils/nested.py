"""Pytree helpers for arbitrarily nested call arguments and model outputs.

Inputs of a tensor-parallel forward are walked leaf by leaf so that tensors can be
replicated to every rank while non-tensor leaves (``None``, ints, per-device KV caches)
are passed through untouched.  Behaviour to preserve (reference:
``src/tensor_parallel/utils.py:16-106``): dict entries are visited in sorted-key order,
namedtuples and Hugging Face ``ModelOutput`` containers are rebuilt with their own type.
"""
from __future__ import annotations

from typing import Any, Callable, Iterator, List


def _is_namedtuple(obj: Any) -> bool:
    return isinstance(obj, tuple) and hasattr(type(obj), "_fields")


def _kind(obj: Any) -> str:
    if isinstance(obj, dict):
        return "map"
    if isinstance(obj, (list, tuple)):
        return "seq"
    return "leaf"


def nested_flatten(tree: Any) -> Iterator[Any]:
    """Yield the leaves of ``tree`` depth-first; mapping values come in sorted-key order."""
    stack: List[Any] = [tree]
    while stack:
        node = stack.pop()
        kind = _kind(node)
        if kind == "seq":
            stack.extend(reversed(list(node)))
        elif kind == "map":
            stack.extend(node[k] for k in sorted(node.keys(), reverse=True))
        else:
            yield node


def _rebuild(leaves: Iterator[Any], like: Any) -> Any:
    kind = _kind(like)
    if kind == "seq":
        items = [_rebuild(leaves, child) for child in like]
        if _is_namedtuple(like):
            return type(like)(*items)
        return type(like)(items)
    if kind == "map":
        rebuilt = {k: _rebuild(leaves, like[k]) for k in sorted(like.keys())}
        if type(like) is dict:
            return rebuilt
        try:  # ModelOutput-style containers accept a mapping / keyword arguments
            return type(like)(**rebuilt)
        except Exception:
            try:
                return type(like)(rebuilt)
            except Exception:
                return rebuilt
    return next(leaves)


def nested_pack(flat, structure: Any) -> Any:
    """Inverse of :func:`nested_flatten`: fill ``structure``'s shape with the leaves in ``flat``."""
    return _rebuild(iter(flat), structure)


def nested_compare(a: Any, b: Any) -> bool:
    """True when ``a`` and ``b`` have the same container skeleton (leaf values are ignored)."""
    ka, kb = _kind(a), _kind(b)
    if ka != kb:
        return ka == "leaf" and kb == "leaf"
    if ka == "seq":
        return isinstance(b, type(a)) and len(a) == len(b) and all(nested_compare(x, y) for x, y in zip(a, b))
    if ka == "map":
        return set(a.keys()) == set(b.keys()) and all(nested_compare(a[k], b[k]) for k in a)
    return True


def nested_map(fn: Callable, *trees: Any) -> Any:
    """Apply ``fn`` leaf-wise over one or more identically shaped trees."""
    if not trees:
        raise ValueError("nested_map needs at least one tree")
    for other in trees[1:]:
        if not nested_compare(trees[0], other):
            raise ValueError(f"nested structures differ: {trees[0]!r} vs {other!r}")
    return nested_pack(map(fn, *map(nested_flatten, trees)), trees[0])
