"""A small pytree implementation with JAX's flattening rules.

The reference leans on jax.tree_util for three things: flattening nested containers in a
deterministic order (dict keys sorted), naming every leaf by its path, and comparing tree
structures.  This module provides exactly that for dict / list / tuple / NamedTuple / None
containers; anything else (tensors, numbers, arrays) is a leaf.  Paths are tuples of dict
keys, sequence indices and NamedTuple field names, the form the reference normalises JAX
key paths to (flashoptim_jax/utils.py:76-91).
"""

from __future__ import annotations

from typing import Any, Callable, List, Optional, Sequence, Tuple

_LEAF = "*"


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


class TreeDef:
    """Structure of a pytree: container kinds, keys and leaf count; hashable and comparable."""

    __slots__ = ("kind", "meta", "children", "num_leaves")

    def __init__(self, kind: str, meta: Any, children: Tuple["TreeDef", ...]):
        self.kind = kind
        self.meta = meta
        self.children = children
        self.num_leaves = 1 if kind == _LEAF else sum(c.num_leaves for c in children)

    def _key(self):
        meta = self.meta
        if self.kind == "namedtuple":
            meta = (meta.__module__, meta.__qualname__, meta._fields)
        return (self.kind, meta, tuple(c._key() for c in self.children))

    def __eq__(self, other):
        return isinstance(other, TreeDef) and self._key() == other._key()

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(self._key())

    def __repr__(self):
        if self.kind == _LEAF:
            return "*"
        if self.kind == "none":
            return "None"
        inner = ", ".join(repr(c) for c in self.children)
        if self.kind == "dict":
            inner = ", ".join(f"{k!r}: {c!r}" for k, c in zip(self.meta, self.children))
            return "{" + inner + "}"
        if self.kind == "list":
            return "[" + inner + "]"
        if self.kind == "tuple":
            return "(" + inner + ")"
        return f"{self.meta.__name__}({inner})"

    def unflatten(self, leaves: Sequence[Any]) -> Any:
        leaves = list(leaves)
        if len(leaves) != self.num_leaves:
            raise ValueError(f"treedef expects {self.num_leaves} leaves, got {len(leaves)}")
        out, used = self._build(leaves, 0)
        assert used == len(leaves)
        return out

    def _build(self, leaves: List[Any], pos: int):
        if self.kind == _LEAF:
            return leaves[pos], pos + 1
        if self.kind == "none":
            return None, pos
        items = []
        for c in self.children:
            v, pos = c._build(leaves, pos)
            items.append(v)
        if self.kind == "dict":
            return dict(zip(self.meta, items)), pos
        if self.kind == "list":
            return items, pos
        if self.kind == "tuple":
            return tuple(items), pos
        return self.meta(*items), pos


def _flatten(x: Any, path: Tuple[Any, ...], is_leaf: Optional[Callable[[Any], bool]], out: List[Tuple[Tuple[Any, ...], Any]]) -> TreeDef:
    if is_leaf is not None and is_leaf(x):
        out.append((path, x))
        return TreeDef(_LEAF, None, ())
    if x is None:
        return TreeDef("none", None, ())
    if isinstance(x, dict):
        try:
            keys = tuple(sorted(x.keys()))
        except TypeError:
            keys = tuple(x.keys())
        return TreeDef("dict", keys, tuple(_flatten(x[k], path + (k,), is_leaf, out) for k in keys))
    if _is_namedtuple(x):
        fields = type(x)._fields
        return TreeDef("namedtuple", type(x), tuple(_flatten(getattr(x, f), path + (f,), is_leaf, out) for f in fields))
    if isinstance(x, list):
        return TreeDef("list", len(x), tuple(_flatten(v, path + (i,), is_leaf, out) for i, v in enumerate(x)))
    if isinstance(x, tuple):
        return TreeDef("tuple", len(x), tuple(_flatten(v, path + (i,), is_leaf, out) for i, v in enumerate(x)))
    out.append((path, x))
    return TreeDef(_LEAF, None, ())


def tree_flatten(tree: Any, is_leaf: Optional[Callable[[Any], bool]] = None) -> Tuple[List[Any], TreeDef]:
    out: List[Tuple[Tuple[Any, ...], Any]] = []
    treedef = _flatten(tree, (), is_leaf, out)
    return [leaf for _, leaf in out], treedef


def tree_flatten_with_path(tree: Any, is_leaf: Optional[Callable[[Any], bool]] = None):
    out: List[Tuple[Tuple[Any, ...], Any]] = []
    treedef = _flatten(tree, (), is_leaf, out)
    return out, treedef


_CONTAINERS = (dict, tuple, list)


def _walk(x: Any, is_leaf: Optional[Callable[[Any], bool]], out: List[Any], sig: Optional[List[Any]]) -> None:
    """The leaves of x in flattening order, without paths or TreeDef objects; `sig`, when given, receives one
    entry per container in pre-order (kind with keys / type / length, and the number of leaves seen before
    it): two trees have the same structure iff their leaf counts and these lists agree (a child slot whose
    turn comes when the leaf count equals the next container's offset must be that container)."""
    if is_leaf is not None and is_leaf(x):
        out.append(x)
        return
    if x is None:
        if sig is not None:
            sig.append((None, len(out)))
        return
    if isinstance(x, dict):
        try:
            keys = sorted(x)
        except TypeError:
            keys = list(x)
        if sig is not None:
            sig.append(("dict", tuple(keys), len(out)))
        children = [x[k] for k in keys]
    elif isinstance(x, tuple):
        if sig is not None:
            sig.append((type(x) if hasattr(type(x), "_fields") else "tuple", len(x), len(out)))
        children = x
    elif isinstance(x, list):
        if sig is not None:
            sig.append(("list", len(x), len(out)))
        children = x
    else:
        out.append(x)
        return
    for v in children:  # leaves are taken here, without a call of their own
        if v is not None and not isinstance(v, _CONTAINERS) and (is_leaf is None or not is_leaf(v)):
            out.append(v)
        else:
            _walk(v, is_leaf, out, sig)


def tree_leaves(tree: Any, is_leaf: Optional[Callable[[Any], bool]] = None) -> List[Any]:
    out: List[Any] = []
    _walk(tree, is_leaf, out, None)
    return out


def tree_leaves_and_signature(tree: Any, is_leaf: Optional[Callable[[Any], bool]] = None) -> Tuple[List[Any], List[Any]]:
    """Leaves plus a cheap structural signature (see _walk): equal signatures and leaf counts mean equal
    tree structures.  For hot paths that re-check a structure on every call."""
    out: List[Any] = []
    sig: List[Any] = []
    _walk(tree, is_leaf, out, sig)
    return out, sig


def tree_structure(tree: Any, is_leaf: Optional[Callable[[Any], bool]] = None) -> TreeDef:
    return tree_flatten(tree, is_leaf)[1]


def tree_unflatten(treedef: TreeDef, leaves: Sequence[Any]) -> Any:
    return treedef.unflatten(leaves)


def tree_map(fn: Callable[..., Any], tree: Any, *rest: Any, is_leaf: Optional[Callable[[Any], bool]] = None) -> Any:
    leaves, treedef = tree_flatten(tree, is_leaf)
    others = []
    for r in rest:
        r_leaves, r_def = tree_flatten(r, is_leaf)
        if r_def != treedef:
            raise ValueError(f"tree_map: tree structures differ: {treedef} vs {r_def}")
        others.append(r_leaves)
    return treedef.unflatten([fn(*args) for args in zip(leaves, *others)])
