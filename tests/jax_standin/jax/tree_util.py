"""Pytree flattening with JAX's ordering rules: dict keys sorted, tuples / lists / named tuples in
field order, None an empty node, everything else a leaf."""
from __future__ import annotations

from typing import Any, Callable, List, Optional, Tuple


class DictKey:
    def __init__(self, key):
        self.key = key

    def __repr__(self):
        return f"[{self.key!r}]"

    def __eq__(self, other):
        return isinstance(other, DictKey) and self.key == other.key

    def __hash__(self):
        return hash(("d", self.key))


class SequenceKey:
    def __init__(self, idx):
        self.idx = idx

    def __repr__(self):
        return f"[{self.idx}]"

    def __eq__(self, other):
        return isinstance(other, SequenceKey) and self.idx == other.idx

    def __hash__(self):
        return hash(("s", self.idx))


class GetAttrKey:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f".{self.name}"

    def __eq__(self, other):
        return isinstance(other, GetAttrKey) and self.name == other.name

    def __hash__(self):
        return hash(("a", self.name))


def _is_namedtuple(x) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


class PyTreeDef:
    """Structure of a pytree: a nested description with `*` for leaves."""

    def __init__(self, spec):
        self.spec = spec

    def __eq__(self, other):
        return isinstance(other, PyTreeDef) and self.spec == other.spec

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(repr(self.spec))

    def __repr__(self):
        return f"PyTreeDef({self.spec!r})"

    @property
    def num_leaves(self) -> int:
        def count(s):
            if s == "*":
                return 1
            if s is None:
                return 0
            return sum(count(c) for c in s[2])
        return count(self.spec)

    def unflatten(self, leaves):
        it = iter(leaves)

        def build(s):
            if s == "*":
                return next(it)
            if s is None:
                return None
            kind, meta, children = s
            built = [build(c) for c in children]
            if kind == "dict":
                return dict(zip(meta, built))
            if kind == "list":
                return list(built)
            if kind == "tuple":
                return tuple(built)
            if kind == "namedtuple":
                return meta(*built)
            raise TypeError(kind)

        out = build(self.spec)
        rest = list(it)
        if rest:
            raise ValueError("too many leaves for this tree structure")
        return out


def _flatten(tree, is_leaf, path, out):
    if is_leaf is not None and is_leaf(tree):
        out.append((path, tree))
        return "*"
    if tree is None:
        return None
    if isinstance(tree, dict):
        keys = sorted(tree.keys())
        return ("dict", tuple(keys), tuple(_flatten(tree[k], is_leaf, path + (DictKey(k),), out) for k in keys))
    if _is_namedtuple(tree):
        return ("namedtuple", type(tree), tuple(
            _flatten(getattr(tree, f), is_leaf, path + (GetAttrKey(f),), out) for f in type(tree)._fields))
    if isinstance(tree, (list, tuple)):
        kind = "list" if isinstance(tree, list) else "tuple"
        return (kind, None, tuple(_flatten(c, is_leaf, path + (SequenceKey(i),), out) for i, c in enumerate(tree)))
    out.append((path, tree))
    return "*"


def tree_flatten_with_path(tree, is_leaf: Optional[Callable[[Any], bool]] = None):
    out: List[Tuple[tuple, Any]] = []
    spec = _flatten(tree, is_leaf, (), out)
    return out, PyTreeDef(spec)


def tree_flatten(tree, is_leaf: Optional[Callable[[Any], bool]] = None):
    path_leaves, treedef = tree_flatten_with_path(tree, is_leaf)
    return [leaf for _, leaf in path_leaves], treedef


def tree_leaves(tree, is_leaf=None):
    return tree_flatten(tree, is_leaf)[0]


def tree_structure(tree, is_leaf=None):
    return tree_flatten(tree, is_leaf)[1]


def tree_unflatten(treedef, leaves):
    return treedef.unflatten(leaves)


def tree_map(fn, tree, *rest, is_leaf=None):
    leaves, treedef = tree_flatten(tree, is_leaf)
    others = []
    for r in rest:
        # the other trees are flattened up to the first tree's structure
        r_leaves, r_def = tree_flatten(r, is_leaf=lambda x, _d=treedef: False if is_leaf is None else is_leaf(x))
        if r_def != treedef:
            r_leaves = _flatten_up_to(treedef.spec, r)
        others.append(r_leaves)
    return treedef.unflatten([fn(*args) for args in zip(leaves, *others)])


def _flatten_up_to(spec, tree):
    out = []

    def walk(s, t):
        if s == "*":
            out.append(t)
            return
        if s is None:
            return
        kind, meta, children = s
        if kind == "dict":
            for k, c in zip(meta, children):
                walk(c, t[k])
        elif kind == "namedtuple":
            for f, c in zip(meta._fields, children):
                walk(c, getattr(t, f))
        else:
            for i, c in enumerate(children):
                walk(c, t[i])

    walk(spec, tree)
    return out
