"""bench.py and __graft_entry__.py only run on a GPU box; a name that is not defined where it is
used would surface there, at the end of a run.  This checks every function statically."""

import ast
import builtins
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bound_names(node):
    """Names bound anywhere inside `node` (assignments, imports, defs, loop / with / except targets, arguments)."""
    out = set()
    for n in ast.walk(node):
        if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            out.add(n.name)
        if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.Lambda)):
            a = n.args
            for arg in a.posonlyargs + a.args + a.kwonlyargs + ([a.vararg] if a.vararg else []) + ([a.kwarg] if a.kwarg else []):
                out.add(arg.arg)
        elif isinstance(n, ast.Name) and isinstance(n.ctx, (ast.Store, ast.Del)):
            out.add(n.id)
        elif isinstance(n, (ast.Import, ast.ImportFrom)):
            for alias in n.names:
                out.add((alias.asname or alias.name).split(".")[0])
        elif isinstance(n, ast.ExceptHandler) and n.name:
            out.add(n.name)
        elif isinstance(n, (ast.Global, ast.Nonlocal)):
            out.update(n.names)
    return out


@pytest.mark.parametrize("name", ["bench.py", "__graft_entry__.py"])
def test_every_name_used_in_a_function_is_bound_somewhere_visible(name):
    tree = ast.parse(open(os.path.join(ROOT, name)).read())
    module_names = set(dir(builtins)) | {"__file__", "__name__"}
    for node in tree.body:  # module level only (not what functions bind locally)
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            module_names.add(node.name)
        else:
            module_names |= _bound_names(node)

    problems = []

    def visit(fn, visible):
        visible = visible | _bound_names(fn)  # a function sees what it and its nested functions bind (over-approximation)
        for n in ast.walk(fn):
            if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Load) and n.id not in visible:
                problems.append(f"{name}:{n.lineno}: {n.id} in {fn.name}")

    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)):
            visit(node, module_names)
    assert not problems, problems
