"""Every `module.attribute` that names a module of this package resolves: the
benchmark drivers, the model and the tests reach the ops through aliases such
as `smr.`, `ops.` and `symm_mem.`; an attribute that the module does not
export would raise only on the line that uses it."""
import ast
import importlib
import pathlib
import types

ROOT = pathlib.Path(__file__).resolve().parent.parent
PKG = "symm_mem_recipes_b200"
FILES = sorted(list((ROOT / PKG).rglob("*.py")) + list((ROOT / "tests").glob("*.py")) +
               [ROOT / "bench.py", ROOT / "__graft_entry__.py"])


def _package_of(path: pathlib.Path) -> str:
    rel = path.relative_to(ROOT)
    if rel.parts[0] != PKG:
        return ""
    return ".".join(rel.parts[:-1])


def _module_aliases(tree: ast.AST, package: str) -> dict:
    """alias -> module object, for imports (anywhere in the file) of modules of this package."""
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name.split(".")[0] == PKG and a.asname:
                    found[a.asname] = importlib.import_module(a.name)
        elif isinstance(node, ast.ImportFrom):
            if node.level:
                base = package.split(".") if package else []
                if node.level > 1:
                    base = base[: len(base) - (node.level - 1)]
                mod = ".".join(base + ([node.module] if node.module else []))
            else:
                mod = node.module or ""
            if mod.split(".")[0] != PKG:
                continue
            parent = importlib.import_module(mod)
            for a in node.names:
                # what the import statement binds: the attribute if the module has one of that name
                # (`from .. import ops`; `ops.matmul_reduce_scatter` is the function, not the submodule)
                if hasattr(parent, a.name):
                    obj = getattr(parent, a.name)
                else:
                    try:
                        obj = importlib.import_module(f"{mod}.{a.name}")
                    except ImportError:
                        continue
                if isinstance(obj, types.ModuleType) and (obj.__name__.split(".")[0] == PKG):
                    found[a.asname or a.name] = obj
    return found


def test_attributes_of_package_modules_exist():
    problems, checked = [], 0
    for path in FILES:
        tree = ast.parse(path.read_text(), filename=str(path))
        aliases = _module_aliases(tree, _package_of(path))
        # an alias that is also assigned or used as a parameter somewhere in the file may be something else
        rebound = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store)}
        rebound |= {a.arg for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.Lambda))
                    for a in n.args.args + n.args.kwonlyargs}
        for node in ast.walk(tree):
            if (isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id in aliases
                    and node.value.id not in rebound and isinstance(node.ctx, ast.Load)):
                mod = aliases[node.value.id]
                if mod.__name__.endswith("._C"):
                    continue
                checked += 1
                if not hasattr(mod, node.attr):
                    problems.append(f"{path.relative_to(ROOT)}:{node.lineno}: {mod.__name__} has no attribute "
                                    f"'{node.attr}'")
    assert not problems, "\n".join(problems)
    assert checked > 300


def test_calls_into_package_modules_fit_the_signatures():
    """`alias.function(...)` with a Python function of this package: keywords that the function
    takes, no more positional arguments than it has parameters, no required parameter left out."""
    import inspect

    problems, checked = [], 0
    for path in FILES:
        tree = ast.parse(path.read_text(), filename=str(path))
        aliases = _module_aliases(tree, _package_of(path))
        rebound = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store)}
        rebound |= {a.arg for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.Lambda))
                    for a in n.args.args + n.args.kwonlyargs}
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)
                    and isinstance(node.func.value, ast.Name) and node.func.value.id in aliases
                    and node.func.value.id not in rebound):
                continue
            fn = getattr(aliases[node.func.value.id], node.func.attr, None)
            target = fn.__init__ if inspect.isclass(fn) else fn
            if not (inspect.isfunction(target) or inspect.ismethod(target)):
                continue
            try:
                sig = inspect.signature(fn)
            except (TypeError, ValueError):
                continue
            params = list(sig.parameters.values())
            has_var_kw = any(p.kind is p.VAR_KEYWORD for p in params)
            has_var_pos = any(p.kind is p.VAR_POSITIONAL for p in params)
            positional = [p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
            n_pos = sum(1 for a in node.args if not isinstance(a, ast.Starred))
            starred = any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords)
            kw = [k.arg for k in node.keywords if k.arg is not None]
            where = f"{path.relative_to(ROOT)}:{node.lineno}: {node.func.value.id}.{node.func.attr}"
            checked += 1
            if n_pos > len(positional) and not has_var_pos:
                problems.append(f"{where}: {n_pos} positional arguments, {len(positional)} accepted")
            names = {p.name for p in params if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)}
            for k in kw:
                if k not in names and not has_var_kw:
                    problems.append(f"{where}: no parameter '{k}'")
            if not starred:
                for i, p in enumerate(positional):
                    if p.default is p.empty and i >= n_pos and p.name not in kw:
                        problems.append(f"{where}: required parameter '{p.name}' not supplied")
                for p in params:
                    if p.kind is p.KEYWORD_ONLY and p.default is p.empty and p.name not in kw:
                        problems.append(f"{where}: required keyword '{p.name}' not supplied")
    assert not problems, "\n".join(problems)
    assert checked > 150
