"""Every name a function reads resolves: to a local, an enclosing scope, a
module-level definition or a builtin.  A stand-in for a linter on a machine
that has none; it finds the misspelt or never-imported name that would
otherwise raise NameError only on the path that reaches it (the benchmark
drivers' GPU-only branches, for instance)."""
import builtins
import pathlib
import symtable

ROOT = pathlib.Path(__file__).resolve().parent.parent
FILES = sorted(list((ROOT / "symm_mem_recipes_b200").rglob("*.py")) + list((ROOT / "tests").glob("*.py")) +
               list((ROOT / "baseline").glob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"])
MODULE_IMPLICIT = {"__file__", "__name__", "__doc__", "__package__", "__spec__", "__builtins__", "__class__"}


def _undefined(table: symtable.SymbolTable, module_names: set, path: str, out: list) -> None:
    for sym in table.get_symbols():
        name = sym.get_name()
        if not sym.is_referenced():
            continue
        if table.get_type() == "module":
            resolved = sym.is_assigned() or sym.is_imported() or sym.is_namespace()
        else:
            # local, parameter, free (enclosing function) or class-body names are bound where they are used
            resolved = not sym.is_global() or sym.is_assigned() and not sym.is_declared_global()
            if sym.is_declared_global():
                resolved = False
        if resolved or name in module_names or hasattr(builtins, name) or name in MODULE_IMPLICIT:
            continue
        out.append(f"{path}:{table.get_lineno()}: '{name}' in {table.get_type()} '{table.get_name()}' is not defined")
    for child in table.get_children():
        _undefined(child, module_names, path, out)


def test_no_undefined_names():
    problems = []
    assert len(FILES) > 40
    for path in FILES:
        src = path.read_text()
        top = symtable.symtable(src, str(path), "exec")
        module_names = {s.get_name() for s in top.get_symbols()
                        if s.is_assigned() or s.is_imported() or s.is_namespace()}
        # names bound through `global x` inside functions count as module names
        def collect_globals(t):
            for s in t.get_symbols():
                if t.get_type() != "module" and s.is_declared_global() and s.is_assigned():
                    module_names.add(s.get_name())
            for c in t.get_children():
                collect_globals(c)
        collect_globals(top)
        _undefined(top, module_names, str(path.relative_to(ROOT)), problems)
    assert not problems, "\n".join(problems)
