"""Every `C.<function>(...)` call in the package against the signature the
built extension publishes for that function (pybind11 writes it into the
docstring): enough positional arguments for the parameters without a default,
not more than there are parameters, keywords that exist.  A call site that
drifted from its binding fails here, on the CPU, instead of on the first GPU
run."""
import ast
import pathlib

import pytest

from symm_mem_recipes_b200._ext import C

PKG = pathlib.Path(__file__).resolve().parent.parent / "symm_mem_recipes_b200"
ROOT_FILES = [PKG.parent / "bench.py", PKG.parent / "__graft_entry__.py"]


def _split_top_level(text: str) -> list[str]:
    parts, depth, cur = [], 0, ""
    for ch in text:
        if ch in "[(":
            depth += 1
        elif ch in "])":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur.strip())
    return parts


def _published_signatures(name: str) -> list[list[tuple[str, bool]]]:
    """[(parameter name, has default), ...] per overload of C.<name>."""
    doc = getattr(C, name).__doc__ or ""
    sigs = []
    for line in doc.splitlines():
        line = line.strip()
        if line[:2].isdigit() or line[:1].isdigit():          # "1. name(...)" lines of an overload set
            line = line.split(". ", 1)[1] if ". " in line else line
        if not line.startswith(name + "("):
            continue
        inner = line[len(name) + 1:line.rindex(")")]
        params = []
        for p in _split_top_level(inner):
            if p in ("*", "/"):
                continue
            pname = p.split(":", 1)[0].strip()
            params.append((pname, " = " in p))
        sigs.append(params)
    return sigs


def _call_sites():
    files = [p for p in PKG.rglob("*.py")] + [p for p in ROOT_FILES if p.exists()]
    for path in sorted(files):
        tree = ast.parse(path.read_text(), filename=str(path))
        for node in ast.walk(tree):
            if (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)
                    and isinstance(node.func.value, ast.Name) and node.func.value.id == "C"):
                yield path, node


def _fits(params, n_pos, kw_names, has_star):
    named = {p for p, _ in params}
    positional_only_names = all(p.startswith("arg") and p[3:].isdigit() for p, _ in params) and bool(params)
    if n_pos > len(params):
        return f"{n_pos} positional arguments for {len(params)} parameters"
    if kw_names and positional_only_names:
        return "keywords passed to a binding without parameter names"
    for k in kw_names:
        if k not in named:
            return f"no parameter named {k!r}"
        if k in [p for p, _ in params[:n_pos]]:
            return f"{k!r} given twice"
    if has_star:
        return None                                            # *args / **kwargs: only the checks above
    for i, (p, has_default) in enumerate(params):
        if i >= n_pos and not has_default and p not in kw_names:
            return f"parameter {p!r} (position {i}) not supplied"
    return None


def test_every_native_call_site_fits_its_binding():
    checked, problems = 0, []
    for path, node in _call_sites():
        name = node.func.attr
        fn = getattr(C, name, None)
        if fn is None:
            problems.append(f"{path.name}:{node.lineno}: C.{name} does not exist")
            continue
        if not callable(fn) or isinstance(fn, type):
            continue                                           # constants and classes
        sigs = _published_signatures(name)
        if not sigs:
            continue
        n_pos = sum(1 for a in node.args if not isinstance(a, ast.Starred))
        has_star = any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords)
        kw_names = [k.arg for k in node.keywords if k.arg is not None]
        verdicts = [_fits(params, n_pos, kw_names, has_star) for params in sigs]
        checked += 1
        if all(v is not None for v in verdicts):
            problems.append(f"{path.relative_to(PKG.parent)}:{node.lineno}: C.{name}: {verdicts[0]}")
    assert not problems, "\n".join(problems)
    assert checked >= 30                                       # the walk really found the call sites


@pytest.mark.parametrize("name,expected", [
    ("ag_matmul", ["a", "b", "c", "mode", "aout_alloc", "aout_offset", "a_out", "block_n", "num_sms", "timeout_ns",
                   "tail_scratch", "epilogue", "trace", "lead", "push_ahead", "push_plain_stores",
                   "push_pieces", "panel_w"]),
    ("matmul_reduce_scatter", ["a", "b", "out", "workspace", "num_sms", "timeout_ns", "trace", "panel_w"]),
    ("matmul_all_reduce", ["a", "b", "out", "out_alloc", "out_offset", "workspace", "num_sms", "timeout_ns",
                           "panel_w"]),
    ("gemv_all_reduce", ["x", "w", "out", "workspace", "ws_offset", "timeout_ns", "tensor_core", "num_sms",
                         "tagged", "weights_nk"]),
    ("rms_norm", ["x", "residual", "w", "sum_out", "out", "eps"]),
])
def test_stand_ins_of_the_flow_tests_follow_the_bindings(name, expected):
    """The CPU flow tests replace these entry points by host functions written
    with these parameter lists; the bindings must keep publishing the same."""
    (params,) = _published_signatures(name)
    assert [p for p, _ in params] == expected
