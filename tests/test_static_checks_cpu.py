"""Static checks of the Python sources that guard the branches only a GPU run reaches: every kernel entry point is
called with as many arguments as its prototype takes, and no function reads a global name that nothing defines."""
import ast
import builtins
import pathlib
import symtable

from ksa_b200.ops import _lib

ROOT = pathlib.Path(__file__).resolve().parent.parent
SOURCES = sorted(p for d in ("ksa_b200", "recipes", "baseline", "examples") for p in (ROOT / d).rglob("*.py")
                 if "_ref" not in p.parts and "_ref_kernels" not in p.parts) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]


def test_kernel_entry_points_are_called_with_the_prototypes_argument_counts():
    sig = _lib._SIGNATURES
    checked, problems = 0, []
    for f in SOURCES:
        for node in ast.walk(ast.parse(f.read_text())):
            if not isinstance(node, ast.Call) or not node.args:
                continue
            fn = node.func
            if isinstance(fn, ast.Attribute) and isinstance(fn.value, ast.Name) and fn.value.id == "_lib":
                kind = fn.attr
            elif isinstance(fn, ast.Name) and f.name == "_lib.py":
                kind = fn.id
            else:
                continue
            if kind not in ("call", "call_nostream", "call_on"):
                continue
            first = node.args[0]
            if not (isinstance(first, ast.Constant) and isinstance(first.value, str)):
                continue
            name = first.value
            if name not in sig:
                problems.append(f"{f.name}:{node.lineno}: {name} has no bound signature")
                continue
            if any(isinstance(a, ast.Starred) for a in node.args):
                continue
            n = len(node.args) - 1
            n += 1 if kind == "call" else 0            # `call` appends the stream; `call_on` takes it in second place
            checked += 1
            if n != len(sig[name]):
                problems.append(f"{f.name}:{node.lineno}: {name} gets {n} arguments, its prototype takes {len(sig[name])}")
    assert not problems, problems
    assert checked >= 50


def _defined_at_module_level(tree) -> set:
    names = set()
    for node in ast.walk(tree):
        if isinstance(node, (ast.Import, ast.ImportFrom)):
            names.update((a.asname or a.name).split(".")[0] for a in node.names)
        elif isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            names.add(node.name)
        elif isinstance(node, ast.Name) and isinstance(node.ctx, (ast.Store, ast.Del)):
            names.add(node.id)
        elif isinstance(node, ast.Global):
            names.update(node.names)
    return names


def _undefined(path: pathlib.Path, src: str) -> list:
    known = _defined_at_module_level(ast.parse(src)) | set(dir(builtins)) | {"__file__", "__name__", "__doc__", "__class__"}
    out = []

    def walk(tab):
        for sym in tab.get_symbols():
            free = sym.is_global() or (tab.get_type() == "module" and not sym.is_assigned() and not sym.is_imported())
            if free and sym.is_referenced() and sym.get_name() not in known:
                out.append(f"{path.name}: {sym.get_name()!r} in {tab.get_name()}")
        for child in tab.get_children():
            walk(child)
    walk(symtable.symtable(src, str(path), "exec"))
    return out


def test_no_function_reads_a_name_that_nothing_defines():
    assert _undefined(pathlib.Path("probe.py"), "import os\ndef f(x):\n    return missing(x) + os.sep\n") == \
        ["probe.py: 'missing' in f"]                   # the check sees what it is meant to see
    problems = []
    for f in SOURCES + sorted((ROOT / "tests").glob("*.py")):
        problems += _undefined(f, f.read_text())
    assert not problems, problems
