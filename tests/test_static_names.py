"""Every name a function reads as a global must exist at module level or be a builtin.
Branches that only run on a GPU (fused collectives, native kernels, the benchmark
driver) are never executed by the CPU suite; a misspelt name in them would otherwise
first show on hardware."""
import builtins
import os
import symtable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DUNDER = {"__file__", "__name__", "__doc__", "__path__", "__spec__", "__package__", "__class__"}


def _undefined(path):
    src = open(path).read()
    top = symtable.symtable(src, path, "exec")
    module_names = {s.get_name() for s in top.get_symbols() if s.is_assigned() or s.is_imported() or s.is_namespace()}
    out = []

    def walk(tab):
        for sym in tab.get_symbols():
            if sym.is_referenced() and sym.is_global() and not sym.is_assigned() and not sym.is_imported():
                name = sym.get_name()
                if name not in module_names and not hasattr(builtins, name) and name not in DUNDER:
                    out.append(f"{os.path.relpath(path, ROOT)}: {tab.get_name()} reads undefined '{name}'")
        for child in tab.get_children():
            walk(child)

    walk(top)
    return out


def test_no_function_reads_an_undefined_global():
    files = [os.path.join(ROOT, f) for f in ("bench.py", "__graft_entry__.py", "setup.py")]
    for base in ("flextrain_b200", "benchmarks", "examples", "baseline"):
        for root, dirs, names in os.walk(os.path.join(ROOT, base)):
            dirs[:] = [d for d in dirs if d not in ("_ref", "__pycache__", "_native")]
            files += [os.path.join(root, n) for n in names if n.endswith(".py")]
    assert len(files) > 50
    problems = [p for f in files for p in _undefined(f)]
    assert not problems, "\n".join(problems)
