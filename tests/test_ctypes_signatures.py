"""Every ``argtypes`` list in the package against the C signature it binds: the C entry
points are parsed out of ``csrc`` and compared parameter by parameter (pointer / 32-bit
int / 64-bit int / float / double).  A mismatch here would be silent garbage or a fault
on the GPU, so it is caught on the CPU."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


RETURNS = {}


def _c_signatures():
    sigs = {}
    for path in glob.glob(os.path.join(ROOT, "csrc", "**", "*.c*"), recursive=True):
        if os.sep + "selftest" + os.sep in path:
            continue
        text = open(path).read()
        text = re.sub(r"//[^\n]*", "", text)
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"\n(?:static\s+)?([A-Za-z_][\w \*]*?)\s+(ft_\w+)\s*\(([^)]*)\)\s*\{", text):
            ret, name, params = m.group(1).strip(), m.group(2), m.group(3)
            if "static" in m.group(0).split(name)[0]:
                continue
            kinds = []
            for p in [x.strip() for x in params.split(",") if x.strip() and x.strip() != "void"]:
                if "*" in p or "cudaStream_t" in p:
                    kinds.append("P")
                elif re.search(r"\b(int64_t|uint64_t|long long|size_t|ssize_t|off_t)\b", p):
                    kinds.append("L")
                elif re.search(r"\bdouble\b", p):
                    kinds.append("D")
                elif re.search(r"\bfloat\b", p):
                    kinds.append("F")
                elif re.search(r"\b(int|uint32_t|int32_t|unsigned|bool)\b", p):
                    kinds.append("I")
                else:
                    kinds.append("?" + p)
            sigs[name] = kinds
            RETURNS[name] = 'P' if '*' in ret else ('L' if re.search(r'\b(int64_t|uint64_t|long long|size_t)\b', ret) else 'I')
    return sigs


def _kind(ct):
    if ct in (ctypes.c_void_p, ctypes.c_char_p) or (isinstance(ct, type) and issubclass(ct, ctypes._Pointer)):
        return "P"
    if ct in (ctypes.c_int64, ctypes.c_uint64, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_size_t,
              ctypes.c_ssize_t, ctypes.c_long, ctypes.c_ulong):
        return "L"
    if ct in (ctypes.c_int, ctypes.c_uint, ctypes.c_int32, ctypes.c_uint32, ctypes.c_bool):
        return "I"
    if ct is ctypes.c_float:
        return "F"
    if ct is ctypes.c_double:
        return "D"
    return "?" + repr(ct)


def _declared():
    """Load both libraries and run every module-level declaration helper of the package."""
    from flextrain_b200.ops.native import cuda_lib, host_lib
    libs = [host_lib(), cuda_lib()]
    # modules that declare signatures lazily: touch their declaring helpers
    from flextrain_b200.parallel import fused
    fused._lib()
    fused._ag_lib()
    try:
        from flextrain_b200.parallel import symm_mem
        for name in ("_lib", "_declare"):
            if hasattr(symm_mem, name):
                getattr(symm_mem, name)()
    except Exception:
        pass
    from flextrain_b200.memory import nvme_swapper, pin_memory
    for mod in (nvme_swapper, pin_memory):
        if hasattr(mod, "_lib"):
            mod._lib()
    from flextrain_b200.ops import attention_native
    if hasattr(attention_native, "_lib"):
        attention_native._lib()
    # bindings declared at their first use
    import torch
    t = pin_memory.new_cpu_locked_tensor(1024, torch.float32)
    pin_memory.host_memcpy(t, torch.ones(1024))
    pin_memory.free_cpu_locked_tensor(t)
    fused.set_wait_seconds(10.0)
    libs[1].ft_comm_set_spin_budget(0)
    libs[1].ft_ag_set_spin_budget(0)
    return libs


def test_every_declared_argtypes_matches_its_c_signature():
    c = _c_signatures()
    assert len(c) > 60, "the parser lost most entry points"
    libs = _declared()
    checked, bad = 0, []
    for name, kinds in c.items():
        for lib in libs:
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue
            if fn.argtypes is None:
                continue
            got = [_kind(a) for a in fn.argtypes]
            checked += 1
            if got != kinds:
                bad.append(f"{name}: C {''.join(kinds)} vs ctypes {''.join(got)}")
    assert not bad, "\n".join(bad)
    assert checked > 55, f"only {checked} bindings carry argtypes"
    # whoever takes a pointer or a 64-bit value must not rely on ctypes' default (C int)
    from_python = set()
    for root, _, files in os.walk(os.path.join(ROOT, "flextrain_b200")):
        for f in files:
            if f.endswith(".py"):
                from_python.update(re.findall(r"\b(ft_\w+)\b", open(os.path.join(root, f)).read()))
    loose = []
    for name, kinds in c.items():
        if name not in from_python or not any(k in ("P", "L", "F", "D") for k in kinds):
            continue
        for lib in libs:
            fn = getattr(lib, name, None)
            if fn is not None and fn.argtypes is None:
                loose.append(name)
    assert not loose, f"called from Python with pointer / 64-bit / float arguments but without argtypes: {loose}"


def test_pointer_and_wide_return_types_are_declared():
    """ctypes assumes a C int return: a pointer or a 64-bit count comes back truncated unless
    ``restype`` says otherwise."""
    c = _c_signatures()
    libs = _declared()
    from_python = set()
    for root, _, files in os.walk(os.path.join(ROOT, "flextrain_b200")):
        for f in files:
            if f.endswith(".py"):
                from_python.update(re.findall(r"\b(ft_\w+)\b", open(os.path.join(root, f)).read()))
    bad = []
    for name in c:
        want = RETURNS.get(name, "I")
        if want == "I" or name not in from_python:
            continue
        for lib in libs:
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            got = _kind(fn.restype) if fn.restype is not None else "void"
            if got != want:
                bad.append(f"{name}: returns {want} in C, restype is {fn.restype}")
    assert not bad, "\n".join(bad)


def test_every_entry_point_named_in_python_exists_in_a_library():
    libs = _declared()
    named = set()
    for base in ("flextrain_b200", "benchmarks", "tests"):
        for root, dirs, files in os.walk(os.path.join(ROOT, base)):
            dirs[:] = [d for d in dirs if d != "__pycache__"]
            for f in files:
                if f.endswith(".py"):
                    named.update(re.findall(r"\b(?:lib|_lib\(\)|cuda_lib\(\)|host_lib\(\)|_ag_lib\(\))\.(ft_\w+)",
                                            open(os.path.join(root, f)).read()))
    assert len(named) > 50
    missing = [n for n in sorted(named) if not any(hasattr(lib, n) for lib in libs)]
    assert not missing, f"not exported by libft_cuda / libft_host: {missing}"


def test_call_sites_pass_as_many_arguments_as_the_c_function_takes():
    import ast
    c = _c_signatures()
    checked, bad = 0, []
    for base in ("flextrain_b200", "benchmarks"):
        for root, dirs, files in os.walk(os.path.join(ROOT, base)):
            dirs[:] = [d for d in dirs if d != "__pycache__"]
            for f in files:
                if not f.endswith(".py"):
                    continue
                path = os.path.join(root, f)
                for node in ast.walk(ast.parse(open(path).read())):
                    if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)):
                        continue
                    name = node.func.attr
                    if not name.startswith("ft_") or name not in c:
                        continue
                    if node.keywords or any(isinstance(a, ast.Starred) for a in node.args):
                        continue
                    checked += 1
                    if len(node.args) != len(c[name]):
                        bad.append(f"{os.path.relpath(path, ROOT)}:{node.lineno} {name}: {len(node.args)} arguments, "
                                   f"C takes {len(c[name])}")
    assert not bad, "\n".join(bad)
    assert checked > 60, f"only {checked} call sites were found"
