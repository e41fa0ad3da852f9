"""ctypes mirror of include/trainlib_b200_abi.h.

The struct layouts are read from the header itself at import time, so the Python side can
never drift from the C ABI.  Every pointer field is a ``c_void_p`` (an address: host numpy
memory, a device pointer, or the address of another struct); ``float`` -> ``c_float``,
``int`` -> ``c_int``, a by-value ``fp16`` -> ``c_uint16`` (raw IEEE binary16 bits).

The same classes describe the argument structs of the reference library
(lib/include/pulp_*.h), which is what lets one test body drive both implementations.
"""
import ctypes
import os
import re

HEADER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include", "trainlib_b200_abi.h")

_SCALARS = {"float": ctypes.c_float, "int": ctypes.c_int, "fp16": ctypes.c_uint16}


def _strip_comments(src):
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return re.sub(r"//[^\n]*", "", src)


def parse_structs(path=HEADER):
    """Return {struct name: [(field name, kind)]}, kind in {'ptr', 'float', 'int', 'fp16'}."""
    src = _strip_comments(open(path).read())
    out = {}
    for m in re.finditer(r"struct\s+(\w+)\s*\{(.*?)\}\s*;", src, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = decl.replace("__restrict__", " ").strip()
            if not decl:
                continue
            name = re.search(r"(\w+)\s*$", decl).group(1)
            if "*" in decl:
                kind = "ptr"
            else:
                kind = decl[: decl.rfind(name)].strip().split()[-1]
                if kind not in _SCALARS:
                    raise ValueError("unknown by-value type in '%s' of struct %s" % (decl, m.group(1)))
            fields.append((name, kind))
        out[m.group(1)] = fields
    return out


def parse_functions(path=HEADER):
    """Names of all `void f(void *)` entry points the header declares (plus the three scalars)."""
    src = _strip_comments(open(path).read())
    names = re.findall(r"\bvoid\s+(\w+)\s*\(\s*void\s*\*\s*\w*\s*\)\s*;", src)
    return names


STRUCT_FIELDS = parse_structs()
FUNCTIONS = parse_functions()


def _make(name, fields):
    cfields = [(f, ctypes.c_void_p if k == "ptr" else _SCALARS[k]) for f, k in fields]
    return type(name, (ctypes.Structure,), {"_fields_": cfields})


STRUCTS = {name: _make(name, fields) for name, fields in STRUCT_FIELDS.items()}
globals().update(STRUCTS)


def addr(obj):
    """Address of a ctypes struct / numpy array / int (device pointer) / None."""
    if obj is None:
        return None
    if isinstance(obj, int):
        return obj
    if isinstance(obj, ctypes.Structure) or isinstance(obj, ctypes.Array):
        return ctypes.addressof(obj)
    if hasattr(obj, "ctypes"):          # numpy array
        return obj.ctypes.data
    raise TypeError("cannot take the address of %r" % (obj,))
