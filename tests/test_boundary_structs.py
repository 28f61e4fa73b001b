"""The three statements of the C-ABI structs - include/kronos_cuda_ffi.h, the ctypes classes of kronos_2t_b200.ffi and
the #[repr(C)] blocks a Rust host would copy from INTEGRATION.md - must list the same fields, in the same order, with
the same machine types.  (A host built from a shorter struct would make the library read past its end.)"""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_KINDS = {"uint32_t": "u32", "int32_t": "i32", "float": "f32", "uint64_t": "u64", "size_t": "usize", "int8_t": "i8"}
RUST_KINDS = {"u32": "u32", "i32": "i32", "f32": "f32", "u64": "u64", "usize": "usize"}
CTYPES_KINDS = {C.c_uint32: "u32", C.c_int32: "i32", C.c_float: "f32", C.c_uint64: "u64", C.c_size_t: "usize", C.c_void_p: "ptr"}
if C.sizeof(C.c_size_t) == C.sizeof(C.c_uint64):
    CTYPES_KINDS[C.c_size_t] = "usize"      # ctypes aliases c_size_t to c_uint64 / c_ulong on LP64: compared by size below


def header_struct(name):
    text = open(os.path.join(ROOT, "include", "kronos_cuda_ffi.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if not decl:
            continue
        m = re.match(r"(const )?(\w+) (.*)", decl)
        base, rest = m.group(2), m.group(3)
        for item in rest.split(","):
            item = item.strip()
            ptr = item.startswith("*")
            item = item.lstrip("* ")
            arr = re.match(r"(\w+)\[(\d+)\]", item)
            if arr:
                fields.append((arr.group(1), "%s[%s]" % (C_KINDS[base], arr.group(2))))
            elif ptr:
                fields.append((item, "ptr"))
            elif base in C_KINDS:
                fields.append((item, C_KINDS[base]))
            else:
                fields.append((item, "struct " + base))
    return fields


def rust_struct(name):
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    body = re.search(r"#\[repr\(C\)\]\s*pub struct %s \{(.*?)\n\}" % name, text, re.S).group(1)
    body = re.sub(r"//[^\n]*", "", body)
    fields = []
    for item in body.split(","):
        item = " ".join(item.split())
        if not item:
            continue
        fname, ftype = [x.strip() for x in item.split(":", 1)]
        if ftype.startswith("*"):
            kind = "ptr"
        elif ftype.startswith("["):
            t, n = re.match(r"\[(\w+); (\d+)\]", ftype).groups()
            kind = "%s[%s]" % (t, n)
        elif ftype in RUST_KINDS:
            kind = RUST_KINDS[ftype]
        else:
            kind = "struct " + ftype
        fields.append((fname, kind))
    return fields


def ctypes_struct(cls):
    fields = []
    for fname, ftype in cls._fields_:
        if isinstance(ftype, type) and issubclass(ftype, C.Structure):
            kind = "struct KronosCuda" + ftype.__name__
        elif isinstance(ftype, type) and issubclass(ftype, C.Array):
            kind = "i8[%d]" % ftype._length_
        else:
            kind = CTYPES_KINDS[ftype]
        fields.append((fname, kind))
    return fields


def same(a, b):
    """usize and u64 are one type to ctypes on LP64; everything else must match exactly."""
    norm = lambda k: "u64" if k == "usize" and C.sizeof(C.c_size_t) == 8 else k
    return [(n, norm(k)) for n, k in a] == [(n, norm(k)) for n, k in b]


@pytest.mark.parametrize("name,cls_name", [("KronosCudaMatrixDesc", "MatrixDesc"), ("KronosCudaEngineConfig", "EngineConfig"),
                                           ("KronosCudaLayerDesc", "LayerDesc")])
def test_struct_layouts_agree(name, cls_name):
    from kronos_2t_b200 import ffi
    h, r, c = header_struct(name), rust_struct(name), ctypes_struct(getattr(ffi, cls_name))
    assert len(h) > 3
    assert h == r, ("header vs INTEGRATION.md", [x for x in zip(h, r) if x[0] != x[1]], len(h), len(r))
    assert same(h, c), ("header vs ffi.py", [x for x in zip(h, c) if x[0] != x[1]], len(h), len(c))


def test_engine_config_size_is_what_the_library_checks():
    """struct_size travels in the first field; the ctypes layout must have the size a C compiler gives the header's struct
    (4-byte fields, one 8-byte field on an 8-byte boundary)."""
    from kronos_2t_b200 import ffi
    fields = header_struct("KronosCudaEngineConfig")
    off = 0
    for _, kind in fields:
        sz = 8 if kind in ("u64", "usize", "ptr") else 4
        off = (off + sz - 1) // sz * sz + sz
    assert (off + 7) // 8 * 8 == C.sizeof(ffi.EngineConfig)
    assert fields[0] == ("struct_size", "u32")
