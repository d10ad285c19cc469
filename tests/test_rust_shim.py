"""The Rust binding crate (oneiron-luminal_b200/host/rust/luminal_b200) cannot be compiled where this repository is built (no Rust
toolchain), so it ships as reviewed source.  What can be checked mechanically is checked here: its raw declarations
(src/ffi.rs) against the C header — every function, in the header's order, with the same argument names and types; every field
of the #[repr(C)] structs; every enum value it mirrors — and the ctypes mirror of the same structs against both.
"""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CRATE = os.path.join(ROOT, "oneiron-luminal_b200", "host", "rust", "luminal_b200")

SCALAR = {"int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64", "size_t": "usize", "float": "f32", "double": "f64",
          "char": "c_char", "int8_t": "i8", "uint8_t": "u8", "void": "c_void", "lum_rt": "lum_rt", "lum_st": "lum_st", "lum_config": "lum_config",
          "lum_model_desc": "lum_model_desc", "lum_stats": "lum_stats", "lum_sampling": "lum_sampling"}


def strip_comments(text):
    return re.sub(r"//[^\n]*", "", re.sub(r"/\*.*?\*/", "", text, flags=re.S))


def c_type_to_rust(tokens):
    """['const', 'char', '*', 'const', '*'] -> '*const *const c_char'"""
    toks = list(tokens)
    base_const = False
    if toks[0] == "const":
        base_const = True
        toks = toks[1:]
    base = SCALAR[toks[0]]
    rest = toks[1:]
    # each '*' may be followed by 'const' (constness of that pointer level's TARGET is the qualifier to its left)
    levels = []        # constness of what each pointer points to, innermost first
    target_const = base_const
    i = 0
    while i < len(rest):
        assert rest[i] == "*", tokens
        levels.append(target_const)
        target_const = i + 1 < len(rest) and rest[i + 1] == "const"
        i += 2 if target_const else 1
    out = base
    for is_const in levels:
        out = ("*const " if is_const else "*mut ") + out
    return out


def header_functions():
    text = strip_comments(open(os.path.join(ROOT, "include", "lum_b200.h")).read())
    fns = []
    for m in re.finditer(r"^([A-Za-z_][\w \*]*?)\b(lum_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.M | re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        ret_toks = re.findall(r"\w+|\*", ret)
        rust_ret = None if ret_toks == ["void"] else c_type_to_rust(ret_toks)
        params = []
        if args and args != "void":
            for a in args.split(","):
                toks = re.findall(r"\w+|\*", a)
                params.append((toks[-1], c_type_to_rust(toks[:-1])))
        fns.append((name, params, rust_ret))
    return fns


def rust_functions():
    text = strip_comments(open(os.path.join(CRATE, "src", "ffi.rs")).read())
    block = re.search(r'extern "C" \{(.*?)\n\}', text, flags=re.S).group(1)
    fns = []
    for m in re.finditer(r"pub fn (\w+)\((.*?)\)\s*(?:->\s*([^;]+?))?;", block, flags=re.S):
        params = []
        for a in filter(None, (p.strip() for p in m.group(2).split(","))):
            n, t = a.split(":", 1)
            params.append((n.strip(), " ".join(t.split())))
        fns.append((m.group(1), params, m.group(3).strip() if m.group(3) else None))
    return fns


def test_extern_block_matches_the_header():
    h, r = header_functions(), rust_functions()
    assert len(h) >= 70
    assert [f[0] for f in r] == [f[0] for f in h], "functions differ or are in another order"
    for hf, rf in zip(h, r):
        assert hf == rf, f"{hf[0]}: header says {hf[1:]}, ffi.rs says {rf[1:]}"


def c_struct_fields(name):
    text = strip_comments(open(os.path.join(ROOT, "include", "lum_b200.h")).read())
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, flags=re.S).group(1)
    out = []
    for decl in filter(None, (d.strip() for d in body.split(";"))):
        toks = decl.replace(",", " , ").split()
        ty = SCALAR[toks[0]]
        out += [(n, ty) for n in toks[1:] if n != ","]
    return out


def rust_struct_fields(name):
    text = strip_comments(open(os.path.join(CRATE, "src", "ffi.rs")).read())
    body = re.search(r"pub struct %s \{(.*?)\}" % name, text, flags=re.S).group(1)
    return [(m.group(1), m.group(2)) for m in re.finditer(r"pub (\w+): (\w+),", body)]


@pytest.mark.parametrize("name, mirror", [("lum_config", "Config"), ("lum_model_desc", "ModelDesc"), ("lum_stats", "Stats"), ("lum_sampling", "Sampling")])
def test_repr_c_structs_match_the_header_and_the_ctypes_mirror(pkg, name, mirror):
    import ctypes as C
    c, r = c_struct_fields(name), rust_struct_fields(name)
    assert c == r
    ct = {C.c_int32: "i32", C.c_uint32: "u32", C.c_float: "f32", C.c_uint64: "u64", C.c_double: "f64", C.c_int64: "i64"}
    assert [(n, ct[t]) for n, t in getattr(pkg, mirror)._fields_] == c


def test_enum_values_match_the_headers():
    rs = strip_comments(open(os.path.join(CRATE, "src", "ffi.rs")).read())
    consts = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"pub const (LUM_\w+): [iu]32 = (-?\w+);", rs)}
    values = {}
    for hdr in ("lum_llir.h", "lum_b200.h"):
        text = strip_comments(open(os.path.join(ROOT, "include", hdr)).read())
        for body in re.findall(r"enum\s*\w*\s*\{(.*?)\}", text, flags=re.S):
            nxt = 0
            for item in filter(None, (i.strip() for i in body.split(","))):
                if "=" in item:
                    k, v = (s.strip() for s in item.split("="))
                    nxt = int(v, 0)
                else:
                    k = item
                if k.startswith("LUM_"):
                    values[k] = nxt
                nxt += 1
        for m in re.finditer(r"#define (LUM_LLIR_\w+) (\w+?)u?\n", text):
            values[m.group(1)] = int(m.group(2), 0)
    for k, v in consts.items():
        assert values.get(k) == v, (k, v, values.get(k))
    for k in ("LUM_Q8_0", "LUM_P_DTYPE", "LUM_T_LT", "LUM_E_NOMEM", "LUM_LLIR_MAGIC"):
        assert k in consts


def test_every_slot_the_binding_names_exists(pkg):
    """src/runtime.rs maps safetensors labels and Input nodes to slots by the header's enum names."""
    text = strip_comments(open(os.path.join(ROOT, "include", "lum_b200.h")).read())
    body = re.search(r"typedef enum lum_slot \{(.*?)\} lum_slot;", text, flags=re.S).group(1)
    names = [n.strip().split("=")[0].strip() for n in body.split(",") if n.strip()]
    assert [n[len("LUM_S_"):].lower() for n in names] == [k for k, _ in sorted(pkg.SLOT.items(), key=lambda kv: kv[1])]


def test_crate_sources_are_present_and_cite_the_trait():
    for f in ("Cargo.toml", "build.rs", "src/lib.rs", "src/ffi.rs", "src/wire.rs", "src/ops.rs", "src/runtime.rs"):
        assert os.path.getsize(os.path.join(CRATE, f)) > 200, f
    rt = open(os.path.join(CRATE, "src", "runtime.rs")).read()
    for needle in ("impl Runtime for B200Runtime", "fn load_llir", "fn execute", "fn profile", "fn allocate_dummy_input", "fn clear_intermediate_buffers"):
        assert needle in rt, needle
