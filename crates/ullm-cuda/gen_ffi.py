#!/usr/bin/env python
"""Generates ``src/ffi.rs`` (the raw ``extern "C"`` bindings of the ``ullm-cuda`` crate) from the C headers
``include/ullm_cuda.h``, ``include/ullm_gguf.h`` and ``include/ullm_safetensors.h``.

The headers are the single statement of the boundary; this script turns every function, ``#[repr(C)]``
struct, opaque handle, enum constant and integer ``#define`` in them into Rust.  ``python gen_ffi.py``
rewrites ``src/ffi.rs``; ``python gen_ffi.py --check`` exits non-zero when the committed file differs from
what the headers say (the repository's tests run this check, so the bindings cannot fall behind the header).
The parser understands the subset of C these headers use: one declaration per ``;``, pointer declarators,
comma-separated members, ``typedef struct {...} name;``, ``typedef struct tag name;``, anonymous and named
enums with explicit or running values.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
HEADERS = ["ullm_cuda.h", "ullm_gguf.h", "ullm_safetensors.h"]

SCALARS = {
    "int": "c_int", "unsigned": "c_uint", "unsigned int": "c_uint", "float": "f32", "double": "f64", "size_t": "usize", "char": "c_char",
    "uint8_t": "u8", "int8_t": "i8", "uint16_t": "u16", "int16_t": "i16", "uint32_t": "u32", "int32_t": "i32", "uint64_t": "u64",
    "int64_t": "i64", "void": "c_void",
}


RUST_KEYWORDS = {"in", "type", "fn", "ref", "mod", "move", "match", "loop", "impl", "use", "where", "self", "box", "as", "dyn", "priv"}


def ident(name: str) -> str:
    return f"r#{name}" if name in RUST_KEYWORDS else name


def strip_comments(src: str) -> str:
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    return re.sub(r"//[^\n]*", " ", src)


def rust_type(base: str, ptrs: list[bool], known: set[str]) -> str:
    """``base`` is the C base type (``const`` removed, flag passed separately in ptrs[0] logic below).
    ``ptrs`` lists, innermost first, whether the pointee of each ``*`` is const."""
    base = base.replace("struct ", "").strip()
    if base in SCALARS:
        t = SCALARS[base]
    elif base in known:
        t = base
    else:
        raise ValueError(f"unknown C type {base!r}")
    for is_const in ptrs:
        t = ("*const " if is_const else "*mut ") + t
    return t


def parse_declarator(decl: str):
    """'const float *const *d_x' -> (base 'float', ptr constness innermost-first [True, True], name 'd_x')."""
    decl = decl.strip()
    m = re.match(r"^(.*?)([A-Za-z_][A-Za-z0-9_]*)?(\[[^\]]*\])?$", decl)
    left, name, arr = m.group(1), m.group(2), m.group(3)
    if name in SCALARS or name in ("const", "struct"):  # unnamed parameter whose last word is the type
        left, name = decl, None
    toks = re.findall(r"\*|[A-Za-z_][A-Za-z0-9_]*", left)
    base_words, ptrs, pending_const = [], [], False
    # constness that precedes the first '*' applies to the base; a 'const' after a '*' applies to that pointer itself,
    # i.e. to what the NEXT '*' (or the variable) points at
    consts_after = []
    seen_star = False
    base_const = False
    for t in toks:
        if t == "*":
            seen_star = True
            consts_after.append(False)
        elif t == "const":
            if seen_star:
                consts_after[-1] = True
            else:
                base_const = True
        else:
            if seen_star:
                raise ValueError(f"unexpected token after '*' in {decl!r}")
            base_words.append(t)
    n = len(consts_after)
    # pointee constness of star i: the base for i == 0, else the const that followed star i-1
    ptrs = [base_const if i == 0 else consts_after[i - 1] for i in range(n)]
    return " ".join(base_words), ptrs, name, arr


def parse(src: str):
    src = strip_comments(src)
    defines = re.findall(r"^\s*#define\s+([A-Z][A-Z0-9_]*)\s+\(?\s*([0-9][0-9a-fxu]*)\s*(?:<<\s*([0-9]+))?\s*\)?\s*$", src, flags=re.M)
    src = re.sub(r"^\s*#.*$", "", src, flags=re.M)
    src = src.replace('extern "C" {', "").replace("}\n#endif", "")
    items = {"opaque": [], "structs": [], "consts": [], "fns": []}
    for name, val, shift in defines:
        if name.endswith("_H"):
            continue
        v = int(re.sub(r"u$", "", val), 0)
        items["consts"].append((name, v << int(shift) if shift else v))
    # enums
    for m in re.finditer(r"(?:typedef\s+)?enum\s*([A-Za-z_0-9]*)\s*\{(.*?)\}\s*([A-Za-z_0-9]*)\s*;", src, flags=re.S):
        nxt = 0
        for ent in m.group(2).split(","):
            ent = ent.strip()
            if not ent:
                continue
            if "=" in ent:
                k, v = [x.strip() for x in ent.split("=")]
                nxt = int(v, 0)
            else:
                k = ent
            items["consts"].append((k, nxt))
            nxt += 1
    src = re.sub(r"(?:typedef\s+)?enum\s*[A-Za-z_0-9]*\s*\{.*?\}\s*[A-Za-z_0-9]*\s*;", "", src, flags=re.S)
    # structs with bodies
    for m in re.finditer(r"typedef\s+struct\s*([A-Za-z_0-9]*)\s*\{(.*?)\}\s*([A-Za-z_0-9]+)\s*;", src, flags=re.S):
        fields = []
        for stmt in m.group(2).split(";"):
            stmt = stmt.strip()
            if not stmt:
                continue
            first, *rest = [p.strip() for p in stmt.split(",")]
            base, ptrs, name, arr = parse_declarator(first)
            fields.append((base, ptrs, name, arr))
            for r in rest:
                stars = len(r) - len(r.lstrip("* "))
                nm = r.lstrip("* ").strip()
                pc = [ptrs[0] if ptrs else ("const" in first.split(base)[0])] * r.count("*")
                # members after a comma share the base type and its constness
                base_const = bool(re.match(r"^\s*const\b", first))
                fields.append((base, [base_const] * r.count("*"), nm, None))
        items["structs"].append((m.group(3), m.group(1), fields))
    src = re.sub(r"typedef\s+struct\s*[A-Za-z_0-9]*\s*\{.*?\}\s*[A-Za-z_0-9]+\s*;", "", src, flags=re.S)
    # opaque handles: typedef struct tag name;  and bare forward declarations  struct tag;
    for m in re.finditer(r"typedef\s+struct\s+([A-Za-z_0-9]+)\s+([A-Za-z_0-9]+)\s*;", src):
        items["opaque"].append(m.group(2))
    src = re.sub(r"typedef\s+struct\s+[A-Za-z_0-9]+\s+[A-Za-z_0-9]+\s*;", "", src)
    for m in re.finditer(r"(?<![A-Za-z_0-9])struct\s+([A-Za-z_0-9]+)\s*;", src):
        items["opaque"].append(m.group(1))
    src = re.sub(r"(?<![A-Za-z_0-9])struct\s+[A-Za-z_0-9]+\s*;", "", src)
    # functions
    for stmt in src.split(";"):
        stmt = " ".join(stmt.split())
        m = re.match(r"^(.*?)\b([A-Za-z_][A-Za-z0-9_]*)\s*\((.*)\)$", stmt)
        if not m or not m.group(2).startswith("ullm_"):
            continue
        ret_base, ret_ptrs, _, _ = parse_declarator(m.group(1) + " x")
        args = []
        if m.group(3).strip() not in ("", "void"):
            for a in m.group(3).split(","):
                args.append(parse_declarator(a))
        items["fns"].append((m.group(2), (ret_base, ret_ptrs), args))
    return items


def render(all_items) -> str:
    struct_alias = {}
    known = set()
    for it in all_items:
        known.update(it["opaque"])
        for name, tag, _ in it["structs"]:
            known.add(name)
            if tag:
                struct_alias[tag] = name
    out = ["// Raw bindings of libullm_cuda.so.  GENERATED by gen_ffi.py from include/*.h - do not edit by hand.",
           "#![allow(non_camel_case_types, non_upper_case_globals, dead_code)]", "",
           "use std::os::raw::{c_char, c_int, c_uint, c_void};", ""]
    seen = set()
    for it in all_items:
        for name in it["opaque"]:
            if name in struct_alias or name in seen:
                continue
            seen.add(name)
            out += ["#[repr(C)]", f"pub struct {name} {{", "    _private: [u8; 0],", "}"]
    out.append("")
    for it in all_items:
        for k, v in it["consts"]:
            if k in seen:
                continue
            seen.add(k)
            out.append(f"pub const {k}: {'usize' if k.endswith('_BYTES') or k.endswith('_RANKS') else 'c_int'} = {v};")
    out.append("")

    def ty(base, ptrs):
        b = base.replace("struct ", "").strip()
        b = struct_alias.get(b, b)
        return rust_type(b, ptrs, known)

    for it in all_items:
        for name, tag, fields in it["structs"]:
            out += ["#[repr(C)]", "#[derive(Clone, Copy)]", f"pub struct {name} {{"]
            for base, ptrs, fname, arr in fields:
                t = ty(base, ptrs)
                if arr:  # fixed-size array member
                    t = f"[{t}; {int(arr.strip('[]'), 0)}]"
                out.append(f"    pub {ident(fname)}: {t},")
            out += ["}", ""]
    out += ['#[link(name = "ullm_cuda")]', 'extern "C" {']
    for it in all_items:
        for name, (rb, rp), args in it["fns"]:
            a = ", ".join(f"{ident(an or f'arg{i}')}: {ty(b, p)}" for i, (b, p, an, _) in enumerate(args))
            ret = "" if (rb == "void" and not rp) else f" -> {ty(rb, rp)}"
            out.append(f"    pub fn {name}({a}){ret};")
    out += ["}", ""]
    return "\n".join(out)


def generate() -> str:
    return render([parse(open(os.path.join(ROOT, "include", h)).read()) for h in HEADERS])


def main() -> int:
    target = os.path.join(HERE, "src", "ffi.rs")
    text = generate()
    if "--check" in sys.argv:
        if not os.path.exists(target) or open(target).read() != text:
            print("crates/ullm-cuda/src/ffi.rs is out of date: run python crates/ullm-cuda/gen_ffi.py", file=sys.stderr)
            return 1
        return 0
    with open(target, "w") as f:
        f.write(text)
    print(f"wrote {target}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
