"""Generates ffi.rs (raw Rust bindings) from include/t0b200.h.

    python rust-gpu_b200/rust/gen_ffi.py [--check]

The Rust side of the boundary cannot be compiled where this library is built (no Rust toolchain), so the bindings
are produced mechanically from the one header both sides agree on: every `t0_*` prototype becomes an `extern "C"`
declaration, every record a `#[repr(C)]` struct, every enumerator and `#define`d integer a constant.  `--check` exits
non-zero when the committed ffi.rs differs from what the header gives.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "..", "include", "t0b200.h")
OUT = os.path.join(HERE, "ffi.rs")

SCALARS = {"int": "c_int", "unsigned": "c_uint", "long": "c_long", "char": "c_char", "float": "f32", "double": "f64", "size_t": "usize",
           "uint8_t": "u8", "uint16_t": "u16", "uint32_t": "u32", "uint64_t": "u64", "int32_t": "i32", "int64_t": "i64", "void": "c_void"}


def strip_comments(text: str) -> str:
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def rust_type(ctype: str, opaque: set[str]) -> str:
    ctype = ctype.strip()
    const = False
    stars = ctype.count("*")
    base = ctype.replace("*", " ")
    toks = [t for t in base.split() if t not in ("struct",)]
    if "const" in toks:
        const = True
        toks = [t for t in toks if t != "const"]
    name = " ".join(toks)
    rt = SCALARS.get(name, name)
    for i in range(stars):
        # only the innermost pointer carries the const of `const T*`
        rt = ("*const " if (const and i == 0) else "*mut ") + rt
    return rt


def parse(text: str):
    text = strip_comments(text)
    consts = []
    for m in re.finditer(r"#define\s+(T0_[A-Z0-9_]+)\s+(\d+)\b", text):
        consts.append((m.group(1), int(m.group(2))))
    for m in re.finditer(r"enum\s*(?:t0_[a-z_]+\s*)?\{(.*?)\}", text, flags=re.S):
        value = -1
        for item in m.group(1).split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, v = [s.strip() for s in item.split("=")]
                value = int(v, 0)
            else:
                name, value = item, value + 1
            consts.append((name, value))
    structs = []
    for m in re.finditer(r"typedef\s+struct\s+(t0_[a-z0-9_]+)\s*\{(.*?)\}\s*(t0_[a-z0-9_]+)\s*;", text, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            mm = re.match(r"(.+?)\s+([A-Za-z_][A-Za-z0-9_\[\], ]*)$", decl)
            ctype, names = mm.group(1), mm.group(2)
            for nm in names.split(","):
                nm = nm.strip()
                arr = re.match(r"([A-Za-z_][A-Za-z0-9_]*)\[([A-Za-z0-9_]+)\]", nm)
                fields.append((arr.group(1), ctype, arr.group(2)) if arr else (nm, ctype, None))
        structs.append((m.group(3), fields))
    opaque = sorted(set(re.findall(r"typedef\s+struct\s+(t0_[a-z0-9_]+)\s+(t0_[a-z0-9_]+)\s*;", text)))
    funcs = []
    for m in re.finditer(r"(?m)^([A-Za-z_][A-Za-z0-9_ \*]*?)\b(t0_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                arr = re.match(r"(.+?)\s*\b([A-Za-z_][A-Za-z0-9_]*)\[(\w*)\]$", a)
                if arr:
                    params.append((arr.group(2), arr.group(1) + "*"))
                    continue
                mm = re.match(r"(.+?[\s\*])([A-Za-z_][A-Za-z0-9_]*)$", a)
                params.append((mm.group(2), mm.group(1)))
        funcs.append((name, ret, params))
    return consts, structs, [o[1] for o in opaque], funcs


KEYWORDS = {"type", "ref", "box", "move", "in", "fn", "mod", "use", "self", "super", "match", "loop"}


def emit(consts, structs, opaque, funcs) -> str:
    out = ["// Raw bindings to libt0b200, generated from include/t0b200.h by gen_ffi.py: do not edit.",
           "// Never compiled where the library is built (no Rust toolchain there); checked only against the header.",
           "#![allow(non_camel_case_types, non_upper_case_globals, dead_code)]",
           "use std::os::raw::{c_char, c_int, c_long, c_uint, c_void};", ""]
    for name, value in consts:
        out.append(f"pub const {name}: u32 = {value};")
    out.append("")
    for name in opaque:
        out += ["#[repr(C)]", f"pub struct {name} {{ _private: [u8; 0] }}"]
    out.append("")
    known = set(opaque)
    for name, fields in structs:
        known.add(name)
        out += ["#[repr(C)]", "#[derive(Clone, Copy)]", f"pub struct {name} {{"]
        for fname, ctype, arr in fields:
            rt = rust_type(ctype, known)
            if arr:
                rt = f"[{rt}; {arr} as usize]" if not arr.isdigit() else f"[{rt}; {arr}]"
            if fname in KEYWORDS:
                fname = "r#" + fname
            out.append(f"    pub {fname}: {rt},")
        out += ["}", ""]
    out.append('extern "C" {')
    for name, ret, params in funcs:
        ps = ", ".join(f"{('r#' + p) if p in KEYWORDS else p}: {rust_type(t, known)}" for p, t in params)
        r = rust_type(ret, known)
        tail = "" if r == "c_void" else f" -> {r}"
        out.append(f"    pub fn {name}({ps}){tail};")
    out += ["}", ""]
    return "\n".join(out)


def main() -> int:
    text = emit(*parse(open(HEADER).read()))
    if "--check" in sys.argv:
        same = os.path.exists(OUT) and open(OUT).read() == text
        print("ffi.rs is up to date" if same else "ffi.rs differs from the header: run gen_ffi.py")
        return 0 if same else 1
    with open(OUT, "w") as f:
        f.write(text)
    print(f"wrote {OUT}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
