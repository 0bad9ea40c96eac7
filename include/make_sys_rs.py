#!/usr/bin/env python
"""Generate the Rust `-sys` binding of include/t0b200.h: one `extern "C"` item per exported function, one
`#[repr(C)]` struct per C struct, the error / enum constants as `pub const`.

    python include/make_sys_rs.py            # rewrites include/t0b200_sys.rs
    python include/make_sys_rs.py --check    # exit 1 when the committed file is out of date

The output is the file a maintainer of the reference crate adds as `src/t0b200_sys.rs` (the integration guide at the
repository root embeds a copy).
It is generated, not hand-written, so that it cannot drift from the header; tests/test_host_api.py regenerates it
and compares.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "t0b200.h")
OUT = os.path.join(HERE, "t0b200_sys.rs")

SCALARS = {"int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "int64_t": "i64", "size_t": "usize", "float": "f32",
           "double": "f64", "uint8_t": "u8", "uint16_t": "u16", "int": "i32", "char": "c_char", "void": "c_void"}
KEYWORDS = {"async": "is_async", "type": "kind", "ref": "reference", "in": "input", "loop": "loop_", "match": "match_",
            "move": "move_", "fn": "func", "mod": "module", "self": "this", "box": "box_"}


def strip_comments(text: str) -> str:
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def rust_type(ctype: str, array: bool) -> str:
    """`ctype` is a C parameter type without its name, e.g. 'const t0b_gemm_config*' or 'uint64_t'."""
    t = " ".join(ctype.replace("*", " * ").split())
    const = False
    toks = t.split()
    if toks and toks[0] == "const":
        const = True
        toks = toks[1:]
    base = toks[0]
    if base == "struct":
        base = toks[1]
        toks = toks[1:]
    stars = toks.count("*") + (1 if array else 0)
    inner = SCALARS.get(base, base)
    if stars == 0:
        return inner
    out = inner
    for level in range(stars):
        out = ("*const " if (const and level == 0) else "*mut ") + out
    return out


def parse_params(arglist: str):
    arglist = arglist.strip()
    if arglist in ("", "void"):
        return []
    params = []
    for raw in arglist.split(","):
        raw = " ".join(raw.split())
        m = re.match(r"^(.*?)(\w+)\s*(\[\s*\d*\s*\])?$", raw)
        ctype, name, arr = m.group(1).strip(), m.group(2), m.group(3)
        params.append((KEYWORDS.get(name, name), rust_type(ctype, arr is not None)))
    return params


def generate() -> str:
    with open(HEADER) as f:
        text = strip_comments(f.read())
    out = ["// Generated from include/t0b200.h by include/make_sys_rs.py -- do not edit.",
           "// The `-sys` layer of the B200 backend: `extern \"C\"` declarations of libt0b200.so, one per exported function.",
           "#![allow(non_camel_case_types, dead_code)]", "use std::os::raw::{c_char, c_void};", ""]
    # enum constants
    for body in re.findall(r"enum\s*\{(.*?)\}\s*;", text, flags=re.S):
        nxt = 0
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, val = [x.strip() for x in item.split("=")]
                nxt = int(val, 0)
            else:
                name = item
            out.append(f"pub const {name}: i32 = {nxt};")
            nxt += 1
    out.append("")
    out.append("#[repr(C)] pub struct t0b_ctx { _private: [u8; 0] }")
    # structs
    for body, name in re.findall(r"typedef\s+struct\s+\w+\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        out.append("")
        out.append("#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq)]")
        out.append(f"pub struct {name} {{")
        for decl in body.split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            ctype, names = decl.split(" ", 1)
            for n in names.split(","):
                n = n.strip()
                m = re.match(r"^(\w+)\s*\[\s*(\d+)\s*\]$", n)
                if m:
                    out.append(f"    pub {m.group(1)}: [{SCALARS[ctype]}; {m.group(2)}],")
                else:
                    out.append(f"    pub {n}: {SCALARS[ctype]},")
        out.append("}")
    # functions
    out.append("")
    out.append('extern "C" {')
    for ret, name, args in re.findall(r"T0B_API\s+([\w\s\*]+?)\s*\b(t0b_\w+)\s*\((.*?)\)\s*;", text, flags=re.S):
        params = ", ".join(f"{n}: {t}" for n, t in parse_params(args))
        ret = " ".join(ret.split())
        r = rust_type(ret, False)
        arrow = "" if r == "c_void" else f" -> {r}"
        out.append(f"    pub fn {name}({params}){arrow};")
    out.append("}")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    text = generate()
    if "--check" in sys.argv:
        with open(OUT) as f:
            sys.exit(0 if f.read() == text else 1)
    with open(OUT, "w") as f:
        f.write(text)
    print(OUT)
