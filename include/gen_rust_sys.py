"""Generates the Rust `-sys` module for `vyre_b200.h` (the block shown in INTEGRATION.md section 1).

    python include/gen_rust_sys.py            # prints the module
    python include/gen_rust_sys.py --check    # exit 1 when INTEGRATION.md does not hold exactly this text

The header is the single source: every `typedef struct`, every `#define` constant and every function declaration is
translated mechanically, in header order, so the binding a vyre maintainer pastes into `vyre-driver-cuda` cannot drift
from the C ABI. tests/test_integration_doc.py runs the check.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "vyre_b200.h")
DOC = os.path.join(HERE, "..", "INTEGRATION.md")

SCALARS = {"uint8_t": "u8", "int8_t": "i8", "uint16_t": "u16", "uint32_t": "u32", "int32_t": "i32", "uint64_t": "u64",
           "int64_t": "i64", "size_t": "usize", "float": "f32", "double": "f64", "char": "c_char", "void": "c_void"}


def strip_comments(text: str) -> str:
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def rust_type(ctype: str, array: str | None, in_struct: bool) -> str:
    """ctype: e.g. 'const vyb_program*', 'uint32_t', 'vyb_payload**'; array: '[32]' or None."""
    t = ctype.strip()
    stars = t.count("*")
    words = t.replace("*", " ").split()
    # const applies to the pointee next to it: `const T*` and `const T**` (pointer to pointer to const T)
    const = bool(words) and words[0] == "const"
    base = [w for w in words if w not in ("const", "struct")][0]
    r = SCALARS.get(base, base)
    for level in range(stars):
        r = ("*const " if (const and level == 0) else "*mut ") + r
    if array:
        n = array.strip("[]")
        if in_struct:
            r = f"[{r}; {n}]"
        else:  # an array parameter is a pointer to its first element
            r = ("*const " if const else "*mut ") + r
    return r


def parse(header: str):
    text = strip_comments(header)
    items = []  # (pos, kind, payload)
    for m in re.finditer(r"#define\s+(VYB_\w+)\s+([0-9A-Fa-fxX]+)(u?)\s*$", text, flags=re.M):
        items.append((m.start(), "const", (m.group(1), m.group(2), m.group(3))))
    for m in re.finditer(r"typedef\s+struct\s+(\w+)\s+(\w+)\s*;", text):
        items.append((m.start(), "opaque", m.group(2)))
    for m in re.finditer(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            # `uint32_t a, b[3]` declares several fields of one base type
            first, *rest = [p.strip() for p in decl.split(",")]
            fm = re.match(r"(.+?[\s\*])(\w+)(\[\d+\])?$", first)
            ctype = fm.group(1)
            fields.append((fm.group(2), rust_type(ctype, fm.group(3), True)))
            for extra in rest:
                em = re.match(r"(\w+)(\[\d+\])?$", extra)
                fields.append((em.group(1), rust_type(ctype, em.group(2), True)))
        items.append((m.start(), "struct", (m.group(3), fields)))
    for m in re.finditer(r"^([\w\s\*]+?[\s\*])(vyb_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.M | re.S):
        ret = " ".join(m.group(1).split())
        if ret.startswith("typedef"):
            continue
        params = []
        plist = " ".join(m.group(3).split())
        if plist and plist != "void":
            for p in plist.split(","):
                pm = re.match(r"(.+?[\s\*])(\w+)(\[\d+\])?$", p.strip())
                params.append((pm.group(2), rust_type(pm.group(1), pm.group(3), False)))
        items.append((m.start(), "fn", (m.group(2), ret, params)))
    items.sort(key=lambda it: it[0])
    return items


RUST_KEYWORDS = {"type", "in", "ref", "match", "move", "box", "fn", "use", "mod", "impl", "loop", "where"}


def ident(name: str) -> str:
    return "r#" + name if name in RUST_KEYWORDS else name


def generate() -> str:
    with open(HEADER) as fh:
        items = parse(fh.read())
    out = ["#![allow(non_camel_case_types)]", "use std::os::raw::{c_char, c_void};", ""]
    fns = []
    for _, kind, payload in items:
        if kind == "const":
            name, value, unsigned = payload
            ty = "u32" if unsigned or name.startswith(("VYB_DT_", "VYB_ACCESS_", "VYB_LAUNCH_", "VYB_ABI")) else "i32"
            out.append(f"pub const {name}: {ty} = {value};")
        elif kind == "opaque":
            out.append(f"#[repr(C)] pub struct {payload} {{ _private: [u8; 0] }}")
        elif kind == "struct":
            name, fields = payload
            out.append("#[repr(C)] #[derive(Clone, Copy)]")
            out.append(f"pub struct {name} {{")
            out.extend(f"    pub {ident(f)}: {t}," for f, t in fields)
            out.append("}")
        else:
            fns.append(payload)
    out += ["", '#[link(name = "vyre_b200")]', 'extern "C" {']
    for name, ret, params in fns:
        args = ", ".join(f"{ident(p)}: {t}" for p, t in params)
        r = "" if ret == "void" else " -> " + rust_type(ret, None, False)
        out.append(f"    pub fn {name}({args}){r};")
    out.append("}")
    return "\n".join(out) + "\n"


BEGIN, END = "<!-- generated by include/gen_rust_sys.py: begin -->", "<!-- generated by include/gen_rust_sys.py: end -->"


def doc_block() -> str | None:
    with open(DOC) as fh:
        doc = fh.read()
    if BEGIN not in doc or END not in doc:
        return None
    body = doc.split(BEGIN, 1)[1].split(END, 1)[0]
    m = re.search(r"```rust\n(.*?)```", body, flags=re.S)
    return m.group(1) if m else None


if __name__ == "__main__":
    text = generate()
    if "--check" in sys.argv:
        sys.exit(0 if doc_block() == text else 1)
    sys.stdout.write(text)
