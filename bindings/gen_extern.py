"""Writes the `extern "C"` block of bindings/ava_engine.rs from include/ava_engine.h, prototype by prototype.

    python bindings/gen_extern.py           rewrite the block between the two marker lines of ava_engine.rs
    python bindings/gen_extern.py --check   exit 1 when the block in the file is not what the header gives

The rest of ava_engine.rs (the structs and the safe wrapper) is written by hand and left alone.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "ava_engine.h")
RS = os.path.join(HERE, "ava_engine.rs")
BEGIN = "    // ---- begin: generated from include/ava_engine.h by bindings/gen_extern.py"
END = "    // ---- end: generated"

BASE = {"int": "c_int", "int32_t": "i32", "int64_t": "i64", "uint32_t": "u32", "uint64_t": "u64", "uint8_t": "u8", "int8_t": "i8",
        "unsigned char": "u8", "float": "f32", "double": "f64", "char": "c_char", "void": "c_void", "size_t": "usize",
        "ava_engine": "AvaEngine", "ava_state": "AvaState", "ava_ckpt": "AvaCkpt", "ava_trace": "AvaTrace", "ava_config": "AvaConfig"}
CALLBACKS = {"ava_pick_fn": "Option<extern \"C\" fn(*mut c_void, i32, *const f32, i32) -> u32>",
             "ava_stop_fn": "Option<extern \"C\" fn(*mut c_void, i32, *const u32, i32) -> c_int>"}
RUST_KEYWORDS = {"type", "in", "ref", "box", "move", "fn", "impl", "loop", "match", "mod", "use", "where", "self"}


def rust_type(c: str) -> str:
    """`const float*` -> `*const f32`, `ava_state**` -> `*mut *mut AvaState`, `const ava_state* const*` -> `*const *const AvaState`."""
    c = c.strip()
    if c in CALLBACKS:
        return CALLBACKS[c]
    # split into the base (with its const) and the pointer levels (each with an optional const after it)
    m = re.match(r"^(const\s+)?((?:unsigned\s+)?\w+)\s*((?:\*\s*(?:const\s*)?)*)$", c)
    if not m:
        raise ValueError(f"type not understood: {c!r}")
    base_const, base, stars = bool(m.group(1)), m.group(2), m.group(3)
    if base not in BASE:
        raise ValueError(f"base type not known: {base!r} in {c!r}")
    levels = re.findall(r"\*\s*(const)?", stars)   # left to right: nearest the base first
    out = BASE[base]
    for i, lvl_const in enumerate(levels):
        pointee_const = base_const if i == 0 else bool(levels[i - 1])
        out = ("*const " if pointee_const else "*mut ") + out
    return out


def prototypes():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    text = re.sub(r"typedef[^;]*;", "", text, flags=re.S)
    text = re.sub(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    out = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(ava_[a-z0-9_]+)\s*\(([^;{}]*)\)\s*;", text, flags=re.S):
        ret, name, args = " ".join(m.group(1).split()), m.group(2), " ".join(m.group(3).split())
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                am = re.match(r"^(.*?)(\w+)(\[\d*\])?$", a)
                ty, pname = am.group(1).strip(), am.group(2)
                if am.group(3):
                    ty += "*"
                params.append((pname + "_" if pname in RUST_KEYWORDS else pname, rust_type(ty)))
        out.append((name, None if ret == "void" else rust_type(ret), params))
    return out


def block() -> str:
    lines = [BEGIN]
    for name, ret, params in prototypes():
        sig = f"    pub fn {name}(" + ", ".join(f"{p}: {t}" for p, t in params) + ")" + (f" -> {ret}" if ret else "") + ";"
        lines.append(sig)
    lines.append(END)
    return "\n".join(lines)


def main():
    src = open(RS).read()
    i0, i1 = src.index(BEGIN), src.index(END) + len(END)
    new = src[:i0] + block() + src[i1:]
    if "--check" in sys.argv:
        sys.exit(0 if new == src else 1)
    open(RS, "w").write(new)


if __name__ == "__main__":
    main()
