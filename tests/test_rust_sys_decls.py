"""The Rust `-sys` crate cannot be compiled in this environment (no Rust toolchain); this test keeps its
declarations in step with the C header by text: every function `include/rwkv7_b200.h` declares appears in
`src/lib.rs` with the same number of parameters, the status and dtype constants carry the header's values,
and the tensor descriptor has the header's fields in the header's order."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rwkv7_b200.h")
LIB_RS = os.path.join(ROOT, "rwkv-rs-stable_b200", "rust", "rwkv7-b200-sys", "src", "lib.rs")


def _strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", " ", re.sub(r"//[^\n]*", " ", text), flags=re.S)


def _c_functions(text):
    out = {}
    for m in re.finditer(r"\b(?:int|size_t|int64_t|const char \*)\s*(rwkv7_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    return out


def _rust_functions(text):
    text = re.sub(r"//[^\n]*", " ", text)
    out = {}
    for m in re.finditer(r"pub fn (rwkv7_\w+)\s*\(([^)]*)\)", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if not args else len([a for a in args.split(",") if a.strip()])
    return out


def test_every_header_function_is_declared_with_the_same_arity():
    c = _c_functions(_strip_c_comments(open(HEADER).read()))
    rs = _rust_functions(open(LIB_RS).read())
    assert len(c) >= 30
    assert set(c) == set(rs), (sorted(set(c) - set(rs)), sorted(set(rs) - set(c)))
    wrong = {n: (c[n], rs[n]) for n in c if c[n] != rs[n]}
    assert not wrong, wrong


def test_constants_and_descriptor_match_the_header():
    h = _strip_c_comments(open(HEADER).read())
    rs = open(LIB_RS).read()
    enums = dict((n, int(v)) for n, v in re.findall(r"\b(RWKV7_[A-Z0-9_]+)\s*=\s*(-?\d+)", h))
    assert len(enums) >= 25
    for name, value in enums.items():
        m = re.search(r"pub const %s: \w+ = (-?\d+);" % name, rs)
        assert m, name
        assert int(m.group(1)) == value, name
    fields_c = re.findall(r"\b(\w+)(?:\[\w+\])?;", re.search(r"typedef struct rwkv7_tensor \{(.*?)\}", h, flags=re.S).group(1))
    fields_rs = re.findall(r"pub (\w+):", re.search(r"pub struct rwkv7_tensor \{(.*?)\}", rs, flags=re.S).group(1))
    assert fields_c == fields_rs == ["data", "dtype", "device", "ndim", "reserved", "shape", "stride"]
