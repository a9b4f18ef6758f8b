"""The Rust binding (muser-cuda/src/ffi.rs, not compiled here) stays in step with include/muser_cuda.h:
every entry point is declared, with the same number of arguments, and every shared constant has the same value."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "muser_cuda.h").read_text()
FFI = (ROOT / "muser-cuda" / "src" / "ffi.rs").read_text()


def strip_comments(text, rust=False):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//.*", "", text) if rust else text


def arity(arglist):
    arglist = arglist.strip()
    if arglist in ("", "void"):
        return 0
    return len([a for a in arglist.split(",") if a.strip()])


def header_functions():
    text = strip_comments(HEADER)
    return {m.group(1): arity(m.group(2)) for m in re.finditer(r"MUSER_CUDA_API[^;(]*?\b(muser_cuda_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)}


def ffi_functions():
    text = strip_comments(FFI, rust=True)
    return {m.group(1): arity(m.group(2)) for m in re.finditer(r"pub fn (muser_cuda_\w+)\s*\(([^;]*?)\)\s*(?:->[^;]*)?;", text, flags=re.S)}


def test_every_entry_point_is_bound_with_the_same_arity():
    h, r = header_functions(), ffi_functions()
    assert len(h) >= 35
    assert set(h) == set(r), (sorted(set(h) - set(r)), sorted(set(r) - set(h)))
    assert {n: (h[n], r[n]) for n in h if h[n] != r[n]} == {}


def test_argument_names_agree():
    text_h, text_r = strip_comments(HEADER), strip_comments(FFI, rust=True)
    for name in header_functions():
        args_h = re.search(rf"\b{name}\s*\(([^;]*?)\)\s*;", text_h, flags=re.S).group(1)
        args_r = re.search(rf"pub fn {name}\s*\(([^;]*?)\)\s*(?:->[^;]*)?;", text_r, flags=re.S).group(1)
        names_h = [re.search(r"(\w+)\s*(?:\[\d*\])?\s*$", a.strip()).group(1) for a in args_h.split(",") if a.strip() not in ("", "void")]
        names_r = [a.strip().split(":")[0].strip() for a in args_r.split(",") if a.strip()]
        assert names_h == names_r, name


def test_constants_agree():
    defines = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+(MUSER_\w+)\s+(\d+)u\b", HEADER)}
    consts = {m.group(1): int(m.group(2)) for m in re.finditer(r"pub const (MUSER_\w+): \w+ = (\d+);", FFI)}
    assert set(defines) == set(consts), (sorted(set(defines) ^ set(consts)))
    assert defines == consts


def test_status_codes_agree():
    enum_h = re.search(r"typedef enum muser_cuda_status \{(.*?)\}", strip_comments(HEADER), flags=re.S).group(1)
    enum_r = re.search(r"pub enum muser_cuda_status \{(.*?)\}", strip_comments(FFI, rust=True), flags=re.S).group(1)
    pairs = lambda s: dict(re.findall(r"(MUSER_CUDA_\w+)\s*=\s*(\d+)", s))
    assert pairs(enum_h) == pairs(enum_r) and len(pairs(enum_h)) == 10


def test_struct_fields_agree():
    for struct in ("muser_cuda_shard", "muser_cuda_epilogue", "muser_cuda_weight_info", "muser_cuda_group_item"):
        body_h = re.search(rf"typedef struct {struct} \{{(.*?)\}} {struct};", strip_comments(HEADER), flags=re.S).group(1)
        fields_h = []
        for decl in body_h.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            parts = [p.strip() for p in decl.split(",")]
            fields_h.append(re.search(r"(\w+)$", parts[0]).group(1))
            fields_h += [re.search(r"(\w+)$", p).group(1) for p in parts[1:]]
        body_r = re.search(rf"pub struct {struct} \{{(.*?)\}}", strip_comments(FFI, rust=True), flags=re.S).group(1)
        fields_r = re.findall(r"pub (\w+):", body_r)
        assert fields_h == fields_r, struct
