"""The Rust FFI crate (source only: no Rust toolchain exists here) declares exactly the entry points of
include/ruai_b200.h, each with the header's number of arguments, and mirrors its constants and structs."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CRATE = os.path.join(ROOT, "include", "ruai-b200-sys")


def header_functions():
    text = open(os.path.join(ROOT, "include", "ruai_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for name, args in re.findall(r"\b(ruai_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        args = args.strip()
        out[name] = 0 if args in ("", "void") else len(args.split(","))
    return out


def rust_functions():
    text = open(os.path.join(CRATE, "src", "lib.rs")).read()
    out = {}
    for name, args in re.findall(r"pub fn (ruai_[a-z0-9_]+)\s*\(([^)]*)\)", text):
        out[name] = len([a for a in args.split(",") if a.strip()])
    return out


def test_crate_files_exist():
    for f in ("Cargo.toml", "build.rs", "src/lib.rs", "src/backend.rs"):
        assert os.path.exists(os.path.join(CRATE, f)), f


def test_every_entry_point_is_declared_with_the_same_arity():
    h, r = header_functions(), rust_functions()
    assert h and set(h) == set(r), set(h) ^ set(r)
    assert {n: a for n, a in h.items() if r[n] != a} == {}


def test_constants_and_structs_match_the_header():
    h = open(os.path.join(ROOT, "include", "ruai_b200.h")).read()
    r = open(os.path.join(CRATE, "src", "lib.rs")).read()
    for name, val in re.findall(r"\b(RUAI_(?:OK|ERR_[A-Z]+|F32|F16|BF16))\s*=\s*(\d+)", h):
        assert re.search(rf"pub const {name}: c_int = {val};", r), name
    for struct in ("ruai_llama_config", "ruai_gpt2_config", "ruai_tp"):
        body = re.search(r"typedef struct \{([^}]*)\}\s*" + struct, h).group(1)
        fields = [f.strip() for decl in body.split(";") for f in re.sub(r"\b(uint32_t|float)\b", "", decl).split(",") if f.strip()]
        rbody = re.search(r"pub struct " + struct + r" \{([^}]*)\}", r).group(1)
        assert re.findall(r"pub (\w+):", rbody) == fields, struct
    assert "pub const RUAI_IPC_HANDLE_BYTES: usize = 64;" in r and "#define RUAI_IPC_HANDLE_BYTES 64" in h


def test_safe_layer_uses_only_declared_entry_points():
    used = set(re.findall(r"\b(ruai_[a-z0-9_]+)\s*\(", open(os.path.join(CRATE, "src", "backend.rs")).read()))
    assert used <= set(rust_functions()), used - set(rust_functions())
