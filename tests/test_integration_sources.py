"""The reference-side sources under integration/ stay in lockstep with the C ABI: every function include/et_cuda.h declares
appears in crates/runtime-cuda/src/ffi.rs with the same name, the same number of parameters and pointer/scalar kinds in
the same places, and every symbol the safe layer and the addon call exists in ffi.rs."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "et_cuda.h")
CRATE = os.path.join(ROOT, "integration", "crates", "runtime-cuda", "src")


def header_functions():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for decl in re.findall(r"ETC_API\s+([^;{]+\([^;]*\))\s*;", text):
        decl = " ".join(decl.split())
        m = re.match(r"^(.*?)(\w+)\((.*)\)$", decl)
        args = [] if m.group(3).strip() == "void" else [a.strip() for a in m.group(3).split(",")]
        out[m.group(2)] = ["ptr" if "*" in a else "value" for a in args]
    return out


def rust_functions():
    text = open(os.path.join(CRATE, "ffi.rs")).read()
    block = text[text.index('extern "C" {'):]
    out = {}
    for name, args in re.findall(r"pub fn (\w+)\(([^)]*)\)", block, flags=re.S):
        params = [a.strip() for a in args.split(",") if a.strip()]
        out[name] = ["ptr" if re.search(r":\s*\*(const|mut)", a) else "value" for a in params]
    return out


def test_every_header_symbol_is_bound_with_the_same_arity_and_argument_kinds():
    c, rust = header_functions(), rust_functions()
    assert len(c) > 80
    assert sorted(c) == sorted(rust)
    for name, kinds in c.items():
        assert rust[name] == kinds, name


def test_the_safe_layer_and_the_addon_only_call_bound_symbols():
    rust = rust_functions()
    for path in ("lib.rs", os.path.join("napi", "mod.rs")):
        text = open(os.path.join(CRATE, path)).read()
        for name in set(re.findall(r"ffi::(etc_\w+)", text)):
            assert name in rust, f"{path} calls {name}, which ffi.rs does not declare"


def test_structs_mirror_the_header_field_for_field():
    header = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    rust = open(os.path.join(CRATE, "ffi.rs")).read()
    for c_name, rust_name in (("etc_capabilities", "EtcCapabilities"), ("etc_decoder_config", "EtcDecoderConfig"), ("etc_lane", "EtcLane")):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (c_name, c_name), header, flags=re.S).group(1)
        c_fields = []
        for statement in body.split(";"):
            statement = " ".join(statement.split())
            if not statement:
                continue
            names = statement.split(" ", 1)[1] if " " in statement else statement
            names = re.sub(r"^(int|double|char|uint32_t|uint64_t|int64_t)\s+", "", statement)
            c_fields += [re.sub(r"\[.*\]", "", n).strip() for n in names.split(",")]
        rust_body = re.search(r"pub struct %s \{(.*?)\n\}" % rust_name, rust, flags=re.S).group(1)
        rust_fields = re.findall(r"pub (\w+):", rust_body)
        assert rust_fields == c_fields, (c_name, c_fields, rust_fields)
