"""The Rust `turq-sys` crate cannot be compiled here (no Rust toolchain), so its extern block is
checked textually: every function include/turq.h declares must appear in rust/turq-sys/src/lib.rs
with the same name, arity, argument names and pointer / integer types, and the constants must
match. The safe wrapper may only call functions the -sys crate declares."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gen():
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(ROOT, "rust", "turq-sys", "gen_bindings.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_extern_block_matches_the_header_signature_by_signature():
    gen = _gen()
    c_funcs, consts, enums = gen.parse_header()
    r_funcs = {name: (ret, args) for name, ret, args in gen.parse_rust()}
    assert len(c_funcs) >= 40
    for name, ret, args in c_funcs:
        assert name in r_funcs, f"{name} is missing from the Rust extern block"
        rret, rargs = r_funcs[name]
        assert rret == ("()" if ret == "c_void" else ret), (name, rret, ret)
        assert rargs == args, f"{name}: Rust {rargs} vs C {args}"
    assert set(r_funcs) == {n for n, _, _ in c_funcs}, "the Rust block declares something the header does not"
    text = open(os.path.join(ROOT, "rust", "turq-sys", "src", "lib.rs")).read()
    for ename, items in enums:
        for iname, ival in items:
            assert re.search(rf"pub const {iname}: i32 = {ival};", text), iname
    for name, _ in consts:
        assert f"pub const {name}:" in text
    assert text == gen.render(), "rust/turq-sys/src/lib.rs is stale: run python rust/turq-sys/gen_bindings.py"


def test_type_translation():
    gen = _gen()
    t = gen.c_type_to_rust
    assert t("const turq_qtensor* const*") == "*const *const turq_qtensor"
    assert t("float* const*") == "*const *mut f32"
    assert t("const float* const*") == "*const *const f32"
    assert t("turq_ctx**") == "*mut *mut turq_ctx"
    assert t("const void*") == "*const c_void" and t("void*") == "*mut c_void"
    assert t("int64_t") == "i64" and t("size_t") == "usize" and t("const char*") == "*const c_char"


def test_safe_wrapper_only_calls_declared_functions_and_never_panics():
    gen = _gen()
    declared = {n for n, _, _ in gen.parse_rust()}
    src = open(os.path.join(ROOT, "rust", "turq", "src", "lib.rs")).read()
    code = re.sub(r"//.*", "", src)
    used = set(re.findall(r"sys::(turq_\w+)\s*\(", code))
    assert used and used <= declared, used - declared
    for banned in (".unwrap()", ".expect(", "panic!(", "unreachable!(", "todo!(", "unimplemented!("):
        assert banned not in code, f"the wrapper must not use {banned} (the reference denies it: Cargo.toml:79-86)"
    assert "impl Drop for QTensor" in code and "#[derive(Clone)]\npub struct QMatMul" in src
