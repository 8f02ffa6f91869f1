"""INTEGRATION.md's Rust `-sys` block is generated from include/vyre_b200.h: it must hold exactly the generator's
output, and every declaration must agree with the header symbol by symbol (name, arity, argument order)."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "include"))


def test_rust_block_in_integration_md_is_the_generated_one():
    import gen_rust_sys

    block = gen_rust_sys.doc_block()
    assert block is not None, "INTEGRATION.md lost its generated block"
    assert block == gen_rust_sys.generate(), "regenerate: python include/gen_rust_sys.py"


def test_rust_declarations_match_the_header_symbol_by_symbol():
    import gen_rust_sys

    rust = gen_rust_sys.doc_block()
    rust_fns = {m.group(1): [a.split(":")[0].strip() for a in m.group(2).split(",") if a.strip()]
                for m in re.finditer(r"pub fn (\w+)\((.*?)\)", rust)}
    header = gen_rust_sys.strip_comments(open(os.path.join(ROOT, "include", "vyre_b200.h")).read())
    c_fns = {}
    for m in re.finditer(r"\b(vyb_\w+)\s*\(([^;{}]*?)\)\s*;", header, flags=re.S):
        params = " ".join(m.group(2).split())
        names = [] if params in ("", "void") else [re.sub(r"\[\d+\]$", "", p.strip()).split()[-1].lstrip("*") for p in params.split(",")]
        c_fns[m.group(1)] = names
    assert set(rust_fns) == set(c_fns)
    for name, params in c_fns.items():
        got = [p.replace("r#", "") for p in rust_fns[name]]
        assert got == params, (name, got, params)
    # the two signatures a maintainer is most likely to paste
    assert rust_fns["vyb_submit"] == ["instance", "artifact_digest", "bindings", "n_bindings", "config", "submission"]
    assert "artifact_digest: *const u8" in rust and "config: *const vyb_dispatch_config" in rust


def test_generator_check_mode():
    assert subprocess.run([sys.executable, os.path.join(ROOT, "include", "gen_rust_sys.py"), "--check"]).returncode == 0
