"""The Rust -sys crate under bindings/ against the C header: every function the header declares is declared in
bindings/hearth-b200-sys/src/lib.rs with the same name and the same number of parameters, every status code and type
id has the same value, and the committed file is what the generator produces from the current header.  Runs without a
Rust toolchain (text comparison only)."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _generator():
    spec = importlib.util.spec_from_file_location("hb200_bindgen", os.path.join(ROOT, "bindings", "generate.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_bindings_are_current():
    gen = _generator()
    assert open(gen.OUT).read() == gen.generate(), "run `python bindings/generate.py` after changing include/hb200.h"


def test_every_header_function_is_bound_with_the_same_arity():
    gen = _generator()
    header = open(gen.HEADER).read()
    rust = open(gen.OUT).read()
    protos = gen.prototypes(header)
    names = [n for n, _, _ in protos]
    assert len(names) == len(set(names)) >= 70
    # independent of the generator's own parser: count the HB200_API markers
    assert len(re.findall(r"^HB200_API\b", gen.strip_comments(header), flags=re.M)) == len(names)
    bound = dict(re.findall(r"pub fn (hb200_\w+)\((.*?)\)", rust))
    assert sorted(bound) == sorted(names)
    for name, _, args in protos:
        n_rust = 0 if not bound[name].strip() else bound[name].count(":")
        assert n_rust == len(args), (name, args, bound[name])
    from hearth_b200 import lib as L
    assert sorted(L.SIGNATURES) == sorted(names)
    for name, _, args in protos:
        assert len(L.SIGNATURES[name][1]) == len(args), name


def test_constants_match_the_header():
    gen = _generator()
    header = gen.strip_comments(open(gen.HEADER).read())
    rust = dict(re.findall(r"pub const (HB200_\w+): \w+ = (-?\d+);", open(gen.OUT).read()))
    for k, v in re.findall(r"(HB200_\w+)\s*=\s*(-?\d+)", header):
        assert rust[k] == v, k
    for k in ("HB200_MAX_SEQ_LEN", "HB200_NOALLOC_MAX_TOKENS", "HB200_NOALLOC_MAX_COLS", "HB200_PEER_HANDLE_BYTES", "HB200_MAX_PEERS"):
        assert k in rust
    from hearth_b200 import lib as L
    for code, name in L.STATUS.items():
        assert int(rust[name]) == code
