"""The Rust side of the boundary, as source: rust/tangq-sys declares every entry point of include/tangq.h.

No Rust toolchain exists here, so nothing is compiled.  What can be checked is that the committed declarations are
exactly what the generator produces from the current header (nobody edited one without the other), that every symbol
the header exports is declared with the right number of arguments, and that the same names are what the ctypes
mirror binds — i.e. the Rust block, the header and the tested Python host all describe one ABI.
"""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gen():
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(ROOT, "rust", "tangq-sys", "gen_bindings.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_bindings_match_the_header():
    gen = _gen()
    committed = open(os.path.join(ROOT, "rust", "tangq-sys", "src", "lib.rs")).read()
    assert committed == gen.generate(), "rust/tangq-sys/src/lib.rs is stale: run python rust/tangq-sys/gen_bindings.py"


def test_every_exported_symbol_is_declared_with_its_arity():
    from tang_b200 import _lib

    gen = _gen()
    structs, funcs, enums = gen.parse(open(os.path.join(ROOT, "include", "tangq.h")).read())
    header = open(os.path.join(ROOT, "include", "tangq.h")).read()
    exported = set(re.findall(r"TQ_API[^;(]*?\b(tq_\w+)\s*\(", header))
    declared = {name: params for name, _ret, params in funcs}
    assert set(declared) == exported
    assert set(declared) == set(_lib.PROTOTYPES)
    for name, params in declared.items():
        assert len(params) == len(_lib.PROTOTYPES[name][1]), name
    # by-value structs of the ABI are #[repr(C)] with every field of the header
    names = {n for n, _ in structs}
    assert names == {"tq_sampler_config", "tq_llama_config", "tq_moe_config", "tq_mla_config"}
    cfg = dict(structs)["tq_llama_config"]
    assert [f for f, _ in cfg] == ["n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "max_seq",
                                   "max_batch", "eps", "rope_base"]
    assert dict(cfg)["eps"] == "f32" and dict(cfg)["rope_base"] == "f64" and dict(cfg)["max_seq"] == "u32"
    assert dict(enums["tq_status"])["TQ_ETIMEOUT"] == 4
