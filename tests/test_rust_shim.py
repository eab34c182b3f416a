"""The Rust shim (rust-shim/src/lib.rs) cannot be compiled where this library is built (no rustc), so
its FFI mirror is checked as text against include/llmini_b200.h: every exported function with the same
number of arguments, every struct with the same fields in the same order, and the constants.  The
forwarding layer must carry every hot-path method of the reference's `OptimizerModule` and
`Nvfp4QuantModule`."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = open(os.path.join(ROOT, "include", "llmini_b200.h")).read()
SHIM = open(os.path.join(ROOT, "rust-shim", "src", "lib.rs")).read()


def _strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def _strip_rust_comments(text):
    return re.sub(r"//[^\n]*", "", text)


def header_functions():
    """name -> argument count of every function the header declares."""
    text = _strip_c_comments(HEADER)
    out = {}
    for m in re.finditer(r"\b(b2_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    return out


def header_structs():
    """name -> field names in declaration order."""
    text = _strip_c_comments(HEADER)
    out = {}
    for m in re.finditer(r"typedef\s+struct\s+(b2_[a-z0-9_]+)\s*\{(.*?)\}\s*\1\s*;", text, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                name = re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[[^\]]*\])?\s*$", part.strip())
                assert name, decl
                fields.append(name[0])
        out[m.group(1)] = fields
    return out


def shim_functions():
    text = _strip_rust_comments(SHIM)
    block = re.search(r'extern\s+"C"\s*\{(.*?)\n    \}', text, flags=re.S).group(1)
    out = {}
    for m in re.finditer(r"pub fn (b2_[a-z0-9_]+)\s*\((.*?)\)\s*(?:->\s*[^;]+)?;", block, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if not args else len([a for a in args.split(",") if a.strip()])
    return out


def shim_structs():
    text = _strip_rust_comments(SHIM)
    out = {}
    for m in re.finditer(r"#\[repr\(C\)\][^{;]*?pub struct (b2_[a-z0-9_]+)\s*\{(.*?)\n    \}", text, flags=re.S):
        out[m.group(1)] = re.findall(r"pub ([a-z0-9_]+)\s*:", m.group(2))
    return out


def test_every_exported_function_is_bound_with_the_same_arity():
    h, s = header_functions(), shim_functions()
    assert len(h) >= 50
    assert sorted(h) == sorted(s), (sorted(set(h) - set(s)), sorted(set(s) - set(h)))
    assert {n: (h[n], s[n]) for n in h if h[n] != s[n]} == {}


def test_every_struct_has_the_same_fields_in_the_same_order():
    h, s = header_structs(), shim_structs()
    assert set(h) == {"b2_muon_slot_descriptor", "b2_symexp_lin_slot_descriptor", "b2_muon_options", "b2_muon_step_args",
                      "b2_schedule_free_materialize_args", "b2_adamw_update_args", "b2_adamw_slot_descriptor",
                      "b2_symexp_lin_adamw_args", "b2_gradient_clip_args", "b2_peer_group"}
    for name, fields in h.items():
        assert s.get(name) == fields, name


def test_constants_agree():
    text = _strip_c_comments(HEADER)
    for name, value in re.findall(r"#define\s+(B2_[A-Z0-9_]+)\s+\(?([0-9]+)u?", text):
        m = re.search(rf"pub const {name}: [a-z0-9]+ = ([0-9]+)", SHIM)
        if m:
            assert int(m.group(1)) == int(value), name
    assert re.search(r"pub const B2_ABI_VERSION: u32 = (\d+)", SHIM).group(1) == re.search(
        r"#define B2_ABI_VERSION (\d+)u", HEADER).group(1)
    for enum in re.findall(r"enum\s*\{([^}]*)\}", text, flags=re.S):
        for name, value in re.findall(r"(B2_[A-Z0-9_]+)\s*=\s*([0-9]+)", enum):
            m = re.search(rf"pub const {name}: u32 = ([0-9]+)", SHIM)
            assert m and int(m.group(1)) == int(value), name


def test_forwarding_layer_has_every_reference_method_of_the_path():
    # crates/cuda-kernels/src/gpt/optimizer/launcher/{mod,muon_mega,update,adam,grad_clip,symexp_lin}.rs and
    # crates/cuda-kernels/src/utils/nvfp4/quant/{amax,four_six}.rs
    methods = ["verify_storage_layout", "materialize_master", "muon_mega_update", "muon_tma_prepare_polar",
               "muon_tma_prepare_polar_cooperative_reference", "muon_tma_finish_update",
               "muon_tma_finish_update_deferred_quantization", "muon_tma_finish_hyperball_update_deferred_quantization",
               "muon_tma_sign_update_deferred_quantization", "muon_tma_finish_update_cooperative_reference",
               "materialize_schedule_free_precomputed", "materialize_schedule_free", "apply_adamw_update",
               "apply_adamw_update_deferred_quantization", "zero_f32_pointer_table", "apply_fp32_adamw_update",
               "clip_gradients", "symexp_lin_zero_scale_grads", "symexp_lin_scale_adamw_update",
               "symexp_lin_congruent_inverse_in_place", "tensor_amax_f32", "tensor_amax_from_chunks_f32",
               "fp32_to_nvfp4_four_six"]
    for m in methods:
        assert re.search(rf"pub fn {m}\s*\(", SHIM), m
    # struct literals are complete: every field of the FFI struct is named where the shim builds one
    structs = shim_structs()
    text = _strip_rust_comments(SHIM)
    for name in ("b2_muon_step_args", "b2_adamw_update_args", "b2_gradient_clip_args", "b2_symexp_lin_adamw_args",
                 "b2_schedule_free_materialize_args"):
        literals = re.findall(rf"(?<!struct )(?<!-> )\b{name} \{{\n(.*?)\n        \}}", text, flags=re.S)
        assert literals, name
        for body in literals:
            named = re.findall(r"^\s*([a-z0-9_]+)\s*[:,]", body, flags=re.M)
            assert named == structs[name], (name, named)
