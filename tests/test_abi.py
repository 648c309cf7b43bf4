"""CPU checks of the C-ABI boundary: the library builds, loads without a GPU, exports every symbol
the header declares, and rejects bad arguments without touching a device."""
import ctypes
import os
import re

from kernl_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kernl_b200.h")
DEBUG_HEADER = os.path.join(ROOT, "include", "kernl_b200_debug.h")


def declared_functions(header=HEADER):
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kb_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    lib = ctypes.CDLL(build.LIB_PATH)
    names = declared_functions()
    assert "kb_attention_fwd" in names and "kb_linear_fwd" in names and "kb_norm_fwd" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/kernl_b200.h but not exported"
    for name in _lib.EXPORTED_SYMBOLS:
        assert name in names
    # the unstable test hooks are declared apart, and nothing is exported that neither header declares
    hooks = declared_functions(DEBUG_HEADER)
    assert hooks and all(h.startswith("kb_debug_") for h in hooks)
    for name in hooks:
        assert hasattr(lib, name), f"{name} is declared in include/kernl_b200_debug.h but not exported"
    import subprocess

    exported = subprocess.run(["nm", "-D", "--defined-only", build.LIB_PATH], capture_output=True, text=True).stdout
    for sym in re.findall(r"\bT (kb_\w+)", exported):
        assert sym in names or sym in hooks, f"{sym} is exported but declared in no header"


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.kb_version() >= 100
    assert _lib.status_str(0) == "ok"
    for code in range(-6, 0):
        assert _lib.status_str(code) != "unknown status"


def test_bad_arguments_are_rejected_before_any_device_call():
    lib = _lib.load()
    assert lib.kb_norm_fwd(None, None) == -1
    assert lib.kb_linear_fwd(None, None) == -1
    assert lib.kb_attention_fwd(None, None) == -1
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=4, K=0)
    assert lib.kb_linear_fwd(p, None) == -1
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=4, K=12, x_row_stride=12, y_row_stride=4)
    assert lib.kb_linear_fwd(p, None) == -2  # K not a multiple of 8
    gated = _lib.ACTIVATIONS["swiglu"]
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=24, K=16, x_row_stride=16, y_row_stride=12, activation=gated)
    assert lib.kb_linear_fwd(p, None) == -1  # gate/up rows come in blocks of eight: N a multiple of 16
    p = _lib.LinearParams(x=16, w=16, y=16, act_inputs=16, M=4, N=32, K=16, x_row_stride=16, y_row_stride=16,
                          activation=gated)
    assert lib.kb_linear_fwd(p, None) == -1  # no pre-activation output with the gated epilogue
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=32, K=16, x_row_stride=16, y_row_stride=16, activation=7)
    assert lib.kb_linear_fwd(p, None) == -1
    assert lib.kb_attention_decode_scratch_bytes(2, 3, 1, 1500, 64) == 2 * 3 * 1 * 12 * 66 * 4
    assert lib.kb_attention_decode_scratch_bytes(1, 1, 1, 128 * 256 + 1, 64) == 129 * 66 * 4


def test_struct_layouts_match_the_header():
    # sizes follow from the field lists in include/kernl_b200.h (LP64)
    assert ctypes.sizeof(_lib.NormParams) == 6 * 8 + 6 * 8 + 3 * 4 + 4 + 2 * 8
    assert ctypes.sizeof(_lib.LinearParams) == 5 * 8 + 5 * 8 + 2 * 4 + 2 * 8
    assert ctypes.sizeof(_lib.AttnParams) == 5 * 8 + 5 * 8 + 5 * 32 + 5 * 4 + 4 + 8  # 4 bytes of padding before kv_len_dev


def header_structs():
    """{struct name: [field names in order]} parsed from the header's `typedef struct {...} name;`."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for body, name in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # `const void* q`, `int64_t B, H, M`, `int64_t q_strides[4]`, `uint32_t* flags[8]`
            first, *rest = decl.split(",")
            fields.append(re.findall(r"(\w+)\s*(?:\[\w+\])?\s*$", first.strip())[0])
            fields += [re.findall(r"(\w+)\s*(?:\[\w+\])?\s*$", r.strip())[0] for r in rest]
        out[name] = fields
    return out


def test_ctypes_structs_follow_the_header_field_by_field():
    structs = header_structs()
    pairs = {"kb_norm_params": _lib.NormParams, "kb_linear_params": _lib.LinearParams, "kb_attn_params": _lib.AttnParams,
             "kb_rope_params": _lib.RopeParams, "kb_allreduce_params": _lib.AllReduceParams}
    for name, cls in pairs.items():
        assert name in structs, f"{name} not found in the header"
        assert [f[0] for f in cls._fields_] == structs[name], name


def test_binding_stub_in_the_integration_notes_follows_the_header():
    """The ctypes stub shown to a maintainer of the reference must list the header's fields, all of
    them and in order: a stub that stops early hands the library a struct that is too short."""
    structs = header_structs()
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    found = re.findall(r"class (kb_\w+)\(Structure\):\s*_fields_ = \[(.*?)\]\n", text, flags=re.S)
    assert found, "no ctypes stub found in INTEGRATION.md"
    for name, body in found:
        assert re.findall(r'\("(\w+)"', body) == structs[name], name


def test_reference_import_paths_resolve_to_this_package():
    """`kernl.*` module paths of the reference (src/kernl/...) are served by the modules of the same
    name under kernl_b200, as the same module objects."""
    import importlib

    import pytest

    for path, names in {
        "model_optimization": ["optimize_model"],
        "implementations.attention": ["attention_forward", "attention_reference", "closest_power_of_2"],
        "implementations.attention_skinny": ["skinny_attention_forward"],
        "implementations.linear_layer": ["linear_layer"],
        "implementations.layer_norm": ["layer_norm", "pytorch_naive_layernorm", "pytorch_naive_rmsnorm"],
        "optimizer.attention": ["attention_wrapper", "fuse_attention_pattern_1", "fuse_attention_pattern_2", "fuse_attention_pattern_3"],
        "optimizer.linear": ["linear_wrapper", "linear_wrapper_functional", "replace_all_linear"],
        "optimizer.layer_norm": ["layer_norm_wrapper", "layer_norm_rms_wrapper", "replace_layer_norm", "replace_layer_norm_rms"],
        "optimizer.dropout": ["remove_dropout"],
        "optimizer.normalizer": ["normalize_operators"],
        "optimizer.dynamo_backend": ["dynamo_backend_ofi"],
        "optimizer.cuda_graph": ["cuda_graphs_wrapper", "static_inputs_pool", "prepare_inputs", "get_pool_size", "argsort"],
        "optimizer.pool_cuda_graphs": ["CudaGraphPool", "get_aligned_size"],
        "utils.extended_matcher": ["replace_pattern"],
        "utils.fx": ["static_args_are_equal"],
    }.items():
        alias = importlib.import_module("kernl." + path)
        assert alias is importlib.import_module("kernl_b200." + path)
        for n in names:
            assert hasattr(alias, n), f"kernl.{path}.{n}"
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("kernl.debugger")
