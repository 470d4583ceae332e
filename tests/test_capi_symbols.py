"""The C-ABI library loads here (no GPU) and exports exactly what include/vtlb.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "vtlb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vtlb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_groups():
    names = declared_functions()
    for must in ("vtlb_ctx_create", "vtlb_alloc", "vtlb_gemm_f32", "vtlb_linear_fwd_f32",
                 "vtlb_linear_bwd_f32", "vtlb_adam_step_f32", "vtlb_adamw_step_f32",
                 "vtlb_quant_rows_i8", "vtlb_gemm_i8_i32", "vtlb_linear_i8_fwd",
                 "vtlb_allreduce_sum_f32_async"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from vtl_b200 import capi
    lib = capi.load()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in vtlb.h but not exported: {missing}"


def test_python_binding_covers_every_declared_symbol():
    from vtl_b200 import capi
    bound = set(capi._PROTOS) | {"vtlb_last_error", "vtlb_launch_count", "vtlb_stream", "vtlb_ckpt_text_len"}
    assert set(declared_functions()) <= bound, set(declared_functions()) - bound


def test_no_cpu_fallback_without_gpu():
    """Without a GPU, creating a context fails loudly (VTLB_ECUDA); nothing computes on the CPU."""
    from vtl_b200 import capi
    if capi.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(capi.VtlbError) as e:
        capi.Device(0)
    assert e.value.code == capi.ECUDA
    rc = capi.load().vtlb_sync(None)
    assert rc == capi.EINVAL


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "vtl_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


def test_v_declarations_follow_the_header():
    """vtl_b200/vglue/c_d_b200.v (the `fn C.vtlb_*` declarations a `-d b200` build of vtl includes)
    is what gen_c_decls.py derives from include/vtlb.h: one line per prototype, none missing, and
    every vtlb_* call in the hook files beside it is declared."""
    import importlib.util
    import re
    vdir = os.path.join(ROOT, "vtl_b200", "vglue")
    spec = importlib.util.spec_from_file_location("gen_c_decls", os.path.join(vdir, "gen_c_decls.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    committed = open(os.path.join(vdir, "c_d_b200.v")).read()
    assert committed == gen.render(), "run python vtl_b200/vglue/gen_c_decls.py"
    declared = set(re.findall(r"^fn C\.(vtlb_\w+)\(", committed, re.M))
    header = open(os.path.join(ROOT, "include", "vtlb.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    in_header = set(re.findall(r"\b(vtlb_\w+)\s*\(", header))
    assert declared == in_header
    for f in os.listdir(vdir):
        if f.endswith(".v") and f != "c_d_b200.v":
            used = set(re.findall(r"C\.(vtlb_\w+)\(", open(os.path.join(vdir, f)).read()))
            assert used <= declared, (f, used - declared)
