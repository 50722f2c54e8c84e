"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import __graft_entry__ as entry


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    declared = entry.declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(pkg.SIGNATURES) == declared, "host bindings and header disagree"
    assert b"sm_100a" in lib.p92b_version()


def test_header_is_plain_c_and_cites_the_reference():
    text = open(os.path.join(entry.ROOT, "include", "p92b_moe.h")).read()
    assert "torch" not in text and "std::" not in text and "at::" not in text
    body = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    assert "class " not in body and "template" not in body
    for cite in ("include/p92/kernels.h", "src/executor.cpp", "src/model.cpp", "cuda/nvfp4_grouped.cu"):
        assert cite in text


def test_expert_projection_layout_matches_reference_struct(pkg):
    # p92::cuda::Nvfp4ExpertProjection is three pointers (include/p92/kernels.h:12-16)
    assert ctypes.sizeof(pkg.ExpertProjection) == 24


def test_argument_validation_needs_no_gpu(pkg):
    lib = pkg.load_library()
    assert lib.p92b_nvfp4_swizzled_scale_bytes(1024, 160) == 163840
    assert lib.p92b_nvfp4_swizzled_scale_bytes(2560, 64) == 163840
    assert lib.p92b_nvfp4_swizzled_scale_bytes(4, 160) == 128 * 160
    assert lib.p92b_nvfp4_swizzled_scale_bytes(0, 4) == 0
    assert lib.p92b_nvfp4_quantize(None, None, None, 16, 1.0, None) == 1        # cudaErrorInvalidValue
    assert lib.p92b_router_top8_rows(None, None, None, None, 1, 2.5, None) == 1
    assert lib.p92b_moe_forward(None, None, None, None, None, None, 1, 2.5, None) == 1
    lib.p92b_plan_destroy(None)     # null-safe, like nvfp4_grouped_plan_destroy
    lib.p92b_bank_destroy(None)
    assert lib.p92b_plan_last_launches(None) == 0
