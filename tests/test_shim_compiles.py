"""The shim that puts the library behind the reference's operator entry points must compile against the
reference's OWN header (include/p92/kernels.h): its functions are defined with the reference's signatures, so any
drift between the two interfaces is a compile error.  Needs the reference checkout ($P92_REFERENCE, or a directory
named "reference" beside the repository) and a C++17 compiler; skipped otherwise.  Compile only: nothing is linked or
run."""
import os
import shutil
import subprocess

import pytest

import __graft_entry__ as entry

SHIM = os.path.join(entry.PACKAGE_DIR, "shim", "p92b_kernels_shim.cpp")


def test_shim_compiles_against_the_reference_header():
    header = os.path.join(entry.REFERENCE, "include", "p92", "kernels.h")
    compiler = shutil.which("g++")
    cuda_include = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if not os.path.exists(header) or compiler is None or not os.path.exists(os.path.join(cuda_include, "cuda_runtime_api.h")):
        pytest.skip("reference checkout, g++ or the CUDA headers are not available")
    result = subprocess.run([compiler, "-std=c++17", "-fsyntax-only", "-Wall", "-Wextra", "-Werror",
                             "-I", os.path.join(entry.REFERENCE, "include"), "-I", os.path.join(entry.ROOT, "include"),
                             "-I", cuda_include, SHIM], capture_output=True, text=True)
    assert result.returncode == 0, result.stderr


def test_shim_defines_every_moe_entry_point_of_the_reference_header():
    text = open(SHIM).read()
    for name in ("nvfp4_grouped_plan_create", "nvfp4_grouped_plan_destroy", "nvfp4_grouped_m1", "nvfp4_grouped_rows",
                 "bf16_gemv_f32", "bf16_gemm_f32", "router_top8", "router_top8_rows", "nvfp4_quantize",
                 "nvfp4_swizzled_scale_bytes", "nvfp4_swizzle_scales", "swiglu", "expert_combine", "expert_combine_rows",
                 "add_inplace", "rmsnorm", "rmsnorm_strided"):
        assert f" {name}(" in text, name
