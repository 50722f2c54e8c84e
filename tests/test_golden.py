"""Golden vectors: outputs of the reference's own kernels (cuda/nvfp4_ops.cu compiled unmodified for sm_100a)
recorded on a B200 by tests/golden/make_golden.py.  The CPU tests pin the oracle against them; the GPU tests
pin the library against them, so the comparison holds even where oracle/_ref is not built."""
import hashlib
import os

import numpy as np
import pytest

from conftest import from_u16, u16

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_b200.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


# ------------------------------------------------------------------ CPU: oracle vs the reference's outputs

@pytest.mark.parametrize("rows", [1, 4])
def test_oracle_logits_are_bit_exact_with_reference_kernels(orc, gold, rows):
    logits = orc.router_logits(gold[f"router{rows}_x"], gold["router_w"])          # IEEE fmaf chains, same order
    assert np.array_equal(logits.view(np.uint32), gold[f"router{rows}_logits"].view(np.uint32))


@pytest.mark.parametrize("rows", [1, 4])
def test_oracle_routing_matches_reference_kernels(orc, gold, rows):
    ids, weights, margin = orc.router_top8(gold[f"router{rows}_logits"], gold["router_bias"])
    safe = margin > 2e-6            # the reference's sigmoid is the fast-math one; exclude razor-thin margins
    assert safe.all()
    assert np.array_equal(ids, gold[f"router{rows}_ids"])
    assert np.abs(weights - gold[f"router{rows}_weights"]).max() < 2e-6


def test_oracle_quantiser_against_reference_kernel(orc, gold):
    packed, scales = orc.nvfp4_quantize(gold["quant_in"])
    assert np.array_equal(scales, gold["quant_scales"])
    g = gold["quant_packed"]
    mismatch = ((packed & 15) != (g & 15)).sum() + ((packed >> 4) != (g >> 4)).sum()
    assert mismatch <= 2                                   # exact division vs fast-math reciprocal on rounding ties
    assert not g[0, :8].any() and gold["quant_scales"][0, 0] == 0        # the all-zero block


def test_oracle_swiglu_and_combine_against_reference_kernels(orc, gold):
    out = np.empty(4096, np.uint16)
    orc.cpu().orc_swiglu(gold["swiglu_gate"], gold["swiglu_up"], out, 4096)
    a, b = orc.bf16_to_f32(out), orc.bf16_to_f32(gold["swiglu_out"])
    assert (out != gold["swiglu_out"]).mean() < 0.02       # libm expf vs ex2.approx: a last-bit BF16 flip at most
    assert np.abs(a - b).max() <= 2.0 ** -6 * np.abs(b).max()
    comb = np.empty((3, 2560), np.uint16)
    orc.cpu().orc_expert_combine_rows(gold["combine_rows"].reshape(-1), gold["combine_weights"].reshape(-1),
                                      comb.reshape(-1), 3, 8, 2560)
    assert np.array_equal(comb, gold["combine_out"])        # IEEE fmaf chain: bit-exact


# ------------------------------------------------------------------ GPU: library vs the reference's outputs

@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 4])
def test_library_router_bit_exact_with_golden(cuda, pkg, gold, rows):
    torch = cuda
    x = from_u16(gold[f"router{rows}_x"])
    w = from_u16(gold["router_w"])
    bias = torch.from_numpy(gold["router_bias"]).cuda()
    logits = torch.empty((rows, 256), dtype=torch.float32, device="cuda")
    if rows == 1:
        pkg.bf16_gemv_f32(x, w, logits)
    else:
        pkg.bf16_gemm_f32(x, w, logits, rows)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), gold[f"router{rows}_logits"].view(np.uint32))
    ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
    wt = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
    pkg.router_top8_rows(logits, bias, ids, wt, rows)
    assert np.array_equal(ids.cpu().numpy(), gold[f"router{rows}_ids"])
    assert np.array_equal(wt.cpu().numpy().view(np.uint32), gold[f"router{rows}_weights"].view(np.uint32))


@pytest.mark.gpu
def test_library_elementwise_bit_exact_with_golden(cuda, pkg, gold):
    torch = cuda
    x = from_u16(gold["quant_in"])
    packed = torch.empty((6, 512), dtype=torch.uint8, device="cuda")
    scales = torch.empty((6, 64), dtype=torch.uint8, device="cuda")
    pkg.nvfp4_quantize(x, packed, scales, 6 * 1024, 1.0)
    assert np.array_equal(packed.cpu().numpy(), gold["quant_packed"])
    assert np.array_equal(scales.cpu().numpy(), gold["quant_scales"])
    out = torch.empty(4096, dtype=torch.bfloat16, device="cuda")
    pkg.swiglu(from_u16(gold["swiglu_gate"]), from_u16(gold["swiglu_up"]), out, 4096)
    assert np.array_equal(u16(out), gold["swiglu_out"])
    comb = torch.empty((3, 2560), dtype=torch.bfloat16, device="cuda")
    pkg.expert_combine_rows(from_u16(gold["combine_rows"]), torch.from_numpy(gold["combine_weights"]).cuda(), comb, 3, 8,
                            2560)
    assert np.array_equal(u16(comb), gold["combine_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("path", [2, 3])
@pytest.mark.parametrize("rows", [1, 4])
def test_library_block_against_golden(cuda, pkg, orc, gold, layer0, rows, path):
    torch = cuda
    raw = layer0.raw
    digest = hashlib.sha256()
    for t in (raw.packed[:9], raw.scales_linear[:9], raw.packed[-3:], raw.alpha):
        digest.update(t.cpu().numpy().tobytes())
    if not np.array_equal(np.frombuffer(digest.digest(), dtype=np.uint8), gold["layer_digest"]):
        pytest.skip("the synthetic layer regenerated differently from the one the golden file was made on")
    x = from_u16(gold[f"block{rows}_x"])
    out = torch.empty_like(x)
    plan = pkg.MoePlan(max_rows=4)
    plan.set_path(path)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan).run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    v = plan.views(rows)
    assert np.array_equal(v["expert_ids"].cpu().numpy(), gold[f"block{rows}_ids"])            # bit-exact routing
    assert np.array_equal(v["expert_weights"].cpu().numpy().view(np.uint32), gold[f"block{rows}_weights"].view(np.uint32))
    got, want = orc.bf16_to_f32(u16(out)), orc.bf16_to_f32(gold[f"block{rows}_out"])
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    assert rel <= 1e-2 and float(np.abs(got - want).max()) <= 2e-2, (rel,)
    plan.close()
