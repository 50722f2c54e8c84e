"""The stand-ins for the reference's grouped-projection call (nvfp4_grouped_plan_create / nvfp4_grouped_rows,
include/p92/kernels.h:25-53) and for the two executor methods built on it (src/executor.cpp:39-107), replayed the
way tests/moe_forward_test.cpp drives them: the grouped dispatch of one token (:209-221), the M=4 verifier fixture
whose rows must equal the M=1 result bit for bit (:258-285), and the numerical gate against the serial chain
(:286-304, cosine >= 0.9999), here against the reference's software NVFP4 product on the same GPU."""
import ctypes

import numpy as np
import pytest

from conftest import u16

pytestmark = pytest.mark.gpu

HIDDEN, INTER = 2560, 1024


def _stream(torch):
    return torch.cuda.current_stream().cuda_stream


def _device_table(torch, raw):
    """Nvfp4ExpertProjection[257 * 3] on the device, pointing at the reference-format tensors of the layer."""
    n = raw.packed.shape[0]
    table = np.zeros((n, 3), dtype=np.uint64)
    for i in range(n):
        table[i] = (raw.packed[i].data_ptr(), raw.scales_swizzled[i].data_ptr(), raw.alpha[i:i + 1].data_ptr())
    return torch.from_numpy(table.view(np.int64)).cuda()


def _quantise_rows(torch, pkg, rows_bf16):
    n, width = rows_bf16.shape
    packed = torch.empty((n, width // 2), dtype=torch.uint8, device="cuda")
    linear = torch.empty((n, width // 16), dtype=torch.uint8, device="cuda")
    pkg.nvfp4_quantize(rows_bf16, packed, linear, n * width, 1.0)
    tiled = torch.empty(pkg.nvfp4_swizzled_scale_bytes(n, width // 16), dtype=torch.uint8, device="cuda")
    pkg.nvfp4_swizzle_scales(linear, tiled, n, width // 16)
    return packed, linear, tiled


def _routed(torch, pkg, layer0, x, rows):
    logits = torch.empty((rows, 256), dtype=torch.float32, device="cuda")
    ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
    weights = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
    if rows == 1:
        pkg.bf16_gemv_f32(x, layer0.router_weight, logits)
    else:
        pkg.bf16_gemm_f32(x, layer0.router_weight, logits, rows)
    pkg.router_top8_rows(logits, layer0.bias, ids, weights, rows)
    return ids, weights


def _grouped_chain(torch, pkg, table, ids, weights, x, rows):
    """project_expert_gate_up -> swiglu -> project_expert_down -> expert_combine_rows with the kernel-level calls,
    quantising the rows the way ProjectionExecutor does (src/executor.cpp:53-59,85-95)."""
    xq, _, xs = _quantise_rows(torch, pkg, x)
    gate = torch.full((rows * 8, INTER), float("nan"), dtype=torch.bfloat16, device="cuda")
    up = torch.full_like(gate, float("nan"))
    gu_plan = pkg.GroupedPlan(rows * 16, INTER, HIDDEN)
    gu_plan.grouped_rows(xq, xs, table, ids, gate, up, 0, rows, False)
    gate_only = torch.full_like(gate, float("nan"))
    one_plan = pkg.GroupedPlan(rows * 8, INTER, HIDDEN)
    one_plan.grouped_rows(xq, xs, table, ids, gate_only, None, 0, rows, False)
    up_only = torch.full_like(gate, float("nan"))
    one_plan.grouped_rows(xq, xs, table, ids, up_only, None, 1, rows, False)
    torch.cuda.synchronize()
    assert gu_plan.status() == 0 and one_plan.status() == 0
    assert torch.equal(gate.view(torch.int16), gate_only.view(torch.int16))       # one matrix alone = its half of the pair
    assert torch.equal(up.view(torch.int16), up_only.view(torch.int16))
    hidden_rows = torch.empty_like(gate)
    pkg.swiglu(gate, up, hidden_rows, gate.numel())
    hq, _, hs = _quantise_rows(torch, pkg, hidden_rows)
    down = torch.full((rows * 8, HIDDEN), float("nan"), dtype=torch.bfloat16, device="cuda")
    dn_plan = pkg.GroupedPlan(rows * 8, HIDDEN, INTER)
    dn_plan.grouped_rows(hq, hs, table, ids, down, None, 2, rows, True)
    routed = torch.empty((rows, HIDDEN), dtype=torch.bfloat16, device="cuda")
    pkg.expert_combine_rows(down, weights, routed, rows, 8, HIDDEN)
    torch.cuda.synchronize()
    assert dn_plan.status() == 0
    for plan in (gu_plan, one_plan, dn_plan):
        plan.close()
    return gate, up, down, routed


def _reference_serial(torch, orc, raw, ids, weights, x, rows):
    """The serial chain with the reference's own kernels: per (row, slot) software NVFP4 products."""
    ref = orc.ref()
    st = _stream(torch)
    xq = torch.empty((rows, HIDDEN // 2), dtype=torch.uint8, device="cuda")
    xs = torch.empty((rows, HIDDEN // 16), dtype=torch.uint8, device="cuda")
    assert ref.ref_nvfp4_quantize(x.data_ptr(), xq.data_ptr(), xs.data_ptr(), rows * HIDDEN, 1.0, st) == 0
    host_ids = ids.cpu().numpy().reshape(-1)
    alphas = raw.alpha.cpu().numpy()
    n = rows * 8
    gate = torch.empty((n, INTER), dtype=torch.bfloat16, device="cuda")
    up = torch.empty_like(gate)
    for a in range(n):
        e, r = int(host_ids[a]), a // 8
        for kind, dst in ((0, gate), (1, up)):
            assert ref.ref_nvfp4_gemv(xq[r].data_ptr(), raw.packed[e * 3 + kind].data_ptr(), xs[r].data_ptr(),
                                      raw.scales_linear[e * 3 + kind].data_ptr(), dst[a].data_ptr(), INTER, HIDDEN,
                                      float(alphas[e * 3 + kind]), st) == 0
    act = torch.empty_like(gate)
    assert ref.ref_swiglu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), n * INTER, st) == 0
    hq = torch.empty((n, INTER // 2), dtype=torch.uint8, device="cuda")
    hs = torch.empty((n, INTER // 16), dtype=torch.uint8, device="cuda")
    assert ref.ref_nvfp4_quantize(act.data_ptr(), hq.data_ptr(), hs.data_ptr(), n * INTER, 1.0, st) == 0
    down = torch.empty((n, HIDDEN), dtype=torch.bfloat16, device="cuda")
    for a in range(n):
        e = int(host_ids[a])
        assert ref.ref_nvfp4_gemv(hq[a].data_ptr(), raw.packed[e * 3 + 2].data_ptr(), hs[a].data_ptr(),
                                  raw.scales_linear[e * 3 + 2].data_ptr(), down[a].data_ptr(), HIDDEN, INTER,
                                  float(alphas[e * 3 + 2]), st) == 0
    routed = torch.empty((rows, HIDDEN), dtype=torch.bfloat16, device="cuda")
    assert ref.ref_expert_combine_rows(down.data_ptr(), weights.data_ptr(), routed.data_ptr(), rows, 8, HIDDEN, st) == 0
    torch.cuda.synchronize()
    return gate, up, down, routed


def _cosine(a, b):
    a, b = a.float().flatten().double(), b.float().flatten().double()
    return float((a @ b) / (a.norm() * b.norm()))


def test_grouped_dispatch_of_one_token_and_the_four_row_verifier_fixture(cuda, pkg, orc, layer0):
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    table = _device_table(torch, layer0.raw)
    x1 = synth.make_activations(901, 0, 1)
    ids1, w1 = _routed(torch, pkg, layer0, x1, 1)
    gate1, up1, down1, routed1 = _grouped_chain(torch, pkg, table, ids1, w1, x1, 1)
    # numerical gate against the serial chain (tests/moe_forward_test.cpp:286-304)
    r_gate, r_up, r_down, r_routed = _reference_serial(torch, orc, layer0.raw, ids1, w1, x1, 1)
    assert _cosine(gate1, r_gate) >= 0.9999 and _cosine(up1, r_up) >= 0.9999 and _cosine(down1, r_down) >= 0.9999
    assert _cosine(routed1, r_routed) >= 0.9999
    assert float((routed1.float() - r_routed.float()).abs().max()) <= 2e-2
    # M=4: the same token and the same ids four times; every row bit-equal to the M=1 result (:258-285)
    x4 = x1.repeat(4, 1).contiguous()
    ids4 = ids1.repeat(4, 1).contiguous()
    w4 = w1.repeat(4, 1).contiguous()
    gate4, up4, down4, routed4 = _grouped_chain(torch, pkg, table, ids4, w4, x4, 4)
    for row in range(4):
        assert torch.equal(routed4[row].view(torch.int16), routed1[0].view(torch.int16))
        assert torch.equal(gate4[row * 8:(row + 1) * 8].view(torch.int16), gate1.view(torch.int16))
        assert torch.equal(down4[row * 8:(row + 1) * 8].view(torch.int16), down1.view(torch.int16))


@pytest.mark.parametrize("rows", [1, 3, 4, 16])
def test_grouped_rows_on_distinct_tokens_equals_the_bank_based_stage_entry_points(cuda, pkg, orc, layer0, rows):
    """Weights read in place from the caller's table give the same numbers as the retiled bank; both against the
    reference's software product."""
    torch = cuda
    from p92moe_b200 import synth

    table = _device_table(torch, layer0.raw)
    x = synth.make_activations(902, rows, rows)
    ids, weights = _routed(torch, pkg, layer0, x, rows)
    gate, up, down, routed = _grouped_chain(torch, pkg, table, ids, weights, x, rows)
    plan = pkg.MoePlan(max_rows=rows)
    block = pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan)
    s_gate = torch.full_like(gate, float("nan"))
    s_up = torch.full_like(up, float("nan"))
    block.project_expert_gate_up(ids, x, s_gate, s_up, rows)
    act = torch.empty_like(gate)
    pkg.swiglu(s_gate, s_up, act, act.numel())
    s_down = torch.full_like(down, float("nan"))
    block.project_expert_down(ids, act, s_down, rows)
    torch.cuda.synchronize()
    assert plan.status() == 0
    assert torch.equal(gate.view(torch.int16), s_gate.view(torch.int16))
    assert torch.equal(up.view(torch.int16), s_up.view(torch.int16))
    assert torch.equal(down.view(torch.int16), s_down.view(torch.int16))
    if orc.have_ref() and rows <= 4:
        r_gate, r_up, r_down, r_routed = _reference_serial(torch, orc, layer0.raw, ids, weights, x, rows)
        assert _cosine(gate, r_gate) >= 0.9999 and _cosine(down, r_down) >= 0.9999 and _cosine(routed, r_routed) >= 0.9999
    plan.close()


@pytest.mark.parametrize("rows", [33, 64])
def test_stage_entry_points_at_prefill_block_sizes(cuda, pkg, orc, layer0, rows):
    """The reference's executor methods stop at four rows (include/p92/executor.h:61-62); the stand-ins take any row
    count the plan holds.  Checked against the whole-block call on the same rows: combine of the staged down rows +
    the shared expert's contribution must reproduce its output within the block tolerance."""
    torch = cuda
    from p92moe_b200 import synth

    x = synth.make_activations(903, rows, rows)
    ids, weights = _routed(torch, pkg, layer0, x, rows)
    plan = pkg.MoePlan(max_rows=rows)
    block = pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan)
    gate = torch.full((rows * 8, INTER), float("nan"), dtype=torch.bfloat16, device="cuda")
    up = torch.full_like(gate, float("nan"))
    block.project_expert_gate_up(ids, x, gate, up, rows)
    pkg.swiglu(gate, up, gate, gate.numel())
    down = torch.full((rows * 8, HIDDEN), float("nan"), dtype=torch.bfloat16, device="cuda")
    block.project_expert_down(ids, gate, down, rows)
    torch.cuda.synchronize()
    assert plan.status() == 0 and bool(torch.isfinite(down.float()).all())
    out = torch.empty_like(x)
    block.run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    views = plan.views(rows)
    assert torch.equal(views["expert_ids"], ids)
    mixed = views["mixed"][: rows * 8]                      # the whole-block call's per-assignment down rows
    assert torch.equal(mixed.view(torch.int16), down.view(torch.int16))
    plan.close()


def test_grouped_rows_rejects_what_the_reference_rejects(cuda, pkg, layer0):
    torch = cuda
    lib = pkg.load_library()
    table = _device_table(torch, layer0.raw)
    plan = pkg.GroupedPlan(32, INTER, HIDDEN)               # 2 rows x 16
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    ids = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.zeros((16, INTER), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.P92Error) as err:                # groups do not match batch_rows (cuda/nvfp4_grouped.cu:358)
        plan.grouped_rows(buf, buf, table, ids, out, out, 0, 4, False)
    assert err.value.code == 1
    with pytest.raises(pkg.P92Error):                       # a gate/up plan asked for the down matrix
        plan.grouped_rows(buf, buf, table, ids, out, None, 2, 4, True)
    with pytest.raises(pkg.P92Error):
        pkg.GroupedPlan(0, INTER, HIDDEN)
    handle = ctypes.c_void_p()
    assert lib.p92b_nvfp4_grouped_plan_create(ctypes.byref(handle), 16, 100, HIDDEN) == 1
    lib.p92b_nvfp4_grouped_plan_destroy(None)               # null-safe like the reference's destroy
    plan.close()
