"""The callers either side of the MoE block: the two RMSNorms around it (src/model.cpp:211-218,1210-1217) and the
dense SwiGLU MLP of layers 0-1 (src/model.cpp:1476-1484,1668-1675), against the reference's own kernels
(oracle/_ref) on the GPU and against the CPU restatement."""
import numpy as np
import pytest

from conftest import from_u16, u16

REL_L2 = 1e-2
MAX_ABS = 2e-2
EPS = 1.0e-5


def _stream(torch):
    return torch.cuda.current_stream().cuda_stream


def _rel(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)), float(np.abs(got - want).max())


def _norm_weight(torch, seed, n=2560):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.empty(n, dtype=torch.float32, device="cuda").normal_(1.0, 0.1, generator=g).to(torch.bfloat16)


# ------------------------------------------------------------------ CPU: the oracle's rmsnorm

def test_oracle_rmsnorm_matches_a_plain_float64_evaluation(orc):
    rng = np.random.default_rng(3)
    x = orc.f32_to_bf16(rng.standard_normal((5, 2560)).astype(np.float32) * 3.0)
    w = orc.f32_to_bf16((1.0 + 0.1 * rng.standard_normal(2560)).astype(np.float32))
    got = orc.bf16_to_f32(orc.rmsnorm(x, w, EPS)).astype(np.float64)
    xf, wf = orc.bf16_to_f32(x).astype(np.float64), orc.bf16_to_f32(w).astype(np.float64)
    want = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + EPS) * wf
    assert np.abs(got - want).max() <= 2.0 ** -8 * np.abs(want).max()          # one BF16 rounding of the result
    zero = orc.rmsnorm(np.zeros((1, 2560), np.uint16), w, EPS)
    assert not zero.any()


# ------------------------------------------------------------------ GPU

@pytest.mark.gpu
@pytest.mark.parametrize("rows,elements", [(1, 2560), (4, 2560), (64, 2560), (3, 1024), (2, 10240)])
def test_rmsnorm_operator_bit_exact_with_reference_kernel(cuda, pkg, orc, rows, elements):
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(rows * elements)
    x = (torch.empty((rows, elements), dtype=torch.float32, device="cuda").normal_(0, 2.0, generator=g)).to(torch.bfloat16)
    w = _norm_weight(torch, 11, elements)
    out = torch.empty_like(x)
    pkg.rmsnorm(x, w, out, rows, elements, EPS)
    # CPU restatement: equal up to the last BF16 place (hardware rsqrt and division approximations)
    want = orc.bf16_to_f32(orc.rmsnorm(u16(x), u16(w), EPS))
    got = orc.bf16_to_f32(u16(out))
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()
    assert (u16(out) != orc.rmsnorm(u16(x), u16(w), EPS)).mean() < 0.05
    if orc.have_ref() and hasattr(orc.ref(), "ref_rmsnorm"):
        ref_out = torch.empty_like(x)
        assert orc.ref().ref_rmsnorm(x.data_ptr(), w.data_ptr(), ref_out.data_ptr(), rows, elements, EPS, _stream(torch)) == 0
        assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16))        # bit-exact
    # in place
    y = x.clone()
    pkg.rmsnorm(y, w, y, rows, elements, EPS)
    assert torch.equal(y.view(torch.int16), out.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 3, 4, 8, 9, 16, 33])
@pytest.mark.parametrize("which", ["both", "pre", "post"])
def test_block_with_fused_norms_against_reference_chain(cuda, pkg, orc, layer0, rows, which):
    """rmsnorm(pre_mlp_norm) -> run_moe_rows -> rmsnorm(post_mlp_norm) in one call: the pre-normalised rows must be
    the reference operator's bit for bit (so the routing is the reference's), the result within the block tolerance."""
    torch = cuda
    if not (orc.have_ref() and hasattr(orc.ref(), "ref_rmsnorm")):
        pytest.skip("oracle/_ref with rmsnorm was not built")
    from p92moe_b200 import synth

    ref = orc.ref()
    mixed = (synth.make_activations(77, rows, rows).float() * 1.7 + 0.05).to(torch.bfloat16)
    pre_w = _norm_weight(torch, 21) if which in ("both", "pre") else None
    post_w = _norm_weight(torch, 22) if which in ("both", "post") else None
    plan = pkg.MoePlan(max_rows=max(rows, 4))
    block = pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan)
    out = torch.full_like(mixed, float("nan"))
    for _ in range(2):                                   # twice: the launch counters of the fused kernel move on
        block.run_moe_rows_normed(mixed, pre_w, post_w, out, rows, EPS)
    torch.cuda.synchronize()
    assert plan.status() == 0
    views = plan.views(rows)
    # reference chain
    normalized = mixed
    if pre_w is not None:
        normalized = torch.empty_like(mixed)
        assert ref.ref_rmsnorm(mixed.data_ptr(), pre_w.data_ptr(), normalized.data_ptr(), rows, 2560, EPS, _stream(torch)) == 0
    raw = layer0.raw
    hidden = torch.empty_like(mixed)
    ref_ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
    ref_w = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
    assert ref.ref_moe_forward_rows(normalized.data_ptr(), layer0.router_weight.data_ptr(), layer0.bias.data_ptr(),
                                    raw.packed.data_ptr(), raw.scales_linear.data_ptr(), raw.alpha.cpu().numpy(),
                                    raw.packed.shape[1], raw.scales_linear.shape[1], hidden.data_ptr(), rows, 2560, 1024,
                                    256, 2.5, None, ref_ids.data_ptr(), ref_w.data_ptr(), None, _stream(torch)) == 0
    want = hidden
    if post_w is not None:
        want = torch.empty_like(hidden)
        assert ref.ref_rmsnorm(hidden.data_ptr(), post_w.data_ptr(), want.data_ptr(), rows, 2560, EPS, _stream(torch)) == 0
    assert torch.equal(views["expert_ids"], ref_ids)               # same normalised rows -> same routing, bit for bit
    assert torch.equal(views["expert_weights"], ref_w)
    rel, max_abs = _rel(orc.bf16_to_f32(u16(out)), orc.bf16_to_f32(u16(want)))
    # the post-norm rescales rows of RMS ~0.03 to RMS ~1: the relative bar is the block's, the absolute one scales with it
    assert rel <= REL_L2, (rel, max_abs)
    scale = 1.0 if post_w is None else float(orc.bf16_to_f32(u16(want)).std() / max(orc.bf16_to_f32(u16(hidden)).std(), 1e-9))
    assert max_abs <= MAX_ABS * max(1.0, scale), (rel, max_abs, scale)
    # and the un-fused sequence of the same library calls gives the same bits
    seq_in = mixed
    if pre_w is not None:
        seq_in = torch.empty_like(mixed)
        pkg.rmsnorm(mixed, pre_w, seq_in, rows, 2560, EPS)
    seq = torch.empty_like(mixed)
    block.run_moe_rows(seq_in, seq, rows)
    if post_w is not None:
        pkg.rmsnorm(seq, post_w, seq, rows, 2560, EPS)
    assert torch.equal(seq.view(torch.int16), out.view(torch.int16))
    plan.close()


def _dense_layer(torch, pkg, seed, hidden=2560, inter=9216):
    """(bank, reference-format tensors) of one dense MLP drawn ~N(0,0.02) and quantised by the a12 law."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    tensors = []
    for kind in range(3):
        rows, cols = (inter, hidden) if kind < 2 else (hidden, inter)
        w = torch.empty((rows, cols), dtype=torch.float32, device="cuda").normal_(0, 0.02, generator=g).to(torch.bfloat16)
        packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device="cuda")
        linear = torch.empty((rows, cols // 16), dtype=torch.uint8, device="cuda")
        alpha = torch.empty(1, dtype=torch.float32, device="cuda")
        pkg.nvfp4_pack_weight(w, packed, linear, alpha)
        swizzled = torch.empty(pkg.nvfp4_swizzled_scale_bytes(rows, cols // 16), dtype=torch.uint8, device="cuda")
        pkg.nvfp4_swizzle_scales(linear, swizzled, rows, cols // 16)
        tensors.append((packed, linear, swizzled, alpha))
    bank = pkg.ExpertBank([(p, s, a) for p, _, s, a in tensors], first_expert=0, local_experts=0, hidden=hidden,
                          intermediate=inter)
    return bank, tensors


def _reference_dense(torch, orc, tensors, x, rows, hidden=2560, inter=9216):
    """run_dense_rows with the reference's kernels: quantise, software NVFP4 product per row, SwiGLU, again."""
    ref = orc.ref()
    st = _stream(torch)
    xq = torch.empty((rows, hidden // 2), dtype=torch.uint8, device="cuda")
    xs = torch.empty((rows, hidden // 16), dtype=torch.uint8, device="cuda")
    assert ref.ref_nvfp4_quantize(x.data_ptr(), xq.data_ptr(), xs.data_ptr(), rows * hidden, 1.0, st) == 0
    gate = torch.empty((rows, inter), dtype=torch.bfloat16, device="cuda")
    up = torch.empty_like(gate)
    for kind, dst in ((0, gate), (1, up)):
        packed, linear, _, alpha = tensors[kind]
        for r in range(rows):
            assert ref.ref_nvfp4_gemv(xq[r].data_ptr(), packed.data_ptr(), xs[r].data_ptr(), linear.data_ptr(),
                                      dst[r].data_ptr(), inter, hidden, float(alpha[0]), st) == 0
    assert ref.ref_swiglu(gate.data_ptr(), up.data_ptr(), gate.data_ptr(), rows * inter, st) == 0
    hq = torch.empty((rows, inter // 2), dtype=torch.uint8, device="cuda")
    hs = torch.empty((rows, inter // 16), dtype=torch.uint8, device="cuda")
    assert ref.ref_nvfp4_quantize(gate.data_ptr(), hq.data_ptr(), hs.data_ptr(), rows * inter, 1.0, st) == 0
    out = torch.empty((rows, hidden), dtype=torch.bfloat16, device="cuda")
    packed, linear, _, alpha = tensors[2]
    for r in range(rows):
        assert ref.ref_nvfp4_gemv(hq[r].data_ptr(), packed.data_ptr(), hs[r].data_ptr(), linear.data_ptr(),
                                  out[r].data_ptr(), hidden, inter, float(alpha[0]), st) == 0
    torch.cuda.synchronize()
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 4, 17, 64, 150])
def test_dense_mlp_against_reference_kernels(cuda, pkg, orc, rows):
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    bank, tensors = _dense_layer(torch, pkg, 31)
    plan = pkg.MoePlan(max_rows=rows, hidden=2560, intermediate=9216)
    x = synth.make_activations(78, rows, rows)
    out = torch.full_like(x, float("nan"))
    pkg.run_dense_rows(plan, bank, x, out, rows)
    pkg.run_dense_rows(plan, bank, x, out, rows)
    torch.cuda.synchronize()
    assert plan.status() == 0
    want = _reference_dense(torch, orc, tensors, x, rows)
    got = orc.bf16_to_f32(u16(out))
    assert np.isfinite(got).all()
    rel, max_abs = _rel(got, orc.bf16_to_f32(u16(want)))
    assert rel <= REL_L2 and max_abs <= MAX_ABS, (rel, max_abs)
    plan.close()
    bank.close()


@pytest.mark.gpu
def test_dense_entry_point_rejects_mismatched_shapes(cuda, pkg, layer0):
    torch = cuda
    plan = pkg.MoePlan(max_rows=4, hidden=2560, intermediate=9216)
    x = torch.zeros((4, 2560), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.P92Error) as err:
        pkg.run_dense_rows(plan, layer0.bank, x, x.clone(), 4)          # a 1024-wide expert bank with a 9216-wide plan
    assert err.value.code == 1
    plan.close()
