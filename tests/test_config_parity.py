"""Parity at the sizes of the benchmark configurations, against the reference's own kernels.

A token's output depends on nothing but its own routing and its own row, so the reference chain
(oracle/_ref: cuda/nvfp4_ops.cu compiled unmodified, driven in run_moe_rows order) can check any subset
of a large batch exactly: router logits, expert ids and route weights are compared on EVERY row, the
permutation against the CPU restatement of the ranking law, and the output rows of a sample that is
chosen to cover the hottest expert (many 128-row tiles), an expert with 129..256 rows (the two-half
items of the paired gate/up kernel), an expert with a single row, and random tokens.
tests/moe_forward_test.cpp:143-157,286-304 are the gates this follows.
"""
import numpy as np
import pytest

from conftest import u16

pytestmark = pytest.mark.gpu

REL_L2 = 1e-2
MAX_ABS = 2e-2
FAST_ROUTER_ROWS = 9         # from this batch size on the block takes tensor-core logits with exact repair


def _stream(torch):
    return torch.cuda.current_stream().cuda_stream


def _rel(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)), float(np.abs(got - want).max())


def _reference_rows(torch, orc, layer0, bias, x_rows):
    """ref_moe_forward_rows on a subset of token rows (at least two, so the T>1 logits order applies)."""
    raw = layer0.raw
    n = x_rows.shape[0]
    assert n >= 2
    out = torch.empty_like(x_rows)
    ids = torch.empty((n, 8), dtype=torch.int32, device="cuda")
    weights = torch.empty((n, 8), dtype=torch.float32, device="cuda")
    code = orc.ref().ref_moe_forward_rows(x_rows.data_ptr(), layer0.router_weight.data_ptr(), bias.data_ptr(),
                                          raw.packed.data_ptr(), raw.scales_linear.data_ptr(), raw.alpha.cpu().numpy(),
                                          raw.packed.shape[1], raw.scales_linear.shape[1], out.data_ptr(), n, 2560, 1024,
                                          256, 2.5, None, ids.data_ptr(), weights.data_ptr(), None, _stream(torch))
    assert code == 0
    return out, ids, weights


def _sample_tokens(ids, counts, how_many, seed):
    """Tokens of the hottest expert (first, middle, last of its rows), of one expert with 129..256 rows
    if there is one, of the smallest non-empty expert, and random ones."""
    rng = np.random.default_rng(seed)
    picked = []

    def tokens_of(expert):
        return np.nonzero((ids == expert).any(axis=1))[0]

    hot = int(np.argmax(counts))
    t = tokens_of(hot)
    picked += [int(t[0]), int(t[len(t) // 2]), int(t[-1])] + [int(v) for v in rng.choice(t, min(12, len(t)), replace=False)]
    mid = np.nonzero((counts >= 129) & (counts <= 256))[0]
    if len(mid):
        t = tokens_of(int(mid[0]))
        picked += [int(t[0]), int(t[63 if len(t) > 63 else -1]), int(t[64 if len(t) > 64 else -1]), int(t[128]), int(t[-1])]
    small = np.where(counts > 0, counts, 1 << 30)
    picked += [int(v) for v in tokens_of(int(np.argmin(small)))[:4]]
    picked += [int(v) for v in rng.choice(ids.shape[0], how_many, replace=False)]
    return np.array(sorted(set(picked))[:max(how_many, 64) + 32], dtype=np.int64)


def _check_block_against_reference(torch, pkg, orc, layer0, bias, x, out, views, rows, seed, samples=64):
    # every row: logits, ids, weights bit-equal to the reference kernels
    ref_logits = torch.empty((rows, 256), dtype=torch.float32, device="cuda")
    assert orc.ref().ref_bf16_gemm_f32(x.data_ptr(), layer0.router_weight.data_ptr(), ref_logits.data_ptr(), rows, 256,
                                       2560, _stream(torch)) == 0
    if rows < FAST_ROUTER_ROWS:
        assert torch.equal(views["logits"], ref_logits)
    ref_ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
    ref_w = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
    assert orc.ref().ref_router_top8_rows(ref_logits.data_ptr(), bias.data_ptr(), ref_ids.data_ptr(), ref_w.data_ptr(),
                                          rows, 2.5, _stream(torch)) == 0
    assert torch.equal(views["expert_ids"], ref_ids)
    assert torch.equal(views["expert_weights"], ref_w)
    if rows >= FAST_ROUTER_ROWS:
        # larger batches: tensor-core logits, exact only where they can decide the routing.  The selected experts' logits
        # are the reference's bit for bit; everywhere else the deviation must stay far (8x) inside the bound the repair
        # assumes, 2^-14 * ||x|| * ||w|| (about 3e-3 here)
        picked = ref_ids.long()
        assert torch.equal(torch.gather(views["logits"], 1, picked), torch.gather(ref_logits, 1, picked))
        x_norm = x.float().norm(dim=1, keepdim=True)
        w_norm = layer0.router_weight.float().norm(dim=1)[None, :]
        ratio = ((views["logits"] - ref_logits).abs() / (x_norm * w_norm * 2.0 ** -14)).max()
        stats = views["router_stats"].cpu().numpy()
        print(f"rows {rows}: max |approximate - exact| / bound = {float(ratio):.4f}; exactly recomputed logits so far "
              f"{int(stats[0])} ({int(stats[0]) / rows:.2f} per token if one call), whole rows {int(stats[1])}")
        assert float(ratio) <= 0.125
    ids = ref_ids.cpu().numpy()
    # router invariants of tests/moe_forward_test.cpp:143-157 on every row
    assert (np.sort(ids, axis=1)[:, 1:] != np.sort(ids, axis=1)[:, :-1]).all() and ids.min() >= 0 and ids.max() < 256
    w = ref_w.cpu().numpy()
    assert (w > 0).all() and np.abs(w.sum(axis=1) - 2.5).max() <= 1e-5
    # permutation: the ranking law over the whole batch
    o_order, o_pos, o_counts, o_offsets = orc.permute(ids)
    assert np.array_equal(views["order"].cpu().numpy(), o_order)
    assert np.array_equal(views["position"].cpu().numpy(), o_pos)
    assert np.array_equal(views["counts"].cpu().numpy(), o_counts)
    assert np.array_equal(views["offsets"].cpu().numpy(), o_offsets)
    # sampled rows: whole block through the reference's kernels
    sample = _sample_tokens(ids, o_counts, samples, seed)
    index = torch.from_numpy(sample).cuda()
    want, s_ids, _ = _reference_rows(torch, orc, layer0, bias, x[index].contiguous())
    assert torch.equal(s_ids, ref_ids[index])
    got = out[index]
    assert bool(torch.isfinite(out.float()).all())
    rel, max_abs = _rel(orc.bf16_to_f32(u16(got)), orc.bf16_to_f32(u16(want)))
    assert rel <= REL_L2 and max_abs <= MAX_ABS, (rel, max_abs)
    worst = max(_rel(orc.bf16_to_f32(u16(got[i:i + 1])), orc.bf16_to_f32(u16(want[i:i + 1])))[0] for i in range(len(sample)))
    assert worst <= 2 * REL_L2, worst                       # no single row hides behind the aggregate
    return o_counts, len(sample)


def test_prefill_4096_zipf_against_reference_kernels(cuda, pkg, orc, layer0):
    """Config 2: T=4096, Zipf(1.2) routing, the multi-kernel tcgen05 pipeline."""
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    rows = 4096
    bias, achieved = synth.fit_zipf_bias(layer0.router_weight, 1.2, 4242)
    bias = bias.contiguous()
    x = synth.make_activations(4242, 1, rows)
    out = torch.full_like(x, float("nan"))
    plan = pkg.MoePlan(max_rows=rows)
    plan.set_path(2)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, bias, plan).run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    views = plan.views(rows)
    assert int(views["status"][0]) == 0
    counts, n = _check_block_against_reference(torch, pkg, orc, layer0, bias, x, out, views, rows, seed=1)
    assert counts.max() > 1024 and n >= 64                  # the skew is real: an expert with many token tiles
    assert ((counts >= 129) & (counts <= 256)).any()
    plan.close()


def test_prefill_16384_uniform_against_reference_kernels(cuda, pkg, orc, layer0):
    """Config 3's batch on one GPU: T=16384, zero bias."""
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    rows = 16384
    bias = torch.zeros(256, dtype=torch.float32, device="cuda")
    x = synth.make_activations(4243, 1, rows)
    out = torch.full_like(x, float("nan"))
    plan = pkg.MoePlan(max_rows=rows)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, bias, plan).run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    views = plan.views(rows)
    assert int(views["status"][0]) == 0
    _check_block_against_reference(torch, pkg, orc, layer0, bias, x, out, views, rows, seed=2)
    plan.close()


@pytest.mark.parametrize("rows", [64, 512])
def test_block_of_64_and_512_rows_against_reference_kernels(cuda, pkg, orc, layer0, rows):
    """64 rows is the reference's prefill block (kMaximumBlockRows, src/model.cpp:53,257-271); 512 is the
    serving-decode batch of config 4 on one GPU."""
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    x = synth.make_activations(4244, rows, rows)
    out = torch.full_like(x, float("nan"))
    plan = pkg.MoePlan(max_rows=rows)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan).run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    views = plan.views(rows)
    assert int(views["status"][0]) == 0
    _check_block_against_reference(torch, pkg, orc, layer0, layer0.bias, x, out, views, rows, seed=3, samples=min(rows, 64))
    plan.close()


@pytest.mark.parametrize("rows", [9, 10, 17, 31, 32, 33, 100, 255, 256, 257, 300])
def test_router_either_side_of_the_small_batch_switch(cuda, pkg, orc, layer0, rows):
    """The tensor-core router runs in two forms: up to 256 rows K is split over blocks and a block of eight warps
    repairs one token; above, one warp per token.  Ids and route weights of every row must be the reference
    kernels' bits in both (cuda/nvfp4_ops.cu:178-207,357-433), also with a bias that crowds the scores."""
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import synth

    for seed, bias in ((4300 + rows, layer0.bias), (4400 + rows, torch.zeros_like(layer0.bias))):
        x = synth.make_activations(seed, rows, rows)
        out = torch.empty_like(x)
        plan = pkg.MoePlan(max_rows=rows)
        plan.set_path(2)
        pkg.MoeBlock(layer0.bank, layer0.router_weight, bias, plan).run_moe_rows(x, out, rows)
        torch.cuda.synchronize()
        views = plan.views(rows)
        assert int(views["status"][0]) == 0
        _, ref_ids, ref_w = _reference_rows(torch, orc, layer0, bias, x)
        assert torch.equal(views["expert_ids"], ref_ids)
        assert torch.equal(views["expert_weights"], ref_w)
        plan.close()


def test_gathered_exchange_path_300_rows_against_reference_kernels(cuda, pkg, orc, layer0):
    """The multi-kernel expert-parallel path (one GPU owning all experts): its own routing lists, the window
    round trip and the grouped products, checked against the reference chain on sampled rows."""
    torch = cuda
    if not orc.have_ref():
        pytest.skip("oracle/_ref was not built")
    from p92moe_b200 import ep, synth

    rows = 300
    window = ep.EpWindow(0, 1, 512)
    plan = pkg.MoePlan(max_rows=512)
    try:
        x = synth.make_activations(4245, 0, rows)
        out = torch.full_like(x, float("nan"))
        ep.forward_gathered(window, plan, layer0.bank, layer0.router_weight, layer0.bias, x, out, rows)
        torch.cuda.synchronize()
        assert plan.status() == 0
        ref_ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
        sample = np.unique(np.random.default_rng(4).choice(rows, 64, replace=False))
        index = torch.from_numpy(sample).cuda()
        want, s_ids, s_w = _reference_rows(torch, orc, layer0, layer0.bias, x[index].contiguous())
        v = plan.views(rows)
        assert torch.equal(v["expert_ids"][index], s_ids) and torch.equal(v["expert_weights"][index], s_w)
        rel, max_abs = _rel(orc.bf16_to_f32(u16(out[index])), orc.bf16_to_f32(u16(want)))
        assert rel <= REL_L2 and max_abs <= MAX_ABS, (rel, max_abs)
        del ref_ids
    finally:
        window.close()


def test_device_combine_law_against_the_host_scheduled_law_at_33_rows(cuda, pkg, orc, layer0, layer0_host):
    """Above four rows the reference combines on the host-scheduled branch: BF16 read-modify-write per expert
    in ascending expert id (src/model.cpp:1509-1563, cuda/nvfp4_ops.cu:616-632), while this library keeps the
    device law (FP32 in slot order, one rounding, cuda/nvfp4_ops.cu:124-142) at every size.  Both laws are in
    the CPU oracle; the gap between them, and between the library and the host law, stays inside the block
    tolerance - equality with the reference at prefill sizes is tolerance-level by construction."""
    torch = cuda
    from p92moe_b200 import synth

    rows = 33
    x = synth.make_activations(4246, 0, rows)
    out = torch.empty_like(x)
    plan = pkg.MoePlan(max_rows=rows)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan).run_moe_rows(x, out, rows)
    torch.cuda.synchronize()
    host = layer0_host
    laws = {}
    for name, flag in (("device", False), ("host", True)):
        laws[name] = orc.bf16_to_f32(orc.moe_forward(u16(x), host["router"], host["bias"], host["packed"], host["scales"],
                                                     host["alpha"], pkg.HIDDEN, pkg.INTERMEDIATE, host_law=flag))
    got = orc.bf16_to_f32(u16(out))
    _, _, margin = orc.router_top8(orc.router_logits(u16(x), host["router"]), host["bias"])
    safe = margin > 2e-6
    gap_laws = _rel(laws["host"][safe], laws["device"][safe])
    gap_library = _rel(got[safe], laws["host"][safe])
    print(f"host law vs device law: rel_l2={gap_laws[0]:.3e} max_abs={gap_laws[1]:.3e}; "
          f"library vs host law: rel_l2={gap_library[0]:.3e} max_abs={gap_library[1]:.3e}")
    assert gap_laws[0] <= REL_L2 and gap_laws[1] <= MAX_ABS
    assert gap_library[0] <= REL_L2 and gap_library[1] <= MAX_ABS
    plan.close()
