"""The allocation-free permutation entry point (p92b_moe_permute_static) against the plan-based one.

Collected last on purpose (file name), so that a run that stops at the first failure has already
run every other test.  Some hosts of the library cannot allocate device memory at call time - an
engine that gave the whole card to its own arena, a process that forbids further CUDA allocations,
a decode loop that must not meet an allocation's device-wide synchronisation - so this entry point
keeps its scratch in a fixed array inside the library instead of in a plan.  The test calls it
through the C ABI twice in a row with different inputs (the array keeps the previous call's
contents) and requires bit-identical results to p92b_moe_permute; sizes beyond the built-in limit
must be refused.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _make_ids(rows, seed, hot=None):
    rng = np.random.default_rng(seed)
    ids = np.argsort(rng.random((rows, 256)), axis=1)[:, :8].astype(np.int32)
    if hot is not None:
        ids[:, 0] = hot
    return ids


def _run_both(torch, pkg, lib, ids, orc=None):
    n = ids.size
    d_ids = torch.from_numpy(ids).cuda()
    stream = torch.cuda.current_stream().cuda_stream

    def buffers():
        return (torch.full((n,), -1, dtype=torch.int32, device="cuda"),
                torch.full((n,), -1, dtype=torch.int32, device="cuda"),
                torch.full((256,), -1, dtype=torch.int32, device="cuda"),
                torch.full((257,), -1, dtype=torch.int32, device="cuda"))

    got = buffers()
    code = lib.p92b_moe_permute_static(d_ids.data_ptr(), n, got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(),
                                       got[3].data_ptr(), stream)
    assert code == 0
    want = buffers()
    plan = pkg.MoePlan(max_rows=ids.shape[0])
    plan.permute(d_ids, *want)
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    plan.close()
    if orc is not None:
        # and against the CPU restatement of the reference's ranking law directly
        for g, w in zip(got, orc.permute(ids)):
            assert np.array_equal(g.cpu().numpy(), w)
    assert pkg.moe_permute_static_status() == 0
    return got


def test_static_permutation_matches_plan_based_entry_point_twice_in_a_row(cuda, pkg, orc):
    torch = cuda
    lib = pkg.load_library()
    # multi-block path (uses the built-in histogram scratch), then a different, smaller multi-block
    # case whose chunks are a subset of the first call's: stale histograms must not leak
    first = _run_both(torch, pkg, lib, _make_ids(4096, seed=1), orc)
    second = _run_both(torch, pkg, lib, _make_ids(1500, seed=2, hot=200), orc)
    assert first[0].numel() == 4096 * 8 and second[0].numel() == 1500 * 8
    # single-block path and the largest size the array serves
    _run_both(torch, pkg, lib, _make_ids(5, seed=3), orc)
    _run_both(torch, pkg, lib, _make_ids(8192, seed=4), orc)


@pytest.mark.parametrize("rows", [6, 2000])
def test_static_permutation_reports_an_out_of_range_id_and_accepts_null_outputs(cuda, pkg, orc, rows):
    """An id outside 0..255 is counted as expert 0 / 255 (no fault) and leaves 1 in the status word,
    which the accessor copies out; the next clean call reads 0 again.  order and position are optional."""
    torch = cuda
    lib = pkg.load_library()
    ids = _make_ids(rows, seed=10 + rows)
    bad = ids.copy()
    bad[rows // 2, 3] = 256
    stream = torch.cuda.current_stream().cuda_stream
    for case, expect in ((bad, 1), (ids, 0)):
        d_ids = torch.from_numpy(case).cuda()
        counts = torch.full((256,), -1, dtype=torch.int32, device="cuda")
        offsets = torch.full((257,), -1, dtype=torch.int32, device="cuda")
        assert lib.p92b_moe_permute_static(d_ids.data_ptr(), case.size, None, None, counts.data_ptr(), offsets.data_ptr(),
                                           stream) == 0
        assert pkg.moe_permute_static_status() == expect
        clamped = np.minimum(case, 255)
        _, _, o_counts, o_offsets = orc.permute(clamped)
        assert np.array_equal(counts.cpu().numpy(), o_counts)
        assert np.array_equal(offsets.cpu().numpy(), o_offsets)


def test_static_permutation_rejects_sizes_beyond_the_built_in_scratch(cuda, pkg):
    torch = cuda
    lib = pkg.load_library()
    n = pkg.STATIC_PERMUTE_MAX_ASSIGNMENTS + 8
    ids = torch.zeros(n, dtype=torch.int32, device="cuda")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    counts = torch.full((256,), -7, dtype=torch.int32, device="cuda")
    offsets = torch.empty(257, dtype=torch.int32, device="cuda")
    code = lib.p92b_moe_permute_static(ids.data_ptr(), n, out.data_ptr(), out.data_ptr(), counts.data_ptr(),
                                       offsets.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == 1                                   # cudaErrorInvalidValue
    torch.cuda.synchronize()
    assert int(counts[0]) == -7                        # nothing was launched
    with pytest.raises(pkg.P92Error):
        pkg.moe_permute_static(ids, out, out, counts, offsets)
