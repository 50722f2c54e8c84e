"""Expert parallelism.  CPU: the host-side exchange logic over gloo with two processes.  GPU: all
ranks emulated in one process on one GPU (same device code as the NCCL path) against the
single-GPU block."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    entry.load_package()
    from p92moe_b200 import ep

    local = 256 // world
    rng = np.random.default_rng(100 + rank)
    rows = 5 + rank * 3
    ids = np.stack([rng.choice(256, 8, replace=False) for _ in range(rows)]).astype(np.int32).reshape(-1)
    order = np.argsort(ids, kind="stable")                       # the stable permutation by expert id
    counts = np.bincount(ids, minlength=256).astype(np.int32)
    # a row is tagged (home rank, flat index, expert) so its journey can be checked
    send = torch.tensor([[rank, int(i), int(ids[i])] for i in order], dtype=torch.int32)
    counts_by_dst = torch.from_numpy(counts).view(world, local).contiguous()
    assert ep.split_sizes(counts.tolist(), world) == counts_by_dst.sum(dim=1).tolist()
    recv, recv_counts, send_sizes, recv_sizes = ep.exchange_dispatch(send, counts_by_dst)
    first, n_local = ep.shard_range(rank, world)
    ok = True
    # arrivals: runs by source, inside a run experts ascending and flat index ascending per expert
    at = 0
    for s in range(world):
        run = recv[at:at + recv_sizes[s]]
        at += recv_sizes[s]
        ok &= bool((run[:, 0] == s).all())
        ok &= bool(((run[:, 2] >= first) & (run[:, 2] < first + n_local)).all())
        keys = (run[:, 2].long() * 100000 + run[:, 1].long()).tolist()
        ok &= keys == sorted(keys)
        ok &= recv_counts[s].tolist() == np.bincount(run[:, 2].numpy() - first, minlength=n_local).tolist()
    # per expert, concatenating the sources' runs gives the global stable order (home rank, flat)
    for e in range(first, first + n_local):
        rows_e = recv[recv[:, 2] == e]
        keys = (rows_e[:, 0].long() * 100000 + rows_e[:, 1].long()).tolist()
        ok &= keys == sorted(keys)
    back = ep.exchange_return(recv * 2, send_sizes, recv_sizes)
    ok &= bool(torch.equal(back, send * 2))                      # every row returns to its slot
    result[rank] = ok
    dist.destroy_process_group()


def test_exchange_logic_over_gloo_two_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_gloo_worker, args=(world, port, result), nprocs=world, join=True)
        assert dict(result) == {0: True, 1: True}


def test_shard_ranges():
    entry.load_package()
    from p92moe_b200 import ep

    assert [ep.shard_range(r, 8) for r in (0, 7)] == [(0, 32), (224, 32)]
    assert ep.shard_range(1, 2) == (128, 128) and ep.shard_range(3, 4) == (192, 64)
    with pytest.raises(ValueError):
        ep.shard_range(0, 3)


@pytest.mark.gpu
@pytest.mark.parametrize("exchange", ["exact", "fixed"])
@pytest.mark.parametrize("world,rows", [(2, [5, 3]), (4, [2, 7, 4, 3]), (8, [4] * 8), (2, [130, 70]), (4, [1, 1, 1, 1])])
def test_expert_parallel_block_matches_single_gpu(cuda, pkg, layer0, world, rows, exchange):
    torch = cuda
    from p92moe_b200 import ep, synth

    raw = layer0.raw
    entries = raw.entries()
    xs = [synth.make_activations(500 + r, 0, n) for r, n in enumerate(rows)]
    states = []
    for r in range(world):
        first, local = ep.shard_range(r, world)
        shard = entries[first * 3:(first + local) * 3] + entries[256 * 3:]
        bank = pkg.ExpertBank(shard, first_expert=first, local_experts=local)
        states.append(ep.EpRank(r, world, bank, layer0.router_weight, layer0.bias, max_local_rows=max(rows),
                                max_arrival_rows=world * max(rows)))
    outs = [torch.full_like(x, float("nan")) for x in xs]
    if exchange == "exact":
        ep.forward_emulated(states, xs, outs, rows)
    else:
        ep.forward_emulated_fixed(states, xs, outs, rows)
    # single GPU on all tokens at once
    x_all = torch.cat(xs).contiguous()
    total = x_all.shape[0]
    plan = pkg.MoePlan(max_rows=total)
    plan.set_path(2)
    want = torch.empty_like(x_all)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan).run_moe_rows(x_all, want, total)
    torch.cuda.synchronize()
    ids_all = plan.views(total)["expert_ids"]
    at = 0
    for r, n in enumerate(rows):
        v = states[r].home.views(n)
        assert torch.equal(v["expert_ids"], ids_all[at:at + n])              # routing is per token: identical ids
        got = outs[r].float().cpu().numpy()
        ref = want[at:at + n].float().cpu().numpy()
        assert np.isfinite(got).all()
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 1e-2 and np.abs(got - ref).max() <= 2e-2, (r, rel)
        at += n


# ---- fused small-batch kernel: exchanges inside the kernel -----------------------------------------

def _single_gpu_reference(pkg, layer0, x, rows):
    plan = pkg.MoePlan(max_rows=max(rows, 1))
    plan.set_path(2)
    want = x.new_empty(x.shape)
    pkg.MoeBlock(layer0.bank, layer0.router_weight, layer0.bias, plan).run_moe_rows(x, want, rows)
    import torch
    torch.cuda.synchronize()
    return want, plan.views(rows)


@pytest.mark.gpu
@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("rows", [1, 2, 4, 5, 8])
def test_fused_kernel_world_one_matches_block(cuda, pkg, layer0, rows, wide, monkeypatch):
    """One GPU owning all experts: the fused kernel's gather, routing lists, tiles, direct placement
    and combine all run (to and from its own window), both token widths, several calls in a row so
    that both halves of the double-buffered window are used."""
    torch = cuda
    from p92moe_b200 import ep, synth

    if wide:
        monkeypatch.setenv("P92B_EP_WIDE", "1")
    window = ep.EpWindow(0, 1, 8)
    plan = pkg.MoePlan(max_rows=32)
    try:
        for call in range(3):
            x = synth.make_activations(700 + call, 0, rows)
            out = torch.full_like(x, float("nan"))
            ep.forward_fused(window, plan, layer0.bank, layer0.router_weight, layer0.bias, x, out, rows)
            torch.cuda.synchronize()
            v = plan.views(rows)
            assert int(v["status"][0]) == 0
            want, ref = _single_gpu_reference(pkg, layer0, x, rows)
            assert torch.equal(v["expert_ids"], ref["expert_ids"])
            assert torch.equal(v["expert_weights"], ref["expert_weights"])
            assert torch.equal(v["counts"][:256], ref["counts"][:256])
            got, exp = out.float().cpu().numpy(), want.float().cpu().numpy()
            assert np.isfinite(got).all()
            rel = np.linalg.norm(got - exp) / np.linalg.norm(exp)
            assert rel <= 1e-2 and np.abs(got - exp).max() <= 2e-2, (call, rel)
    finally:
        window.close()


@pytest.mark.gpu
def test_fused_kernel_gives_up_when_a_peer_never_arrives(cuda, pkg, layer0):
    """Two windows in this process, only rank 0 launches: its wait for rank 1's flag runs out after
    about a second, the kernel returns, the status word says so and the context stays usable."""
    torch = cuda
    from p92moe_b200 import ep, synth

    windows = [ep.EpWindow(r, 2, 4, connect=False) for r in range(2)]
    ep.EpWindow.connect_local(windows)
    entries = layer0.raw.entries()
    bank = pkg.ExpertBank(entries[:128 * 3] + entries[256 * 3:], first_expert=0, local_experts=128)
    plan = pkg.MoePlan(max_rows=8)
    x = synth.make_activations(720, 0, 4)
    out = torch.zeros_like(x)
    try:
        ep.forward_fused(windows[0], plan, bank, layer0.router_weight, layer0.bias, x, out, 4)
        torch.cuda.synchronize()
        assert int(plan.views(4)["status"][0]) == 2
        assert float((x.float() * 2).sum().cpu()) == float(x.float().sum().cpu()) * 2     # the GPU still answers
    finally:
        for w in windows:
            w.close()


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 4, 33, 100, 300])
def test_gathered_path_world_one_matches_block(cuda, pkg, layer0, rows):
    """One GPU owning all experts: push into its own window, permutation law over the batch, grouped
    tcgen05 products, result rows placed through the window, combine; both window parities."""
    torch = cuda
    from p92moe_b200 import ep, synth

    window = ep.EpWindow(0, 1, 512)
    plan = pkg.MoePlan(max_rows=512)
    try:
        for call in range(3):
            x = synth.make_activations(740 + call, 0, rows)
            out = torch.full_like(x, float("nan"))
            ep.forward_gathered(window, plan, layer0.bank, layer0.router_weight, layer0.bias, x, out, rows)
            torch.cuda.synchronize()
            v = plan.views(rows)
            assert int(v["status"][0]) == 0
            want, ref = _single_gpu_reference(pkg, layer0, x, rows)
            assert torch.equal(v["expert_ids"], ref["expert_ids"])
            assert torch.equal(v["expert_weights"], ref["expert_weights"])
            got, exp = out.float().cpu().numpy(), want.float().cpu().numpy()
            assert np.isfinite(got).all()
            rel = np.linalg.norm(got - exp) / np.linalg.norm(exp)
            assert rel <= 1e-2 and np.abs(got - exp).max() <= 2e-2, (call, rel)
    finally:
        window.close()


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [40, 700, 2048])
def test_bulk_path_world_one_matches_block(cuda, pkg, layer0, rows):
    """One GPU owning all experts: rows and ids stored into its own window, flags, the permutation restricted to the
    local range (here everything), grouped products, result rows placed through the window, combine.  Fewer rows
    than the window holds on the second call (empty slots carry id -1 and are skipped)."""
    torch = cuda
    from p92moe_b200 import ep, synth

    window = ep.EpWindow(0, 1, rows, bulk=True)
    plan = pkg.MoePlan(max_rows=rows)
    try:
        for call, n in enumerate((rows, rows - 7, rows)):
            x = synth.make_activations(760 + call, 0, n)
            out = torch.full_like(x, float("nan"))
            ep.forward_bulk(window, plan, layer0.bank, layer0.router_weight, layer0.bias, x, out, n)
            torch.cuda.synchronize()
            assert plan.status() == 0
            want, ref = _single_gpu_reference(pkg, layer0, x, n)
            v = plan.views(n)
            assert torch.equal(v["expert_ids"], ref["expert_ids"])
            assert torch.equal(v["expert_weights"], ref["expert_weights"])
            assert torch.equal(v["counts"], ref["counts"])
            # same kernels, same per-expert row order, same combine law: the same bits
            assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    finally:
        window.close()


@pytest.mark.gpu
def test_other_calls_refuse_a_bulk_window(cuda, pkg, layer0):
    torch = cuda
    from p92moe_b200 import ep, synth

    window = ep.EpWindow(0, 1, 8, bulk=True)
    plan = pkg.MoePlan(max_rows=8)
    x = synth.make_activations(770, 0, 4)
    out = torch.zeros_like(x)
    try:
        for call in (ep.forward_fused, ep.forward_gathered):
            with pytest.raises(pkg.P92Error) as err:
                call(window, plan, layer0.bank, layer0.router_weight, layer0.bias, x, out, 4)
            assert err.value.code == 801
    finally:
        window.close()
