"""The expert-parallel block on REAL GPUs, one process per GPU: the fused small-batch kernel (exchanges by
peer stores inside the kernel) and the two NCCL orchestrations, each rank's output checked against the
single-GPU block run on all tokens at once.  Needs two or more GPUs; skipped otherwise."""
import os
import socket

import numpy as np
import pytest

import __graft_entry__ as entry


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def _worker(rank: int, world: int, port: int, schedule, result) -> None:
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg = entry.load_package()
    from p92moe_b200 import ep, synth

    layer = synth.make_layer(seed=11, layer=0, keep_raw=True)          # same seed: same bytes on every GPU
    entries = layer.raw.entries()
    first, local = ep.shard_range(rank, world)
    bank = pkg.ExpertBank(entries[first * 3:(first + local) * 3] + entries[256 * 3:], first_expert=first,
                          local_experts=local)
    rows_per_gpu = max(max(rows) for rows in schedule)
    window = ep.EpWindow(rank, world, rows_per_gpu)
    wide_rows = 24                                                    # a second window for the gathered path at a larger batch
    wide_window = ep.EpWindow(rank, world, wide_rows)
    wide_plan = pkg.MoePlan(max_rows=world * wide_rows)
    fused_plan = pkg.MoePlan(max_rows=world * rows_per_gpu)
    state = ep.EpRank(rank, world, bank, layer.router_weight, layer.bias, max_local_rows=rows_per_gpu)
    ok, worst = True, 0.0
    for call, rows in enumerate(schedule):
        xs = [synth.make_activations(900 + 16 * call + r, 0, n) for r, n in enumerate(rows)]
        x_all = torch.cat(xs).contiguous()
        total = x_all.shape[0]
        plan = pkg.MoePlan(max_rows=total)
        plan.set_path(2)
        want = torch.empty_like(x_all)
        pkg.MoeBlock(layer.bank, layer.router_weight, layer.bias, plan).run_moe_rows(x_all, want, total)
        torch.cuda.synchronize()
        at = sum(rows[:rank])
        mine, n = xs[rank], rows[rank]
        ref = want[at:at + n].float().cpu().numpy()
        ref_ids = plan.views(total)["expert_ids"][at:at + n]
        for kind in ("fused", "gathered", "fixed", "exact"):
            out = torch.full_like(mine, float("nan"))
            if kind == "fused":
                ep.forward_fused(window, fused_plan, bank, layer.router_weight, layer.bias, mine, out, n)
                torch.cuda.synchronize()
                ok &= int(fused_plan.views(n)["status"][0]) == 0
                ok &= bool(torch.equal(fused_plan.views(n)["expert_ids"], ref_ids))
            elif kind == "gathered":
                ep.forward_gathered(window, fused_plan, bank, layer.router_weight, layer.bias, mine, out, n)
                torch.cuda.synchronize()
                ok &= fused_plan.status() == 0
            elif kind == "fixed":
                ep.forward_nccl_fixed(state, mine, out, n, 8 * rows_per_gpu)
            else:
                ep.forward_nccl(state, mine, out, n)
            torch.cuda.synchronize()
            got = out.float().cpu().numpy()
            rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
            worst = max(worst, rel)
            ok &= bool(np.isfinite(got).all()) and rel <= 1e-2 and float(np.abs(got - ref).max()) <= 2e-2
    # the gathered path at 24 tokens per GPU, ragged: rank r brings 24 - r tokens
    for call in range(2):
        rows = [wide_rows - r for r in range(world)]
        xs = [synth.make_activations(1300 + 16 * call + r, 0, n) for r, n in enumerate(rows)]
        x_all = torch.cat(xs).contiguous()
        total = x_all.shape[0]
        plan = pkg.MoePlan(max_rows=total)
        plan.set_path(2)
        want = torch.empty_like(x_all)
        pkg.MoeBlock(layer.bank, layer.router_weight, layer.bias, plan).run_moe_rows(x_all, want, total)
        at, n = sum(rows[:rank]), rows[rank]
        out = torch.full_like(xs[rank], float("nan"))
        ep.forward_gathered(wide_window, wide_plan, bank, layer.router_weight, layer.bias, xs[rank], out, n)
        torch.cuda.synchronize()
        ok &= wide_plan.status() == 0
        got, ref = out.float().cpu().numpy(), want[at:at + n].float().cpu().numpy()
        rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
        worst = max(worst, rel)
        ok &= bool(np.isfinite(got).all()) and rel <= 1e-2 and float(np.abs(got - ref).max()) <= 2e-2
    # the large-batch path: 300 home tokens per GPU, then ragged (rank r brings 300 - 11 r)
    bulk_rows = 300
    bulk_window = ep.EpWindow(rank, world, bulk_rows, bulk=True)
    bulk_plan = pkg.MoePlan(max_rows=world * bulk_rows)
    for call in range(3):
        rows = [bulk_rows - (11 * r if call == 1 else 0) for r in range(world)]
        xs = [synth.make_activations(1700 + 16 * call + r, 0, n) for r, n in enumerate(rows)]
        x_all = torch.cat(xs).contiguous()
        total = x_all.shape[0]
        plan = pkg.MoePlan(max_rows=total)
        want = torch.empty_like(x_all)
        pkg.MoeBlock(layer.bank, layer.router_weight, layer.bias, plan).run_moe_rows(x_all, want, total)
        at, n = sum(rows[:rank]), rows[rank]
        out = torch.full_like(xs[rank], float("nan"))
        ep.forward_bulk(bulk_window, bulk_plan, bank, layer.router_weight, layer.bias, xs[rank], out, n)
        torch.cuda.synchronize()
        ok &= bulk_plan.status() == 0
        ok &= bool(torch.equal(bulk_plan.views(n)["expert_ids"], plan.views(total)["expert_ids"][at:at + n]))
        # per expert the rows are in the single-GPU order and the combine is the single-GPU law: the same bits
        ok &= bool(torch.equal(out.view(torch.int16), want[at:at + n].view(torch.int16)))
        plan.close()
    dist.barrier()
    torch.cuda.synchronize()
    window.close()
    wide_window.close()
    bulk_window.close()
    result[rank] = (bool(ok), worst)
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_on_real_gpus(world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    # home tokens per GPU, call by call: even, ragged, one token each
    schedule = [[4] * world, [(r % 4) + 1 for r in range(world)], [1] * world, [4] * world]
    port = _free_port()
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_worker, args=(world, port, schedule, result), nprocs=world, join=True)
        got = dict(result)
    assert all(got[r][0] for r in range(world)), got
