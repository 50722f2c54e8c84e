"""Expert-parallel MoE block: host orchestration of the two all-to-all exchanges.

256 routed experts are sharded contiguously over G GPUs (128 / 64 / 32 per GPU at G = 2 / 4 / 8);
router weight, correction bias and the shared expert are replicated; every GPU is home to its own
tokens.  One process per GPU; the exchanges are NCCL all-to-alls issued through torch.distributed,
everything else is the C ABI (p92b_ep_route / p92b_ep_experts / p92b_ep_combine).

The reference has no expert parallelism (its CUDA backend is one device and one stream,
src/executor.cpp:20-23); the contract kept here is its single-device one: per expert, rows are
ordered by global flat index (home GPU, token, slot), so the permutation restricted to a GPU's
experts is what one GPU would compute, and the combine is the device law in slot order.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import (EXPERTS, HIDDEN, INTERMEDIATE, ROUTED_SCALE, TOP_K, ExpertBank, MoePlan, _check, _ptr, _stream,
               load_library)

ROW_BYTES = HIDDEN // 2 + HIDDEN // 16


def shard_range(rank: int, world: int, experts: int = EXPERTS) -> tuple:
    """[first, first + count) of the experts GPU `rank` owns."""
    if experts % world != 0:
        raise ValueError("world size must divide the expert count")
    per = experts // world
    return rank * per, per


def split_sizes(counts: Sequence[int], world: int) -> List[int]:
    """Rows this GPU sends to each destination, from its per-expert histogram."""
    per = len(counts) // world
    return [int(sum(counts[d * per:(d + 1) * per])) for d in range(world)]


class EpRank:
    """One GPU's share: its expert shard, two plans (arrivals; home tokens + shared expert)."""

    def __init__(self, rank: int, world: int, bank: ExpertBank, router_weight, correction_bias,
                 max_local_rows: int, max_arrival_rows: Optional[int] = None, routed_scale: float = ROUTED_SCALE,
                 share_scratch_with: Optional["EpRank"] = None):
        self.rank, self.world = rank, world
        self.first, self.local = shard_range(rank, world)
        if bank.first_expert != self.first or bank.local_experts != self.local:
            raise ValueError("bank does not hold this rank's expert shard")
        self.bank, self.router_weight, self.bias, self.routed_scale = bank, router_weight, correction_bias, routed_scale
        # worst case every assignment of every GPU lands here
        arrival_rows = max_arrival_rows if max_arrival_rows is not None else max_local_rows * world
        self.max_local_rows = max_local_rows
        if share_scratch_with is not None:
            # layers of one rank run one after the other on one stream: they can use the same plans and buffers
            other = share_scratch_with
            if other.max_local_rows < max_local_rows or other.arrivals.max_rows < arrival_rows:
                raise ValueError("the scratch to share is too small")
            self.home, self.shared, self.arrivals = other.home, other.shared, other.arrivals
            self.send, self._fixed = other.send, other._fixed
            return
        self.home = MoePlan(max_rows=max_local_rows)
        self.shared = MoePlan(max_rows=max_local_rows)
        self.arrivals = MoePlan(max_rows=arrival_rows)
        self.send = torch.empty((max_local_rows * TOP_K, ROW_BYTES), dtype=torch.uint8, device="cuda")
        self._fixed = {}

    # ---- fixed-capacity exchange buffers (small batches) -----------------------------------
    def fixed_buffers(self, cap_rows: int):
        """(send blocks, receive blocks, outgoing result slots, returned result slots) for `cap_rows`
        row slots per (source, destination) pair; allocated once per capacity."""
        if cap_rows not in self._fixed:
            if cap_rows * self.world > self.arrivals.max_rows * TOP_K:
                raise ValueError("arrival plan too small for this capacity")
            block = load_library().p92b_ep_fixed_block_bytes(HIDDEN, self.local, cap_rows)
            self._fixed[cap_rows] = (
                torch.zeros((self.world, block), dtype=torch.uint8, device="cuda"),
                torch.zeros((self.world, block), dtype=torch.uint8, device="cuda"),
                torch.zeros((self.world, cap_rows, HIDDEN), dtype=torch.bfloat16, device="cuda"),
                torch.zeros((self.world, cap_rows, HIDDEN), dtype=torch.bfloat16, device="cuda"))
        return self._fixed[cap_rows]

    def route_fixed(self, x, rows: int, cap_rows: int, send_blocks) -> None:
        _check(load_library().p92b_ep_route_fixed(self.home.handle, _ptr(x), _ptr(self.router_weight), _ptr(self.bias),
                                                  rows, self.routed_scale, _ptr(send_blocks), self.world, cap_rows,
                                                  _stream()), "ep_route_fixed")

    def experts_fixed(self, recv_blocks, cap_rows: int, out_slots) -> None:
        _check(load_library().p92b_ep_experts_fixed(self.arrivals.handle, self.bank.handle, _ptr(recv_blocks), self.world,
                                                    cap_rows, _ptr(out_slots), _stream()), "ep_experts_fixed")

    def combine_fixed(self, x, returned_slots, out, rows: int) -> None:
        _check(load_library().p92b_ep_combine_fixed(self.home.handle, self.shared.handle, self.bank.handle, _ptr(x),
                                                    _ptr(returned_slots), _ptr(out), rows, _stream()), "ep_combine_fixed")

    # ---- device halves ---------------------------------------------------------------------
    def route(self, x, rows: int):
        """-> (send rows [8*rows, 1440] in destination order, per-expert counts [256] on the device)."""
        _check(load_library().p92b_ep_route(self.home.handle, _ptr(x), _ptr(self.router_weight), _ptr(self.bias), rows,
                                            self.routed_scale, _ptr(self.send), _stream()), "ep_route")
        return self.send[: rows * TOP_K], self.home.device_counts()

    def experts(self, recv_rows, recv_counts, total_rows: int):
        """recv_counts int32 [world, local] on the device -> BF16 down rows [total_rows, hidden] in arrival order."""
        out = torch.empty((total_rows, HIDDEN), dtype=torch.bfloat16, device="cuda")
        _check(load_library().p92b_ep_experts(self.arrivals.handle, self.bank.handle, _ptr(recv_rows) if total_rows else 0,
                                              _ptr(recv_counts), self.world, total_rows,
                                              _ptr(out) if total_rows else 0, _stream()), "ep_experts")
        return out

    def combine(self, x, returned_rows, out, rows: int) -> None:
        _check(load_library().p92b_ep_combine(self.home.handle, self.shared.handle, self.bank.handle, _ptr(x),
                                              _ptr(returned_rows), _ptr(out), rows, _stream()), "ep_combine")


def exchange_dispatch(send, counts_by_dst, group=None):
    """Exchange 1.  send: rows in destination order; counts_by_dst int32 [world, local] = rows per
    (destination, its local expert).  Returns (arrived rows: the runs of sources 0..world-1
    concatenated, recv_counts [world(source), local], send_sizes, recv_sizes).  Works on any backend
    (NCCL on GPUs, gloo on CPU tensors); the split sizes cross to the host once."""
    import torch.distributed as dist

    recv_counts = torch.empty_like(counts_by_dst)
    dist.all_to_all_single(recv_counts, counts_by_dst, group=group)
    sizes = torch.stack([counts_by_dst.sum(dim=1), recv_counts.sum(dim=1)]).cpu().tolist()
    send_sizes, recv_sizes = [int(v) for v in sizes[0]], [int(v) for v in sizes[1]]
    recv = torch.empty((sum(recv_sizes),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send, output_split_sizes=recv_sizes, input_split_sizes=send_sizes, group=group)
    return recv, recv_counts, send_sizes, recv_sizes


def exchange_return(rows_out, send_sizes, recv_sizes, group=None):
    """Exchange 2: rows computed for the arrivals go back to their homes, splits reversed; the result
    is in the order the home GPU sent its rows."""
    import torch.distributed as dist

    returned = torch.empty((sum(send_sizes),) + tuple(rows_out.shape[1:]), dtype=rows_out.dtype, device=rows_out.device)
    dist.all_to_all_single(returned, rows_out, output_split_sizes=send_sizes, input_split_sizes=recv_sizes, group=group)
    return returned


def forward_nccl(state: EpRank, x, out, rows: int, group=None) -> dict:
    """The block on `rows` home tokens of this rank, exchanges over NCCL.  Returns split statistics."""
    send, counts = state.route(x, rows)
    counts_by_dst = counts.view(state.world, state.local).contiguous()
    recv, recv_counts, send_sizes, recv_sizes = exchange_dispatch(send, counts_by_dst, group)
    down = state.experts(recv, recv_counts, recv.shape[0])
    returned = exchange_return(down, send_sizes, recv_sizes, group)
    state.combine(x, returned, out, rows)
    return {"sent_rows": send_sizes, "received_rows": int(recv.shape[0])}


FUSED_MAX_ROWS = 8       # home tokens per GPU the fused kernel takes ...
FUSED_MAX_TOKENS = 32    # ... and tokens in flight over all GPUs


class EpWindow:
    """This GPU's exchange window for the fused small-batch kernel, connected to all peers' windows.
    Collective over `group` when world > 1 (the 64-byte handles are all-gathered); one window serves all
    layers.  Every rank must make the same sequence of forward_fused calls on it."""

    def __init__(self, rank: int, world: int, rows_per_gpu: int, group=None, connect: bool = True, bulk: bool = False,
                 hidden: int = HIDDEN):
        """bulk=True makes the window of the large-batch path (forward_bulk): another layout, any rows_per_gpu."""
        lib = load_library()
        handle = ctypes.c_void_p()
        if bulk:
            _check(lib.p92b_ep_window_create_bulk(ctypes.byref(handle), rank, world, rows_per_gpu, hidden),
                   "ep_window_create_bulk")
        else:
            _check(lib.p92b_ep_window_create(ctypes.byref(handle), rank, world, rows_per_gpu), "ep_window_create")
        self.handle, self.rank, self.world, self.rows_per_gpu = handle, rank, world, rows_per_gpu
        if not connect:
            return
        if world > 1:
            import torch.distributed as dist

            mine = (ctypes.c_uint8 * 64)()
            _check(lib.p92b_ep_window_handle(handle, mine), "ep_window_handle")
            device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
            local = torch.tensor(list(mine), dtype=torch.uint8, device=device)
            gathered = [torch.empty_like(local) for _ in range(world)]
            dist.all_gather(gathered, local, group=group)
            blob = bytes(torch.stack(gathered).cpu().flatten().tolist())
            everyone = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(blob)
            _check(lib.p92b_ep_window_connect(handle, everyone), "ep_window_connect")
        else:
            _check(lib.p92b_ep_window_connect(handle, None), "ep_window_connect")

    @staticmethod
    def connect_local(windows: Sequence["EpWindow"]) -> None:
        """Connect windows that all live in this process (rank order)."""
        array = (ctypes.c_void_p * len(windows))(*[w.handle.value for w in windows])
        for w in windows:
            _check(load_library().p92b_ep_window_connect_local(w.handle, array), "ep_window_connect_local")

    def close(self) -> None:
        if self.handle:
            load_library().p92b_ep_window_destroy(self.handle)
            self.handle = None


def forward_fused(window: EpWindow, plan: MoePlan, bank: ExpertBank, router_weight, correction_bias, x, out, rows: int,
                  routed_scale: float = ROUTED_SCALE) -> None:
    """The block on this GPU's `rows` home tokens as one kernel launch; the exchanges happen inside it.
    `plan` needs max_rows >= world * rows_per_gpu; it can be shared by all layers of a rank."""
    _check(load_library().p92b_ep_forward_fused(plan.handle, bank.handle, window.handle, _ptr(x), _ptr(router_weight),
                                                _ptr(correction_bias), _ptr(out), rows, routed_scale, _stream()),
           "ep_forward_fused")


def forward_fused_host_async(window: EpWindow, plan: MoePlan, bank: ExpertBank, router_weight, correction_bias,
                             pinned_in, pinned_out, rows: int, routed_scale: float = ROUTED_SCALE) -> None:
    """forward_fused with page-locked host tensors, copies pipelined on the plan's own streams; outputs are valid
    after ``plan.host_flush()`` and a synchronisation of the current stream."""
    _check(load_library().p92b_ep_forward_fused_host_async(plan.handle, bank.handle, window.handle, pinned_in.data_ptr(),
                                                           _ptr(router_weight), _ptr(correction_bias),
                                                           pinned_out.data_ptr(), rows, routed_scale, _stream()),
           "ep_forward_fused_host_async")


GATHERED_MAX_ROWS = 512      # home tokens per GPU the gathered multi-kernel path takes ...
GATHERED_MAX_TOKENS = 1024   # ... and tokens in flight over all GPUs


def forward_gathered(window: EpWindow, plan: MoePlan, bank: ExpertBank, router_weight, correction_bias, x, out, rows: int,
                     routed_scale: float = ROUTED_SCALE) -> None:
    """The block on this GPU's `rows` home tokens, exchanges by the library's own kernels (peer stores and
    polled words, no NCCL, no host synchronisation).  `plan` needs max_rows >= world * rows_per_gpu."""
    _check(load_library().p92b_ep_forward_gathered(plan.handle, bank.handle, window.handle, _ptr(x), _ptr(router_weight),
                                                   _ptr(correction_bias), _ptr(out), rows, routed_scale, _stream()),
           "ep_forward_gathered")


def forward_bulk(window: EpWindow, plan: MoePlan, bank: ExpertBank, router_weight, correction_bias, x, out, rows: int,
                 routed_scale: float = ROUTED_SCALE) -> None:
    """The block on this GPU's `rows` home tokens for large batches: all-gather dispatch and direct placement of the
    result rows by the library's own kernels (16-byte peer stores, one flag per peer and exchange), no NCCL, no host
    synchronisation.  `window` was created with bulk=True; `plan` needs max_rows >= world * rows_per_gpu."""
    _check(load_library().p92b_ep_forward_bulk(plan.handle, bank.handle, window.handle, _ptr(x), _ptr(router_weight),
                                               _ptr(correction_bias), _ptr(out), rows, routed_scale, _stream()),
           "ep_forward_bulk")


FIXED_MAX_ROWS = 64      # per-GPU batch up to which forward_auto takes the fixed-capacity exchange


def forward_nccl_fixed(state: EpRank, x, out, rows: int, cap_rows: int, group=None) -> None:
    """The block on `rows` home tokens with fixed-capacity exchange blocks: two equal-split all-to-alls
    and no host synchronisation anywhere in the layer.  cap_rows (>= 8 * rows) must agree on all ranks."""
    import torch.distributed as dist

    send, recv, slots_out, slots_back = state.fixed_buffers(cap_rows)
    state.route_fixed(x, rows, cap_rows, send)
    dist.all_to_all_single(recv, send, group=group)
    state.experts_fixed(recv, cap_rows, slots_out)
    dist.all_to_all_single(slots_back, slots_out, group=group)
    state.combine_fixed(x, slots_back, out, rows)


def forward_auto(state: EpRank, x, out, rows: int, max_rows_any_rank: int, group=None) -> None:
    """Fixed-capacity exchange for small batches (latency-bound, the padding is cheap), exact-size
    exchange otherwise (bandwidth-bound).  max_rows_any_rank must be the same number on all ranks."""
    if max_rows_any_rank <= FIXED_MAX_ROWS:
        forward_nccl_fixed(state, x, out, rows, TOP_K * max_rows_any_rank, group)
    else:
        forward_nccl(state, x, out, rows, group)


def forward_emulated_fixed(states: Sequence[EpRank], xs: Sequence, outs: Sequence, rows: Sequence[int]) -> None:
    """forward_nccl_fixed for all ranks in one process: the all-to-all is a transpose of the blocks."""
    world = len(states)
    cap = TOP_K * max(rows)
    bufs = [st.fixed_buffers(cap) for st in states]
    for st, x, r, b in zip(states, xs, rows, bufs):
        st.route_fixed(x, r, cap, b[0])
    for d in range(world):
        for s in range(world):
            bufs[d][1][s].copy_(bufs[s][0][d])
    for st, b in zip(states, bufs):
        st.experts_fixed(b[1], cap, b[2])
    for s in range(world):
        for d in range(world):
            bufs[s][3][d].copy_(bufs[d][2][s])
    for st, x, o, r, b in zip(states, xs, outs, rows, bufs):
        st.combine_fixed(x, b[3], o, r)
    torch.cuda.synchronize()


def forward_emulated(states: Sequence[EpRank], xs: Sequence, outs: Sequence, rows: Sequence[int]) -> None:
    """All ranks in ONE process on one GPU, the exchanges done by tensor slicing: the same device code
    path as forward_nccl without NCCL, for single-GPU tests of the multi-GPU logic."""
    world = len(states)
    sends, counts = [], []
    for st, x, r in zip(states, xs, rows):
        s, c = st.route(x, r)
        sends.append(s.clone())
        counts.append(c.view(world, st.local).clone())
    torch.cuda.synchronize()
    host_counts = [c.cpu() for c in counts]
    downs = []
    for d, st in enumerate(states):
        recv_counts = torch.stack([counts[s][d] for s in range(world)]).contiguous()
        pieces = []
        for s in range(world):
            start = int(host_counts[s][:d].sum())
            n = int(host_counts[s][d].sum())
            pieces.append(sends[s][start:start + n])
        recv = torch.cat(pieces) if pieces else torch.empty((0, ROW_BYTES), dtype=torch.uint8, device="cuda")
        downs.append(st.experts(recv.contiguous(), recv_counts, recv.shape[0]))
    torch.cuda.synchronize()
    for s, st in enumerate(states):
        pieces = []
        for d in range(world):
            # rows rank s sent to d sit in d's arrival buffer after the runs of sources < s
            before = sum(int(host_counts[t][d].sum()) for t in range(s))
            n = int(host_counts[s][d].sum())
            pieces.append(downs[d][before:before + n])
        returned = torch.cat(pieces).contiguous()
        st.combine(xs[s], returned, outs[s], rows[s])
    torch.cuda.synchronize()
