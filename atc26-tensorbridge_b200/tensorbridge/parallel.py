"""Sharding of the two GEMM families over the GPUs of one node (one process per GPU, `torch.distributed`).

The reference has no multi-GPU code: tensor- and expert-parallel shapes reach it already sharded by the serving
framework (`tensorbridge/vllm_moe.py:130-132`).  These helpers provide that sharding for stand-alone use:

* dense layers split column-parallel on N (`shard_columns`); each rank computes its own output columns with no
  collective, and `gather_columns` all-gathers the BF16 output only when the caller needs it whole;
* MoE layers shard experts `E / world` per rank under the masked layout; `dispatch_masked` moves each routed token to
  the rank that owns its expert with one all-to-all of counts and one of packed rows (FP8 row + scales),
  `combine_masked` returns the expert outputs to the ranks and route slots they came from.

All functions take plain tensors and work on any backend (NCCL on GPUs; the tests run them over gloo on CPU).  On CUDA
tensors the integer bookkeeping and the row movement run in the library's kernels (`tb_ep_*`, `tb_gather_rows`); on
CPU tensors the same plan is worked out with torch ops, which is also what the GPU tests check the kernels against.
"""
from __future__ import annotations

import ctypes
import dataclasses
import os

import torch
import torch.distributed as dist


def shard_columns(packed: torch.Tensor, scale: torch.Tensor, rank: int, world: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Rank `rank`'s channel slice of a checkpoint weight (`packed` uint8 `[N, K/2]`, `scale` E4M3 `[N, K/16]`).
    The global scale is shared by all shards."""
    n = packed.size(0)
    if n % (world * 8):
        raise ValueError(f"N = {n} does not split into {world} shards of a multiple of 8 channels")
    per = n // world
    return packed[rank * per:(rank + 1) * per].contiguous(), scale[rank * per:(rank + 1) * per].contiguous()


def gather_columns(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """`[M, N/world]` per rank -> the full `[M, N]` on every rank (one all-gather)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    m, n_local = local_out.shape
    gathered = torch.empty((world * m, n_local), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, local_out.contiguous(), group=group)
    return gathered.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


def expert_range(num_experts: int, rank: int, world: int) -> tuple[int, int]:
    """(first global expert, local expert count) of `rank` under contiguous placement."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split over {world} ranks")
    per = num_experts // world
    return rank * per, per


def local_experts(num_experts: int, rank: int, world: int, placement: str = "contiguous") -> list[int]:
    """Global ids of the experts `rank` owns, in local order.  `contiguous`: a block of E / world consecutive experts;
    `interleaved`: experts rank, rank + world, ... (spreads popularity that correlates with the expert index)."""
    _, per = expert_range(num_experts, rank, world)
    if placement == "contiguous":
        return list(range(rank * per, (rank + 1) * per))
    if placement == "interleaved":
        return list(range(rank, num_experts, world))
    raise ValueError(f"unknown placement {placement!r}")


def _placed(flat: torch.Tensor, per: int, world: int, placement: str) -> torch.Tensor:
    """Global expert id -> owner rank * E_local + local index."""
    if placement == "contiguous":
        return flat
    if placement == "interleaved":
        return (flat % world) * per + flat // world
    raise ValueError(f"unknown placement {placement!r}")


@dataclasses.dataclass
class MaskedDispatch:
    """What `dispatch_masked` returns: the local masked GEMM inputs and the bookkeeping to send results back."""

    a: torch.Tensor  # FP8 (as stored) [E_local * capacity, K]
    a_scale: torch.Tensor  # FP32 [E_local * capacity, groups]
    counts: torch.Tensor  # int32 [E_local], clamped to capacity
    capacity: int
    recv_rows: torch.Tensor  # int32 [received]: row of `a` each received route landed in (-1 = dropped, over capacity)
    send_pos: torch.Tensor  # int32 [T * top_k]: row of every route in the send order (-1 = not sent)
    send_splits: list[int]
    recv_splits: list[int]


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, group) -> None:
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)


def packed_row_bytes(width: int, groups: int) -> int:
    """Bytes of one packed dispatch row: FP8 row, then its FP32 scales, padded to a multiple of 16."""
    return (width + 4 * groups + 15) // 16 * 16


# ---- the two halves of a dispatch on either side of the exchange, as torch ops (any device; what the CPU tests run) and
# ---- as the library's kernels (CUDA tensors).  Both produce the same integers and bytes.
def _plan_torch(x_q, x_scale, topk_ids, num_experts, world, placement, row_bytes):
    t, top_k = topk_ids.shape
    e_local = num_experts // world
    flat = topk_ids.reshape(-1).to(torch.int64)
    local = (flat >= 0) & (flat < num_experts)
    placed = torch.where(local, _placed(flat.clamp(0, num_experts - 1), e_local, world, placement), torch.full_like(flat, num_experts))
    order = torch.argsort(placed, stable=True)  # by owner rank, then local expert, then route id; unsent routes last
    send_counts = torch.bincount(placed, minlength=num_experts + 1)[:num_experts].to(torch.int32)
    send_pos = torch.empty_like(flat, dtype=torch.int32)
    send_pos[order] = torch.arange(flat.numel(), device=flat.device, dtype=torch.int32)
    send_pos = torch.where(local, send_pos, torch.full_like(send_pos, -1))
    width, groups = x_q.size(1), x_scale.reshape(t, -1).size(1)
    rows = torch.div(order, top_k, rounding_mode="floor")
    send = torch.zeros((flat.numel(), row_bytes), dtype=torch.uint8, device=x_q.device)
    send[:, :width] = x_q.view(torch.uint8)[rows]
    send[:, width:width + 4 * groups] = x_scale.reshape(t, -1)[rows].contiguous().view(torch.uint8).reshape(-1, 4 * groups)
    return send_counts, send_pos, send


def _plan_native(x_q, x_scale, topk_ids, num_experts, world, placement, row_bytes):
    from tensorbridge import _native  # noqa: PLC0415
    lib = _native.load()
    device = x_q.device
    t, top_k = topk_ids.shape
    ids = topk_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    routes = t * top_k
    width, groups = x_q.size(1), x_scale.reshape(t, -1).size(1)
    send_counts = torch.empty(num_experts, dtype=torch.int32, device=device)
    send_pos = torch.empty(routes, dtype=torch.int32, device=device)
    send = torch.empty((routes, row_bytes), dtype=torch.uint8, device=device)
    scale = x_scale.reshape(t, -1).contiguous()
    with torch.cuda.device(device):
        stream = _native.stream_ptr(device)
        _native.check(lib.tb_ep_plan(stream, ids.data_ptr(), int(ids.dtype == torch.int64), routes, num_experts, world,
                                     int(placement == "interleaved"), send_counts.data_ptr(), send_pos.data_ptr(), None))
        _native.check(lib.tb_ep_pack(stream, x_q.data_ptr(), scale.data_ptr(), send_pos.data_ptr(), routes, top_k, width, groups,
                                     row_bytes, send.data_ptr()))
    return send_counts, send_pos, send


def plan_local(topk_ids: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Routes of one rank sorted by expert: int32 `counts[E]` and, per route, its position in expert order (int32
    `[routes]`, -1 for ids outside `[0, E)`; routes of one expert keep their order).  The send plan of a world of
    one: the dispatch plan kernel on CUDA (`E <= 1024`), torch ops elsewhere."""
    ids = topk_ids.reshape(-1).contiguous()
    if not ids.is_cuda:
        flat = ids.to(torch.int64)
        local = (flat >= 0) & (flat < num_experts)
        keyed = torch.where(local, flat, torch.full_like(flat, num_experts))
        order = torch.argsort(keyed, stable=True)
        counts = torch.bincount(keyed, minlength=num_experts + 1)[:num_experts].to(torch.int32)
        positions = torch.empty_like(order)
        positions[order] = torch.arange(flat.numel(), device=flat.device)
        return counts, torch.where(local, positions, torch.full_like(positions, -1)).to(torch.int32)
    from tensorbridge import _native  # noqa: PLC0415
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    counts = torch.empty(num_experts, dtype=torch.int32, device=ids.device)
    positions = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        _native.check(_native.load().tb_ep_plan(_native.stream_ptr(ids.device), ids.data_ptr(), int(ids.dtype == torch.int64),
                                                ids.numel(), num_experts, 1, 0, counts.data_ptr(), positions.data_ptr(), None))
    return counts, positions


def _place_torch(recv, recv_counts, capacity, width, groups, fp8_dtype):
    world, e_local = recv_counts.shape
    device = recv.device
    rc = recv_counts.to(torch.int64)
    before = torch.cumsum(rc, 0) - rc  # rows of earlier source ranks, per expert
    expert_of = torch.repeat_interleave(torch.arange(e_local, device=device).repeat(world), rc.reshape(-1))
    source_of = torch.repeat_interleave(torch.arange(world, device=device).repeat_interleave(e_local), rc.reshape(-1))
    starts = torch.cumsum(rc.reshape(-1), 0) - rc.reshape(-1)  # start of each (source, expert) run in the receive buffer
    within = torch.arange(recv.size(0), device=device) - torch.repeat_interleave(starts, rc.reshape(-1))
    slot = before[source_of, expert_of] + within
    keep = slot < capacity
    recv_rows = torch.where(keep, expert_of * capacity + slot, torch.full_like(slot, -1)).to(torch.int32)
    a = torch.zeros((e_local * capacity, width), dtype=torch.uint8, device=device)
    a_scale = torch.ones((e_local * capacity, groups), dtype=torch.float32, device=device)
    dest = recv_rows[keep].to(torch.int64)
    a[dest] = recv[keep][:, :width]
    a_scale[dest] = recv[keep][:, width:width + 4 * groups].contiguous().view(torch.float32).reshape(-1, groups)
    counts = rc.sum(0).clamp(max=capacity).to(torch.int32)
    return a.view(fp8_dtype), a_scale, counts, recv_rows


def _place_native(recv, recv_counts, capacity, width, groups, fp8_dtype):
    from tensorbridge import _native  # noqa: PLC0415
    lib = _native.load()
    world, e_local = recv_counts.shape
    device = recv.device
    rows, row_bytes = recv.shape
    # rows no route owns are never read by the masked GEMM (it stops at each expert's count): no need to clear them
    a = torch.empty((e_local * capacity, width), dtype=torch.uint8, device=device)
    a_scale = torch.empty((e_local * capacity, groups), dtype=torch.float32, device=device)
    seg = torch.empty((2, world * e_local), dtype=torch.int32, device=device)
    counts = torch.empty(e_local, dtype=torch.int32, device=device)
    recv_rows = torch.empty(rows, dtype=torch.int32, device=device)
    rc = recv_counts.contiguous()
    with torch.cuda.device(device):
        stream = _native.stream_ptr(device)
        _native.check(lib.tb_ep_layout(stream, rc.data_ptr(), world, e_local, capacity, seg[0].data_ptr(), seg[1].data_ptr(),
                                       counts.data_ptr()))
        _native.check(lib.tb_ep_place(stream, recv.data_ptr(), rows, row_bytes, width, groups, seg[0].data_ptr(),
                                      seg[1].data_ptr(), world, e_local, capacity, a.data_ptr(), a_scale.data_ptr(),
                                      recv_rows.data_ptr()))
    return a.view(fp8_dtype), a_scale, counts, recv_rows


def gather_rows(src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """`out[i] = src[index[i]]`, zeros where `index[i] < 0`; rows must be a multiple of 16 bytes on CUDA."""
    if not src.is_cuda:
        out = torch.zeros((index.numel(), src.size(1)), dtype=src.dtype, device=src.device)
        keep = index >= 0
        out[keep] = src[index[keep].to(torch.int64)]
        return out
    from tensorbridge import _native  # noqa: PLC0415
    src = src.contiguous()
    row_bytes = src.size(1) * src.element_size()
    if row_bytes % 16:
        raise ValueError("rows must be a multiple of 16 bytes")
    out = torch.empty((index.numel(), src.size(1)), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        _native.check(_native.load().tb_gather_rows(_native.stream_ptr(src.device), src.data_ptr(),
                                                    index.to(torch.int32).contiguous().data_ptr(), index.numel(), row_bytes,
                                                    out.data_ptr()))
    return out


def dispatch_masked(x_q: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor, num_experts: int, capacity: int,
                    group=None, placement: str = "contiguous") -> MaskedDispatch:
    """Send every route `(token, slot)` of this rank's `x_q` `[T, K]` (FP8) / `x_scale` `[T, groups]` to the rank that
    owns expert `topk_ids[token, slot]`, and lay the received rows out as `E_local` blocks of `capacity` rows, expert
    `e`'s rows ordered by source rank then by route id.  Rows beyond an expert's capacity are dropped (their count is
    clamped, as a masked buffer of fixed capacity must).

    Two exchanges: the per-(rank, expert) counts (fixed size), then one all-to-all of packed rows (FP8 row + scales).
    On CUDA tensors the bookkeeping on both sides runs in the library's kernels and the only value read back to the
    host is the list of split sizes the second exchange needs, so call this outside any CUDA-graph capture."""
    world = dist.get_world_size(group)
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split over {world} ranks")
    if placement not in ("contiguous", "interleaved"):
        raise ValueError(f"unknown placement {placement!r}")
    e_local = num_experts // world
    t, _ = topk_ids.shape
    width, groups = x_q.size(1), x_scale.reshape(t, -1).size(1)
    row_bytes = packed_row_bytes(width, groups)
    native = x_q.is_cuda
    send_counts, send_pos, send = (_plan_native if native else _plan_torch)(x_q, x_scale, topk_ids, num_experts, world,
                                                                              placement, row_bytes)
    send_counts = send_counts.view(world, e_local)
    recv_counts = torch.empty_like(send_counts)  # [source rank, local expert]
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).tolist()  # the one read-back of a dispatch
    send_splits, recv_splits = both
    recv = torch.empty((sum(recv_splits), row_bytes), dtype=torch.uint8, device=x_q.device)
    _all_to_all(recv, send[:sum(send_splits)], recv_splits, send_splits, group)
    a, a_scale, counts, recv_rows = (_place_native if native else _place_torch)(recv, recv_counts, capacity, width, groups,
                                                                                x_q.dtype)
    return MaskedDispatch(a, a_scale, counts, capacity, recv_rows, send_pos, send_splits, recv_splits)


def combine_masked(local_out: torch.Tensor, plan: MaskedDispatch, num_routes: int, group=None) -> torch.Tensor:
    """Return the masked GEMM output rows `[E_local * capacity, N]` to the ranks their routes came from: `[T * top_k, N]`
    in route order on every rank; routes that were dropped for capacity (or never sent) come back as zeros."""
    n = local_out.size(1)
    back = gather_rows(local_out, plan.recv_rows)
    returned = torch.empty((sum(plan.send_splits), n), dtype=local_out.dtype, device=local_out.device)
    _all_to_all(returned, back, plan.send_splits, plan.recv_splits, group)
    if plan.send_pos.numel() != num_routes:
        raise ValueError(f"the plan covers {plan.send_pos.numel()} routes, not {num_routes}")
    return gather_rows(returned, plan.send_pos)


# ---------------------------------------------------------------------------------------------------------------------
# The same step over peer memory: each rank writes its routes straight into the owner's masked buffer and reads the
# results back from the owner's output buffer (NVLink loads and stores issued by the library's kernels), with rank-to-rank
# barriers on flags in that memory.  No collective library call, no host read, no staging copy in a step.
# ---------------------------------------------------------------------------------------------------------------------
class _DeviceView:
    """`__cuda_array_interface__` over raw device memory, so that torch can alias it as a tensor."""

    def __init__(self, pointer: int, shape: tuple, typestr: str) -> None:
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (pointer, False), "version": 2}


def _alias(pointer: int, shape: tuple, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    typestr, view = {torch.uint8: ("|u1", None), torch.float32: ("<f4", None), torch.int32: ("<i4", None),
                     torch.bfloat16: ("<u2", torch.bfloat16), torch.float8_e4m3fn: ("|u1", torch.float8_e4m3fn)}[dtype]
    t = torch.as_tensor(_DeviceView(pointer, shape, typestr), device=device)
    return t if view is None else t.view(view)


@dataclasses.dataclass
class PeerDispatch:
    """What `PeerMaskedExchange.dispatch` returns: the masked GEMM inputs (views of this rank's peer-mapped buffers)."""

    a: torch.Tensor  # FP8 [E_local * capacity, K]
    a_scale: torch.Tensor  # FP32 [E_local * capacity, groups]
    counts: torch.Tensor  # int32 [E_local], clamped to capacity
    out: torch.Tensor  # BF16 [E_local * capacity, N]: where the masked GEMM must write (`out=`)
    dest_row: torch.Tensor  # int32 [T * top_k]: row of every route in its owner's buffers (-1 = dropped)
    topk_ids: torch.Tensor
    scatter: object = None  # `tensorbridge.PeerScatter` for the GEMM when the combine is fused into its epilogue
    routes: torch.Tensor | None = None  # BF16 [T * top_k, N]: where the fused combine delivers this rank's routes


class PeerMaskedExchange:
    """Expert-parallel masked dispatch and combine over peer memory for a fixed (experts, capacity, K, groups, N).

    Construction is collective (every rank of `group`, same arguments): each rank allocates one slab (masked
    activations, their scales, the GEMM output, a `[world, E]` count matrix, arrival flags), exports it and maps its
    peers' slabs (CUDA IPC; all ranks on one node, one GPU each).  A step is

        plan = exchange.dispatch(x_q, x_scale, topk_ids)            # plan, barrier (+ counts), push, barrier
        tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, experts, tb.MaskedRouting(plan.counts), m, out=plan.out)
        y = exchange.combine(plan)                                   # barrier, pull

    or, with the combine fused into the GEMM's epilogue (every output row stored over NVLink into the route buffer of the
    rank it came from, tile by tile as the GEMM produces it):

        plan = exchange.dispatch(x_q, x_scale, topk_ids, fused_combine=True)
        tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, experts, tb.MaskedRouting(plan.counts), m, out=plan.out,
                                  scatter=plan.scatter)
        y = exchange.finish(plan)                                    # barrier

    and launches nothing but this library's kernels: no host read, so it can follow a quantiser and precede the next
    layer without a synchronisation.  The masked buffers are reused by the next `dispatch`: consume `y` (a fresh
    tensor) as you like, but read `plan.a` / `plan.out` only before the next step.  `wait_us` bounds every barrier wait
    (ten seconds by default: ranks reach their first barrier at different times, after loading kernels); a barrier that
    runs out writes `100 + peer` to the status words (`tensorbridge.check_status()` raises).  `close()` unmaps and frees."""

    def __init__(self, num_experts: int, capacity: int, k: int, groups: int, n: int, group=None,
                 placement: str = "interleaved", wait_us: int = 10_000_000, max_routes: int = 0) -> None:
        from tensorbridge import _native  # noqa: PLC0415
        self._native, self._lib = _native, _native.load()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not split over {self.world} ranks")
        if placement not in ("contiguous", "interleaved"):
            raise ValueError(f"unknown placement {placement!r}")
        if k % 16 or (2 * n) % 16:
            raise ValueError("K must be a multiple of 16 and N of 8")
        self.num_experts, self.capacity, self.k, self.groups, self.n = num_experts, capacity, k, groups, n
        self.e_local = num_experts // self.world
        self.placement, self.wait_us = placement, wait_us
        self.device = torch.device("cuda", torch.cuda.current_device())
        rows = self.e_local * capacity
        self.max_routes = max_routes
        sizes = [rows * k, rows * groups * 4, rows * n * 2, self.world * num_experts * 4, 256, rows * 4, max(max_routes, 1) * n * 2]
        self._offsets, total = [], 0
        for size in sizes:
            self._offsets.append(total)
            total += (size + 255) // 256 * 256
        base = ctypes.c_void_p()
        _native.check(self._lib.tb_peer_alloc(total, ctypes.byref(base)))
        self._base = base.value
        handle = ctypes.create_string_buffer(64)
        _native.check(self._lib.tb_ipc_export(self._base, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, (os.getpid(), handle.raw), group=group)
        self._peer_bases, self._opened = [], []
        failure = None
        for r, (pid, raw) in enumerate(handles):
            if r == self.rank or pid == os.getpid():
                self._peer_bases.append(self._base)
                continue
            mapped = ctypes.c_void_p()
            code = self._lib.tb_ipc_open(raw, ctypes.byref(mapped))
            if code:
                failure = f"mapping the slab of rank {r}: {self._lib.tb_last_error().decode()}"
                break
            self._peer_bases.append(mapped.value)
            self._opened.append(mapped.value)
        # every rank learns whether every rank could map every slab: either all go on or all give up together, so that
        # no rank is left waiting in a collective for one that raised
        agreed = torch.tensor([0 if failure is None else 1], dtype=torch.int32, device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=group)
        if int(agreed.item()):
            for pointer in self._opened:
                self._lib.tb_ipc_close(pointer)
            dist.barrier(group=group)
            self._lib.tb_peer_free(self._base)
            self._base, self._opened = None, []
            raise RuntimeError(failure or "a peer could not map the slabs of the exchange")

        def pointers(index: int):
            return (ctypes.c_void_p * self.world)(*[b + self._offsets[index] for b in self._peer_bases])

        self._peer_a, self._peer_scale, self._peer_y = pointers(0), pointers(1), pointers(2)
        self._peer_counts, self._peer_flags = pointers(3), pointers(4)
        self._peer_targets, self._peer_routes = pointers(5), pointers(6)
        self.row_target = _alias(self._base + self._offsets[5], (rows,), torch.int32, self.device)
        self.routes = _alias(self._base + self._offsets[6], (max(max_routes, 1), n), torch.bfloat16, self.device)
        self.a = _alias(self._base + self._offsets[0], (rows, k), torch.float8_e4m3fn, self.device)
        self.a_scale = _alias(self._base + self._offsets[1], (rows, groups), torch.float32, self.device)
        self.out = _alias(self._base + self._offsets[2], (rows, n), torch.bfloat16, self.device)
        self.all_counts = _alias(self._base + self._offsets[3], (self.world, num_experts), torch.int32, self.device)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._send_counts = torch.empty(num_experts, dtype=torch.int32, device=self.device)
        self.counts = torch.empty(self.e_local, dtype=torch.int32, device=self.device)
        dist.barrier(group=group)  # every rank has mapped every slab before anybody writes into one

    def _barrier(self, stream: int, payload: torch.Tensor | None = None) -> None:
        native = self._native
        native.check(self._lib.tb_peer_barrier(
            stream, self._peer_flags, self._peer_counts, None if payload is None else payload.data_ptr(),
            0 if payload is None else payload.numel(), self.rank, self.world, self._epoch.data_ptr(), self.wait_us,
            native.status_words(self.device.index).data_ptr()))

    def dispatch(self, x_q: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor, *, fused_combine: bool = False
                 ) -> PeerDispatch:
        """Plan, exchange the counts, push the rows.  With `fused_combine` (needs `max_routes >= T * top_k` at
        construction) the push also tells every owner which rank and route each of its rows belongs to, clears this
        rank's rows of dropped routes, and the returned plan carries the `scatter` to hand to
        `fp8_nvfp4_grouped_gemm(..., scatter=plan.scatter)`: the GEMM's epilogue then stores every output row into the
        route buffer of the rank it came from, and `finish(plan)` (one barrier) returns this rank's routes."""
        native = self._native
        t, top_k = topk_ids.shape
        if fused_combine and t * top_k > self.max_routes:
            raise ValueError(f"{t * top_k} routes exceed the exchange's max_routes = {self.max_routes}")
        if x_q.size(1) != self.k or x_scale.reshape(t, -1).size(1) != self.groups or not x_q.is_contiguous():
            raise ValueError("activations do not match the exchange's K / scale groups")
        ids = topk_ids if topk_ids.dtype in (torch.int32, torch.int64) and topk_ids.is_contiguous() else topk_ids.to(torch.int64).contiguous()
        scale = x_scale.reshape(t, -1).contiguous()
        routes = t * top_k
        route_rank = torch.empty(routes, dtype=torch.int32, device=self.device)
        dest_row = torch.empty(routes, dtype=torch.int32, device=self.device)
        interleaved = int(self.placement == "interleaved")
        with torch.cuda.device(self.device):
            stream = native.stream_ptr(self.device)
            native.check(self._lib.tb_ep_plan(stream, ids.data_ptr(), int(ids.dtype == torch.int64), routes, self.num_experts,
                                              self.world, interleaved, self._send_counts.data_ptr(), None, route_rank.data_ptr()))
            self._barrier(stream, self._send_counts)  # every rank now holds every rank's counts
            args = native.PushArgs(ids.data_ptr(), int(ids.dtype == torch.int64), top_k, routes, x_q.data_ptr(), scale.data_ptr(),
                                   self.k, self.groups, route_rank.data_ptr(), self.all_counts.data_ptr(), self.num_experts,
                                   self.world, self.rank, interleaved, self.capacity, 0, self._peer_a, self._peer_scale,
                                   dest_row.data_ptr(), self.counts.data_ptr(),
                                   self._peer_targets if fused_combine else None,
                                   self.routes.data_ptr() if fused_combine else None, self.n * 2)
            native.check(self._lib.tb_ep_push(stream, ctypes.byref(args)))
            self._barrier(stream)  # every rank's rows have landed
        if fused_combine:
            from tensorbridge.gemm import PeerScatter  # noqa: PLC0415
            return PeerDispatch(self.a, self.a_scale, self.counts, self.out, dest_row, ids,
                                PeerScatter(self.row_target, self._peer_routes, self.world), self.routes[:routes])
        return PeerDispatch(self.a, self.a_scale, self.counts, self.out, dest_row, ids)

    def finish(self, plan: PeerDispatch) -> torch.Tensor:
        """After the GEMM of a `fused_combine` step: waits (one barrier) until every rank's epilogue has delivered, and
        returns this rank's routes `[T * top_k, N]` -- a view of the exchange's buffer, valid until the next dispatch."""
        if plan.routes is None:
            raise ValueError("finish() follows dispatch(fused_combine=True); use combine() otherwise")
        with torch.cuda.device(self.device):
            self._barrier(self._native.stream_ptr(self.device))
        return plan.routes

    def combine(self, plan: PeerDispatch) -> torch.Tensor:
        """`[T * top_k, N]` in route order: every route's row of the owner's GEMM output, zeros for dropped routes."""
        native = self._native
        routes = plan.dest_row.numel()
        out = torch.empty((routes, self.n), dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            stream = native.stream_ptr(self.device)
            self._barrier(stream)  # every rank's GEMM has written its output buffer
            native.check(self._lib.tb_ep_pull(stream, plan.topk_ids.data_ptr(), int(plan.topk_ids.dtype == torch.int64),
                                              plan.dest_row.data_ptr(), routes, self.num_experts, self.world,
                                              int(self.placement == "interleaved"), self._peer_y, self.n * 2, out.data_ptr()))
        return out

    def close(self) -> None:
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody still reads or writes a peer's slab
        for pointer in self._opened:
            self._native.check(self._lib.tb_ipc_close(pointer))
        self._native.check(self._lib.tb_peer_free(self._base))
        self._base, self._opened = None, []
