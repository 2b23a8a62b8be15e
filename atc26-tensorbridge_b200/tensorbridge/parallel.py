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

import dataclasses

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
                                     int(placement == "interleaved"), send_counts.data_ptr(), send_pos.data_ptr()))
        _native.check(lib.tb_ep_pack(stream, x_q.data_ptr(), scale.data_ptr(), send_pos.data_ptr(), routes, top_k, width, groups,
                                     row_bytes, send.data_ptr()))
    return send_counts, send_pos, send


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
