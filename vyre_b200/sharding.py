"""Sharding of the quantized-linear / MoE path over the GPUs of one box (one process per GPU, torch.distributed).

Two partitionings, both without any exchange inside a contraction:

* column-parallel linear: every reference kernel computes one output element independently of the others
  (vyre-libs/src/nn/linear/inner/linear_4bit.rs:710-742), so rank r owns rows [begin, end) of W and its scales,
  x is replicated, and one all-gather assembles [m, n];
* expert-parallel MoE: experts are independent programs with disjoint weights
  (vyre-libs/src/nn/moe/expert_mlp.rs:18-150), routing is per token (vyre-libs/src/nn/moe/gating.rs:19-69) and the
  combine is a per-token weighted sum (vyre-libs/src/nn/moe/moe_layer.rs:57-101): tokens are split over the ranks,
  rows travel to the rank that owns their expert (all-to-all), come back (all-to-all) and are combined at home.

The planning functions are pure numpy and the exchanges are plain torch.distributed calls, so they run under gloo
on CPU as well as under NCCL; the compute stages are the library's CUDA kernels (`KernelOps`) and exist only there.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

PAD = 0xFFFFFFFF
ROW_TILE = 256  # rows per CTA-pair tile of the grouped expert GEMM


# ---- column-parallel linear ---------------------------------------------------------------------------------------
def column_shard(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Rows [begin, end) of an n-row weight owned by `rank`; shard sizes are multiples of `multiple` except the last."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    units = (n + multiple - 1) // multiple
    per, extra = divmod(units, world)
    begin_u = rank * per + min(rank, extra)
    end_u = begin_u + per + (1 if rank < extra else 0)
    return min(n, begin_u * multiple), min(n, end_u * multiple)


def all_gather_columns(y_local, n_total: int, group=None, multiple: int = 1):
    """[m, n_local] per rank -> [m, n_total] on every rank, for shards cut by column_shard(n_total, world, r, multiple):
    one all_gather_into_tensor of shards padded to the widest, then a column interleave."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    m = y_local.shape[0]
    bounds = [column_shard(n_total, world, r, multiple) for r in range(world)]
    rank = dist.get_rank(group)
    if y_local.shape[1] != bounds[rank][1] - bounds[rank][0]:
        raise ValueError(f"rank {rank} holds {y_local.shape[1]} columns but its shard of {n_total} is {bounds[rank]}")
    widest = max(e - b for b, e in bounds)
    padded = y_local
    if y_local.shape[1] != widest:
        padded = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
        padded[:, : y_local.shape[1]] = y_local
    staged = torch.empty((world, m, widest), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(staged.view(-1), padded.contiguous().view(-1), group=group)
    out = torch.empty((m, n_total), dtype=y_local.dtype, device=y_local.device)
    for r, (b, e) in enumerate(bounds):
        out[:, b:e] = staged[r, :, : e - b]
    return out


# ---- expert-parallel MoE: planning (numpy) ------------------------------------------------------------------------
@dataclass
class DispatchPlan:
    send_order: np.ndarray     # [pairs] u32: token of each sent row; rows are sorted by global expert, token order kept
    pos: np.ndarray            # [tokens, topk] u32: row of each (token, slot) pair in the send buffer
    expert_counts: np.ndarray  # [experts] i64: rows per global expert
    send_splits: list          # rows sent to each rank


def plan_dispatch(idx: np.ndarray, experts: int, world: int) -> DispatchPlan:
    if experts % world:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    tokens, topk = idx.shape
    if idx.size and (idx.min() < 0 or idx.max() >= experts):
        raise ValueError("routing index out of range")
    flat = idx.reshape(-1)
    order = np.argsort(flat, kind="stable")  # by expert, then by (token, slot)
    pos = np.empty(flat.size, dtype=np.uint32)
    pos[order] = np.arange(flat.size, dtype=np.uint32)
    counts = np.bincount(flat, minlength=experts).astype(np.int64)
    local = experts // world
    splits = counts.reshape(world, local).sum(axis=1).tolist()
    return DispatchPlan((order // topk).astype(np.uint32), pos.reshape(tokens, topk), counts, [int(v) for v in splits])


@dataclass
class RegroupPlan:
    src_index: np.ndarray    # [max_rows] u32: received row feeding each padded expert-sorted row, PAD for padding rows
    ret_index: np.ndarray    # [n_recv] u32: padded row that holds the result of each received row
    tile_expert: np.ndarray  # [max_tiles] u32: local expert of each 256-row tile (first m_tiles entries are valid)
    m_tiles: int
    max_rows: int


def plan_regroup(recv_counts: np.ndarray, max_rows: int | None = None, row_tile: int = ROW_TILE) -> RegroupPlan:
    """recv_counts[r, e] = rows received from rank r for local expert e; received rows are ordered by (r, e)."""
    rc = np.ascontiguousarray(recv_counts, dtype=np.int64)
    world, local = rc.shape
    n_recv = int(rc.sum())
    per_expert = rc.sum(axis=0)
    padded = (per_expert + row_tile - 1) // row_tile * row_tile
    seg_start = np.concatenate([[0], np.cumsum(padded)])
    need = int(seg_start[-1])
    if max_rows is None:
        max_rows = max(row_tile, need)
    if need > max_rows:
        raise ValueError(f"expert segments need {need} rows but the buffers hold {max_rows}")
    src = np.full(max_rows, PAD, dtype=np.uint32)
    ret = np.empty(n_recv, dtype=np.uint32)
    recv_off = np.concatenate([[0], np.cumsum(rc.reshape(-1))])  # start of block (r, e) in the received order
    fill = np.zeros(local, dtype=np.int64)
    for r in range(world):
        for e in range(local):
            c = int(rc[r, e])
            if c == 0:
                continue
            a = int(recv_off[r * local + e])
            d = int(seg_start[e] + fill[e])
            src[d:d + c] = np.arange(a, a + c, dtype=np.uint32)
            ret[a:a + c] = np.arange(d, d + c, dtype=np.uint32)
            fill[e] += c
    tiles = np.zeros(max_rows // row_tile, dtype=np.uint32)
    m_tiles = need // row_tile
    t = 0
    for e in range(local):
        k = int(padded[e] // row_tile)
        tiles[t:t + k] = e
        t += k
    return RegroupPlan(src, ret, tiles, m_tiles, max_rows)


# ---- exchanges (torch.distributed; gloo on CPU, NCCL on GPU) -------------------------------------------------------
def exchange_counts(expert_counts: np.ndarray, world: int, device, group=None) -> np.ndarray:
    """Every rank tells every other how many rows it sends for each of that rank's local experts.
    Returns recv_counts [world, local_experts] on the host (the row exchange needs the split sizes there)."""
    import torch
    import torch.distributed as dist

    send = torch.as_tensor(np.ascontiguousarray(expert_counts, dtype=np.int64), device=device)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.cpu().numpy().reshape(world, -1)


def exchange_rows(rows, send_splits, recv_splits, group=None):
    import torch
    import torch.distributed as dist

    out = torch.empty((int(sum(recv_splits)),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=[int(v) for v in recv_splits],
                           input_split_sizes=[int(v) for v in send_splits], group=group)
    return out


def expert_parallel_layer(x, idx_host: np.ndarray, wts, experts: int, ops, group=None, max_rows: int | None = None):
    """One MoE FFN layer over the ranks of `group`, given this rank's tokens x [tokens, hidden] and their routing.

    ops supplies the compute stages: gather(src, index_u32_numpy) -> rows, experts(rows_sorted, RegroupPlan) -> rows,
    combine(y_rows, pos_numpy, wts) -> out. Returns out [tokens, hidden].
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    plan = plan_dispatch(idx_host, experts, world)
    recv_counts = exchange_counts(plan.expert_counts, world, x.device, group)
    recv_splits = recv_counts.sum(axis=1).tolist()
    sent = ops.gather(x, plan.send_order)
    received = exchange_rows(sent, plan.send_splits, recv_splits, group)
    regroup = plan_regroup(recv_counts, max_rows)
    sorted_rows = ops.gather(received, regroup.src_index)
    y_sorted = ops.experts(sorted_rows, regroup)
    y_received = ops.gather(y_sorted, regroup.ret_index)
    y_home = exchange_rows(y_received, recv_splits, plan.send_splits, group)
    return ops.combine(y_home, plan.pos, wts)


# ---- compute stages on the device (C-ABI kernels; there is no CPU implementation) ---------------------------------
class KernelOps:
    """gather / experts / combine through the library's kernel-level entry points, for bf16 rows on the current device."""

    def __init__(self, w13, s13, w2, s2, hidden: int, inter: int, local_experts: int, group_size: int = 128):
        import torch

        from . import ffi

        self.ffi, self.lib, self.torch = ffi, ffi.lib(), torch
        self.w13, self.s13, self.w2, self.s2 = w13, s13, w2, s2
        self.hidden, self.inter, self.local_experts, self.group_size = hidden, inter, local_experts, group_size
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._h = None

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _u32(self, a: np.ndarray):
        return self.torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).cuda()

    def gather(self, src, index: np.ndarray):
        torch = self.torch
        rows = int(index.size)
        dst = torch.empty((rows, src.shape[1]), dtype=src.dtype, device="cuda")
        if rows:
            ix = self._u32(index)
            self.ffi.check(self.lib.vyb_k_rows_gather_bf16(src.data_ptr(), ix.data_ptr(), dst.data_ptr(), rows, src.shape[1],
                                                           self._stream()))
        return dst

    def experts(self, rows_sorted, plan: RegroupPlan):
        torch = self.torch
        y = torch.empty((plan.max_rows, self.hidden), dtype=torch.bfloat16, device="cuda")
        if self._h is None or self._h.shape[0] < plan.max_rows:
            self._h = torch.empty((plan.max_rows, self.inter), dtype=torch.bfloat16, device="cuda")
        tiles = self._u32(plan.tile_expert)
        m_tiles = self._u32(np.array([plan.m_tiles], dtype=np.uint32))
        self.ffi.check(self.lib.vyb_k_moe_experts_int4(
            rows_sorted.data_ptr(), self.w13.data_ptr(), self.s13.data_ptr(), self.w2.data_ptr(), self.s2.data_ptr(),
            y.data_ptr(), self._h.data_ptr(), tiles.data_ptr(), m_tiles.data_ptr(), plan.max_rows, self.hidden, self.inter,
            self.local_experts, self.group_size, self._stream(), C.c_void_p(self.status.data_ptr())))
        return y

    def combine(self, y_rows, pos: np.ndarray, wts):
        torch = self.torch
        tokens, topk = pos.shape
        out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16, device="cuda")
        p = self._u32(pos)
        self.ffi.check(self.lib.vyb_k_moe_combine(y_rows.data_ptr(), p.data_ptr(), wts.data_ptr(), out.data_ptr(), tokens,
                                                  self.hidden, topk, self._stream()))
        return out


def route(x, w_router, experts: int, topk: int):
    """Router linear + gate on the device: (idx int32 [tokens, topk], wts f32 [tokens, topk])."""
    import torch

    from . import ffi

    tokens, hidden = x.shape
    idx = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
    wts = torch.empty((tokens, topk), dtype=torch.float32, device="cuda")
    ffi.check(ffi.lib().vyb_k_moe_route(x.data_ptr(), w_router.data_ptr(), idx.data_ptr(), wts.data_ptr(), tokens, hidden,
                                        experts, topk, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return idx, wts


def expert_parallel_moe_ffn(x, w_router, ops: KernelOps, experts: int, topk: int, group=None, max_rows: int | None = None):
    """Full expert-parallel layer for this rank's tokens: route on the device, plan on the host, exchange, compute."""
    idx, wts = route(x, w_router, experts, topk)
    out = expert_parallel_layer(x, idx.cpu().numpy(), wts, experts, ops, group, max_rows)
    return out, idx, wts


# ---- all-gather of column-parallel outputs by the library's peer-store kernel (NVLink, symmetric memory) -------------
class PeerAllGather:
    """Gather buffers for vyb_k_allgather_push: [2][world][m][n] bf16 per rank plus a 32-bit arrival counter, in
    symmetric memory so that every rank holds device addresses of every peer's copy. Halves are used alternately."""

    def __init__(self, m: int, n: int, group=None, slots: int = 2):
        import os

        import torch
        import torch.distributed as dist

        from . import ffi

        self.ffi, self.torch = ffi, torch
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the fused all-gather addresses at most 8 peers")
        if slots < 2:
            raise ValueError("a gather buffer has at least two slots")
        self.m, self.n, self.slots = m, n, slots
        self.data_bytes = (slots * self.world * m * n * 2 + 255) & ~255
        total = self.data_bytes + 256
        if self.world > 1:
            # plain peer mappings are all the kernel needs; no NVLink multicast object is bound to the buffer
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            self.buf = symm.empty(total, dtype=torch.uint8, device="cuda")
            self.buf.zero_()
            torch.cuda.synchronize()
            self.handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device="cuda")
            self.handle = None
            ptrs = [self.buf.data_ptr()]
        self.local = torch.zeros(64, dtype=torch.int32, device="cuda")  # [0] pushes completed
        self.ctx = ffi.AllGatherCtx()
        self.ctx.world, self.ctx.rank = self.world, self.rank
        for r in range(self.world):
            self.ctx.peer_out[r] = ptrs[r]
            self.ctx.peer_flag[r] = ptrs[r] + self.data_bytes
        self.ctx.epoch = self.local.data_ptr()
        self.ctx.slots = slots
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group)  # every counter is zero before anybody launches

    def halves(self):
        """The [world, m, n] bf16 views of the local gather buffer, one per slot (two unless more were asked for)."""
        slots = getattr(self, "slots", 2)
        t = self.buf[: slots * self.world * self.m * self.n * 2].view(self.torch.bfloat16)
        return t.view(slots, self.world, self.m, self.n)

    def local_slice(self, half: int):
        """This rank's [m, n] slice of a buffer half: the output of a plain GEMV that `push` then sends to the peers."""
        return self.halves()[half][self.rank]

    def push(self, half: int, stream, status):
        """Send the local slice of `half` to every peer (kernel on `stream`, normally a side stream)."""
        self.ffi.check(self.ffi.lib().vyb_k_allgather_push(C.byref(self.ctx), half, self.m, self.n, C.c_void_p(stream),
                                                           C.c_void_p(status.data_ptr())))

    def gemv(self, half: int, x, w, scales, k: int, stream, status, flags: int = 0):
        """The shard's decode GEMV and its all-gather in one launch (vyb_k_int4_gemv_allgather): the bf16 outputs go
        straight into this rank's slice of buffer `half` on every rank. Alternate the halves; run `wait` on the stream
        before a gathered result is read."""
        self.ffi.check(self.ffi.lib().vyb_k_int4_gemv_allgather(
            C.byref(self.ctx), half, x.data_ptr(), w.data_ptr(), scales.data_ptr(), self.m, self.n, k, 128, flags,
            C.c_void_p(stream), C.c_void_p(status.data_ptr())))

    def wait(self, stream, status):
        """Bounded device-side wait on `stream` until every gather launched so far is complete in local memory."""
        self.ffi.check(self.ffi.lib().vyb_k_allgather_wait(C.byref(self.ctx), C.c_void_p(stream),
                                                           C.c_void_p(status.data_ptr())))


class PeerColumnGather:
    """Full [m, n_total] output of a column-parallel linear on every rank, assembled by vyb_k_colpar_push: every rank
    stores its columns of a block of rows straight into every rank's buffer (peer stores over NVLink, symmetric
    memory, no staging and no host-side interleave). Blocks are counted: `wait(blocks)` is the consumer-side check.
    The buffer is reused call after call: start the next gather only when its consumers are done on every rank."""

    def __init__(self, m: int, n_total: int, elem_bytes: int, group=None, multiple: int = 4):
        import os

        import torch
        import torch.distributed as dist

        from . import ffi

        self.ffi, self.torch = ffi, torch
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("the peer-store gather addresses at most 8 peers")
        self.m, self.n, self.elem = m, n_total, elem_bytes
        self.begin, self.end = column_shard(n_total, self.world, self.rank, multiple)
        if (n_total * elem_bytes) % 16 or (self.begin * elem_bytes) % 16 or ((self.end - self.begin) * elem_bytes) % 16:
            raise ValueError("rows, shard offsets and shard widths must be multiples of 16 bytes")
        self.data_bytes = (m * n_total * elem_bytes + 255) & ~255
        total = self.data_bytes + 256
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all that is needed
            import torch.distributed._symmetric_memory as symm

            self.buf = symm.empty(total, dtype=torch.uint8, device="cuda")
            self.buf.zero_()
            torch.cuda.synchronize()
            self.handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device="cuda")
            self.handle = None
            ptrs = [self.buf.data_ptr()]
        self.local = torch.zeros(64, dtype=torch.int32, device="cuda")  # launch counters and tickets
        self.ctx = ffi.AllGatherCtx()
        self.ctx.world, self.ctx.rank = self.world, self.rank
        for r in range(self.world):
            self.ctx.peer_out[r] = ptrs[r]
            self.ctx.peer_flag[r] = ptrs[r] + self.data_bytes
        self.ctx.epoch = self.local.data_ptr()
        self.blocks = 0  # blocks pushed so far by every rank (all ranks push the same number)
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group)

    def output(self, dtype):
        return self.buf[: self.m * self.n * self.elem].view(dtype).view(self.m, self.n)

    def push(self, block, row0: int, stream, status):
        """block: this rank's columns [rows, end - begin] of rows [row0, row0 + rows), contiguous."""
        rows, width = block.shape
        assert width == self.end - self.begin and block.is_contiguous()
        self.ffi.check(self.ffi.lib().vyb_k_colpar_push(
            C.byref(self.ctx), block.data_ptr(), rows, width * self.elem, self.n * self.elem,
            (row0 * self.n + self.begin) * self.elem, C.c_void_p(stream), C.c_void_p(status.data_ptr())))
        self.blocks += 1

    def gemm(self, xq, w_rows, stream, status):
        """xq int8 [m, k] . w_rows^T (this rank's rows [begin, end) of W), the int32 outputs stored by the GEMM's own
        epilogue into every rank's full output (vyb_k_int8_gemm_i32_gather): one block delivered everywhere."""
        m, k = xq.shape
        assert m == self.m and w_rows.shape[0] == self.end - self.begin and self.elem == 4
        self.ffi.check(self.ffi.lib().vyb_k_int8_gemm_i32_gather(
            C.byref(self.ctx), xq.data_ptr(), w_rows.data_ptr(), m, w_rows.shape[0], k, self.n * self.elem,
            self.begin * self.elem, C.c_void_p(stream), C.c_void_p(status.data_ptr())))
        self.blocks += 1

    def wait(self, stream, status):
        self.ffi.check(self.ffi.lib().vyb_k_colpar_wait(C.byref(self.ctx), self.blocks, C.c_void_p(stream),
                                                        C.c_void_p(status.data_ptr())))


def column_parallel_int8_linear(gather: PeerColumnGather, xq, w_rows, status, chunks: int = 4, side_stream=None,
                                fused: bool = True):
    """y int32 [m, n_total] = xq int8 [m, k] . W^T with this rank holding rows [begin, end) of W. With more than 128
    rows (the paired tcgen05 kernel) and `fused`, GEMM and gather are one kernel: the epilogue stores every tile into
    every rank's output. Otherwise the GEMM runs in `chunks` row chunks on the current stream, each chunk's columns are
    pushed to every rank on `side_stream` while the next chunk's GEMM runs. Either way the call ends with the bounded
    wait for every rank's blocks. Returns the full output (and the local block of the chunked path, else None)."""
    import torch

    from . import ffi

    L = ffi.lib()
    m, k = xq.shape
    n_local = w_rows.shape[0]
    cur = torch.cuda.current_stream()
    if fused and m > 128 and n_local % 4 == 0 and k % 16 == 0:
        gather.gemm(xq, w_rows, cur.cuda_stream, status)
        gather.wait(cur.cuda_stream, status)
        return gather.output(torch.int32), None
    side = side_stream or cur
    y_local = torch.empty((m, n_local), dtype=torch.int32, device="cuda")
    step = (m + chunks - 1) // chunks
    for r0 in range(0, m, step):
        rows = min(step, m - r0)
        # every chunk but the first runs beside the push of the chunk before it: leave that copy kernel a few SMs
        flags = ffi.LAUNCH_LEAVE_COPY_SMS if (side is not cur and r0 > 0) else 0
        ffi.check(L.vyb_k_int8_gemm_i32_ex(xq[r0:r0 + rows].data_ptr(), w_rows.data_ptr(), y_local[r0:r0 + rows].data_ptr(), rows,
                                           n_local, k, flags, C.c_void_p(cur.cuda_stream), C.c_void_p(status.data_ptr())))
        if side is not cur:
            ev = torch.cuda.Event()
            ev.record(cur)
            side.wait_event(ev)
        gather.push(y_local[r0:r0 + rows], r0, side.cuda_stream, status)
    if side is not cur:
        cur.wait_stream(side)
    gather.wait(cur.cuda_stream, status)
    return gather.output(torch.int32), y_local


# ---- expert-parallel MoE FFN with device-side dispatch / combine (peer stores over NVLink, symmetric memory) --------
class DeviceExpertParallel:
    """One MoE FFN layer over the ranks of a group with no host read-back: vyb_k_moe_ep_ffn_int4.

    Holds the symmetric region (count matrix, arrival counters, expert-sorted activations, return addresses, per-pair
    results) and the local scratch. `w13`, `s13`, `w2`, `s2` are this rank's experts only. Collective: every rank
    calls `forward` the same number of times."""

    def __init__(self, w_router, w13, s13, w2, s2, hidden: int, inter: int, experts: int, topk: int, tokens_local_max: int,
                 tokens_total: int, group_size: int = 128, group=None):
        import os

        import torch
        import torch.distributed as dist

        from . import ffi

        self.ffi, self.torch = ffi, torch
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.w_router, self.w13, self.s13, self.w2, self.s2 = w_router, w13, s13, w2, s2
        self.hidden, self.inter, self.experts, self.topk, self.group_size = hidden, inter, experts, topk, group_size
        self.tokens_local_max, self.tokens_total = tokens_local_max, tokens_total
        self.ctx = ffi.MoeEpCtx()
        sym_bytes, local_bytes = C.c_uint64(0), C.c_uint64(0)
        ffi.check(ffi.lib().vyb_k_moe_ep_sizes(tokens_local_max, tokens_total, hidden, inter, experts, topk, self.world,
                                               C.byref(self.ctx), C.byref(sym_bytes), C.byref(local_bytes)))
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all that is needed
            import torch.distributed._symmetric_memory as symm

            self.region = symm.empty(sym_bytes.value, dtype=torch.uint8, device="cuda")
            self.region.zero_()
            torch.cuda.synchronize()
            self.handle = symm.rendezvous(self.region, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.region = torch.zeros(sym_bytes.value, dtype=torch.uint8, device="cuda")
            self.handle = None
            ptrs = [self.region.data_ptr()]
        self.ctx.world, self.ctx.rank = self.world, self.rank
        for r in range(self.world):
            self.ctx.peer_base[r] = ptrs[r]
        self.local = torch.zeros(local_bytes.value, dtype=torch.uint8, device="cuda")
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group)  # every counter is zero before anybody launches

    def forward(self, x, stream=None):
        """x: this rank's tokens [tokens, hidden] bf16. Returns (out bf16 [tokens, hidden], idx int32, wts f32)."""
        torch = self.torch
        tokens = x.shape[0]
        if tokens > self.tokens_local_max:
            raise ValueError(f"{tokens} tokens exceed the {self.tokens_local_max} this instance was sized for")
        out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16, device="cuda")
        idx = torch.empty((tokens, self.topk), dtype=torch.int32, device="cuda")
        wts = torch.empty((tokens, self.topk), dtype=torch.float32, device="cuda")
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        self.ffi.check(self.ffi.lib().vyb_k_moe_ep_ffn_int4(
            C.byref(self.ctx), x.data_ptr(), self.w_router.data_ptr(), self.w13.data_ptr(), self.s13.data_ptr(),
            self.w2.data_ptr(), self.s2.data_ptr(), out.data_ptr(), idx.data_ptr(), wts.data_ptr(), self.local.data_ptr(),
            tokens, self.tokens_total, self.hidden, self.inter, self.experts, self.topk, self.group_size, C.c_void_p(s),
            C.c_void_p(self.status.data_ptr())))
        return out, idx, wts
