"""Host-side sharding logic under world_size-2 gloo on CPU: column-parallel all-gather and the expert-parallel MoE
exchange (dispatch plan, counts all-to-all, row all-to-all, regrouping into padded expert segments, return, combine).

The compute stages are stand-ins defined here (a fake expert that scales a row by its global expert id + 1); the real
ones are CUDA kernels and are exercised by the GPU tests.
"""
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vyre_b200 import sharding


class TorchOps:
    """CPU stand-ins with the semantics of the device stages."""

    def __init__(self, rank: int, local_experts: int):
        self.rank, self.local = rank, local_experts

    def gather(self, src, index):
        index = np.asarray(index, dtype=np.uint32)
        out = torch.zeros((index.size, src.shape[1]), dtype=src.dtype)
        keep = index != sharding.PAD
        if keep.any():
            out[torch.from_numpy(keep)] = src[torch.from_numpy(index[keep].astype(np.int64))]
        return out

    def experts(self, rows_sorted, plan):
        assert rows_sorted.shape[0] == plan.max_rows and plan.max_rows % sharding.ROW_TILE == 0
        y = torch.full_like(rows_sorted, float("nan"))  # rows past the planned tiles must never be read back
        for t in range(plan.m_tiles):
            e_global = self.rank * self.local + int(plan.tile_expert[t])
            sl = slice(t * sharding.ROW_TILE, (t + 1) * sharding.ROW_TILE)
            y[sl] = rows_sorted[sl] * float(e_global + 1)
        return y

    def combine(self, y_rows, pos, wts):
        pos_t = torch.from_numpy(np.asarray(pos, dtype=np.int64))
        return (y_rows[pos_t] * wts.unsqueeze(-1)).sum(dim=1)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_q):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # ---- column-parallel: ragged shards of n = 10 over 2 ranks ------------------------------------------
        n, m = 10, 3
        b, e = sharding.column_shard(n, world, rank)
        full = torch.arange(m * n, dtype=torch.float32).reshape(m, n)
        got = sharding.all_gather_columns(full[:, b:e].clone(), n)
        assert torch.equal(got, full)

        # ---- expert-parallel: different token counts per rank, an expert nobody picks, one everybody picks ---
        experts, topk, hidden = 4, 2, 8
        tokens = 5 + 300 * rank  # rank 1 sends more than one 256-row tile to a single expert
        g = np.random.default_rng(100 + rank)
        x = torch.from_numpy(g.standard_normal((tokens, hidden)).astype(np.float32))
        idx = np.empty((tokens, topk), dtype=np.int64)
        idx[:, 0] = 3                                   # every token picks expert 3 (owned by rank 1)
        idx[:, 1] = g.integers(0, 2, size=tokens)       # and one of experts 0/1 (rank 0); expert 2 stays empty
        wts = torch.from_numpy(g.uniform(0.1, 0.9, size=(tokens, topk)).astype(np.float32))
        ops = TorchOps(rank, experts // world)
        out = sharding.expert_parallel_layer(x, idx, wts, experts, ops)
        want = sum(wts[:, j:j + 1] * x * torch.from_numpy((idx[:, j] + 1).astype(np.float32)).unsqueeze(-1)
                   for j in range(topk))
        assert torch.allclose(out, want, rtol=1e-6, atol=1e-6)
        result_q.put((rank, "ok"))
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        result_q.put((rank, f"{type(exc).__name__}: {exc}"))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_column_and_expert_parallel_exchange_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_column_shard_covers_rows_once():
    for n, world, mult in [(14336, 8, 128), (28672, 4, 256), (10, 3, 1), (1000, 8, 64)]:
        bounds = [sharding.column_shard(n, world, r, mult) for r in range(world)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        for (b0, e0), (b1, e1) in zip(bounds, bounds[1:]):
            assert e0 == b1 and b0 <= e0
        with pytest.raises(ValueError):
            sharding.column_shard(n, world, world)


def test_dispatch_and_regroup_plans_are_consistent():
    g = np.random.default_rng(3)
    tokens, topk, experts, world = 37, 2, 8, 4
    idx = np.stack([g.permutation(experts)[:topk] for _ in range(tokens)])
    plan = sharding.plan_dispatch(idx, experts, world)
    flat = idx.reshape(-1)
    assert sorted(plan.pos.reshape(-1).tolist()) == list(range(tokens * topk))
    assert np.all(np.diff(flat[np.argsort(plan.pos.reshape(-1))]) >= 0)          # send buffer is sorted by expert
    assert np.array_equal(plan.send_order[plan.pos], np.repeat(np.arange(tokens), topk).reshape(tokens, topk))
    assert sum(plan.send_splits) == tokens * topk
    recv_counts = np.array([[3, 0], [300, 2], [0, 0], [1, 255]])
    rg = sharding.plan_regroup(recv_counts)
    assert rg.m_tiles == 2 + 2 and rg.max_rows >= rg.m_tiles * sharding.ROW_TILE     # 304 -> 2 tiles, 257 -> 2 tiles
    assert rg.tile_expert[: rg.m_tiles].tolist() == [0, 0, 1, 1]
    valid = rg.src_index != sharding.PAD
    assert np.array_equal(np.sort(rg.src_index[valid]), np.arange(recv_counts.sum()))
    assert np.array_equal(rg.src_index[rg.ret_index], np.arange(recv_counts.sum()))
    with pytest.raises(ValueError):
        sharding.plan_regroup(recv_counts, max_rows=512)
    with pytest.raises(ValueError):
        sharding.plan_dispatch(idx, experts, 3)
