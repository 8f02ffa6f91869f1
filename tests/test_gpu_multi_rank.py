"""Two ranks on two GPUs (NCCL): expert-parallel MoE FFN and column-parallel int8 linear against the single-GPU kernels.

Skipped on a box with fewer than two GPUs. Each rank is a child process; results must be bit-identical to the
single-GPU path because every output row is computed by the same kernel arithmetic wherever it is placed.
"""
import ctypes as C
import datetime
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    from vyre_b200 import ffi, sharding, synth

    torch.cuda.set_device(rank)
    # a short collective timeout: if one rank fails between collectives, the other's next collective ends with an
    # error instead of waiting forever
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=45))
    failed = False
    try:
        L = ffi.lib()
        stream = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
        # ---- expert-parallel MoE FFN -------------------------------------------------------------------------
        tokens, hidden, inter, experts, topk = 640, 512, 768, 8, 2
        x, wr, w13, s13, w2, s2 = synth.moe_ffn_inputs(tokens, hidden, inter, experts, seed=11)
        dev = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()  # noqa: E731
        tx, twr, tw13, ts13, tw2, ts2 = (dev(a) for a in (x, wr, w13, s13, w2, s2))
        tx = tx.view(torch.bfloat16)  # NCCL moves bf16 rows, not int16 views
        # single-GPU reference: the fused layer over all tokens
        need = C.c_uint64(0)
        ffi.check(L.vyb_k_moe_ffn_int4_scratch_bytes(tokens, hidden, inter, experts, topk, C.byref(need)))
        ref_out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
        ref_idx = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
        ref_w = torch.empty((tokens, topk), dtype=torch.float32, device="cuda")
        scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        ffi.check(L.vyb_k_moe_ffn_int4(tx.data_ptr(), twr.data_ptr(), tw13.data_ptr(), ts13.data_ptr(), tw2.data_ptr(),
                                       ts2.data_ptr(), ref_out.data_ptr(), ref_idx.data_ptr(), ref_w.data_ptr(),
                                       scratch.data_ptr(), need.value, tokens, hidden, inter, experts, topk, 128, stream(),
                                       C.c_void_p(status.data_ptr())))
        torch.cuda.synchronize()
        assert status.cpu().tolist() == [0, 0, 0, 0]
        # expert-parallel: this rank's tokens and experts
        local = experts // world
        t0, t1 = rank * tokens // world, (rank + 1) * tokens // world
        ops = sharding.KernelOps(tw13[rank * local:(rank + 1) * local].contiguous(), ts13[rank * local:(rank + 1) * local].contiguous(),
                                 tw2[rank * local:(rank + 1) * local].contiguous(), ts2[rank * local:(rank + 1) * local].contiguous(),
                                 hidden, inter, local)
        out, idx, wts = sharding.expert_parallel_moe_ffn(tx[t0:t1].contiguous(), twr, ops, experts, topk)
        torch.cuda.synchronize()
        assert ops.status.cpu().tolist() == [0, 0, 0, 0]
        assert torch.equal(idx, ref_idx[t0:t1]) and torch.equal(wts, ref_w[t0:t1])
        assert torch.equal(out.view(torch.int16), ref_out[t0:t1].view(torch.int16))

        # ---- the same layer with device-side dispatch / combine over peer memory: several layers in a row ------------
        dep = sharding.DeviceExpertParallel(twr, ops.w13, ops.s13, ops.w2, ops.s2, hidden, inter, experts, topk,
                                            tokens_local_max=t1 - t0, tokens_total=tokens)
        for rep in range(3):
            out2, idx2, wts2 = dep.forward(tx[t0:t1].contiguous())
            torch.cuda.synchronize()
            assert dep.status.cpu().tolist() == [0, 0, 0, 0], f"layer {rep}"
            assert torch.equal(idx2, ref_idx[t0:t1]) and torch.equal(wts2, ref_w[t0:t1])
            assert torch.equal(out2.view(torch.int16), ref_out[t0:t1].view(torch.int16)), f"layer {rep}"

        # ---- column-parallel dynamic int8 linear + all-gather ----------------------------------------------------
        m, n, k = 256, 1000, 512
        g = torch.Generator().manual_seed(5)
        xa = (torch.randn(m, k, generator=g) * 2).to(torch.bfloat16).cuda()
        wa = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda()

        def int8_linear(w_rows):
            xq = torch.empty((m, k), dtype=torch.int8, device="cuda")
            sc = torch.empty(m, dtype=torch.float32, device="cuda")
            y = torch.empty((m, w_rows.shape[0]), dtype=torch.int32, device="cuda")
            ffi.check(L.vyb_k_quantize_per_token_int8(xa.data_ptr(), xq.data_ptr(), sc.data_ptr(), m, k, stream()))
            ffi.check(L.vyb_k_int8_gemm_i32(xq.data_ptr(), w_rows.data_ptr(), y.data_ptr(), m, w_rows.shape[0], k, stream(),
                                            C.c_void_p(status.data_ptr())))
            return y

        full = int8_linear(wa)
        b, e = sharding.column_shard(n, world, rank, multiple=8)
        gathered = sharding.all_gather_columns(int8_linear(wa[b:e].contiguous()), n, multiple=8)
        torch.cuda.synchronize()
        assert status.cpu().tolist() == [0, 0, 0, 0]
        assert torch.equal(gathered, full)
        # the same through the library's own peer-store gather: chunks of rows, pushes on a side stream, twice in a row
        xq = torch.empty((m, k), dtype=torch.int8, device="cuda")
        sc = torch.empty(m, dtype=torch.float32, device="cuda")
        ffi.check(L.vyb_k_quantize_per_token_int8(xa.data_ptr(), xq.data_ptr(), sc.data_ptr(), m, k, stream()))
        pcg = sharding.PeerColumnGather(m, n, 4, multiple=8)
        side = torch.cuda.Stream()
        for rep in range(4):  # twice by copy kernels behind row chunks, twice by the GEMM's own gathering epilogue
            got, _ = sharding.column_parallel_int8_linear(pcg, xq, wa[pcg.begin:pcg.end].contiguous(), status, chunks=3,
                                                          side_stream=side, fused=rep >= 2)
            torch.cuda.synchronize()
            assert status.cpu().tolist() == [0, 0, 0, 0]
            assert torch.equal(got, full), f"peer-store column gather, pass {rep}"
            dist.barrier()
            got.zero_()
            torch.cuda.synchronize()
            dist.barrier()
        # ---- decode GEMV + the library's peer-store all-gather, against NCCL's all-gather ---------------------------
        # two batch rows: the plain launch and the gathering launch run the same integer kernel, so the gathered bytes
        # must equal NCCL's all-gather of the plain results bit for bit (from three rows on the plain launch takes the f16
        # tensor path, whose results agree with the gathering form only to rounding)
        m, n, k = 2, 2048, 4096
        xg, wg, sg = synth.int4_linear_inputs(m, n, k, seed=40 + rank)
        xg = synth.int4_linear_inputs(m, n, k, seed=40)[0]  # activations are replicated
        tx2, tw2_, ts2_ = dev(xg), torch.from_numpy(wg).cuda(), dev(sg)
        cur = torch.cuda.current_stream().cuda_stream
        y_local = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ffi.check(L.vyb_k_int4_gemv_ex(tx2.data_ptr(), tw2_.data_ptr(), ts2_.data_ptr(), y_local.data_ptr(), m, n, k, 128,
                                       ffi.DT_BF16, 0, C.c_void_p(cur), C.c_void_p(status.data_ptr())))
        want_all = torch.empty((world, m, n), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want_all.view(-1), y_local.view(-1))
        # plain GEMV into the local slice of a buffer half, then the push kernel; both halves, several times
        pag2 = sharding.PeerAllGather(m, n)
        for step in range(4):
            half = step & 1
            ffi.check(L.vyb_k_int4_gemv_ex(tx2.data_ptr(), tw2_.data_ptr(), ts2_.data_ptr(), pag2.local_slice(half).data_ptr(),
                                           m, n, k, 128, ffi.DT_BF16, 0, C.c_void_p(cur), C.c_void_p(status.data_ptr())))
            pag2.push(half, cur, status)
            pag2.wait(cur, status)
            torch.cuda.synchronize()
            assert status.cpu().tolist() == [0, 0, 0, 0]
            assert torch.equal(pag2.halves()[half].view(torch.int16), want_all.view(torch.int16)), f"push step {step}"
            pag2.halves()[half].zero_()
            torch.cuda.synchronize()
            dist.barrier()
        # ---- GEMV and gather in one launch (peer stores from the reduction), a chain of launches, then the wait ------
        pag3 = sharding.PeerAllGather(m, n)
        for rounds in range(4):  # two rounds with the stores in the producing launch, two with the pipelined form
            flags = ffi.LAUNCH_CONSTANT_WEIGHTS | (ffi.LAUNCH_PIPELINED_GATHER if rounds >= 2 else 0)
            for step in range(6):  # halves alternate; programmatic chain, no host sync in between
                pag3.gemv(step & 1, tx2, tw2_, ts2_, k, cur, status, flags)
            pag3.wait(cur, status)
            torch.cuda.synchronize()
            assert status.cpu().tolist() == [0, 0, 0, 0]
            for half in (0, 1):
                assert torch.equal(pag3.halves()[half].view(torch.int16), want_all.view(torch.int16)), f"fused gather {rounds}/{half}"
            dist.barrier()
            pag3.halves().zero_()
            torch.cuda.synchronize()
            dist.barrier()
        q.put((rank, "ok"))
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        import traceback

        failed = True
        q.put((rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        torch.cuda.synchronize()
        if not failed:  # a failed rank leaves between steps with nothing in flight; its peer times out on the host
            dist.barrier()
            dist.destroy_process_group()


def _run(world: int):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in procs:
        try:
            results.append(q.get(timeout=150))
        except Exception:  # noqa: BLE001 - a rank that was aborted by the collective timeout reports nothing
            results.append((-1, "no report"))
    for p in procs:
        p.join(timeout=90)
        if p.is_alive():
            p.terminate()
    assert sorted(results) == [(r, "ok") for r in range(world)], results


def test_sharded_path_with_one_rank_matches_single_gpu():
    """World of one: the whole expert-parallel / column-parallel flow (plans, exchanges with itself, kernels)."""
    _run(1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_and_column_parallel_match_single_gpu():
    _run(2)
