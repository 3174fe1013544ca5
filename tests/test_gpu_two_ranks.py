"""GPU, two or more devices: the multi-rank entry points across real NVLink -- one process per GPU, outputs in peer-mapped
buffers (torch symmetric memory for the mapping only), every result bit for bit against the oracle.

  * N split: rq_w4a4_mul_mat_push stores each rank's columns into every rank's [M][N] output, rq_rank_barrier releases
    them; M = 1 and 9 take the GEMV, M = 200 the tensor-core kernel (a pair of CTAs).
  * K split: every rank multiplies its slice of x by its block columns, rq_w4a4_sum_partials adds the partials in rank
    order, one shot and two shot; the oracle adds the same partials in the same order.
  * shared quantizer: every rank rotates and quantizes its own range of tokens, rq_w4a4_share_rows carries the range
    into the other ranks' workspaces, and every rank then multiplies all tokens.

Skipped with fewer than two devices.  A rank that fails checks its asserts only after its stream is idle, and the waits
of rq_rank_barrier are bounded, so a failure ends the test instead of hanging it; NVLS is off for NCCL.
"""
import os
import socket
import traceback

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import datetime

    import torch.distributed as dist

    failures = []
    try:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
        import torch.distributed._symmetric_memory as symm

        import oracle
        import ruquant_b200 as rq
        from tests import inputs

        rq.lib()
        port_ = oracle.Port()

        def mapped(n, dtype=torch.float32):
            t = symm.empty(n, dtype=dtype, device=dev)
            t.zero_()
            h = symm.rendezvous(t, dist.group.WORLD)
            return t, [int(p) for p in h.buffer_ptrs], h

        flags, flag_ptrs, keep_f = mapped(64, torch.int32)
        epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        dist.barrier()

        def meet():
            rq.rank_barrier(flag_ptrs, rank, epoch, status)

        def check(got, want, what):
            if not (inputs.bits(got) == inputs.bits(want)).all():
                failures.append("%s: %d of %d outputs differ on rank %d" % (what, int((inputs.bits(got) != inputs.bits(want)).sum()), want.size, rank))

        # ---- N split: rank r holds rows [r*nl, (r+1)*nl)
        K, N = 1536, 128 * world
        nl = N // world
        wb = port_.quantize_weights(inputs.normal_weights(N, K, 6100), 45)
        w = rq.Weight(torch.from_numpy(wb[rank * nl:(rank + 1) * nl].copy()).to(dev).view(-1), 45, K, N=nl)
        order = [rank] + [r for r in range(world) if r != rank]          # own buffer first
        for M in (1, 9, 200):
            x = inputs.outlier_activations(M, K, 6110 + M)
            y, y_ptrs, keep_y = mapped(M * N)
            meet()                                                      # every rank's buffer is zeroed before anyone stores
            rq.mul_mat_push([w], torch.from_numpy(x).to(dev), [[y_ptrs[d] + 4 * rank * nl] for d in order], [N])
            meet()
            torch.cuda.synchronize()
            check(y.view(M, N).cpu().numpy(), port_.mul_mat(wb, 45, K, x), "N split, M=%d" % M)
            del keep_y

        # ---- K split: a slice is a W4A4H tensor of its own (its own rotation block, its own range per token)
        ks, Nk = 1024, 320
        wf = inputs.normal_weights(Nk, ks * world, 6200)
        slices = [port_.quantize_weights(np.ascontiguousarray(wf[:, r * ks:(r + 1) * ks]), 45) for r in range(world)]
        wk = rq.Weight(torch.from_numpy(slices[rank]).to(dev).view(-1), 45, ks, N=Nk)
        for M in (1, 130):
            x = inputs.outlier_activations(M, ks * world, 6210 + M)
            want = None
            for r in range(world):
                p = port_.mul_mat(slices[r], 45, ks, np.ascontiguousarray(x[:, r * ks:(r + 1) * ks]))
                want = p if want is None else (want + p).astype(np.float32)
            part, part_ptrs, keep_p = mapped(M * Nk)
            y1 = torch.zeros(M * Nk, dtype=torch.float32, device=dev)
            y2, y2_ptrs, keep_2 = mapped(M * Nk)
            xs = torch.from_numpy(np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks])).to(dev)
            rq.mul_mat(wk, xs, out=part.view(M, Nk))
            meet()
            rq.sum_partials(part_ptrs, rank, M * Nk, [y1.data_ptr() if r == rank else 0 for r in range(world)])
            rq.sum_partials(part_ptrs, rank, M * Nk, y2_ptrs, two_shot=True)
            meet()
            torch.cuda.synchronize()
            check(y1.view(M, Nk).cpu().numpy(), want, "K split one shot, M=%d" % M)
            check(y2.view(M, Nk).cpu().numpy(), want, "K split two shot, M=%d" % M)
            del keep_p, keep_2
        # ---- shared quantizer: token ranges quantized apart, exchanged through workspaces mapped into one another
        K, N, M = 5120, 192, 70
        wb = port_.quantize_weights(inputs.normal_weights(N, K, 6300), 45)
        w = rq.Weight(torch.from_numpy(wb).to(dev).view(-1), 45, K, N=N)
        x = inputs.outlier_activations(M, K, 6301)
        ws, ws_ptrs, keep_w = mapped(rq.workspace_bytes(K, M), torch.uint8)
        rq.init_workspace(ws, K, M)
        lo, hi = rank * M // world, (rank + 1) * M // world
        fmt = rq.act_format(w, M)
        meet()                                                          # every workspace is initialised
        rq.quantize_rows(torch.from_numpy(x[lo:hi]).to(dev), M, lo, w.n_rot, 1.0, 64, fmt, ws)
        rq.share_rows(ws_ptrs, rank, ws.numel(), K, M, 64, lo, hi - lo)
        meet()
        y = rq.mul_mat_quantized(w, M, ws, act_group=64)
        torch.cuda.synchronize()
        check(y.cpu().numpy(), port_.mul_mat(wb, 45, K, x), "shared quantizer")
        meet()
        del keep_w
        torch.cuda.synchronize()
        if int(status.item()) != 0:
            failures.append("rank %d: a barrier's bounded wait expired (status %d)" % (rank, int(status.item())))
        dist.barrier()
        del keep_f
        dist.destroy_process_group()
    except Exception:      # noqa: BLE001 -- reported to the parent
        failures.append("rank %d: %s" % (rank, traceback.format_exc()))
        try:
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001
            pass
    results.put((rank, failures))


def test_push_and_partial_sums_across_devices():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    got = []
    try:
        for _ in range(world):
            got.append(results.get(timeout=600))
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    failures = [f for _r, fs in got for f in fs]
    assert len(got) == world and not failures, "\n".join(failures)
