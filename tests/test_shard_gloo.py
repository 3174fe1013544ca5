"""The two multi-rank splits of the node as world_size-2 gloo jobs on CPU: each rank computes its piece with the oracle
(the GPU kernels are checked against the same oracle elsewhere), the exchange goes through torch.distributed."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from ruquant_b200 import shard
from tests import inputs

K, N, M = 2048, 64, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(rot_blocks):
    port = oracle.Port()
    w = inputs.normal_weights(N, K, 8100)
    x = inputs.outlier_activations(M, K, 8101)
    return port, port.quantize_weights(w, 45, rot_blocks=rot_blocks, threads=1), x


def _rows_worker(rank, world, tcp, out):
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % tcp, rank=rank, world_size=world)
    port, wb, x = _case(1)
    mine = np.ascontiguousarray(shard.row_shard(wb, N, K, rank, world))
    y = port.mul_mat(mine, 45, K, x, threads=1)
    full = shard.gather_rows(torch.from_numpy(y))
    want = port.mul_mat(wb, 45, K, x, threads=1)
    ok = bool((full.numpy().view(np.uint32) == want.view(np.uint32)).all())
    if rank == 0:
        with open(out, "w") as f:
            f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def _cols_worker(rank, world, tcp, out):
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % tcp, rank=rank, world_size=world)
    port, wb, x = _case(world)
    ks = K // world
    mine = np.ascontiguousarray(shard.col_shard(wb, N, K, rank, world))
    part = port.mul_mat(mine, 45, ks, np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks]), threads=1)
    total = shard.sum_partials(torch.from_numpy(part))
    want = None
    for r in range(world):   # the same composition on one process, in rank order
        p = port.mul_mat(np.ascontiguousarray(shard.col_shard(wb, N, K, r, world)), 45, ks,
                         np.ascontiguousarray(x[:, r * ks:(r + 1) * ks]), threads=1)
        want = p if want is None else want + p
    ok = bool((total.numpy().view(np.uint32) == want.view(np.uint32)).all())
    gathered = [None] * world
    dist.all_gather_object(gathered, total.numpy().tobytes())
    ok = ok and all(g == gathered[0] for g in gathered)          # every rank holds the same bits
    if rank == 0:
        with open(out, "w") as f:
            f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def _tokens_worker(rank, world, tcp, out):
    """Ranks sharing the quantizer: each quantizes its range of tokens (the oracle stands in for rq_w4a4_quantize_rows),
    the ranges are exchanged in place, every rank then holds what quantizing all tokens gives."""
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % tcp, rank=rank, world_size=world)
    port = oracle.Port()
    Mt = 6
    x = inputs.outlier_activations(Mt, K, 8300)
    whole = port.quantize_act(x, 0.9, 64, K)                              # [Mt, K/256*144] activation blocks
    u_all, m_all, z_all, q_all = oracle.act_fields(whole, 64)
    lo, hi = shard.token_range(Mt, rank, world)
    mine = port.quantize_act(np.ascontiguousarray(x[lo:hi]), 0.9, 64, K)
    u, m, z, q = oracle.act_fields(mine, 64)
    codes = torch.zeros((Mt, K), dtype=torch.int8)
    mult = torch.zeros((Mt, K // 64), dtype=torch.int32)
    unit = torch.zeros((Mt,), dtype=torch.float32)
    codes[lo:hi] = torch.from_numpy((q - np.repeat(z, 64, axis=1)).astype(np.int8))
    mult[lo:hi] = torch.from_numpy(m.astype(np.int32))
    unit[lo:hi] = torch.from_numpy(u)
    shard.exchange_token_ranges([codes, mult, unit], rank)
    ok = bool((codes.numpy() == (q_all - np.repeat(z_all, 64, axis=1))).all() and (mult.numpy() == m_all).all() and
              (unit.numpy().view(np.uint32) == u_all.view(np.uint32)).all())
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        with open(out, "w") as f:
            f.write("ok" if all(flags) else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_rows_worker, _cols_worker, _tokens_worker], ids=["rows", "columns", "tokens"])
def test_two_ranks(tmp_path, worker):
    out = str(tmp_path / "result")
    mp.spawn(worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read() == "ok"


def test_shard_geometry():
    wb = np.arange(4 * 4 * 144, dtype=np.uint32).astype(np.uint8).reshape(4, 4 * 144)
    assert shard.row_shard(wb, 4, 1024, 1, 2).shape == (2, 576) and (shard.row_shard(wb, 4, 1024, 1, 2) == wb[2:]).all()
    c = shard.col_shard(wb, 4, 1024, 1, 2)
    assert c.shape == (4, 288) and (c == wb[:, 288:]).all()
    with pytest.raises(ValueError):
        shard.col_shard(wb, 4, 1024, 0, 8)       # 128 inputs per rank: not whole blocks
    with pytest.raises(ValueError):
        shard.row_range(5, 0, 2)
    # a K slice of a W4A4H tensor rotated over the whole row cannot be multiplied: the oracle refuses, as the reference aborts
    port = oracle.Port()
    w = port.quantize_weights(inputs.normal_weights(8, 1024, 8200), 45)
    with pytest.raises(Exception):
        port.mul_mat(np.ascontiguousarray(shard.col_shard(w, 8, 1024, 0, 2)), 45, 512, np.zeros((1, 512), np.float32))
