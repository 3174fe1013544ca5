"""Splitting a W4A4 / W4A4H MUL_MAT over ranks (host side; the compute stays the one-GPU node on each rank's piece).

Two ways, both from the reference:

* rows (N): rank r holds weight rows [r*N/g, (r+1)*N/g) as ordinary blocks, every rank quantizes the same x, the
  outputs are gathered along N.  No arithmetic crosses ranks, so the result has the one-GPU bits.
* columns (K), the reference's tensor-parallel mode for attn_output / ffn_down: rank r holds the block columns of
  inputs [r*K/g, (r+1)*K/g) and that slice of x, quantizes it on its own (its own range and unit) and produces a
  partial Y; the partials are summed.  A W4A4H tensor must have been converted with a block-diagonal rotation whose
  length divides the slice (`ruquant convert --rot-blocks`, src/convert.rs:120-128; ggml_rq_rot_check,
  patches/llama.cpp-ruquant.patch:2612-2620 aborts otherwise -- here rq_w4a4_prepare returns RQ_ERR_ROTATION).  The sum
  is taken in rank order on every rank, so all ranks hold the same bits and a CPU restatement can reproduce them
  (a ring all-reduce would not promise an order).

* tokens (M), for wide inputs on row-split ranks: the rotate + quantize step is per token, so rank r does tokens
  [r*M/g, (r+1)*M/g) (rq_w4a4_quantize_rows) and the ranks exchange the results -- one byte per input, a multiplier per
  group, a unit per token: a quarter of what x itself takes -- before each multiplies all tokens by its own rows.
  Identical bits by construction.

torch.distributed is used for the exchange only; the functions work with any backend (gloo on CPU tensors in the
tests, NCCL on CUDA tensors on the GPUs).  On the GPUs the outputs of row-split ranks and the partials of column-split
ranks can also travel without a collective: rq_w4a4_mul_mat_push / rq_rank_barrier / rq_w4a4_sum_partials over
peer-mapped buffers (ruquant_b200.mul_mat_push, rank_barrier, sum_partials).
"""
BLOCK_CODES, BLOCK_BYTES = 256, 144


def row_range(N, rank, world):
    if N % world:
        raise ValueError("N = %d does not split over %d ranks" % (N, world))
    n = N // world
    return rank * n, (rank + 1) * n


def row_shard(blocks, N, K, rank, world):
    """blocks: [N, K/256*144] uint8 (numpy or torch).  The rank's rows, a view."""
    lo, hi = row_range(N, rank, world)
    return blocks.reshape(N, K // BLOCK_CODES * BLOCK_BYTES)[lo:hi]


def col_shard(blocks, N, K, rank, world):
    """The rank's block columns [N, (K/world)/256*144]: whole blocks only.  A strided view; make it contiguous before
    handing it to the library."""
    if K % (world * BLOCK_CODES):
        raise ValueError("K = %d does not split into %d slices of whole blocks" % (K, world))
    nb = K // world // BLOCK_CODES
    rows = blocks.reshape(N, K // BLOCK_CODES, BLOCK_BYTES)
    return rows[:, rank * nb:(rank + 1) * nb].reshape(N, nb * BLOCK_BYTES)


def gather_rows(y_local, group=None):
    """[M, N/g] per rank -> [M, N] on every rank (rank r's columns at [r*N/g, (r+1)*N/g))."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [torch.empty_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def sum_partials(y_partial, group=None):
    """[M, N] partial per rank -> the fp32 sum ((p0 + p1) + p2) + ... on every rank, the same bits everywhere."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [torch.empty_like(y_partial) for _ in range(world)]
    dist.all_gather(parts, y_partial.contiguous(), group=group)
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    return total


def token_range(M, rank, world):
    """Tokens [lo, hi) rank `rank` rotates and quantizes when the ranks share that work."""
    if M % world:
        raise ValueError("M = %d does not split over %d ranks" % (M, world))
    n = M // world
    return rank * n, (rank + 1) * n


def exchange_token_ranges(regions, rank, group=None, scratch=None):
    """regions: tensors whose first dimension is the token (the workspace's codes [M, K], multipliers [M, K/G], units
    [M]), each holding this rank's token range already; on return every rank holds all ranges.  In place: the own range
    is copied out first (to `scratch[i]` if given, a tensor shaped like the range), then all-gathered into the region."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    for i, region in enumerate(regions):
        lo, hi = token_range(region.shape[0], rank, world)
        tmp = scratch[i] if scratch is not None else torch.empty_like(region[lo:hi])
        tmp.copy_(region[lo:hi])
        dist.all_gather_into_tensor(region.view(-1), tmp.view(-1), group=group)
