"""Synthetic W4A4 / W4A4H weights built on the GPU, for benchmarks and smoke runs.

`quantize_weights` follows the reference's weight quantizer (quantize_row_w4a4(h)_ref, ggml/src/ggml-quants.c in
patches/llama.cpp-ruquant.patch:2509-2555, 2701-2710): rotate the row (W4A4H), search 13 clip ratios for the scale
s = amax * (1 - 0.025 r) / 7 with the least squared rounding error, round to codes in [-8, 7], pack 144-byte blocks
with the row's unit, code sum, rotation length and clip in each header.  The rotation runs on this library's own
Hadamard kernel; the search is plain torch.  It is an input generator, not part of the MUL_MAT path: the error sums
are accumulated in a different order than the reference's sequential double loop, so a near-tie between two clip
ratios may resolve differently and the blocks are not promised to match the reference's converter bit for bit.
"""
import numpy as np
import torch

from . import BLOCK_BYTES, BLOCK_CODES, TYPE_W4A4H, hadamard_factor, rotate


def quantize_weights(w, type_, clip=0.0, n_rot=None):
    """w: f32 CUDA [N, K] -> uint8 CUDA [N, K/256*144] blocks (legacy header: sum = the row's code sum)."""
    N, K = w.shape
    if type_ == TYPE_W4A4H:
        n_rot = K if n_rot is None else n_rot
        if hadamard_factor(n_rot) is None:
            raise ValueError("no Hadamard of length %d" % n_rot)
        w = rotate(w.contiguous(), n_rot)
    amax = w.abs().amax(dim=1, keepdim=True)
    best_err = torch.full((N, 1), float("inf"), dtype=torch.float64, device=w.device)
    best_s = torch.zeros((N, 1), dtype=torch.float32, device=w.device)
    for r in range(13):
        s = amax * np.float32(1.0 - np.float32(0.025) * np.float32(r)) / np.float32(7.0)
        q = torch.clamp(torch.round(w / torch.where(s > 0, s, torch.ones_like(s))), -8.0, 7.0)
        err = ((q * s - w).double() ** 2).sum(dim=1, keepdim=True)
        better = (err < best_err) & (amax > 0)
        best_err = torch.where(better, err, best_err)
        best_s = torch.where(better, s, best_s)
    safe = torch.where(best_s > 0, best_s, torch.ones_like(best_s))
    codes = torch.where(best_s > 0, torch.clamp(torch.round(w / safe), -8.0, 7.0), torch.zeros_like(w)).to(torch.int32)
    nb = K // BLOCK_CODES
    nib = (codes & 0xF).view(N, nb, 32, 8)
    shifts = (4 * torch.arange(8, device=w.device, dtype=torch.int32)).view(1, 1, 1, 8)
    words = (nib << shifts).sum(dim=-1, dtype=torch.int64).to(torch.int32)            # [N, nb, 32], bit patterns
    hdr = torch.zeros((N, nb, 4), dtype=torch.int32, device=w.device)
    hdr[:, :, 0] = best_s.view(torch.int32).expand(N, nb)
    hdr[:, :, 1] = codes.sum(dim=1, dtype=torch.int32).view(N, 1).expand(N, nb)
    hdr[:, :, 2] = n_rot if type_ == TYPE_W4A4H else K
    hdr[:, :, 3] = int(np.float32(clip).view(np.int32)) if clip > 0 else 0
    blocks = torch.cat([hdr, words], dim=2).contiguous()                               # [N, nb, 36] int32
    return blocks.view(torch.uint8).view(N, nb * BLOCK_BYTES)


def random_weights(N, K, type_, seed, clip=0.0, device="cuda", std=0.02, chunk=4096):
    """fp32 N(0, std) rows, seeded, quantized chunk by chunk to bound the fp32 footprint."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.empty((N, K // BLOCK_CODES * BLOCK_BYTES), dtype=torch.uint8, device=device)
    for r0 in range(0, N, chunk):
        n = min(chunk, N - r0)
        w = torch.randn((n, K), generator=g, device=device, dtype=torch.float32) * std
        out[r0:r0 + n] = quantize_weights(w, type_, clip)
    return out
