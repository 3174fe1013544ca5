"""Synthetic W4A4 / W4A4H weights for benchmarks and smoke runs: seeded fp32 N(0, std) rows quantized by the
library's own GPU weight quantizer (rq_w4a4_quantize_weights, bit-identical to the reference's quantize_w4a4 /
quantize_w4a4h, patches/llama.cpp-ruquant.patch:2775-2789), chunk by chunk to bound the fp32 footprint."""
import torch

from . import BLOCK_BYTES, BLOCK_CODES, quantize_weights


def random_weights(N, K, type_, seed, device="cuda", std=0.02, chunk=4096, wgroup=0, rot_blocks=1):
    """uint8 CUDA [N, K/256*144]: the reference's blocks of N rows drawn from N(0, std) with the given seed."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.empty((N, K // BLOCK_CODES * BLOCK_BYTES), dtype=torch.uint8, device=device)
    for r0 in range(0, N, chunk):
        n = min(chunk, N - r0)
        w = torch.randn((n, K), generator=g, device=device, dtype=torch.float32) * std
        out[r0:r0 + n] = quantize_weights(w, type_, wgroup, rot_blocks)
    return out
