// One-time re-layout of a W4A4 / W4A4H weight into what the contraction kernels stream.  The 144-byte blocks are only
// read.  (The reference re-packs in place on first use: rq_repack_kernel / rq_colsum_kernel / rq_wk_kernel,
// ggml/src/ggml-cuda/rq-w4a4.cu in patches/llama.cpp-ruquant.patch:1842-1880.)
//
//   sw  f32 [N]        the row unit s_w (block 0 of each row; every block of a row repeats it)
//   w4  u32 [ceil(N/16) tiles][K/64 runs][32 lanes][4 words]   decode stream in consumption order: lane l = 4*gid + tig
//                      of the GEMV warp loads its 16 bytes and unpacks word j into two int8x4 registers,
//                      `(w << 4) & 0xF0F0F0F0` = 16*c of row tile*16 + gid and `w & 0xF0F0F0F0` = 16*c of row
//                      tile*16 + gid + 8, inputs run*64 + (j/2)*32 + (j%2)*16 + tig*4 .. +3 -- exactly the A fragment
//                      of mma.m16n8k32 (a nibble moved to the top of its byte is 16*c in two's complement: no sign
//                      fix-up).  Rows beyond N are zero.
//   w8  u8  [N][K]     tensor-core operand: the e4m3 byte of c when every multiplier is 1 (fp8 MMA, fp32 accumulate,
//                      exact on these integers), else int8 k*c (|k*c| <= 120, integer MMA), permuted
//                      inside each run of 64 inputs like the activations (rq_perm64)
//   wk  i8  [N][K/64]  the multiplier of each run of 64 inputs (RQ_W_MULT_G, patch:40-43), only when some k != 1
#include "rq_common.cuh"

namespace {

__global__ void rq_scan_wk_kernel(const rq_block * __restrict__ blocks, int64_t n_blocks, int32_t * flag) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    const int32_t s = blocks[i].sum;
    bool any = false;
    for (int g = 0; g < 4; ++g) any |= rq_wmult(s, g) != 1;
    if (any) atomicOr(flag, 1);
}

// a thread per (row, word of 8 codes)
__global__ void rq_prepack_kernel(const rq_block * __restrict__ blocks, int64_t K, int64_t N, float * __restrict__ sw,
                                  int8_t * __restrict__ w8, int8_t * __restrict__ wk, int wk_mode) {
    const int64_t words = K / 8;
    const int64_t idx = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * words) return;
    const int64_t row = idx / words, w = idx - row * words;
    const rq_block * b = blocks + row * (K / RQ_BLOCK_CODES) + w / 32;
    const uint32_t src = b->qs[w % 32];
    const int g64 = (int) ((w % 32) / 8);
    const int k = rq_wmult(b->sum, g64);
    if (w == 0) sw[row] = b->d;
    if (wk != nullptr && (w % 8) == 0) wk[row * (K / 64) + w / 8] = (int8_t) k;
    if (w8 != nullptr) {
        uint32_t pk[2] = { 0u, 0u };
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = ((int) (((src >> (4 * j)) & 0xFu) << 28)) >> 28;
            // multipliers present: int8 k*c for the integer MMA; else the e4m3 byte of c (|c| <= 8, exact) for the fp8 MMA
            const uint32_t byte = wk_mode ? (uint32_t) ((c * k) & 0xFF) : rq_e4m3_of_int(c);
            pk[j >> 2] |= byte << (8 * (j & 3));
        }
        const int64_t kw = w * 8, run = kw & ~(int64_t) 63;
        const int off = (int) (kw & 63);                     // same permutation as the activations (rq_perm64)
        *reinterpret_cast<uint32_t *>(w8 + row * K + run + rq_perm64(off)) = pk[0];
        *reinterpret_cast<uint32_t *>(w8 + row * K + run + rq_perm64(off + 4)) = pk[1];
    }
}

// a thread per word of the decode stream
__global__ void rq_prepack_stream_kernel(const rq_block * __restrict__ blocks, int64_t K, int64_t N, uint32_t * __restrict__ w4) {
    const int64_t ng64 = K / 64, tiles = (N + 15) / 16;
    const int64_t idx = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tiles * ng64 * 128) return;
    const int j = (int) (idx & 3), lane = (int) ((idx >> 2) & 31);
    const int64_t g64 = (idx >> 7) % ng64, tile = (idx >> 7) / ng64;
    const int gid = lane >> 2, tig = lane & 3;
    const int64_t k0 = g64 * 64 + (j >> 1) * 32 + (j & 1) * 16 + tig * 4;
    uint32_t dst = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int64_t row = tile * 16 + gid + 8 * half;
        if (row < N) {
            const rq_block * b = blocks + row * (K / RQ_BLOCK_CODES) + k0 / RQ_BLOCK_CODES;
            const uint32_t src = b->qs[(k0 % RQ_BLOCK_CODES) / 8] >> (4 * (k0 % 8));     // 4 codes from bit 0
#pragma unroll
            for (int q = 0; q < 4; ++q) dst |= ((src >> (4 * q)) & 0xFu) << (8 * q + 4 * half);
        }
    }
    w4[idx] = dst;
}

}  // namespace

cudaError_t rq_launch_scan_wk(const rq_block * blocks, int64_t n_blocks, int32_t * flag, cudaStream_t stream) {
    rq_scan_wk_kernel<<<(unsigned) ((n_blocks + 255) / 256), 256, 0, stream>>>(blocks, n_blocks, flag);
    return cudaGetLastError();
}

cudaError_t rq_launch_prepack(const rq_block * blocks, int64_t K, int64_t N, float * sw, uint8_t * w4, int8_t * w8,
                              int8_t * wk, int wk_mode, cudaStream_t stream) {
    const int64_t n = N * (K / 8);
    rq_prepack_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, stream>>>(blocks, K, N, sw, w8, wk, wk_mode);
    if (w4 != nullptr) {
        const int64_t nw = ((N + 15) / 16) * (K / 64) * 128;
        rq_prepack_stream_kernel<<<(unsigned) ((nw + 255) / 256), 256, 0, stream>>>(blocks, K, N, reinterpret_cast<uint32_t *>(w4));
    }
    return cudaGetLastError();
}
