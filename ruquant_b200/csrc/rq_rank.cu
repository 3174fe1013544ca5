// All-ranks barrier for N-sharded ranks of one node, over flag words that every rank has mapped (peer access /
// symmetric memory).  It follows the decode GEMVs whose epilogues wrote their outputs straight into the other ranks'
// buffers (rq_w4a4_mul_mat_push): when it returns on a rank, every rank's stores of the preceding kernels on its stream
// have been released, and this rank has seen all of them arrive.
//
// One block of 32 threads per GPU; thread p talks to rank p.  The epoch lives in device memory and counts up with every
// call, so the same captured graph can be replayed.  The wait is bounded (about a second of SM clocks): on expiry the
// status word is set to 3 and the kernel returns; nothing ever waits for a kernel of the same GPU.
#include "rq_common.cuh"

namespace {

struct RankBarrierParams {
    uint32_t * flags[RQ_MAX_RANKS];     // flags[p]: rank p's array of n_ranks words, word r written by rank r
    uint32_t * epoch;
    int32_t * status;
    int rank, n_ranks;
};

__global__ void __launch_bounds__(32) rq_rank_barrier_kernel(const RankBarrierParams prm) {
    const int p = threadIdx.x;
    const uint32_t epoch = *prm.epoch + 1u;
    __syncwarp();
    if (p < prm.n_ranks) {
        // everything this GPU's earlier kernels stored (to any rank) is ordered before the flag
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(prm.flags[p] + prm.rank), "r"(epoch) : "memory");
        const uint32_t * mine = prm.flags[prm.rank] + p;
        const long long t0 = clock64();
        bool seen = false;
        for (uint32_t i = 0; !seen; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            seen = (int32_t) (v - epoch) >= 0;
            if (!seen && (i & 63u) == 63u && clock64() - t0 > 2000000000ll) break;
        }
        if (!seen && prm.status != nullptr) atomicExch(prm.status, 3);
    }
    __syncwarp();
    if (p == 0) *prm.epoch = epoch;
}

// Sum of the ranks' partial outputs for K-split weights (the reference's tensor-parallel mode for attn_output / ffn_down:
// every rank multiplies its block columns by its slice of x, the partial Y are added; its own all-reduce writes packed
// partials into peer staging slots and adds them behind flag barriers, k_broadcast_reduce_16 / k_twoshot_16 in
// patches/mx-llama.cpp-ruquant.patch:5293-5374).  Here every rank's partial sits in a buffer all ranks have mapped; after
// a rank barrier a rank reads the partials with plain peer loads and adds them IN RANK ORDER, ((p0 + p1) + p2) + ..., so
// every rank holds the same bits and a CPU restatement can reproduce them.  Two forms:
//   one shot   every rank adds all `count` elements itself: (g-1) * count * 4 bytes in per rank, one kernel, nothing after it;
//   two shot   rank r adds elements [lo, hi) only and stores the sums into every rank's output (peer stores): 2 * (g-1)/g *
//              count * 4 bytes per rank; a second rank barrier then makes all pieces visible everywhere.
struct PartialSumParams {
    const float * part[RQ_MAX_RANKS];   // part[r]: rank r's partial as mapped on this rank
    float * out[RQ_MAX_RANKS];          // destinations of the sums (one shot: out[0] only)
    int64_t lo, hi;                     // elements this rank adds
    int n_ranks, n_out;
};

__global__ void __launch_bounds__(256) rq_partial_sum_kernel(const PartialSumParams prm) {
    const int64_t n4 = (prm.hi - prm.lo) >> 2;          // lo and hi are multiples of 4 except for the tail of the last piece
    const int64_t stride = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const int64_t e = prm.lo + 4 * i;
        float4 acc = *reinterpret_cast<const float4 *>(prm.part[0] + e);
        for (int r = 1; r < prm.n_ranks; ++r) {
            const float4 v = *reinterpret_cast<const float4 *>(prm.part[r] + e);
            acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
        }
        for (int d = 0; d < prm.n_out; ++d) *reinterpret_cast<float4 *>(prm.out[d] + e) = acc;
    }
    // the last piece's tail
    const int64_t t0 = prm.lo + 4 * n4;
    for (int64_t e = t0 + (int64_t) blockIdx.x * blockDim.x + threadIdx.x; e < prm.hi; e += stride) {
        float acc = prm.part[0][e];
        for (int r = 1; r < prm.n_ranks; ++r) acc = __fadd_rn(acc, prm.part[r][e]);
        for (int d = 0; d < prm.n_out; ++d) prm.out[d][e] = acc;
    }
}

// Ranks that share the quantizer: three byte ranges of this rank's workspace (codes, multipliers, units of its token
// range) go to the same offsets of every other rank's workspace.  16-byte pieces where a range allows them, four loads
// in flight per thread; 4-byte words otherwise (every range is a whole number of them).
struct ShareRowsParams {
    const uint8_t * src;
    uint8_t * dst[RQ_MAX_RANKS - 1];
    uint64_t off[3], bytes[3];
    int n_dst;
};

__global__ void __launch_bounds__(256) rq_share_rows_kernel(const ShareRowsParams prm) {
    const uint64_t tid = (uint64_t) blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t) gridDim.x * blockDim.x;
    for (int seg = 0; seg < 3; ++seg) {
        const uint64_t off = prm.off[seg], bytes = prm.bytes[seg];
        if (((off | bytes) & 15) == 0) {
            const uint64_t n = bytes >> 4;
            for (uint64_t i = tid; i < n; i += 4 * nthr) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i + u * nthr < n) v[u] = __ldcg(reinterpret_cast<const uint4 *>(prm.src + off) + i + u * nthr);
                for (int d = 0; d < prm.n_dst; ++d) {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (i + u * nthr < n) reinterpret_cast<uint4 *>(prm.dst[d] + off)[i + u * nthr] = v[u];
                }
            }
        } else {
            const uint64_t n = bytes >> 2;
            for (uint64_t i = tid; i < n; i += nthr) {
                const uint32_t v = __ldcg(reinterpret_cast<const uint32_t *>(prm.src + off) + i);
                for (int d = 0; d < prm.n_dst; ++d) reinterpret_cast<uint32_t *>(prm.dst[d] + off)[i] = v;
            }
        }
    }
}

}  // namespace

cudaError_t rq_launch_share_rows(const void * src, void * const * dst, int n_dst, const uint64_t * off, const uint64_t * bytes,
                                 cudaStream_t stream) {
    ShareRowsParams prm = {};
    prm.src = static_cast<const uint8_t *>(src);
    for (int d = 0; d < n_dst; ++d) prm.dst[d] = static_cast<uint8_t *>(dst[d]);
    uint64_t total = 0;
    for (int i = 0; i < 3; ++i) { prm.off[i] = off[i]; prm.bytes[i] = bytes[i]; total += bytes[i]; }
    prm.n_dst = n_dst;
    if (n_dst < 1 || total == 0) return cudaSuccess;
    uint64_t blocks = (total / 64 + 255) / 256;       // 64 bytes per thread and sweep
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    rq_share_rows_kernel<<<(unsigned) blocks, 256, 0, stream>>>(prm);
    return cudaGetLastError();
}

cudaError_t rq_launch_partial_sum(const float * const * partials, int n_ranks, int64_t lo, int64_t hi, float * const * outs, int n_out,
                                  cudaStream_t stream) {
    PartialSumParams prm = {};
    for (int r = 0; r < n_ranks; ++r) prm.part[r] = partials[r];
    for (int d = 0; d < n_out; ++d) prm.out[d] = outs[d];
    prm.lo = lo; prm.hi = hi; prm.n_ranks = n_ranks; prm.n_out = n_out;
    if (hi <= lo) return cudaSuccess;
    const int64_t n4 = (hi - lo + 3) / 4;
    int64_t blocks = (n4 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    rq_partial_sum_kernel<<<(unsigned) blocks, 256, 0, stream>>>(prm);
    return cudaGetLastError();
}

cudaError_t rq_launch_rank_barrier(uint32_t * const * flags_of_rank, int rank, int n_ranks, uint32_t * epoch, int32_t * status,
                                   cudaStream_t stream) {
    RankBarrierParams prm = {};
    for (int p = 0; p < n_ranks; ++p) prm.flags[p] = flags_of_rank[p];
    prm.epoch = epoch; prm.status = status; prm.rank = rank; prm.n_ranks = n_ranks;
    rq_rank_barrier_kernel<<<1, 32, 0, stream>>>(prm);
    return cudaGetLastError();
}
