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

}  // namespace

cudaError_t rq_launch_rank_barrier(uint32_t * const * flags_of_rank, int rank, int n_ranks, uint32_t * epoch, int32_t * status,
                                   cudaStream_t stream) {
    RankBarrierParams prm = {};
    for (int p = 0; p < n_ranks; ++p) prm.flags[p] = flags_of_rank[p];
    prm.epoch = epoch; prm.status = status; prm.rank = rank; prm.n_ranks = n_ranks;
    rq_rank_barrier_kernel<<<1, 32, 0, stream>>>(prm);
    return cudaGetLastError();
}
