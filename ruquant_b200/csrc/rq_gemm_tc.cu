// Prefill-width contraction on the sm_100a tensor cores: tcgen05.mma kind::i8 with the accumulator in tensor memory,
// operands staged by TMA, and the reference's per-group integer fold done by the epilogue warps straight out of
// tensor memory while the tensor pipe works on the next group.
//
// Why the accumulator leaves tensor memory every G inputs: the reference shifts each group's term right by 4 before
// the int32 sum (ggml_vec_dot_w4a4_a4, ggml/src/ggml-cpu/quants.c in patches/llama.cpp-ruquant.patch:173), which is
// not linear, so groups cannot be accumulated together.  Operand scaling makes that fold one instruction:
//   A = activations, int8 8*(q - z_g), [M][K] K-major      (tokens are the MMA's M = 128 rows = TMEM lanes)
//   B = weights,     int8 16*c,        [N][K] K-major      (weight rows are the MMA's N = 256 = TMEM columns)
//   D = 128 * S_g after G/32 instructions of K = 32;   total += (m_g * D) >> 11   ( = (m_g*S_g) >> 4, exact)
// An epilogue thread owns one token (one TMEM lane), so m_g is a single register per group.  Weights with
// multipliers k != 1 are stored as k*c instead and folded as (D * m_g) >> 7.
//
// CTA = 128 tokens x 256 weight rows.  Warp 0 lane 0: TMA producer over a ring of 128-input K slices (128B swizzle).
// Warp 1: TMEM allocation, lane 0 issues the MMAs into two 256-column accumulator buffers.  Warps 4-11: fold + final
// fp32 epilogue y = ((float(total) * 16) * u) * s_w.
// The kernel is bound by the L2 -> shared-memory feed of its operands, so above 128 tokens two CTAs work as a pair
// (PAIR, a cluster of 2, tcgen05 cta_group::2): one MMA of M = 256 spans both CTAs' tensor memory, each CTA stages
// its own 128 tokens of A and only HALF of the 256 weight rows of B (32 KB per slice instead of 48 KB, six stages).
// The even CTA issues the MMAs for both; its commits signal the barriers of both CTAs, the odd CTA's TMA bytes and
// epilogue arrivals are counted on the even CTA's barriers.
// Every wait is bounded: on expiry the waiter raises a CTA-wide abort flag and a status word in global memory,
// everyone leaves the pipeline, outstanding TMA transactions are drained and tensor memory is released.
#include <cuda.h>

#include <stdlib.h>

#include "rq_common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int TC_THREADS = 384;
constexpr uint32_t A_BYTES = BM * BK, BH_BYTES = (BN / 2) * BK;     // B travels in halves of 128 weight rows
__host__ __device__ constexpr int stages_of(bool pair) { return pair ? 6 : 4; }
__host__ __device__ constexpr uint32_t stage_bytes_of(bool pair) { return A_BYTES + (pair ? 1u : 2u) * BH_BYTES; }
constexpr uint32_t STAGING_BYTES = 8 * 32 * 32 * 4;      // a 32 x 32 fp32 transposition tile per epilogue warp
__host__ __device__ constexpr uint32_t smem_bytes_of(bool pair) { return stages_of(pair) * stage_bytes_of(pair) + STAGING_BYTES + 1024; }   // + alignment slack
constexpr int MAX_STAGES = 6;
constexpr long long WAIT_CYCLES = 2000000000ll;                // about a second at B200 clocks
constexpr uint32_t TMEM_COLS = 512;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the barrier did not flip within WAIT_CYCLES or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int * abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; return false; }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// the pair's form: the destination is this CTA's shared memory, the barrier may be the partner's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap * map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// address of the same shared-memory object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// K-major operand tile in the canonical 128B-swizzled layout TMA writes: rows of 128 bytes, 8-row atoms 1024 bytes
// apart.  Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (unused for swizzled K-major, 1),
// stride byte offset >> 4 [32,46), descriptor version 1 [46,48), layout type SWIZZLE_128B = 2 [61,64).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t) (1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::i8: D = s32 (2 at [4,6)), A and B signed int8 (1 at [7,10) and [10,13)), both
// K-major (0 at 15, 16), N >> 3 at [17,23), M >> 4 at [24,29)
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);
// kind::f8f6f4: D = f32 (1 at [4,6)), A and B e4m3 (0 at [7,10) and [10,13)), K-major, same N and M fields
constexpr uint32_t IDESC_F8 = (1u << 4) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);
// a pair's instruction covers M = 256 tokens, 128 in each CTA's tensor memory
constexpr uint32_t IDESC_PAIR = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) ((2 * BM) >> 4) << 24);
constexpr uint32_t IDESC_F8_PAIR = (1u << 4) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) ((2 * BM) >> 4) << 24);

// One instruction of K = 32 (128 tokens x 256 weight rows, or 256 x 256 for a pair).  ACC selects between starting and
// continuing an accumulator as two separate instructions with constant predicates: the issuing thread is the
// bottleneck of this kernel the moment it spends more than an instruction's 128 cycles between two issues, so nothing
// is computed per instruction that a template can decide.
template <bool F8, bool PAIR, bool ACC>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db) {
    constexpr uint32_t idesc = PAIR ? (F8 ? IDESC_F8_PAIR : IDESC_PAIR) : (F8 ? IDESC_F8 : IDESC);
    // called by the whole (converged) warp with warp-uniform operands; one elected lane issues
    if (PAIR) {
        if (F8) asm volatile("{\n\t.reg .pred pe, p;\n\telect.sync _|pe, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t@pe tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
        else    asm volatile("{\n\t.reg .pred pe, p;\n\telect.sync _|pe, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t@pe tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
    } else {
        if (F8) asm volatile("{\n\t.reg .pred pe, p;\n\telect.sync _|pe, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t@pe tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
        else    asm volatile("{\n\t.reg .pred pe, p;\n\telect.sync _|pe, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t@pe tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
    }
}
// the commits, like the MMAs, are called by the whole warp and issued by one elected lane
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" :: "r"(bar) : "memory");
}
// the pair's commit arrives on the barrier at this offset in both CTAs (a commit, not a copy: nothing is loaded)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
                 :: "r"(bar), "h"((uint16_t) 3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
// completes this thread's outstanding tensor-memory loads; the values are threaded through as read-write operands
// so that no use of them can be scheduled above the wait
__device__ __forceinline__ void tmem_ld_wait(int (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                   "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :: "memory");
}

// one integer multiply and one shift-add per output per group (measured on B200: 50+ outputs per clock per SM,
// against 30 for a high multiply-add)
// integer path (weights k*c, activations 8*(q - z)): D = 8*k*S, term = (D * m) >> 7
__device__ __forceinline__ void fold32(int (&tot)[128], int base, const int (&v)[32], int mm) {
#pragma unroll
    for (int i = 0; i < 32; ++i) tot[base + i] += (v[i] * mm) >> 7;
}

// fp8 path: D = S exactly (fp32 accumulation of products of small integers).  The running total lives in a float
// kept inside [2^23, 2^24), where the spacing of floats is 1: a round-down fused multiply-add
//     t <- fma.rm(S, m/16, t)
// adds floor(S*m/16) = (m*S) >> 4 exactly (S*m/16 has at most 21 + 4 significant bits below 2^23, the sum is rounded
// once, downwards, to an integer) -- the reference's shifted term in ONE instruction at the full fp32 rate.
constexpr float FOLD_MAGIC = 12582912.0f;        // 1.5 * 2^23
constexpr int FOLD_MAGIC_BITS = 0x4B400000;
__device__ __forceinline__ float fma_rm(float a, float b, float c) {
    float d;
    asm("fma.rm.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
template <int BASE>
__device__ __forceinline__ void fold32_f8(float (&tf)[128], const int (&v)[32], float mf) {
#pragma unroll
    for (int i = 0; i < 32; ++i) tf[BASE + i] = fma_rm(__int_as_float(v[i]), mf, tf[BASE + i]);
}
// Every 1536 inputs the float is re-centred: what it holds above +-2^19 moves, in units of 2^20, into a signed byte
// of a packed carry word, so the float never leaves its window.  Bounds: a group of G inputs adds at most
// 255 * (G*15*8) / 16 in magnitude, 2.94 M per 1536 inputs, on top of at most 2^19 left by the last re-centring:
// |t - magic| < 3.5 M < 2^22; a re-centring moves at most 4 units, K <= 32768 has at most 22 of them: |byte| <= 88.
__device__ __forceinline__ void recenter(float (&tf)[128], int (&carry)[32]) {
#pragma unroll
    for (int i = 0; i < 128; ++i) {
        const int k = __float_as_int(tf[i]) - FOLD_MAGIC_BITS;
        const int c = (k + (1 << 19)) >> 20;
        tf[i] = __int_as_float(FOLD_MAGIC_BITS + (k - (c << 20)));
        carry[i >> 2] += c << (8 * (i & 3));
    }
}

struct TcParams {
    const float * sw;
    const int32_t * msh;
    const float * u;
    float * y;
    float * y_more[RQ_MAX_RANKS - 1];   // further copies of the output (other ranks' buffers, peer-mapped), same layout
    int64_t ldy;
    int32_t * status;
    int K, N, M, G;
    int n_more;
};

struct __align__(8) TcShared {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// F8 = true: multipliers all 1, operands are e4m3 bytes of c and (q - z), fp8 MMA with fp32 accumulators, float fold.
// F8 = false: weight multipliers present, B holds int8 k*c, A int8 8*(q - z), integer MMA and integer fold.
// PAIR = true: launched as clusters of two CTAs; the pair works on token tiles 2p and 2p+1 of the same 256 weight rows.
// The kernel is persistent: CTA (or pair) c takes work units c, c + stride, ... where unit v = n_tile * m_units +
// m_unit -- token tiles fastest, so the CTAs running at one time share their weight slices in L2.  Slots, phases and
// accumulator buffers are running counters that carry over from one unit to the next: the MMAs of the next unit start
// while the epilogue warps still scale and store the previous one.
template <bool F8, bool PAIR, bool PUSH>
__global__ void __launch_bounds__(TC_THREADS, 1)
rq_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TcParams prm) {
    constexpr int STAGES = stages_of(PAIR);
    constexpr uint32_t STAGE_BYTES = stage_bytes_of(PAIR);
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcShared sh;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? (blockIdx.x & 1u) : 0u;      // rank in the cluster; rank 0 issues the pair's MMAs
    const bool leader = rank == 0;
    const int n_ks = prm.K / BK;          // ring slices of 128 inputs
    const int gsteps = prm.G / 64;        // 64-input steps per activation group: 1, 2 or 4
    const int n_ag = prm.K / prm.G;       // activation groups
    const int m_tiles = (prm.M + BM - 1) / BM, n_tiles = (prm.N + BN - 1) / BN;
    const int m_units = PAIR ? (m_tiles + 1) / 2 : m_tiles;
    const int units = m_units * n_tiles;
    const int first = PAIR ? (int) (blockIdx.x >> 1) : (int) blockIdx.x, stride = PAIR ? (int) (gridDim.x >> 1) : (int) gridDim.x;
    volatile int * abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sh.full[s]), 1); mbar_init(smem_u32(&sh.empty[s]), 1); }
        // a pair's accumulator buffer is free when the 8 epilogue warps of BOTH CTAs have arrived (on rank 0's barrier)
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&sh.tmem_full[b]), 1); mbar_init(smem_u32(&sh.tmem_empty[b]), PAIR ? 16 : 8); }
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {   // one warp of each CTA of the pair, same shared-memory slot in both
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         :: "r"(smem_u32(&sh.tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         :: "r"(smem_u32(&sh.tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_barrier();      // the partner's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    // warps 0-3 (TMA, MMA, two idle) give registers back; the two epilogue warpgroups take them
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;              // slices issued, all units
            bool ok = true;
            const uint32_t lbar0 = PAIR ? map_to_cta(smem_u32(&sh.full[0]), 0) : smem_u32(&sh.full[0]);
            RQ_CYC_DECL(c_empty);
            RQ_CYC_DECL(c_total);
            RQ_CYC_BEGIN(c_total);
            for (int v = first; v < units && ok; v += stride) {
                const int n_tile = v / m_units, m_unit = v - n_tile * m_units;
                const int m_tile = PAIR ? 2 * m_unit + (int) rank : m_unit;
                for (int ks = 0; ks < n_ks; ++ks, ++it) {
                    const uint32_t s = it % STAGES;
                    RQ_CYC_BEGIN(c_empty);
                    if (!mbar_wait(smem_u32(&sh.empty[s]), ((it / STAGES) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    RQ_CYC_END(c_empty);
                    const uint32_t dst = ring + s * STAGE_BYTES;
                    if (PAIR) {
                        // both CTAs' bytes are counted on rank 0's barrier; this CTA brings its tokens and its half of B
                        if (leader) mbar_expect_tx(smem_u32(&sh.full[s]), 2 * STAGE_BYTES);
                        const uint32_t lbar = lbar0 + s * 8u;
                        tma_load_2d_pair(dst, &tmap_a, lbar, ks * BK, m_tile * BM);
                        tma_load_2d_pair(dst + A_BYTES, &tmap_b, lbar, ks * BK, n_tile * BN + (int) rank * (BN / 2));
                    } else {
                        const uint32_t bar = smem_u32(&sh.full[s]);
                        mbar_expect_tx(bar, STAGE_BYTES);
                        tma_load_2d(dst, &tmap_a, bar, ks * BK, m_tile * BM);
                        tma_load_2d(dst + A_BYTES, &tmap_b, bar, ks * BK, n_tile * BN);
                        tma_load_2d(dst + A_BYTES + BH_BYTES, &tmap_b, bar, ks * BK, n_tile * BN + BN / 2);
                    }
                }
            }
            RQ_CYC_END(c_total);
            RQ_CYC_REPORT(prm.status, 0x40, c_empty);
            RQ_CYC_REPORT(prm.status, 0x41, c_total);
            if (*abort_flag) {
                // drain: every slice that was issued must land before the CTA's shared memory is given back (rank 1 of a
                // pair cannot see its own copies complete: it gives them time, then meets rank 0 at the final barrier)
                if (!PAIR || leader) {
                    for (uint32_t k = it > (uint32_t) STAGES ? it - STAGES : 0; k < it; ++k) {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(smem_u32(&sh.full[k % STAGES]), (k / STAGES) & 1u) && clock64() - t0 < WAIT_CYCLES) { }
                    }
                } else {
                    const long long t0 = clock64();
                    while (clock64() - t0 < 2000000ll) { }
                }
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // The whole warp walks the loop with warp-uniform values (descriptors and addresses then live in the uniform
            // datapath) and elects a lane at each MMA and commit.  Straight-line issue loop: shifts instead of divisions (gsteps is 1, 2 or 4), slot, phase and accumulator
            // buffer as running counters, descriptors advanced by adding to their address field.
            const uint32_t gmask = (uint32_t) gsteps - 1u;
            const uint64_t da0 = umma_desc(ring), db0 = umma_desc(ring + A_BYTES);
            uint32_t s = 0, ph = 0, gcount = 0;       // ring slot, its phase, accumulator groups issued (all units)
            bool ok = true;
            RQ_CYC_DECL(c_full);
            RQ_CYC_DECL(c_tmem);
            RQ_CYC_DECL(c_mma);
            RQ_CYC_DECL(c_issue);
            RQ_CYC_DECL(c_commit);
            RQ_CYC_BEGIN(c_mma);
            for (int v = first; v < units && ok; v += stride) {
                for (int ks = 0; ks < n_ks && ok; ++ks) {
                    RQ_CYC_BEGIN(c_full);
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.full[s]), ph, abort_flag))) { ok = false; break; }
                    RQ_CYC_END(c_full);
                    tc_fence_after();
                    const uint64_t so = (uint64_t) ((s * STAGE_BYTES) >> 4);
                    const uint64_t da = da0 + so, db = db0 + so;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t gs = (2u * (uint32_t) ks + (uint32_t) h) & gmask;   // 64-input step inside its group
                        const uint32_t buf = gcount & 1u;
                        const uint32_t d = tmem_base + buf * BN;
                        if (gs == 0) {
                            RQ_CYC_BEGIN(c_tmem);
                            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.tmem_empty[buf]), ((gcount >> 1) & 1u) ^ 1u, abort_flag))) { ok = false; break; }
                            RQ_CYC_END(c_tmem);
                            tc_fence_after();
                            RQ_CYC_BEGIN(c_issue);
                            umma<F8, PAIR, false>(d, da + h * 4, db + h * 4);          // bytes >> 4 inside the swizzled row
                        } else {
                            RQ_CYC_BEGIN(c_issue);
                            umma<F8, PAIR, true>(d, da + h * 4, db + h * 4);
                        }
                        umma<F8, PAIR, true>(d, da + h * 4 + 2, db + h * 4 + 2);
                        RQ_CYC_END(c_issue);
                        if (gs == gmask) {
                            RQ_CYC_BEGIN(c_commit);
                            if (PAIR) umma_commit_pair(smem_u32(&sh.tmem_full[buf]));
                            else      umma_commit(smem_u32(&sh.tmem_full[buf]));
                            RQ_CYC_END(c_commit);
                            ++gcount;
                        }
                    }
                    RQ_CYC_BEGIN(c_commit);
                    if (PAIR) umma_commit_pair(smem_u32(&sh.empty[s]));
                    else      umma_commit(smem_u32(&sh.empty[s]));
                    RQ_CYC_END(c_commit);
                    if (++s == (uint32_t) STAGES) { s = 0; ph ^= 1u; }
                }
            }
            RQ_CYC_END(c_mma);
            if (lane == 0) {
            RQ_CYC_REPORT(prm.status, 0x42, c_full);
            RQ_CYC_REPORT(prm.status, 0x43, c_tmem);
            RQ_CYC_REPORT(prm.status, 0x44, c_mma);
            RQ_CYC_REPORT(prm.status, 0x47, c_issue);
            RQ_CYC_REPORT(prm.status, 0x48, c_commit);
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        const int e = warp - 4, quarter = warp & 3, half = e >> 2;
        const uint32_t lane_base = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (half * 128);
        // the quantizer records the format it wrote: refuse to multiply the wrong one
        const bool fmt_ok = prm.status == nullptr || prm.status[1] == (F8 ? RQ_FMT_E4M3 : RQ_FMT_I8);
        const uint32_t empty_bar0 = PAIR ? map_to_cta(smem_u32(&sh.tmem_empty[0]), 0) : smem_u32(&sh.tmem_empty[0]);
        const int recenter_every = 1536 / prm.G;           // G is 64, 128 or 256
        const bool vec = ((prm.ldy & 3) == 0) && ((reinterpret_cast<uintptr_t>(prm.y) & 15) == 0);
        uint32_t gcount = 0;              // accumulator groups folded (all units)
        bool ok = true;
        RQ_CYC_DECL(c_tfull);
        RQ_CYC_DECL(c_epi);
        RQ_CYC_BEGIN(c_epi);
        for (int v = first; v < units && ok; v += stride) {
            const int n_tile = v / m_units, m_unit = v - n_tile * m_units;
            const int m_tile = PAIR ? 2 * m_unit + (int) rank : m_unit;
            const int row = m_tile * BM + quarter * 32 + lane;
            const bool row_ok = row < prm.M;
            const int32_t * mrow = prm.msh + (size_t) (row_ok ? row : 0) * n_ag;
            int tot[F8 ? 1 : 128];
            float tf[F8 ? 128 : 1];
            int carry[F8 ? 32 : 1];
            if (F8) {
#pragma unroll
                for (int i = 0; i < 128; ++i) tf[F8 ? i : 0] = FOLD_MAGIC;
#pragma unroll
                for (int i = 0; i < 32; ++i) carry[F8 ? i : 0] = 0;
            } else {
#pragma unroll
                for (int i = 0; i < 128; ++i) tot[F8 ? 0 : i] = 0;
            }
            int since = 0;
            int mnext = row_ok ? __ldg(mrow) : 0;
            for (int ag = 0; ag < n_ag; ++ag, ++gcount) {
                const uint32_t buf = gcount & 1u;
                const int mm = mnext;
                if (ag + 1 < n_ag) mnext = row_ok ? __ldg(mrow + ag + 1) : 0;
                // the loads below are warp-collective: leave the loop together or not at all
                RQ_CYC_BEGIN(c_tfull);
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.tmem_full[buf]), (gcount >> 1) & 1u, abort_flag))) { ok = false; break; }
                RQ_CYC_END(c_tfull);
                tc_fence_after();
                const uint32_t t0 = lane_base + buf * BN;
                if constexpr (F8) {
                    const float mf = __int_as_float(mm);          // m / 16
                    // four 32-column pieces, the load of piece c+1 in flight while piece c folds
                    int va[32], vb[32];
                    tmem_ld32(t0, va);
                    tmem_ld_wait(va); tmem_ld32(t0 + 32, vb); fold32_f8<0>(tf, va, mf);
                    tmem_ld_wait(vb); tmem_ld32(t0 + 64, va); fold32_f8<32>(tf, vb, mf);
                    tmem_ld_wait(va); tmem_ld32(t0 + 96, vb); fold32_f8<64>(tf, va, mf);
                    tmem_ld_wait(vb);
                    // the accumulator is in registers: hand the buffer back before the last piece is folded
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_cluster(empty_bar0 + buf * 8u);
                        else      mbar_arrive(empty_bar0 + buf * 8u);
                    }
                    fold32_f8<96>(tf, vb, mf);
                } else {
                    // software pipeline over the four 32-column chunks: the load of chunk c+1 is in flight while chunk c folds
                    int va[32], vb[32];
                    tmem_ld32(t0, va);
                    tmem_ld_wait(va);
                    tmem_ld32(t0 + 32, vb);
                    fold32(tot, 0, va, mm);
                    tmem_ld_wait(vb);
                    tmem_ld32(t0 + 64, va);
                    fold32(tot, 32, vb, mm);
                    tmem_ld_wait(va);
                    tmem_ld32(t0 + 96, vb);
                    fold32(tot, 64, va, mm);
                    tmem_ld_wait(vb);
                    fold32(tot, 96, vb, mm);
                }
                if constexpr (!F8) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_cluster(empty_bar0 + buf * 8u);
                        else      mbar_arrive(empty_bar0 + buf * 8u);
                    }
                }
                if constexpr (F8) {
                    if (++since == recenter_every || ag == n_ag - 1) { recenter(tf, carry); since = 0; }
                }
            }
            if (!ok) break;
            if (!fmt_ok) {
                if (lane == 0 && prm.status != nullptr) atomicExch(prm.status, 2);
                continue;
            }
            {
                // Final scaling y = ((float(total) * 16) * u) * s_w and the store.  A thread owns a token's 128 outputs,
                // but a row-per-thread store would scatter 16-byte pieces over 32 rows: the warp transposes 32 x 32
                // pieces through shared memory (16-byte chunks XOR-swizzled by row, conflict-free both ways), after which
                // eight lanes write 128 contiguous bytes of a row and apply s_w, which is per column.
                const float ut = row_ok ? __ldg(prm.u + row) : 0.0f;
                float * stg = reinterpret_cast<float *>(smem_raw + (ring - smem_u32(smem_raw)) + STAGES * STAGE_BYTES) + e * 1024;
                const int jj = lane & 7, rsub = lane >> 3;
                const bool sw_vec = (reinterpret_cast<uintptr_t>(prm.sw) & 15) == 0;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = c * 32 + j * 4;
                        int P = F8 ? carry[F8 ? i >> 2 : 0] : 0;      // four signed byte digits, units of 2^20
                        float f[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            int total;
                            if (F8) {
                                const int d = (int) (signed char) (P & 0xFF);
                                total = d * (1 << 20) + (__float_as_int(tf[F8 ? i + k : 0]) - FOLD_MAGIC_BITS);
                                P = (P - d) >> 8;
                            } else {
                                total = tot[F8 ? 0 : i + k];
                            }
                            f[k] = __fmul_rn(__fmul_rn((float) total, 16.0f), ut);
                        }
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((j ^ (lane & 7)) << 2)) = make_float4(f[0], f[1], f[2], f[3]);
                    }
                    __syncwarp();
                    const int ncol = n_tile * BN + half * 128 + c * 32 + jj * 4;
                    float sc[4];
                    if (sw_vec && ncol + 3 < prm.N) {
                        const float4 q = __ldg(reinterpret_cast<const float4 *>(prm.sw + ncol));
                        sc[0] = q.x; sc[1] = q.y; sc[2] = q.z; sc[3] = q.w;
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) sc[k] = ncol + k < prm.N ? __ldg(prm.sw + ncol + k) : 0.0f;
                    }
#pragma unroll
                    for (int it8 = 0; it8 < 8; ++it8) {
                        const int rr = it8 * 4 + rsub;
                        const int grow = m_tile * BM + quarter * 32 + rr;
                        const float4 q = *reinterpret_cast<const float4 *>(stg + rr * 32 + ((jj ^ (rr & 7)) << 2));
                        const float o0 = __fmul_rn(q.x, sc[0]), o1 = __fmul_rn(q.y, sc[1]), o2 = __fmul_rn(q.z, sc[2]), o3 = __fmul_rn(q.w, sc[3]);
                        if (grow < prm.M) {
                            // destination 0 is this GPU's buffer; N-sharded ranks get the same 128-byte row pieces straight
                            // into their copies of the output while the MMAs of the next unit run
                            for (int dd = 0; dd <= (PUSH ? prm.n_more : 0); ++dd) {
                                float * yr = (!PUSH || dd == 0 ? prm.y : prm.y_more[dd - 1]) + (size_t) grow * prm.ldy + ncol;
                                if (vec && ncol + 3 < prm.N) {
                                    *reinterpret_cast<float4 *>(yr) = make_float4(o0, o1, o2, o3);
                                } else {
                                    if (ncol < prm.N) yr[0] = o0;
                                    if (ncol + 1 < prm.N) yr[1] = o1;
                                    if (ncol + 2 < prm.N) yr[2] = o2;
                                    if (ncol + 3 < prm.N) yr[3] = o3;
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        }
        RQ_CYC_END(c_epi);
        if (warp == 4 && lane == 0) { RQ_CYC_REPORT(prm.status, 0x45, c_tfull); RQ_CYC_REPORT(prm.status, 0x46, c_epi); }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_flag && prm.status != nullptr) atomicExch(prm.status, 1);
    if (PAIR) cluster_barrier();      // neither CTA frees tensor memory or leaves while its partner may still touch it
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t get_encode() {
    static encode_fn_t fn = nullptr;
    if (fn == nullptr) {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<encode_fn_t>(p);
        }
    }
    return fn;
}

}  // namespace

int rq_encode_tmap_i8(void * tmap_out, const void * base, int64_t K, int64_t rows, int box_rows) {
    encode_fn_t fn = get_encode();
    if (fn == nullptr) return -1;
    alignas(64) CUtensorMap map;
    const cuuint64_t dims[2] = { (cuuint64_t) K, (cuuint64_t) rows };
    const cuuint64_t strides[1] = { (cuuint64_t) K };       // bytes between rows
    const cuuint32_t box[2] = { (cuuint32_t) BK, (cuuint32_t) box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
    memcpy(tmap_out, &map, sizeof(map));
    return 0;
}

template <bool F8, bool PAIR, bool PUSH>
static cudaError_t configure_tc() {
    return cudaFuncSetAttribute(rq_gemm_tc_kernel<F8, PAIR, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_of(PAIR));
}

cudaError_t rq_configure_gemm_tc() {
    // <F8, PAIR, PUSH>: fp8 operands (no weight multipliers) or int8; single CTAs or pairs; one or several destinations
    cudaError_t e;
    if ((e = configure_tc<false, false, false>()) != cudaSuccess) return e;
    if ((e = configure_tc<true, false, false>()) != cudaSuccess) return e;
    if ((e = configure_tc<false, true, false>()) != cudaSuccess) return e;
    if ((e = configure_tc<true, true, false>()) != cudaSuccess) return e;
    if ((e = configure_tc<false, false, true>()) != cudaSuccess) return e;
    if ((e = configure_tc<true, false, true>()) != cudaSuccess) return e;
    if ((e = configure_tc<false, true, true>()) != cudaSuccess) return e;
    return configure_tc<true, true, true>();
}

template <bool F8, bool PAIR, bool PUSH>
static cudaError_t launch_tc(const CUtensorMap & ta, const CUtensorMap & tb, const TcParams & prm, int sms, cudaStream_t stream) {
    const int m_tiles = (prm.M + BM - 1) / BM, n_tiles = (prm.N + BN - 1) / BN;
    const int units = (PAIR ? (m_tiles + 1) / 2 : m_tiles) * n_tiles;
    const int slots = PAIR ? sms / 2 : sms;                  // one CTA per SM: the ring takes its whole shared memory
    const int workers = units < slots ? units : slots;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) (PAIR ? 2 * workers : workers));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem_bytes_of(PAIR);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, rq_gemm_tc_kernel<F8, PAIR, PUSH>, ta, tb, prm);
}

cudaError_t rq_launch_gemm_tc(const void * tmap_w8, const float * sw, int fmt, int64_t K, int64_t N,
                              const int8_t * a8, const int32_t * msh, const float * u, int64_t M, int G,
                              float * y, int64_t ldy, int32_t * status, cudaStream_t stream, float * const * y_more, int n_more) {
    static bool configured[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = rq_configure_gemm_tc();
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = dev < 64 && sm_count[dev] > 0 ? sm_count[dev] : 148;
    alignas(64) CUtensorMap ta, tb;
    if (rq_encode_tmap_i8(&ta, a8, K, M, BM) != 0) return cudaErrorInvalidValue;
    memcpy(&tb, tmap_w8, sizeof(tb));
    TcParams prm;
    prm.sw = sw; prm.msh = msh; prm.u = u; prm.y = y; prm.ldy = ldy; prm.status = status;
    prm.K = (int) K; prm.N = (int) N; prm.M = (int) M; prm.G = G;
    prm.n_more = n_more;
    for (int d = 0; d < RQ_MAX_RANKS - 1; ++d) prm.y_more[d] = d < n_more ? y_more[d] : nullptr;
    static const int no_pair = getenv("RQ_TUNE_TC_NOPAIR") ? atoi(getenv("RQ_TUNE_TC_NOPAIR")) : 0;
    const bool pair = M > BM && !no_pair;      // a second token tile exists: let two CTAs share the weight slices
    const bool f8 = fmt == RQ_FMT_E4M3;
    if (n_more > 0) {
        if (f8) return pair ? launch_tc<true, true, true>(ta, tb, prm, sms, stream) : launch_tc<true, false, true>(ta, tb, prm, sms, stream);
        return pair ? launch_tc<false, true, true>(ta, tb, prm, sms, stream) : launch_tc<false, false, true>(ta, tb, prm, sms, stream);
    }
    if (f8) return pair ? launch_tc<true, true, false>(ta, tb, prm, sms, stream) : launch_tc<true, false, false>(ta, tb, prm, sms, stream);
    return pair ? launch_tc<false, true, false>(ta, tb, prm, sms, stream) : launch_tc<false, false, false>(ta, tb, prm, sms, stream);
}
