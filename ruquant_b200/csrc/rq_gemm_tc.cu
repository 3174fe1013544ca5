// Prefill-width contraction on the sm_100a tensor cores: tcgen05.mma with the accumulator in tensor memory, operands
// staged by TMA, and the reference's per-group fold done by the epilogue warps straight out of tensor memory while the
// tensor pipe works on the next group.
//
// Why the accumulator leaves tensor memory every G inputs: the reference shifts each group's term right by 4 before
// the int32 sum (ggml_vec_dot_w4a4_a4, ggml/src/ggml-cpu/quants.c in patches/llama.cpp-ruquant.patch:173), which is
// not linear, so groups cannot be accumulated together.  Two operand formats:
//   F8  (weights without multipliers, the usual case): A = e4m3 byte of (q - z_g) [M][K], B = e4m3 byte of c [N][K],
//       tcgen05.mma kind::f8f6f4 with fp32 accumulators, which hold S_g exactly (sums of products of small integers);
//       the fold (m_g * S_g) >> 4 is ONE round-down FMA per output on a running total kept in [2^23, 2^24).
//   I8  (weights with multipliers k): A = int8 8*(q - z_g), B = int8 k*c, kind::i8, D = 8*k*S_g, term = (D * m_g) >> 7.
// Tokens are the MMA's M rows (TMEM lanes), weight rows its N columns: an epilogue thread owns one token, so m_g is
// one register per group.
//
// CTA = 128 tokens x 256 weight rows.  Warp 0 lane 0: TMA producer over a ring of 128-input K slices (128B swizzle).
// Warp 1: TMEM allocation and MMA issue into two 256-column accumulator buffers.  Warps 4-11: fold + final fp32
// epilogue y = ((float(total) * 16) * u) * s_w.  What bounds the kernel is the epilogue warps: per 64 inputs the two
// MMAs take 256 cycles, 32 K accumulators cross from tensor memory to registers (128 KB) and are folded by 32 K FMAs
// (256 cycles of the fp32 pipe), so the fold loop is written for issue slots: packed two-wide FMAs, the first
// tensor-memory load of a group issued before the last piece of the previous group is folded, multipliers fetched four
// groups at a time.
// Above 128 tokens two CTAs work as a pair (PAIR, a cluster of 2, tcgen05 cta_group::2): one MMA of M = 256 spans both
// CTAs' tensor memory, each CTA stages its own 128 tokens of A and only HALF of the 256 weight rows of B (32 KB per
// slice instead of 48 KB, six stages).  The even CTA issues the MMAs for both; its commits signal the barriers of both
// CTAs, the odd CTA's TMA bytes and epilogue arrivals are counted on the even CTA's barriers.
// PUSH (N-sharded ranks): warps 2 and 3 copy every finished unit from this GPU's output into the other ranks' copies
// (peer stores), so that no folding warp ever waits for NVLink.
// Every wait is bounded: on expiry the waiter raises a CTA-wide abort flag and a status word in global memory,
// everyone leaves the pipeline, outstanding TMA transactions are drained and tensor memory is released.
#include <cuda.h>

#include <stdlib.h>

#include <mutex>
#include <type_traits>

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
// lane 0's arrival as a predicated instruction: no branch, no reconvergence around it
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, int lane) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.s32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" :: "r"(bar), "r"(lane) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_lane0(uint32_t cluster_addr, int lane) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.s32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cluster.b64 _, [%0];\n\t}" :: "r"(cluster_addr), "r"(lane) : "memory");
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
constexpr int BNI = BN;         // weight rows per MMA instruction (two instructions of 128 with accumulators of their own ran slower:
                                // each re-reads the 128 x 32 token operand, 72 cycles per instruction against 150 for one of 256)
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BNI >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);
// kind::f8f6f4: D = f32 (1 at [4,6)), A and B e4m3 (0 at [7,10) and [10,13)), K-major, same N and M fields
constexpr uint32_t IDESC_F8 = (1u << 4) | ((uint32_t) (BNI >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);
// a pair's instruction covers M = 256 tokens, 128 in each CTA's tensor memory
constexpr uint32_t IDESC_PAIR = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BNI >> 3) << 17) | ((uint32_t) ((2 * BM) >> 4) << 24);
constexpr uint32_t IDESC_F8_PAIR = (1u << 4) | ((uint32_t) (BNI >> 3) << 17) | ((uint32_t) ((2 * BM) >> 4) << 24);

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

// integer path (weights k*c, activations 8*(q - z)): D = 8*k*S, term = (D * m) >> 7: one integer multiply and one
// shift-add per output per group (measured on B200: 50+ outputs per clock per SM, against 30 for a high multiply-add)
template <int BASE>
__device__ __forceinline__ void fold32_i8(int (&tot)[128], const int (&v)[32], int mm) {
#pragma unroll
    for (int i = 0; i < 32; ++i) tot[BASE + i] += (v[i] * mm) >> 7;
}

// fp8 path: D = S exactly (fp32 accumulation of products of small integers).  The running total lives in a float
// kept inside [2^23, 2^24), where the spacing of floats is 1: a round-down fused multiply-add
//     t <- fma.rm(S, m/16, t)
// adds floor(S*m/16) = (m*S) >> 4 exactly (S*m/16 has at most 21 + 4 significant bits below 2^23, the sum is rounded
// once, downwards, to an integer) -- the reference's shifted term in ONE instruction.  Two neighbouring columns share
// a 64-bit register pair and one packed instruction (fma.rm.f32x2): half the issue slots of the scalar form.
constexpr int FOLD_MAGIC_BITS = 0x4B400000;      // 1.5 * 2^23
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, uint32_t & lo, uint32_t & hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
template <int BASE>
__device__ __forceinline__ void fold32_f8(uint64_t (&tf)[64], const int (&v)[32], uint64_t mf2) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
#ifdef RQ_TC_SCALAR_FMA
        uint32_t lo, hi, m0, m1;
        unpack2(tf[BASE / 2 + i], lo, hi);
        unpack2(mf2, m0, m1);
        float a, b;
        asm("fma.rm.f32 %0, %1, %2, %3;" : "=f"(a) : "f"(__int_as_float(v[2 * i])), "f"(__uint_as_float(m0)), "f"(__uint_as_float(lo)));
        asm("fma.rm.f32 %0, %1, %2, %3;" : "=f"(b) : "f"(__int_as_float(v[2 * i + 1])), "f"(__uint_as_float(m1)), "f"(__uint_as_float(hi)));
        tf[BASE / 2 + i] = pack2(__float_as_uint(a), __float_as_uint(b));
#else
        asm("fma.rm.f32x2 %0, %1, %2, %0;" : "+l"(tf[BASE / 2 + i]) : "l"(pack2((uint32_t) v[2 * i], (uint32_t) v[2 * i + 1])), "l"(mf2));
#endif
    }
}
// Re-centring.  A float in the window is 2^23 + mantissa with mantissa = 2^22 + t, t the running total since the last
// re-centring; bits 20..22 of the mantissa are floor((t + 2^22) / 2^20), a digit in 0..7 that reads 4 for t in
// [0, 2^20).  Every RECENTER_INPUTS inputs that digit moves into an unsigned byte of a packed carry word and is set
// back to 4: three instructions per output.  Bounds: a group of G inputs adds at most 255 * (G*8*15) / 16 in magnitude,
// 2.94 M per 1536 inputs, on top of t in [0, 2^20): the float stays inside [2^23 + 2^22 - 2.94 M, 2^23 + 2^22 + 2^20 +
// 2.94 M), within the window; K <= 32768 has at most 32 re-centrings (groups of 256 re-centre every 1024 inputs, the
// nearest multiple of four groups), so a byte holds at most 32 * 7 = 224.  At the end
//     total = (sum of digits - 4 * number of re-centrings) * 2^20 + (float - 1.5 * 2^23),
// the last term being t, whatever its size: the end of a unit needs no re-centring of its own.
constexpr int RECENTER_INPUTS = 1536;
// The carry words live in shared memory between re-centrings (the per-warp tile that later stages the transposed
// store; word w of lane l at w * 32 + l: conflict-free) -- the registers they would take are the difference between a
// fold loop that fits and one that spills.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// Integer instructions run at half the rate of the FMAs on this part, so the re-centring counts them: byte 2 of each
// of four floats (mantissa bits 16..23) is gathered with three byte permutes, one shift and one mask turn the four
// bytes into the four digits, already packed as the carry word wants them; one logic op per float resets the digit.
__device__ __forceinline__ void recenter(uint64_t (&tf)[64], uint32_t * carry_smem) {
    const uint32_t base = smem_u32(carry_smem);
#pragma unroll
    for (int i = 0; i < 32; ++i) {          // carry word i: columns 4i .. 4i+3 = pairs 2i, 2i+1
        uint32_t w[4];
        unpack2(tf[2 * i], w[0], w[1]);
        unpack2(tf[2 * i + 1], w[2], w[3]);
        const uint32_t g = prmt(prmt(w[0], w[1], 0x0062u), prmt(w[2], w[3], 0x0062u), 0x5410u);
        const uint32_t cw = (g >> 4) & 0x07070707u;
        // a reduction without a return value: nothing waits for shared memory here (a load-add-store chain per word
        // would, the fold leaves no registers to batch the loads)
        asm volatile("red.shared.add.u32 [%0], %1;" :: "r"(base + (uint32_t) (i * 128)), "r"(cw) : "memory");
        // the digits are reset on the 64-bit pairs where they live: two logic ops per pair on its own halves -- taking the
        // halves apart, changing them and packing them again cost four register moves per pair on top
        tf[2 * i] = (tf[2 * i] & 0xFF8FFFFFFF8FFFFFull) | 0x0040000000400000ull;
        tf[2 * i + 1] = (tf[2 * i + 1] & 0xFF8FFFFFFF8FFFFFull) | 0x0040000000400000ull;
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
    int vec;                            // 16-byte stores are safe: ldy % 4 == 0 and every destination 16-byte aligned
};

struct __align__(8) TcShared {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    unsigned int units_stored;          // PUSH: epilogue warps that have stored a unit, summed over units (8 per unit)
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
    // (the warp index through a shuffle from lane 0: the compiler then knows that it, and every tensor-memory and barrier
    // address derived from it, is the same in all lanes, and keeps them in uniform registers)
    const int warp = __shfl_sync(0xffffffffu, (int) (threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
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
        sh.units_stored = 0;
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
                // drain: every slice that was issued must land before the CTA's shared memory is given back.  In a pair
                // both CTAs' bytes complete on rank 0's barriers, so rank 0's waits cover rank 1's copies of the same
                // slices, and rank 1 cannot leave before them: this thread of rank 0 reaches the cluster barrier at the end
                // of the kernel only after the loop below.  Rank 1 can be at most the slice it has just issued ahead of
                // rank 0 (both producers follow the same commits); it cannot watch a remote barrier, so it gives that one
                // copy 100 us -- it was issued into a free slot, a second after everything else stopped.
                if (!PAIR || leader) {
                    for (uint32_t k = it > (uint32_t) STAGES ? it - STAGES : 0; k < it; ++k) {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(smem_u32(&sh.full[k % STAGES]), (k / STAGES) & 1u) && clock64() - t0 < WAIT_CYCLES) { }
                    }
                } else {
                    const long long t0 = clock64();
                    while (clock64() - t0 < 200000ll) { }
                }
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // The whole warp walks the loop with warp-uniform values (descriptors and addresses then live in the uniform
            // datapath) and elects a lane at each MMA and commit.  Straight-line issue loop: shifts instead of divisions (any number of 64-input steps per accumulator), slot, phase and accumulator
            // buffer as running counters, descriptors advanced by adding to their address field.
            const uint64_t da0 = umma_desc(ring), db0 = umma_desc(ring + A_BYTES);
            uint32_t s = 0, ph = 0, gcount = 0;       // ring slot, its phase, accumulator groups issued (all units)
            uint32_t gs = 0;                          // 64-input step inside the current group
            const uint32_t gsteps_u = (uint32_t) gsteps;
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
                        if (++gs == gsteps_u) {
                            gs = 0;
                            RQ_CYC_BEGIN(c_commit);
                            if (PAIR) umma_commit_pair(smem_u32(&sh.tmem_full[buf]));
                            else      umma_commit(smem_u32(&sh.tmem_full[buf]));
                            RQ_CYC_END(c_commit);
                            ++gcount;
                        }
                    }
                    if (!ok) break;
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
    } else if (PUSH && prm.n_more > 0) {
        // Warps 2 and 3 carry the finished units to the other ranks.  The epilogue warps store a unit into this GPU's
        // output only; these two warps read it back (from L2) and store it into every other rank's copy.  Peer stores
        // drain at NVLink speed -- a quarter of a unit's fold time per destination at best -- and a warp that waits for
        // them cannot fold: issued by the epilogue warps they added their whole duration to the kernel.
        const int pw = warp - 2;
        const bool fmt_ok = prm.status == nullptr || prm.status[1] == (F8 ? RQ_FMT_E4M3 : RQ_FMT_I8);
        volatile unsigned int * stored = &sh.units_stored;
        unsigned int k = 0;
        // (a wrong activation format: the epilogue warps store nothing and count nothing, so there is nothing to wait for)
        for (int v = first; v < units && fmt_ok; v += stride, ++k) {
            bool ok = true;
            const long long t0 = clock64();
            while (*stored < 8u * (k + 1u)) {          // bounded, like every wait of this kernel
                if (*abort_flag) { ok = false; break; }
                if (clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; ok = false; break; }
                __nanosleep(256);
            }
            if (!__all_sync(0xffffffffu, ok)) break;
            __threadfence();
            const int n_tile = v / m_units, m_unit = v - n_tile * m_units;
            const int m_tile = PAIR ? 2 * m_unit + (int) rank : m_unit;
            const int row0 = m_tile * BM, col = n_tile * BN + (pw * 32 + lane) * 4;      // 64 lanes x 4 columns = a unit's row
            const int rows = prm.M - row0 < BM ? prm.M - row0 : BM;
            if (prm.vec && col + 3 < prm.N) {
                // four rows of loads in flight per lane (eight, with registers taken from the epilogue warps, changed
                // nothing: 0.494 against 0.497 ms for the 4096 x 17408 node on 4 GPUs -- the peer stores set the pace, about
                // 3.4 GB/s per SM whichever warps issue them)
                for (int r = 0; r < rows; r += 4) {
                    float4 q[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (r + u < rows) q[u] = __ldcg(reinterpret_cast<const float4 *>(prm.y + (size_t) (row0 + r + u) * prm.ldy + col));
                    for (int d = 0; d < prm.n_more; ++d) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (r + u < rows) *reinterpret_cast<float4 *>(prm.y_more[d] + (size_t) (row0 + r + u) * prm.ldy + col) = q[u];
                    }
                }
            } else if (col < prm.N) {
                for (int r = 0; r < rows; ++r) {
                    const size_t at = (size_t) (row0 + r) * prm.ldy + col;
                    float q[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) q[u] = col + u < prm.N ? __ldcg(prm.y + at + u) : 0.0f;
                    for (int d = 0; d < prm.n_more; ++d) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (col + u < prm.N) prm.y_more[d][at + u] = q[u];
                    }
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        const int e = warp - 4, quarter = warp & 3, half = e >> 2;
        uint32_t lane_base = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (half * 128);
        // (opaque to the compiler from here on: it would otherwise rebuild the address from the warp index -- seven integer
        // instructions -- in front of every tensor-memory load instead of keeping it in a register)
        asm volatile("" : "+r"(lane_base));
        // the quantizer records the format it wrote: refuse to multiply the wrong one
        const bool fmt_ok = prm.status == nullptr || prm.status[1] == (F8 ? RQ_FMT_E4M3 : RQ_FMT_I8);
        const uint32_t empty_bar0 = PAIR ? map_to_cta(smem_u32(&sh.tmem_empty[0]), 0) : smem_u32(&sh.tmem_empty[0]);
        const uint32_t full_bar0 = smem_u32(&sh.tmem_full[0]);
        // groups between two re-centrings of the float totals: a multiple of four (the loop below walks four groups at a time)
        const int recenter_every = prm.G >= 256 ? 4 : RECENTER_INPUTS / prm.G;
        const bool vec = prm.vec != 0;
        const bool m_vec = (n_ag & 3) == 0;            // a token's multipliers start on a 16-byte boundary
        float * stg = reinterpret_cast<float *>(smem_raw + (ring - smem_u32(smem_raw)) + STAGES * STAGE_BYTES) + e * 1024;
        uint32_t * carry_smem = reinterpret_cast<uint32_t *>(stg) + lane;
        uint32_t gcount = 0;              // accumulator groups folded (all units)
        bool ok = true;
        RQ_CYC_DECL(c_tfull);
        RQ_CYC_DECL(c_epi);
        RQ_CYC_DECL(c_hold);
        RQ_CYC_DECL(c_rec);
        RQ_CYC_DECL(c_fin);
        RQ_CYC_DECL(c_tail);
        RQ_CYC_BEGIN(c_epi);
        for (int v = first; v < units && ok; v += stride) {
            const int n_tile = v / m_units, m_unit = v - n_tile * m_units;
            const int m_tile = PAIR ? 2 * m_unit + (int) rank : m_unit;
            const int row = m_tile * BM + quarter * 32 + lane;
            const bool row_ok = row < prm.M;
            const int32_t * mrow = prm.msh + (size_t) (row_ok ? row : 0) * n_ag;
            int row_live = row_ok ? 1 : 0;
            // (kept in registers for the unit: rebuilt from the lane index they cost a dozen integer instructions per load)
            asm volatile("" : "+l"(mrow), "+r"(row_live));
            // the multipliers of four groups at a time (one 16-byte load where a token's row of them is aligned); rows
            // beyond M fold with 0
            auto load_m4 = [&](int ag) -> int4 {
                int4 r = make_int4(0, 0, 0, 0);
                if (!row_live) return r;
                if (m_vec) return __ldg(reinterpret_cast<const int4 *>(mrow + ag));
                r.x = __ldg(mrow + ag);
                if (ag + 1 < n_ag) r.y = __ldg(mrow + ag + 1);
                if (ag + 2 < n_ag) r.z = __ldg(mrow + ag + 2);
                if (ag + 3 < n_ag) r.w = __ldg(mrow + ag + 3);
                return r;
            };
            int tot[F8 ? 1 : 128];
            uint64_t tf[F8 ? 64 : 1];
            if (F8) {
#pragma unroll
                for (int i = 0; i < 64; ++i) tf[F8 ? i : 0] = pack2((uint32_t) FOLD_MAGIC_BITS, (uint32_t) FOLD_MAGIC_BITS);
#pragma unroll
                for (int i = 0; i < 32; ++i) carry_smem[i * 32] = 0u;      // (the previous unit's store ended with a warp barrier)
            } else {
#pragma unroll
                for (int i = 0; i < 128; ++i) tot[F8 ? 0 : i] = 0;
            }
            int since = 0, n_rec = 0;
            int4 mcur = load_m4(0);
            const bool fast4 = (n_ag & 3) == 0;        // then the running group count is a multiple of four at every four groups
            // Software pipeline over 32-column pieces of the accumulator: the tensor-memory load of piece c+1 is in flight
            // while piece c folds, and the first piece of the NEXT group is requested (its barrier permitting) before the
            // last piece of this group folds, so a warp never sits out a whole load latency.
            int va[32], vb[32];
            RQ_CYC_BEGIN(c_tfull);
            if (!__all_sync(0xffffffffu, mbar_wait(full_bar0 + (gcount & 1u) * 8u, (gcount >> 1) & 1u, abort_flag))) { ok = false; break; }
            RQ_CYC_END(c_tfull);
            tc_fence_after();
            tmem_ld32(lane_base + (gcount & 1u) * BN, va);
            for (int ag = 0; ag < n_ag && ok; ag += 4) {
                const int mq[4] = { mcur.x, mcur.y, mcur.z, mcur.w };
                if (ag + 4 < n_ag) mcur = load_m4(ag + 4);
                const int cnt = n_ag - ag < 4 ? n_ag - ag : 4;
                // One group.  FAST: the unit's groups come in fours (always with groups of 64 inputs), so the accumulator
                // buffer and the barrier phase of group j of the four are known when the code is compiled, up to the
                // phase p0 the four start with -- the integer instructions that would derive them from the running
                // count run at half rate and hold the issue port.
                auto group = [&](auto jc, auto fc, uint32_t p0) {
                    constexpr int J = decltype(jc)::value;
                    constexpr bool FAST = decltype(fc)::value;
                    const uint32_t buf = FAST ? (uint32_t) (J & 1) : (gcount & 1u);
                    const uint32_t t0 = lane_base + buf * BN;
                    uint64_t mf2 = 0;
                    if constexpr (F8) mf2 = pack2((uint32_t) mq[J], (uint32_t) mq[J]);      // f32 bits of m / 16, twice
                    const int mm = mq[J];
                    RQ_CYC_BEGIN(c_hold);
                    tmem_ld_wait(va); tmem_ld32(t0 + 32, vb);
                    if constexpr (F8) fold32_f8<0>(tf, va, mf2); else fold32_i8<0>(tot, va, mm);
                    tmem_ld_wait(vb); tmem_ld32(t0 + 64, va);
                    if constexpr (F8) fold32_f8<32>(tf, vb, mf2); else fold32_i8<32>(tot, vb, mm);
                    tmem_ld_wait(va); tmem_ld32(t0 + 96, vb);
                    if constexpr (F8) fold32_f8<64>(tf, va, mf2); else fold32_i8<64>(tot, va, mm);
                    tmem_ld_wait(vb);
                    // the accumulator is in registers: hand the buffer back before the last piece is folded
                    tc_fence_before();
                    __syncwarp();
                    if (PAIR) mbar_arrive_cluster_lane0(empty_bar0 + buf * 8u, lane);
                    else      mbar_arrive_lane0(empty_bar0 + buf * 8u, lane);
                    RQ_CYC_END(c_hold);
                    RQ_CYC_BEGIN(c_tail);
                    ++gcount;
                    if (FAST ? (J < 3 || ag + 4 < n_ag) : (ag + J + 1 < n_ag)) {
                        const uint32_t nbuf = FAST ? (uint32_t) ((J + 1) & 1) : (gcount & 1u);
                        const uint32_t nph = FAST ? (p0 ^ (uint32_t) (((J + 1) >> 1) & 1)) : ((gcount >> 1) & 1u);
                        // the loads are warp-collective: leave the loop together or not at all
                        RQ_CYC_BEGIN(c_tfull);
                        ok = __all_sync(0xffffffffu, mbar_wait(full_bar0 + nbuf * 8u, nph, abort_flag));
                        RQ_CYC_END(c_tfull);
                        if (ok) {
                            tc_fence_after();
                            tmem_ld32(lane_base + nbuf * BN, va);
                        }
                    }
                    if constexpr (F8) fold32_f8<96>(tf, vb, mf2); else fold32_i8<96>(tot, vb, mm);
                    RQ_CYC_END(c_tail);
                };
                if (fast4) {
                    uint32_t p0 = (gcount >> 1) & 1u;
                    asm volatile("" : "+r"(p0));           // (likewise: one value per four groups, not three instructions per use)
                    if (ok) group(std::integral_constant<int, 0>{}, std::true_type{}, p0);
                    if (ok) group(std::integral_constant<int, 1>{}, std::true_type{}, p0);
                    if (ok) group(std::integral_constant<int, 2>{}, std::true_type{}, p0);
                    if (ok) group(std::integral_constant<int, 3>{}, std::true_type{}, p0);
                } else {
                    if (0 < cnt && ok) group(std::integral_constant<int, 0>{}, std::false_type{}, 0u);
                    if (1 < cnt && ok) group(std::integral_constant<int, 1>{}, std::false_type{}, 0u);
                    if (2 < cnt && ok) group(std::integral_constant<int, 2>{}, std::false_type{}, 0u);
                    if (3 < cnt && ok) group(std::integral_constant<int, 3>{}, std::false_type{}, 0u);
                }
                if constexpr (F8) {
                    since += cnt;
                    if (since >= recenter_every) {          // (none at the end of the unit: the final conversion takes the total as it stands)
                        RQ_CYC_BEGIN(c_rec);
                        recenter(tf, carry_smem); since = 0; ++n_rec;
                        RQ_CYC_END(c_rec);
                    }
                }
            }
            if (!ok) break;
            if (!fmt_ok) {
                if (lane == 0 && prm.status != nullptr) atomicExch(prm.status, 2);
                continue;
            }
            RQ_CYC_BEGIN(c_fin);
            {
                // Final scaling y = ((float(total) * 16) * u) * s_w and the store.  A thread owns a token's 128 outputs,
                // but a row-per-thread store would scatter 16-byte pieces over 32 rows: the warp transposes 32 x 32
                // pieces through shared memory (16-byte chunks XOR-swizzled by row, conflict-free both ways), after which
                // eight lanes write 128 contiguous bytes of a row and apply s_w, which is per column.
                // (total * 16) * u as ONE multiply by 16u: the factor 16 is exact on either side (u = R / 3825 with R a
                // finite float difference cannot overflow times 16), so the product is rounded once, from the same real
                const float ut16 = __fmul_rn(row_ok ? __ldg(prm.u + row) : 0.0f, 16.0f);
                const int jj = lane & 7, rsub = lane >> 3;
                // Shared-memory addresses of the transposition, kept in registers (opaque to the compiler, which would
                // otherwise rebuild each from the warp and lane indices -- a dozen integer instructions -- at every access):
                // this lane's row for the stores with its swizzle term, and for the loads row rsub with the term of
                // (row, 16-byte chunk jj); rows it8*4 + rsub differ from it by 512 bytes per step and, in the swizzle, by
                // the bit of it8's parity.
                uint32_t st_addr = smem_u32(stg) + (uint32_t) lane * 128u, st_x = (uint32_t) (lane & 7) << 4;
                uint32_t ld_addr = smem_u32(stg) + (uint32_t) rsub * 128u, ld_x = (uint32_t) (jj ^ rsub) << 4;
                asm volatile("" : "+r"(st_addr), "+r"(st_x), "+r"(ld_addr), "+r"(ld_x));
                const bool sw_vec = (reinterpret_cast<uintptr_t>(prm.sw) & 15) == 0;
                auto piece_col = [&](int c) -> int { return n_tile * BN + half * 128 + c * 32 + jj * 4; };
                // the carry words come back into registers (the fold's load buffers are free now) before the tile is reused
                uint32_t carry[F8 ? 32 : 1];
                if constexpr (F8) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) carry[i] = carry_smem[i * 32];
                    __syncwarp();
                }
                // float(total) without integer conversions (they run at a quarter of the FMA rate): the digit byte becomes
                // the mantissa of 2^23 + digit with one byte permute, both parts are made floats by exact subtractions, and
                // one fused multiply-add forms digit * 2^20 + low with the single round-to-nearest an int -> float
                // conversion of the total would make.  Every re-centring moved a digit that stood for digit - 4 units of
                // 2^20 and left 4 behind; what the float holds beyond 1.5 * 2^23 now is the rest of the total, whatever its
                // digit reads.
                // (the float itself is 1.5 * 2^23 = 12 * 2^20 plus that rest: the 12 goes into the digit's subtrahend and the
                // float enters the multiply-add as it is)
                const float dsub = 8388608.0f + (float) (4 * n_rec + 12);
                {
                // the row units of all four column pieces, requested before anything else: one load latency per unit
                float sc[4][4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int ncol = piece_col(c);
                    if (sw_vec && ncol + 3 < prm.N) {
                        const float4 q = __ldg(reinterpret_cast<const float4 *>(prm.sw + ncol));
                        sc[c][0] = q.x; sc[c][1] = q.y; sc[c][2] = q.z; sc[c][3] = q.w;
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) sc[c][k] = ncol + k < prm.N ? __ldg(prm.sw + ncol + k) : 0.0f;
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = c * 32 + j * 4;
                        float f[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float totalf;
                            if constexpr (F8) {
                                uint32_t w[2];
                                unpack2(tf[F8 ? (i + k) >> 1 : 0], w[0], w[1]);
                                const float df = __fsub_rn(__uint_as_float(prmt(carry[F8 ? i >> 2 : 0], 0x4B000000u, 0x7650u | (uint32_t) k)), dsub);
                                totalf = __fmaf_rn(df, 1048576.0f, __uint_as_float(w[k & 1]));
                            } else {
                                totalf = (float) tot[F8 ? 0 : i + k];
                            }
                            f[k] = __fmul_rn(totalf, ut16);
                        }
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(st_addr + (st_x ^ (uint32_t) (j << 4))), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]) : "memory");
                    }
                    __syncwarp();
                    const int ncol = piece_col(c);
                    float * yrow = prm.y + (size_t) (m_tile * BM + quarter * 32 + rsub) * prm.ldy + ncol;      // row rsub; + 4 rows per step
#pragma unroll
                    for (int it8 = 0; it8 < 8; ++it8) {
                        const int grow = m_tile * BM + quarter * 32 + it8 * 4 + rsub;
                        float4 q;       // row it8*4 + rsub, chunk jj ^ (row & 7) = jj ^ rsub ^ 4*(it8 & 1)
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(q.x), "=f"(q.y), "=f"(q.z), "=f"(q.w)
                                     : "r"(ld_addr + (uint32_t) (it8 * 512) + (ld_x ^ (uint32_t) ((it8 & 1) << 6))) : "memory");
                        const float o0 = __fmul_rn(q.x, sc[c][0]), o1 = __fmul_rn(q.y, sc[c][1]), o2 = __fmul_rn(q.z, sc[c][2]), o3 = __fmul_rn(q.w, sc[c][3]);
                        if (grow < prm.M) {
                            // this GPU's buffer; N-sharded ranks get their copies from warps 2 and 3
                            float * yr = yrow + (size_t) (it8 * 4) * prm.ldy;
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
                    __syncwarp();
                }
                }
            }
            if constexpr (PUSH) {
                // the unit is in this GPU's output: let the pushing warps see it
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(&sh.units_stored, 1u);
            }
            RQ_CYC_END(c_fin);
        }
        RQ_CYC_END(c_epi);
        if (warp == 4 && lane == 0) { RQ_CYC_REPORT(prm.status, 0x45, c_tfull); RQ_CYC_REPORT(prm.status, 0x46, c_epi); RQ_CYC_REPORT(prm.status, 0x49, c_hold);
                                      RQ_CYC_REPORT(prm.status, 0x4a, c_rec); RQ_CYC_REPORT(prm.status, 0x4b, c_fin); RQ_CYC_REPORT(prm.status, 0x4c, c_tail); }
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
    // resolved once; the initialisation of a function-local static is thread-safe
    static const encode_fn_t fn = []() -> encode_fn_t {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            return reinterpret_cast<encode_fn_t>(p);
        }
        return nullptr;
    }();
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
    // first use on a device (normally rq_w4a4_prepare's, outside stream capture); several host threads may get here at once
    static std::mutex mu;
    static bool configured[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    int sms;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            e = rq_configure_gemm_tc();
            if (e != cudaSuccess) return e;
            e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
        sms = sm_count[dev] > 0 ? sm_count[dev] : 148;
    }
    alignas(64) CUtensorMap ta, tb;
    if (rq_encode_tmap_i8(&ta, a8, K, M, BM) != 0) return cudaErrorInvalidValue;
    memcpy(&tb, tmap_w8, sizeof(tb));
    TcParams prm;
    prm.sw = sw; prm.msh = msh; prm.u = u; prm.y = y; prm.ldy = ldy; prm.status = status;
    prm.K = (int) K; prm.N = (int) N; prm.M = (int) M; prm.G = G;
    prm.n_more = n_more;
    // 16-byte stores only when every destination allows them (a peer's buffer may be aligned differently from ours)
    bool vec = (ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    for (int d = 0; d < RQ_MAX_RANKS - 1; ++d) {
        prm.y_more[d] = d < n_more ? y_more[d] : nullptr;
        if (d < n_more) vec = vec && (reinterpret_cast<uintptr_t>(y_more[d]) & 15) == 0;
    }
    prm.vec = vec ? 1 : 0;
    static const int no_pair = rq_env_int("RQ_TUNE_TC_NOPAIR", 0);
    const bool pair = M > BM && !no_pair;      // a second token tile exists: let two CTAs share the weight slices
    const bool f8 = fmt == RQ_FMT_E4M3;
    if (n_more > 0) {
        if (f8) return pair ? launch_tc<true, true, true>(ta, tb, prm, sms, stream) : launch_tc<true, false, true>(ta, tb, prm, sms, stream);
        return pair ? launch_tc<false, true, true>(ta, tb, prm, sms, stream) : launch_tc<false, false, true>(ta, tb, prm, sms, stream);
    }
    if (f8) return pair ? launch_tc<true, true, false>(ta, tb, prm, sms, stream) : launch_tc<true, false, false>(ta, tb, prm, sms, stream);
    return pair ? launch_tc<false, true, false>(ta, tb, prm, sms, stream) : launch_tc<false, false, false>(ta, tb, prm, sms, stream);
}
