// bfloat16 matrix product for many tokens (prefill) on pairs of SMs:
//
//     Y[T, N] = X[T, K] * W[N, K]^T (+ bias[N]),   float32 accumulation, bfloat16 output
//
// (the linear operator of xsmccc/llaisys, src/ops/linear/cpu/linear_cpu.cpp:21-40), and with DUAL
// the fused gate/up product  Y[T, I] = up * gate / (1 + exp(-gate))
// (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21) of a [2I, K] matrix whose up rows lie dual_offset
// rows below the gate rows.
//
// Two CTAs on neighbouring SMs (a cluster of two) work on one tile of 256 weight rows x BN tokens
// with tcgen05.mma.cta_group::2: each CTA holds its own 128 weight rows and HALF of the token
// tile in shared memory, the tensor cores of both SMs read both halves, and each CTA's tensor
// memory receives its 128 rows x BN tokens.  An SM thus fills a third less shared memory per FLOP
// than it would alone.  The pair is persistent: it walks over tiles pair, pair + pairs, ....
// An accumulator is 256 tokens = 256 columns, so tensor memory holds two, and the epilogue of a
// tile (tcgen05.ld, bias or SwiGLU, transposition through shared memory, 16-byte stores) runs while
// the tensor cores work on the next one.
//
// DUAL has two variants.  1 (a short K range): a CTA's 128 weight rows are 64 gate rows followed by
// the 64 up rows of the same outputs (two TMA boxes of 64 rows into one operand tile), so the one
// accumulator holds gate values in lanes 0-63 and up values in lanes 64-127, and the epilogue warps
// of the upper lanes pass theirs to the warps of the lower lanes through shared memory.  2 (a long
// K range): 128 gate rows and 128 up rows with an accumulator each, which fill tensor memory, so the
// next tile's products wait for the epilogue, but an SM takes a third less from the L2 per FLOP.
// (The benchmark's gate/up product at 2,048 tokens, K = 1536: 68 us with the first, 76 with the second.)
//
//   warp 0      TMA producer (one thread): ring of STAGES k-blocks, both CTAs, completion counted on the
//               leader CTA's barrier
//   warp 1      tcgen05.mma issue (one thread of the leader CTA); tcgen05.commit multicast frees the ring
//               slot in both CTAs and, per tile, hands the accumulator to both epilogues
//   warps 2-17  epilogue of this CTA's 128 rows: four warps per 32 rows, each with 8 of every 32 columns, transposed
//               through a buffer of the warp's own (no barrier among the storing warps)
//
// INTO (an instantiation of its own): the product is not stored but added to a float32 stream [T, N]
// (the residual stream: an output projection or a down projection that ends in the residual add of
// src/models/qwen2/layer.hpp:60-66, 75-81).  The pair's work units are then (tile, K range): where one
// round of tiles would leave many pairs idle (48 tiles on 74 pairs), the K range is cut so that the
// units fill the rounds, and every unit adds its partial tile to the stream with one TMA reduction
// (cp.reduce.async.bulk.tensor ... add) per 32 tokens from a float32 staging buffer.  Nothing is
// gathered or re-read: the sums meet in the L2.
//
// Every wait on an mbarrier is bounded; when a bound is hit the role records an error code in
// *err and stops, the other roles run into their own bounds, and both CTAs meet at the final
// cluster barrier, free their tensor memory and return.
#include "common.cuh"
#include "tma_map.cuh"

namespace {

constexpr int BM = 128;        // weight rows of one CTA (half of the pair's UMMA M)
constexpr int BK = 64;         // k elements of a stage: one 128-byte swizzled row of bf16
constexpr int UMMA_K = 16;
constexpr int EPI_SHARE = 4;                       // epilogue warps that share 32 rows (a quarter of tensor memory's lanes)
constexpr int EPI_THREADS = 128 * EPI_SHARE;
constexpr int THREADS = 64 + EPI_THREADS;
constexpr int CHUNK = 32;                          // tokens that the epilogue transposes at a time
constexpr int COLS = CHUNK / EPI_SHARE;            // of which a warp takes this many
constexpr uint32_t WAIT_LIMIT = 1u << 22;

constexpr uint64_t HINT_EVICT_FIRST = 0x12F0000000000000ull;
constexpr uint64_t HINT_EVICT_LAST = 0x14F0000000000000ull;

enum { ERR_TC2_WAIT_FULL = 111, ERR_TC2_WAIT_EMPTY = 112, ERR_TC2_WAIT_ACC_FULL = 113, ERR_TC2_WAIT_ACC_EMPTY = 114 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrival on a barrier of any CTA of the cluster (a shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

// TMA load of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on a barrier that
// may belong to the other CTA of the pair (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y,
                                                 uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y), "l"(hint) : "memory");
}

// K-major tile, 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart (what the TMA box writes).
// Bounded wait of a whole (converged) warp: every lane polls and the vote keeps the control flow uniform (a satisfied
// wait costs about 60 cycles so, several times that with one lane polling in a divergent branch).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return true;
        if ((i & 255u) == 255u && __any_sync(0xffffffffu, *abort_flag != 0)) return false;
    }
    return false;
}
// True in exactly one lane of a converged warp; the compiler knows that what follows runs in one thread.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16: bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair, N = n.
__device__ __forceinline__ uint32_t umma_idesc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs once the MMAs issued so far are complete
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// One row of COLS accumulator columns; the registers hold the values after the next tcgen05.wait::ld.
__device__ __forceinline__ void tmem_ld_cols_nowait(uint32_t taddr, uint32_t* r) {
    static_assert(COLS == 8, "a warp takes 8 of every 32 columns");
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

// The two special-function results of a SwiGLU output as single instructions: without .ftz each of them comes with
// a few more that rescale subnormal arguments and results, which decide nothing here (exp(-gate) below 1e-38 adds
// nothing to 1, and a quotient below 1e-38 is rounded to a bfloat16 zero either way).
__device__ __forceinline__ float ex2_ftz(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_ftz(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

struct Gemm2Args {
    const void* bias;      // [rows_out] or null
    int bias_dtype;
    bf16* Y;               // [T, ldy]
    int T, K, ldy;
    int rows_out;          // N, or the number of gate rows with DUAL
    int dual_offset;
    int tok_tiles, n_tiles, n_pairs;
    int* err;
    int ksplit, chunk_kb;  // INTO: K ranges per tile and k-blocks per range (1 and all of them otherwise)
};

// The loads issued so far have arrived.  The registers pass through the statement so that no use of them is
// scheduled ahead of it (the compiler sees no other dependence between the load, the wait and the use); pin_cols does
// the same for a second set of registers loaded before the wait.
__device__ __forceinline__ void tmem_wait_ld_cols(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]) :: "memory");
}
__device__ __forceinline__ void pin_cols(uint32_t* r) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]) :: "memory");
}

template <int BN, int STAGES, int DUAL, bool INTO = false>
struct Smem2 {
    static constexpr int ACCS = DUAL == 2 ? 2 : 1;                // accumulators of a tile (DUAL 2: gate and up apart)
    static constexpr int A_BYTES = BM * BK * 2;                   // 128 weight rows (DUAL 1: 64 gate rows, then 64 up rows)
    static constexpr int B_BYTES = (BN / 2) * BK * 2;             // this CTA's half of the token tile
    static constexpr int STAGE_BYTES = ACCS * A_BYTES + B_BYTES;
    static constexpr int STG_OFFSET = STAGES * STAGE_BYTES;
    // transposition buffers: INTO two of [32 tokens][128 rows] float32 for all; else two of [COLS tokens][32 rows] bf16
    // per storing warp.  DUAL 1: behind them the exchange buffers, two of [COLS tokens][32 rows] float32 per up warp.
    static constexpr int STG_BYTES = INTO ? 2 * CHUNK * BM * 4 : (EPI_THREADS / 32) * 2 * COLS * 32 * 2;
    static constexpr int XCH_OFFSET = STG_OFFSET + STG_BYTES;
    static constexpr int XCH_BYTES = DUAL == 1 ? (EPI_THREADS / 64) * 2 * COLS * 32 * 4 : 0;
    static constexpr int BAR_OFFSET = XCH_OFFSET + XCH_BYTES;
    static constexpr int N_BARS = 2 * STAGES + 4;
    static constexpr int TOTAL = BAR_OFFSET + N_BARS * 8 + 16 + 1024;   // + slack to align the base
    static constexpr int ACC_COLS = ACCS * BN;                    // tensor-memory columns of one accumulator buffer
    static constexpr int NBUF = 512 / ACC_COLS;                   // buffers in the 512 columns of tensor memory: 2 or 1
    static constexpr int MROWS = DUAL == 1 ? BM / 2 : BM;         // output rows of one CTA's tile
    static_assert(ACC_COLS == 256 || ACC_COLS == 512, "an accumulator buffer is a half or the whole of tensor memory");
    static_assert(TOTAL <= 232448, "a block's shared memory");
};

template <int BN, int STAGES, int DUAL, bool INTO = false>
__global__ void __launch_bounds__(THREADS)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_out, Gemm2Args g) {
    LLB_STAMPS_BEGIN();
    if (threadIdx.x == 64) LLB_STAMP(0);
    using S = Smem2<BN, STAGES, DUAL, INTO>;
    constexpr int ACCS = S::ACCS, ACC_COLS = S::ACC_COLS, NBUF = S::NBUF, MROWS = S::MROWS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base + S::BAR_OFFSET, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_acc_full = bar_empty + 8 * STAGES, bar_acc_empty = bar_acc_full + 16, tmem_slot = bar_acc_empty + 16;
    volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + S::BAR_OFFSET + S::N_BARS * 8);
    __shared__ int s_abort, s_epi_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int kblocks = (g.K + BK - 1) / BK;
    // work units: unit u is tile u % n_tiles over the k-blocks [(u / n_tiles) * chunk_kb, ...) (one unit per tile unless INTO)
    const int n_units = g.n_tiles * g.ksplit;
    auto unit_kb0 = [&](int u) { return (u / g.n_tiles) * g.chunk_kb; };
    auto unit_kb1 = [&](int u) { return min(kblocks, (u / g.n_tiles + 1) * g.chunk_kb); };

    if (tid == 0) {
        s_abort = 0;
        s_epi_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);          // the leader's is used: its producer's expect_tx, bytes of both CTAs
            mbar_init(bar_empty + 8 * s, 1);         // one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);      // one multicast commit per tile
            mbar_init(bar_acc_empty + 8 * b, 2 * (EPI_THREADS / 32));    // the leader's is used: the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {                                 // the same warp of both CTAs allocates, and frees at the end
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // both CTAs' barriers and tensor memory stand before either touches the other's
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;

    // The weight does not depend on any earlier kernel of the step: the first tile's first STAGES k-blocks of it are
    // requested before the grid dependency resolves, while the predecessor is still running.
    const int first_kb0 = unit_kb0(pair);
    const int prefetched = min(STAGES, unit_kb1(pair) - first_kb0);
    if (warp == 0 && lane == 0) {
        const uint32_t full0 = mapa(bar_full, 0);
        const int m0 = (((pair % g.n_tiles) / g.tok_tiles) * 2 + (int)rank) * MROWS;
        for (int i = 0; i < prefetched; ++i) {
            const uint32_t dst = base + i * S::STAGE_BYTES, bar = full0 + 8 * i;
            if (leader) mbar_expect_tx(bar_full + 8 * i, 2u * S::STAGE_BYTES);
            tma_load_2d_pair(dst, &map_w, bar, (first_kb0 + i) * BK, m0, HINT_EVICT_FIRST);      // DUAL 1: the map's box is 64 rows
            if (DUAL) tma_load_2d_pair(dst + S::A_BYTES / (3 - DUAL), &map_w, bar, (first_kb0 + i) * BK, m0 + g.dual_offset, HINT_EVICT_FIRST);
        }
    }
    llb_grid_dependency_sync();      // from here on memory written by earlier kernels is touched

    if (warp == 0) {
        // ---- producer: this CTA's weight rows and its half of the tokens, k-block after k-block, tile after tile.  The
        // warp waits for a free stage as a whole; one elected lane issues the copies.
        const uint32_t full0 = mapa(bar_full, 0);
        if (elect_one()) {   // the activations of the k-blocks whose weight is on its way already
            const int n0 = ((pair % g.n_tiles) % g.tok_tiles) * BN + (int)rank * (BN / 2);
            for (int i = 0; i < prefetched; ++i)
                tma_load_2d_pair(base + i * S::STAGE_BYTES + ACCS * S::A_BYTES, &map_x, full0 + 8 * i, (first_kb0 + i) * BK, n0, HINT_EVICT_LAST);
        }
        __syncwarp();
        int it = prefetched;
        bool ok = true;
        for (int u = pair; u < n_units && ok; u += g.n_pairs) {
            const int t = u % g.n_tiles, kb1 = unit_kb1(u);
            const int m0 = ((t / g.tok_tiles) * 2 + (int)rank) * MROWS;
            const int n0 = (t % g.tok_tiles) * BN + (int)rank * (BN / 2);
            for (int kb = unit_kb0(u) + (u == pair ? prefetched : 0); kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !warp_wait(bar_empty + 8 * s, (uint32_t)(it / STAGES - 1) & 1u, &s_abort)) {
                    if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC2_WAIT_EMPTY); }
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    const uint32_t dst = base + s * S::STAGE_BYTES, bar = full0 + 8 * s;
                    if (leader) mbar_expect_tx(bar_full + 8 * s, 2u * S::STAGE_BYTES);
                    tma_load_2d_pair(dst, &map_w, bar, kb * BK, m0, HINT_EVICT_FIRST);
                    if (DUAL) tma_load_2d_pair(dst + S::A_BYTES / (3 - DUAL), &map_w, bar, kb * BK, m0 + g.dual_offset, HINT_EVICT_FIRST);
                    tma_load_2d_pair(dst + ACCS * S::A_BYTES, &map_x, bar, kb * BK, n0, HINT_EVICT_LAST);
                }
                __syncwarp();
            }
        }
        if (s_abort && leader && lane == 0) {
            // copies in flight (of both CTAs) must land before the pair gives up its shared memory
            int first = it > STAGES ? it - STAGES : 0;
            for (int i = first; i < it; ++i)
                for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try(bar_full + 8 * (i % STAGES), (uint32_t)(i / STAGES) & 1u); ++w) {}
        }
        __syncwarp();
    } else if (warp == 1) {
        if (leader) {
            // ---- tensor-core issue for both SMs: the warp waits as a whole, one elected lane issues; the operand
            // descriptors are made once and a stage's or an instruction's own differ from them by a constant
            const uint32_t idesc = umma_idesc_pair(BN);
            const uint64_t a_desc0 = umma_desc(base), b_desc0 = umma_desc(base + ACCS * S::A_BYTES);
            int it = 0, ti = 0;
            bool ok = true;
            for (int u = pair; u < n_units && ok; u += g.n_pairs, ++ti) {
                const int buf = ti % NBUF, kb0 = unit_kb0(u), kb1 = unit_kb1(u);
                if (ti >= NBUF && !warp_wait(bar_acc_empty + 8 * buf, (uint32_t)(ti / NBUF - 1) & 1u, &s_abort)) {
                    if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC2_WAIT_ACC_EMPTY); }
                    break;
                }
                const uint32_t acc = tmem + buf * ACC_COLS;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!warp_wait(bar_full + 8 * s, (uint32_t)(it / STAGES) & 1u, &s_abort)) {
                        if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC2_WAIT_FULL); }
                        ok = false;
                        break;
                    }
                    if (elect_one()) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t so = (uint64_t)(s * (S::STAGE_BYTES >> 4));
                        const uint64_t ad = a_desc0 + so, bd = b_desc0 + so, ad2 = ad + (uint64_t)(S::A_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint32_t accumulate = (kb > kb0 || k > 0) ? 1u : 0u;
                            const uint64_t step = (uint64_t)(k * UMMA_K * 2 >> 4);      // the start address field counts 16 bytes
                            umma_pair(acc, ad + step, bd + step, idesc, accumulate);
                            if (DUAL == 2) umma_pair(acc + BN, ad2 + step, bd + step, idesc, accumulate);
                        }
                        umma_commit_both(bar_empty + 8 * s);
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (elect_one()) umma_commit_both(bar_acc_full + 8 * buf);
                __syncwarp();
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: warp w may read tensor-memory lanes 32 (w mod 4) .. + 31; a thread owns one weight row and COLS of
        // every 32 columns.  DUAL 1: lanes 0-63 hold gate rows and lanes 64-127 the up rows of the same outputs, so a warp
        // of the upper half hands its values to the warp of the lower half with the same rows and columns through shared
        // memory, with a barrier of the two warps per chunk; the lower warps compute and store.  DUAL 2: a thread reads
        // its row's gate value from the first accumulator and its up value from the second.
        const int et = tid - 64;                                  // 0 .. EPI_THREADS - 1
        const int q = warp & 3, share = (warp - 2) >> 2;
        const int h = share * COLS;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        const uint32_t acc_empty0 = mapa(bar_acc_empty, 0);
        bf16* stg = reinterpret_cast<bf16*>(gen_base + S::STG_OFFSET);
        float* stgf = reinterpret_cast<float*>(gen_base + S::STG_OFFSET);          // INTO: [2][32 tokens][128 rows] float32
        const bool up_warp = DUAL == 1 && q >= 2;
        const int xpair = (q & 1) * EPI_SHARE + share;            // DUAL 1: the two warps' buffers and barrier (ids 2 ..)
        float* xch = reinterpret_cast<float*>(gen_base + S::XCH_OFFSET) + xpair * (2 * COLS * 32);
        const int out_row = DUAL == 1 ? (q & 1) * 32 : q * 32;    // this warp's first output row within the CTA's tile
        const bool stamper = tid == (DUAL == 1 ? 128 : 64);       // (a storing warp's first thread)
        int ti = 0, chunk_i = 0;
        for (int u = pair; u < n_units; u += g.n_pairs, ++ti) {
            const int buf = ti % NBUF, t = u % g.n_tiles;
            const int m0 = ((t / g.tok_tiles) * 2 + (int)rank) * MROWS;
            const int n0 = (t % g.tok_tiles) * BN;
            const int m = m0 + row;
            float bias_v = 0.f;
            if (!DUAL && g.bias && m < g.rows_out && u < g.n_tiles)    // the bias goes in with the first K range only
                bias_v = g.bias_dtype == LLB_F32 ? ((const float*)g.bias)[m] : to_f32(((const bf16*)g.bias)[m]);
            if (!mbar_wait(bar_acc_full + 8 * buf, (uint32_t)(ti / NBUF) & 1u, &s_abort)) {
                s_epi_abort = 1;
                if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC2_WAIT_ACC_FULL); }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            if (stamper && ti < 2) LLB_STAMP(1 + 6 * ti);             // stamps: 1/7 accumulator ready, 2-4 inside a chunk, 5 chunks done, 6/8 handed back
            if (s_epi_abort) break;                               // written before the barrier only: the same for all
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = lane_addr + buf * ACC_COLS;
            // the next columns are on their way from tensor memory while these are worked on
            uint32_t nxt0[COLS], nxt1[COLS];
            tmem_ld_cols_nowait(acc + h, nxt0);
            if (DUAL == 2) tmem_ld_cols_nowait(acc + BN + h, nxt1);
#pragma unroll 1
            for (int c = 0; c < BN; c += CHUNK, ++chunk_i) {
                float v0[COLS], v1[COLS];
                tmem_wait_ld_cols(nxt0);
                if (DUAL == 2) pin_cols(nxt1);                     // (loaded before the wait: valid behind it)
#pragma unroll
                for (int j = 0; j < COLS; ++j) {
                    v0[j] = __uint_as_float(nxt0[j]);
                    if (DUAL == 2) v1[j] = __uint_as_float(nxt1[j]);
                }
                if (c + CHUNK < BN) {
                    tmem_ld_cols_nowait(acc + c + CHUNK + h, nxt0);
                    if (DUAL == 2) tmem_ld_cols_nowait(acc + BN + c + CHUNK + h, nxt1);
                }
                if (INTO) {
                    // this K range's partial sums of 32 tokens x 128 rows, laid out as they lie in the stream, then one
                    // reduction into the stream.  The other buffer is written right after the barrier below (the next
                    // chunk), so the reduction that read it last (the one issued after the barrier before) must have
                    // read it by then: the thread that issues them waits for that before it arrives.
                    float* sf = stgf + (chunk_i & 1) * (CHUNK * BM);
#pragma unroll
                    for (int j = 0; j < COLS; ++j) sf[(h + j) * BM + row] = v0[j] + bias_v;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    if (stamper && ti == 0 && c == CHUNK) LLB_STAMP(2);
                    if (et == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    if (stamper && ti == 0 && c == CHUNK) LLB_STAMP(3);
                    asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                    if (et == 0) {
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                                     ::"l"(&map_out), "r"(m0), "r"(n0 + c), "r"(smem_u32(sf)) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    if (stamper && ti == 0 && c == CHUNK) LLB_STAMP(4);
                    continue;
                }
                if (DUAL == 2) {
#pragma unroll
                    for (int j = 0; j < COLS; ++j)                                  // up * gate / (1 + exp(-gate))
                        v0[j] = v1[j] * v0[j] * rcp_ftz(1.0f + ex2_ftz(-1.4426950408889634f * v0[j]));
                } else if (DUAL == 1) {
                    // The up warp writes buffer chunk_i & 1 and meets the gate warp at their barrier; it writes that buffer
                    // again two chunks on, behind the next chunk's barrier, which the gate warp reaches after these reads.
                    float* xb = xch + (chunk_i & 1) * (COLS * 32);
                    if (up_warp) {
#pragma unroll
                        for (int j = 0; j < COLS; ++j) xb[j * 32 + lane] = v0[j];
                        asm volatile("bar.sync %0, 64;" ::"r"(2 + xpair) : "memory");
                        continue;
                    }
                    asm volatile("bar.sync %0, 64;" ::"r"(2 + xpair) : "memory");
#pragma unroll
                    for (int j = 0; j < COLS; ++j)                                  // up * gate / (1 + exp(-gate))
                        v0[j] = xb[j * 32 + lane] * v0[j] * rcp_ftz(1.0f + ex2_ftz(-1.4426950408889634f * v0[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < COLS; ++j) v0[j] += bias_v;
                }
                // A warp's 32 rows x COLS tokens go through the warp's own two buffers [COLS tokens][32 rows] and out as
                // 64-byte pieces of COLS token rows: no barrier among the storing warps, so one warp's arithmetic runs
                // beside another warp's stores.
                bf16* sw = stg + ((warp - 2) * 2 + (chunk_i & 1)) * (COLS * 32);
#pragma unroll
                for (int j = 0; j < COLS; ++j) sw[j * 32 + lane] = __float2bfloat16_rn(v0[j]);
                if (stamper && ti == 0 && c == 0) LLB_STAMP(2);
                __syncwarp();
                if (stamper && ti == 0 && c == 0) LLB_STAMP(3);
                // four lanes move one token's 32 outputs (64 bytes); eight tokens per pass.  This buffer is written again
                // two chunks on, behind the next chunk's __syncwarp, which every lane passes after these reads.
                const int piece = lane & 3, mcol = m0 + out_row + piece * 8;
                if (mcol < g.rows_out) {
#pragma unroll
                    for (int j = lane >> 2; j < COLS; j += 8) {
                        const int n = n0 + c + h + j;
                        if (n < g.T)
                            *reinterpret_cast<uint4*>(g.Y + (size_t)n * g.ldy + mcol) =
                                *reinterpret_cast<const uint4*>(sw + j * 32 + piece * 8);
                    }
                }
                if (stamper && ti == 0 && c == 0) LLB_STAMP(4);
            }
            if (stamper && ti == 0) LLB_STAMP(5);
            // this buffer may be overwritten by the tile after the next
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8 * buf);
            if (stamper && ti < 2) LLB_STAMP(6 + 2 * ti);
        }
    }

    if (INTO && tid == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");       // the sums have reached memory
    __syncwarp();                              // (that thread's warp goes to the barrier below together)
    // Neither CTA leaves while the other may still signal its barriers, read its shared memory or write its
    // tensor memory.
    __syncthreads();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

template <int BN, int STAGES, int DUAL, bool INTO = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const Gemm2Args& g, cudaStream_t stream) {
    auto k = gemm_tc2_kernel<BN, STAGES, DUAL, INTO>;
    constexpr int smem = Smem2<BN, STAGES, DUAL, INTO>::TOTAL;
    static bool configured[64] = {};         // function attributes belong to a device's copy of the kernel
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -2000 - (int)e;
        configured[dev] = true;
    }
    llb_prefer_max_shared((const void*)k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * g.n_pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (llb_pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaLaunchKernelEx(&cfg, k, mw, mx, mo, g);
    return llb_status();
}

}  // namespace

LLB_DEFINE_SET_STAMPS

// X [T, K] bf16 with row stride ldx; W [N, K] bf16 dense ([2 * dual_offset, K] when dual_offset > 0); Y [T, ldy]
// bf16; bias [N] or null.  max_pairs: how many CTA pairs may run at once (SMs / 2).  Returns
// cudaErrorInvalidValue for what this kernel does not take (the caller then uses the one-CTA kernel).
LLB_API int llb_gemm_tc2(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int T, int N, int K,
                         int ldx, int ldy, int dual_offset, int max_pairs, int* err, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    const int dual = dual_offset > 0;
    const int rows_out = dual ? dual_offset : N;
    if (K <= 0 || K % 8 || ldx % 8 || ldy % 8 || rows_out % 8 || max_pairs < 1 ||
        (((uintptr_t)X | (uintptr_t)W | (uintptr_t)Y) & 15) || (dual && (N != 2 * dual_offset || bias)))
        return (int)cudaErrorInvalidValue;
    const int bn = 256;
    Gemm2Args g;
    g.bias = bias; g.bias_dtype = bias_dtype; g.Y = (bf16*)Y;
    g.T = T; g.K = K; g.ldy = ldy; g.rows_out = rows_out; g.dual_offset = dual_offset;
    g.tok_tiles = (T + bn - 1) / bn;
    // gate/up: with a short K range the one-accumulator variant, whose epilogue runs beside the next tile's products
    // (64 gate and 64 up rows per CTA); with a long one the two-accumulator variant, which takes a third less from the
    // L2 per FLOP and loses little to its exposed epilogue (a prefill step of 2,048 tokens with the first variant: 4 %
    // shorter at K 1536, I 8960; 4 % longer at K 3584, I 18944; the same at K 5120, I 27648).
    const bool side_by_side = dual && K <= 2048;
    const int tile_rows = side_by_side ? BM : 2 * BM;  // output rows of a pair's tile
    const long long tiles = (long long)((rows_out + tile_rows - 1) / tile_rows) * g.tok_tiles;
    if (tiles > (1 << 30)) return (int)cudaErrorInvalidValue;
    g.n_tiles = (int)tiles;
    g.n_pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
    g.err = err;
    g.ksplit = 1;
    g.chunk_kb = (K + BK - 1) / BK;
    CUtensorMap mw, mx;
    int rc = llb_tma::bf16_map_64(W, N, K, K, side_by_side ? BM / 2 : BM, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, K, ldx, bn / 2, &mx);
    if (rc) return rc;
    if (side_by_side) return launch<256, 6, 1>(mw, mx, mw, g, stream);
    return dual ? launch<256, 4, 2>(mw, mx, mw, g, stream) : launch<256, 6, 0>(mw, mx, mw, g, stream);
}

// K ranges per tile for llb_gemm_tc2_into: the count (1 to 4) that minimises rounds of units times the length of a
// unit.  Fitted to measurements at the 1.5B and 7B shapes (2,048 to 8,192 tokens): a k-block of a 256 x 256 tile takes a
// pair 0.37 us, a unit's epilogue (tensor memory -> float32 staging -> reduction) as long as eighteen k-blocks; a cut
// has to win five per cent to be taken.
LLB_API int llb_gemm_tc2_into_ksplit(int T, int N, int K, int max_pairs) {
    const int kblocks = (K + BK - 1) / BK;
    const long long tiles = (long long)((N + 2 * BM - 1) / (2 * BM)) * ((T + 255) / 256);
    const long long whole = ((tiles + max_pairs - 1) / max_pairs) * (kblocks + 18);
    int best = 1;
    long long best_cost = whole;
    for (int ks = 2; ks <= 4 && ks <= kblocks; ++ks) {
        const int chunk = (kblocks + ks - 1) / ks;
        if ((ks - 1) * chunk >= kblocks) continue;                       // an empty range
        const long long rounds = (tiles * ks + max_pairs - 1) / max_pairs, cost = rounds * (chunk + 18);
        if (cost * 100 < whole * 95 && cost < best_cost) { best = ks; best_cost = cost; }
    }
    return best;
}

// stream[T, N] (float32, row stride lds, 16-byte aligned, lds a multiple of 4) += X W^T + bias, for many tokens: the
// same paired kernel, its partial tiles added to the stream by TMA reductions.  ksplit: K ranges per tile (0 chooses).
// The sums of a tile's K ranges meet in the L2 in no fixed order: reproducible up to float32 rounding of that sum.
LLB_API int llb_gemm_tc2_into(const void* X, const void* W, const void* bias, int bias_dtype, float* stream_, int T, int N, int K,
                              int ldx, int lds, int ksplit, int max_pairs, int* err, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || lds % 4 || max_pairs < 1 || !stream_ ||
        (((uintptr_t)X | (uintptr_t)W | (uintptr_t)stream_) & 15))
        return (int)cudaErrorInvalidValue;
    const int bn = 256, kblocks = (K + BK - 1) / BK;
    if (ksplit <= 0) ksplit = llb_gemm_tc2_into_ksplit(T, N, K, max_pairs);
    if (ksplit > kblocks) ksplit = kblocks;
    Gemm2Args g;
    g.bias = bias; g.bias_dtype = bias_dtype; g.Y = nullptr;
    g.T = T; g.K = K; g.ldy = lds; g.rows_out = N; g.dual_offset = 0;
    g.tok_tiles = (T + bn - 1) / bn;
    const long long tiles = (long long)((N + 2 * BM - 1) / (2 * BM)) * g.tok_tiles;
    if (tiles * ksplit > (1 << 30)) return (int)cudaErrorInvalidValue;
    g.n_tiles = (int)tiles;
    g.chunk_kb = (kblocks + ksplit - 1) / ksplit;
    g.ksplit = (kblocks + g.chunk_kb - 1) / g.chunk_kb;                  // no range is empty
    const long long units = tiles * g.ksplit;
    g.n_pairs = (int)(units < max_pairs ? units : max_pairs);
    g.err = err;
    CUtensorMap mw, mx, mo;
    int rc = llb_tma::bf16_map_64(W, N, K, K, BM, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, K, ldx, bn / 2, &mx);
    if (rc) return rc;
    rc = llb_tma::f32_map_plain(stream_, T, N, lds, BM, CHUNK, &mo);
    if (rc) return rc;
    return launch<256, 6, 0, true>(mw, mx, mo, g, stream);
}
