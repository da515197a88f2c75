// The whole SwiGLU feed-forward of a decode step in one launch on the 5th-generation tensor cores:
//
//     residual[T, H] += ( (X Wu^T) * silu(X Wg^T) ) Wd^T          bfloat16 operands, float32 sums
//
// (down(up(x) * silu(gate(x))) of xsmccc/llaisys, src/models/qwen2/mlp.hpp:18-39, swiglu as in
// src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21, followed by the residual add of src/models/qwen2/layer.hpp:75-81.)
//
// For a handful of tokens the three matrices are read once and nothing else matters: the step is
// bound by how steadily the weights stream out of HBM.  Two launches (gate/up, then down) each
// start with an empty pipeline and end with a reduction, and the second cannot prefetch while the
// first one's blocks fill the SMs.  Here the intermediate dimension I is cut into slices of 64
// columns, and a block owns whole slices:
//
//   gate/up   one UMMA tile of M = 128 holds the slice's 64 gate rows (lanes 0-63) and its 64 up rows
//             (lanes 64-127) over the full K = H, so the slice's activations are complete inside the
//             block and SwiGLU needs no reduction across blocks;
//   SwiGLU    the epilogue warps read the accumulator, exchange the up half through shared memory,
//             and write act[token, 64] as bfloat16 into shared memory in the K-major 128-byte-swizzled
//             layout that the tensor core reads;
//   down      act is the B operand (K = 64: one k-block) against the slice's columns of Wd, one tile
//             of 128 output rows at a time, accumulated in tensor memory over all the block's slices;
//   add       each block's partial [T, H] is added to the float32 residual stream by bulk reductions
//             (cp.reduce.async.bulk add.f32) from shared memory, one output tile after the other while the
//             rest of Wd still streams.
//
// So a block's weight traffic is one uninterrupted stream (H/64 k-blocks of gate+up rows, then H/128
// tiles of Wd, per slice) through one ring of TMA stages, issued by one thread that waits for nothing
// but free stages; the first stages are requested before the grid dependency resolves.  No block
// waits for another block.  The sums over slices reach the residual in an order that is not fixed,
// so results are reproducible up to float32 rounding of that last addition, not bit for bit.
//
// Warp roles (192 threads): warp 0 issues TMA, warp 1 owns tensor memory and issues tcgen05.mma,
// warps 2-5 are the epilogue (warp w reads the tensor-memory lanes 32 (w % 4) .. +31).
// Every wait is bounded; a wait that runs out sets the error word and the block leaves in order.
#include "common.cuh"
#include "tma_map.cuh"

namespace {

constexpr int BK = 64;          // k elements of a stage: one 128-byte swizzled row
constexpr int SLICE = 64;       // columns of the intermediate dimension per slice
constexpr int BM = 128;         // rows of a UMMA tile
constexpr int UMMA_K = 16;
constexpr int THREADS = 224;       // warp 0 copies, 1 issues, 2-5 epilogue, 6 hands finished tiles to the copy engine
constexpr int MAX_MT = 32;      // output row tiles of the down projection (tensor memory holds 30 of 16 columns beside the two D1 buffers)
#ifndef LLB_WAIT_LIMIT
#define LLB_WAIT_LIMIT (1u << 22)
#endif
constexpr uint32_t WAIT_LIMIT = LLB_WAIT_LIMIT;
constexpr uint64_t HINT_EVICT_FIRST = 0x12F0000000000000ull;
constexpr uint64_t HINT_EVICT_LAST = 0x14F0000000000000ull;

enum { ERR_MLP_FULL = 131, ERR_MLP_EMPTY = 132, ERR_MLP_D1 = 133, ERR_MLP_EXCH = 134, ERR_MLP_ACT = 135, ERR_MLP_D2 = 136 };   // 136: the output tiles

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait; false when the bound is hit or another thread of the block already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(hint) : "memory");
}
// K-major tile, 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart.
// Bounded wait of a whole (converged) warp: every lane polls and the vote keeps the control flow uniform.
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
// kind::f16: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Programmatic dependent launch, in two halves: every thread lets the next kernel start early; a thread waits for
// the kernels before this one only where it first touches memory that they wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct MlpArgs {
    float* residual;       // [T, H] float32: the result is added here
    int T, H, I;
    int n_slices;          // ceil(I / 64)
    int n_mt;              // ceil(H / 128): output row tiles of the down projection
    int tmem_cols;         // power of two >= 2 BN + n_mt BN
    int* err;
};

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;                  // 16 KB: 64 gate rows + 64 up rows, or 128 rows of Wd
    static constexpr int X_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + X_BYTES;
    static constexpr int ACT_OFFSET = STAGES * STAGE_BYTES;      // two act tiles [BN][64] bf16, swizzled (1024-aligned)
    static constexpr int ACT_BYTES = BN * SLICE * 2;
    static constexpr int EXCH_OFFSET = ACT_OFFSET + 2 * ACT_BYTES;   // two buffers: the up half's exchange [64][BN] float32 during
    static constexpr int EXCH_BYTES = BM * BN * 4;                   // SwiGLU, a staged output tile [BN][128] float32 at the end
    static constexpr int BAR_OFFSET = EXCH_OFFSET + 2 * EXCH_BYTES;
    static constexpr int N_BARS = 2 * STAGES + 10 + MAX_MT;      // full, empty, d1_full[2], exch_full[2], act_full[2], staged[2], unstaged[2], tile[MAX_MT]
    static constexpr int TOTAL = BAR_OFFSET + N_BARS * 8 + 16 + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
mlp_fused_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_up,
                 const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_down,
                 const __grid_constant__ CUtensorMap map_res, MlpArgs g) {
    using S = Smem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    LLB_STAMPS_BEGIN();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base + S::BAR_OFFSET, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_d1 = bar_empty + 8 * STAGES, bar_exch = bar_d1 + 16, bar_act = bar_exch + 16;
    const uint32_t bar_staged = bar_act + 16, bar_unstaged = bar_staged + 16, bar_tile = bar_unstaged + 16;
    const uint32_t tmem_slot = bar_tile + 8 * MAX_MT;
    volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + S::BAR_OFFSET + S::N_BARS * 8);
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB1 = (g.H + BK - 1) / BK;
    // this block's slices: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int my_slices = ((int)blockIdx.x < g.n_slices) ? (g.n_slices - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int per_slice = KB1 + g.n_mt;                   // ring stages a slice takes

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_d1 + 8 * b, 1);
            mbar_init(bar_exch + 8 * b, SLICE);           // the 64 threads that hold up rows
            mbar_init(bar_act + 8 * b, SLICE);            // the 64 threads that hold gate rows
            mbar_init(bar_staged + 8 * b, 128);           // the four epilogue warps have written it to its staging buffer
            mbar_init(bar_unstaged + 8 * b, 1);           // the copy engine has read that buffer
        }
        // One barrier per output tile of the down projection ("complete in tensor memory"), each used once: the issuing
        // thread may be many tiles ahead of the epilogue, and a barrier that completed two phases looks untouched.
        for (int m = 0; m < g.n_mt; ++m) mbar_init(bar_tile + 8 * m, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)g.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;
    const uint32_t tmem_d2 = tmem + 2 * BN;               // D1 buffers at columns [0, BN) and [BN, 2 BN), then n_mt tiles of D2
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (the warp waits, one elected lane issues)
        if (my_slices > 0) {
            // The weights do not depend on any earlier kernel of the step: the first stages' gate and up rows are
            // requested before the grid dependency resolves, their activations after it.
            const int pre = min(STAGES, KB1);
            const int row0 = (int)blockIdx.x * SLICE;
            if (elect_one()) {
                for (int i = 0; i < pre; ++i) {
                    const uint32_t dst = base + i * S::STAGE_BYTES;
                    mbar_expect_tx(bar_full + 8 * i, S::STAGE_BYTES);
                    tma_load_2d(dst, &map_gate, bar_full + 8 * i, i * BK, row0, HINT_EVICT_FIRST);
                    tma_load_2d(dst + S::A_BYTES / 2, &map_up, bar_full + 8 * i, i * BK, row0, HINT_EVICT_FIRST);
                }
            }
            __syncwarp();
            pdl_wait();                                    // the activations are the previous kernel's output
            if (lane == 0) LLB_STAMP(1);                   // stamps: 1 activations ready (grid dependency), 2 first tile of Wd issued,
                                                           //         3 last tile issued, 4 last reduction issued, 5 reductions complete
            if (elect_one()) {
                for (int i = 0; i < pre; ++i)
                    tma_load_2d(base + i * S::STAGE_BYTES + S::A_BYTES, &map_x, bar_full + 8 * i, i * BK, 0, HINT_EVICT_LAST);
            }
            __syncwarp();
            int n = pre;                                   // stages issued so far
            bool ok = true;
            for (int sl = 0; sl < my_slices && ok; ++sl) {
                const int slice = (int)blockIdx.x + sl * (int)gridDim.x;
                for (int j = (sl == 0 ? pre : 0); j < per_slice && ok; ++j, ++n) {
                    const int s = n % STAGES;
                    const uint32_t round = (uint32_t)(n / STAGES);
                    if (round > 0 && !warp_wait(bar_empty + 8 * s, (round - 1) & 1, &s_abort)) {
                        if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_EMPTY); }
                        ok = false;
                        break;
                    }
                    if (elect_one()) {
                        const uint32_t dst = base + s * S::STAGE_BYTES;
                        if (j < KB1) {
                            mbar_expect_tx(bar_full + 8 * s, S::STAGE_BYTES);
                            tma_load_2d(dst, &map_gate, bar_full + 8 * s, j * BK, slice * SLICE, HINT_EVICT_FIRST);
                            tma_load_2d(dst + S::A_BYTES / 2, &map_up, bar_full + 8 * s, j * BK, slice * SLICE, HINT_EVICT_FIRST);
                            tma_load_2d(dst + S::A_BYTES, &map_x, bar_full + 8 * s, j * BK, 0, HINT_EVICT_LAST);
                        } else {
                            mbar_expect_tx(bar_full + 8 * s, S::A_BYTES);
                            tma_load_2d(dst, &map_down, bar_full + 8 * s, slice * SLICE, (j - KB1) * BM, HINT_EVICT_FIRST);
                        }
                    }
                    __syncwarp();
                }
            }
            if (s_abort && lane == 0) {
                // copies in flight must land before this block's shared memory is given up
                const int first = n > STAGES ? n - STAGES : 0;
                for (int i = first; i < n; ++i)
                    for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try(bar_full + 8 * (i % STAGES), (uint32_t)(i / STAGES) & 1u); ++t) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- tensor-core issue
        // The whole warp waits (every lane polls, a vote keeps the warp converged: a satisfied wait costs about 60
        // cycles so, several times that with one lane polling in a divergent branch) and one elected lane issues.
        // The operand descriptors are made once; an instruction's own differs from them by a constant.  Built per
        // instruction by the single issuing thread they cost about as long as a stage takes to arrive.
        if (my_slices > 0) {
            const uint32_t idesc = umma_idesc(BN);
            const uint64_t a_desc0 = umma_desc(base), x_desc0 = umma_desc(base + S::A_BYTES);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int sl = 0; sl < my_slices && ok; ++sl) {
                const int b = sl & 1;
                const uint32_t d1 = tmem + (uint32_t)(b * BN);
                // gate/up: D1[b] = [gate rows; up rows] x X^T over all of K = H
                for (int j = 0; j < KB1; ++j) {
                    if (!warp_wait(bar_full + 8 * s, ph, &s_abort)) {
                        if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_FULL); }
                        ok = false;
                        break;
                    }
                    if (elect_one()) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t so = (uint64_t)(s * (S::STAGE_BYTES >> 4));
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma(d1, a_desc0 + so + (uint64_t)((k * UMMA_K * 2) >> 4), x_desc0 + so + (uint64_t)((k * UMMA_K * 2) >> 4), idesc,
                                 (j > 0 || k > 0) ? 1u : 0u);
                        umma_commit(bar_empty + 8 * s);
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit(bar_d1 + 8 * b);
                __syncwarp();
                // down: D2[m] += Wd[m tile, slice] x act^T, once the epilogue has put act[b] into shared memory
                if (!warp_wait(bar_act + 8 * b, (uint32_t)(sl >> 1) & 1u, &s_abort)) {
                    if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_ACT); }
                    break;
                }
                const uint64_t act_desc0 = umma_desc(base + S::ACT_OFFSET + b * S::ACT_BYTES);
                for (int m = 0; m < g.n_mt; ++m) {
                    if (!warp_wait(bar_full + 8 * s, ph, &s_abort)) {
                        if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_FULL); }
                        ok = false;
                        break;
                    }
                    if (elect_one()) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t so = (uint64_t)(s * (S::STAGE_BYTES >> 4));
#pragma unroll
                        for (int k = 0; k < SLICE / UMMA_K; ++k)
                            umma(tmem_d2 + (uint32_t)(m * BN), a_desc0 + so + (uint64_t)((k * UMMA_K * 2) >> 4),
                                 act_desc0 + (uint64_t)((k * UMMA_K * 2) >> 4), idesc, (sl > 0 || k > 0) ? 1u : 0u);
                        umma_commit(bar_empty + 8 * s);
                        if (sl == my_slices - 1) umma_commit(bar_tile + 8 * m);            // this output tile is final
                        if (sl == my_slices - 1 && m == 0) LLB_STAMP(2);
                        if (sl == my_slices - 1 && m == g.n_mt - 1) LLB_STAMP(3);
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp < 6 && my_slices > 0) {
        // ---------------------------------------------------------------- epilogue (warps 2-5)
        const int q = warp & 3;                            // the quarter of the tensor-memory lanes this warp may read
        const int row = q * 32 + lane;                     // accumulator row: 0-63 gate of column `row`, 64-127 up of column row - 64
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        const bool is_up = row >= SLICE;
        const int col = is_up ? row - SLICE : row;
        bool ok = true;
        for (int sl = 0; sl < my_slices && ok; ++sl) {
            const int b = sl & 1;
            const uint32_t par = (uint32_t)(sl >> 1) & 1u;
            if (!mbar_wait(bar_d1 + 8 * b, par, &s_abort)) {
                if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_D1); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float v[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 16) tmem_ld16(lane_addr + (uint32_t)(b * BN + c), v + c);
            float* exch = reinterpret_cast<float*>(gen_base + S::EXCH_OFFSET + b * S::EXCH_BYTES);       // [64][BN]
            if (is_up) {
#pragma unroll
                for (int n = 0; n < BN; n += 4)
                    *reinterpret_cast<float4*>(exch + col * BN + n) = make_float4(v[n], v[n + 1], v[n + 2], v[n + 3]);
                mbar_arrive(bar_exch + 8 * b);
            } else {
                if (!mbar_wait(bar_exch + 8 * b, par, &s_abort)) {
                    if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_EXCH); }
                    ok = false;
                    break;
                }
                // act[n][col] = up * gate / (1 + exp(-gate)), bfloat16, into the swizzled K-major tile: row n (token) is
                // 128 bytes; its 16-byte piece col / 8 sits at piece (col / 8) ^ (n % 8); groups of 8 rows are 1024 bytes
                uint8_t* act = gen_base + S::ACT_OFFSET + b * S::ACT_BYTES;
#pragma unroll
                for (int n = 0; n < BN; ++n) {
                    const float gate = v[n], up = exch[col * BN + n];
                    const float a = up * __fdividef(gate, 1.0f + __expf(-gate));
                    const int off = (n >> 3) * 1024 + (n & 7) * 128 + ((((col >> 3) ^ (n & 7)) & 7) << 4) + (col & 7) * 2;
                    *reinterpret_cast<bf16*>(act + off) = __float2bfloat16_rn(a);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");        // generic writes -> the tensor core's reads
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(bar_act + 8 * b);
            }
        }
        // ---- the block's partial [T, H] of the down projection, added to the residual stream, tile by tile while the
        // rest of Wd is still streaming.  In the last slice every output tile of 128 rows is final as soon as its
        // tensor-core operations complete.  The four warps copy it from tensor memory into a staging buffer laid out as
        // the rows lie in global memory ([token][128]; two buffers take turns), and warp 6 hands the tile to the copy
        // engine as one tensor reduction (cp.reduce.async.bulk.tensor ... add), which the L2 applies a sector at a time.
        // Measured on the way here: scalar atomics from every thread took 3.6 us at the end of the kernel (1.7 million
        // float adds that reach the L2 one by one); bulk reductions of whole token rows issued after the last tile 2 to
        // 3 us; one bulk reduction per token and tile (96 a block at 8 tokens) were slower still, a reduction costs per
        // operation more than per byte.  Spread over the tiles, one operation each, they hide behind the weight stream.
        // With one of these threads also issuing the reductions, a buffer was handed back only after the next tile's
        // reduction had been issued: staging, hand-over and issue of a tile ran one after the other, 370 ns a tile against
        // 230 ns between the tiles' arrivals, and the last reduction left 1.8 us after the last tile's products.
        bool go = ok && !s_abort;
        for (int m = 0; m < g.n_mt; ++m) {
            const int buf = m & 1;
            const uint32_t par = (uint32_t)(m >> 1) & 1u;
            go = go && mbar_wait(bar_tile + 8 * m, 0, &s_abort);
            go = go && (m < 2 || mbar_wait(bar_unstaged + 8 * buf, par ^ 1u, &s_abort));       // the buffer's last use was read
            if (!__all_sync(0xffffffffu, go)) {              // a warp reads tensor memory together or not at all
                if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_D2); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float v[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 16) tmem_ld16(lane_addr + (uint32_t)(2 * BN + m * BN + c), v + c);
            float* stage = reinterpret_cast<float*>(gen_base + S::EXCH_OFFSET + buf * S::EXCH_BYTES);      // [BN][128]
#pragma unroll
            for (int n = 0; n < BN; ++n)
                if (n < g.T) stage[n * BM + row] = v[n];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // these writes -> the copy engine's reads
            mbar_arrive(bar_staged + 8 * buf);
        }
    } else if (warp == 6 && my_slices > 0) {
        // ---------------------------------------------------------------- staged output tiles -> the copy engine
        for (int m = 0; m < g.n_mt; ++m) {
            const int buf = m & 1;
            if (!warp_wait(bar_staged + 8 * buf, (uint32_t)(m >> 1) & 1u, &s_abort)) {
                if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_MLP_D2); }
                break;
            }
            if (m == 0) pdl_wait();                        // the residual stream was last written by a kernel before this one
            if (lane == 0) {                               // one and the same thread: the copies' groups are its own
                // one reduction for the whole tile: the box is [BN tokens][128 rows of the output]; what lies beyond the
                // step's T tokens or the matrix's H columns is clipped by the copy engine
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&map_res), "r"(m * BM), "r"(0), "r"(base + (uint32_t)(S::EXCH_OFFSET + buf * S::EXCH_BYTES)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the tile has been read: its buffer is free
                mbar_arrive(bar_unstaged + 8 * buf);
            }
            __syncwarp();
        }
        // the sums have reached memory (also after an early stop: no copy may still read this block's shared memory)
        if (lane == 0) {
            LLB_STAMP(4);
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            LLB_STAMP(5);
        }
        __syncwarp();                                      // the warp goes to the block's last barrier together
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)g.tmem_cols) : "memory");
    }
}

template <int BN, int STAGES>
int launch(const CUtensorMap& mg, const CUtensorMap& mu, const CUtensorMap& mx, const CUtensorMap& md, const CUtensorMap& mr,
           const MlpArgs& g, int blocks, cudaStream_t stream) {
    auto k = mlp_fused_kernel<BN, STAGES>;
    constexpr int smem = Smem<BN, STAGES>::TOTAL;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -2000 - (int)e;
        configured[dev] = true;
    }
    llb_launch(k, dim3(blocks), dim3(THREADS), smem, stream, mg, mu, mx, md, mr, g);
    return llb_status();
}

}  // namespace

// 1 when the fused kernel takes these sizes: at most 32 tokens, H and I multiples of 8 (TMA strides), and the
// accumulators of the down projection (ceil(H / 128) tiles of 16 or 32 columns) within tensor memory.
LLB_API int llb_mlp_fused_ok(int T, int H, int I) {
    if (T <= 0 || T > 32 || H <= 0 || I <= 0 || H % 8 || I % 8) return 0;
    const int bn = T <= 16 ? 16 : 32, n_mt = (H + BM - 1) / BM;
    return 2 * bn + n_mt * bn <= 512 && n_mt <= MAX_MT;
}

// X [T, H] bf16 (row stride ldx), Wgu [2 I, H] bf16 dense (gate rows first), Wd [H, I] bf16 dense;
// residual [T, H] float32 dense += the feed-forward of X.  blocks: the most blocks to launch (the SM count).
// stages: depth of the TMA ring (4, 5, 6, 8, and 10 for up to 16 tokens; 0 chooses).
LLB_DEFINE_SET_STAMPS

LLB_API int llb_mlp_fused(const void* X, int ldx, const void* Wgu, const void* Wd, float* residual, int T, int H, int I,
                          int blocks, int stages, int* err, cudaStream_t stream) {
    if (!llb_mlp_fused_ok(T, H, I) || ldx % 8 || blocks <= 0) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)X | (uintptr_t)Wgu | (uintptr_t)Wd | (uintptr_t)residual) & 15) return (int)cudaErrorInvalidValue;
    const int bn = T <= 16 ? 16 : 32;
    MlpArgs g;
    g.residual = residual;
    g.T = T; g.H = H; g.I = I;
    g.n_slices = (I + SLICE - 1) / SLICE;
    g.n_mt = (H + BM - 1) / BM;
    int cols = 2 * bn + g.n_mt * bn, pow2 = 32;
    while (pow2 < cols) pow2 *= 2;
    g.tmem_cols = pow2;
    g.err = err;
    CUtensorMap mg, mu, mx, md, mr;
    int rc = llb_tma::bf16_map_64(Wgu, I, H, H, SLICE, &mg);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64((const bf16*)Wgu + (size_t)I * H, I, H, H, SLICE, &mu);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, H, ldx, bn, &mx);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(Wd, H, I, I, BM, &md);
    if (rc) return rc;
    rc = llb_tma::f32_map_plain(residual, T, H, H, BM, bn, &mr);
    if (rc) return rc;
    const int grid = g.n_slices < blocks ? g.n_slices : blocks;
    if (stages == 0) stages = 6;
#define LLB_MLP(BN_, ST_) if (bn == BN_ && stages == ST_) return launch<BN_, ST_>(mg, mu, mx, md, mr, g, grid, stream)
    LLB_MLP(16, 4); LLB_MLP(16, 5); LLB_MLP(16, 6); LLB_MLP(16, 8); LLB_MLP(16, 10);
    LLB_MLP(32, 4); LLB_MLP(32, 5); LLB_MLP(32, 6); LLB_MLP(32, 8);
#undef LLB_MLP
    return (int)cudaErrorInvalidValue;
}
