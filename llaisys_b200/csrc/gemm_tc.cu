// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//
//     Y[T, N] = X[T, K] * W[N, K]^T (+ bias[N]),   float32 accumulation
//
// (the linear operator of xsmccc/llaisys, src/ops/linear/cpu/linear_cpu.cpp:21-40, whose model
// calls it for the q/k/v, output, gate, up, down and head projections).
//
// The weight is the M operand: a CTA owns 128 consecutive weight rows (one UMMA of M = 128) and a
// tile of BN tokens (the UMMA's N), so the same kernel serves prefill (BN up to 256) and decode
// (BN = 16..64, a handful of tokens against the whole weight) and the weight is read once.
// Both operands are K-major, which is how X and W lie in memory.
//
//   TMA (cp.async.bulk.tensor, 128-byte swizzle) -> shared-memory ring of STAGES k-blocks
//   -> tcgen05.mma issued by one thread, accumulator in tensor memory
//   -> tcgen05.ld by all four warps -> bias -> transposed store to Y.
//
// With `splits` > 1 the K range is divided over gridDim.z CTAs, and their float32 partial tiles
// are added in split order (so the sum does not depend on arrival order) in one of two ways:
//   * cluster (splits 2, 4, 8 or 16, tiles up to 128 tokens): the CTAs of a tile form a thread-block
//     cluster; each leaves its partial tile in its own shared memory, and after a cluster
//     barrier each adds one slice of the rows of all partials through distributed shared
//     memory, applies the bias and stores.  No global memory round trip.
//   * scratch (any split count): each CTA writes its partial tile to `scratch`; the CTA that
//     arrives last at the tile's counter adds them and stores.  Counters return to zero, so the
//     same scratch serves every launch of a stream.
//
// With DUAL the CTA multiplies two 128-row weight blocks (rows m and m + dual_offset: the gate
// and up rows of a fused [2I, K] matrix) into two accumulators and stores
// up * gate / (1 + exp(-gate))  (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21) as [T, I].
//
// Every wait on an mbarrier is bounded; when a bound is hit the CTA records an error code in
// *err, stops issuing, waits (bounded) for the copies it has in flight, frees its tensor
// memory and returns.
#include "common.cuh"
#include "tma_map.cuh"

namespace {

constexpr int BM = 128;        // weight rows of a tile (UMMA M)
constexpr int BK = 64;         // k elements of a stage: one 128-byte swizzled row of bf16
constexpr int UMMA_K = 16;     // k elements of one tcgen05.mma of kind::f16
constexpr int THREADS = 128;
#ifndef LLB_WAIT_LIMIT
#define LLB_WAIT_LIMIT (1u << 22)
#endif
constexpr uint32_t WAIT_LIMIT = LLB_WAIT_LIMIT;      // tries of a bounded wait (a test build makes it small)
// A test build (-DLLB_TEST_STALL=1) can make a wait run out without any fault: a launch that finds TEST_STALL_ARMED
// in its error word arms the first stage's "full" barrier for sixteen bytes more than are ever requested, so that
// the barrier's phase never completes, the issuing thread's wait gives up, and the block leaves by the abort path
// (error word, wait for the copies that are in flight, tensor memory freed).  Not compiled into the product.
constexpr int TEST_STALL_ARMED = -7;

constexpr uint64_t HINT_EVICT_FIRST = 0x12F0000000000000ull;
constexpr uint64_t HINT_EVICT_LAST = 0x14F0000000000000ull;

enum { ERR_TC_WAIT_FULL = 101, ERR_TC_WAIT_EMPTY = 102, ERR_TC_WAIT_ACC = 103, ERR_TC_WAIT_RECV = 104 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait.  Returns false when the bound is hit or another thread already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

// Bounded wait of a whole (converged) warp: every lane polls and the vote keeps the control flow uniform.  A wait that
// is already satisfied costs about 60 cycles this way; one lane polling inside a divergent branch costs several times that.
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                            uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(hint) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled,
// 8-row groups 1024 bytes apart (what the TMA box {64, rows} with SWIZZLE_128B writes).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // start address, bits [0, 14)
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused for swizzled K-major), bits [16, 30)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset: 8 rows * 128 B, bits [32, 46)
    d |= (uint64_t)1 << 46;                             // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                             // layout type: SWIZZLE_128B
    return d;
}

// Instruction descriptor of kind::f16: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4)                    // D format: f32
         | (1u << 7)                    // A format: bf16
         | (1u << 10)                   // B format: bf16
         | ((uint32_t)(n >> 3) << 17)   // N / 8
         | ((uint32_t)(BM >> 4) << 24); // M / 16
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

struct GemmArgs {
    const void* bias;      // [N] or null
    int bias_dtype;
    void* Y;               // [T, ldy]
    int y_dtype;
    int T, N, K, ldy;
    int dual_offset;       // DUAL: rows between the gate block and the up block of W
    int splits;
    int cluster;           // 1: the splits of a tile are a thread-block cluster and reduce by pushing into shared memory
    float* scratch;        // [tiles][splits][accs][BN][BM] float32
    int* counters;         // [tiles], zero between launches
    int* err;
};

template <int BN, int STAGES, bool DUAL>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    // The splits of a cluster reduce by pushing: every CTA receives, from each peer, the partial sums of its share
    // of the tile's rows: [source rank][accumulator][group of 4 tokens][row][4 tokens].  Single-accumulator tiles of
    // up to 32 tokens have a buffer of their own for that, outside the ring (OWN_RECV), so a peer may push as soon as
    // it is done; for the others the buffer is the ring itself, which a peer may write only after a cluster barrier
    // that every CTA passes once its own main loop is over (a buffer of their own would cost the second CTA of an SM).
    static constexpr bool OWN_RECV = BN <= 32 && !DUAL;
    static constexpr int RECV_OFFSET = BAR_OFFSET + (2 * STAGES + 2) * 8 + 16;     // 16-byte aligned (BAR_OFFSET is)
    static constexpr int RECV_BYTES = OWN_RECV ? BN * BM * 4 : 0;
    static constexpr int TOTAL = RECV_OFFSET + RECV_BYTES + 1024;                  // + slack to align the base
};

// INTO (instantiations of their own, so that the others' epilogues do not grow): the product is not stored but added
// to a float32 stream [T, N] (the residual stream: a projection that ends in the residual add).  The K range is
// divided over gridDim.z blocks that need not be a cluster; each stages its partial tile in the idle ring as the rows
// lie in the stream ([token][128 rows]) and hands it to the copy engine as one reduction
// (cp.reduce.async.bulk.tensor ... add), so the sums meet in the L2 and no block waits for another.
template <int BN, int STAGES, bool DUAL, bool INTO = false>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_out, GemmArgs g) {
    using S = Smem<BN, STAGES, DUAL>;
    constexpr int ACCS = DUAL ? 2 : 1;
    LLB_STAMPS_BEGIN();
    constexpr int TMEM_COLS = (ACCS * BN) <= 32 ? 32 : (ACCS * BN) <= 64 ? 64 : (ACCS * BN) <= 128 ? 128 : (ACCS * BN) <= 256 ? 256 : 512;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = base + S::BAR_OFFSET, bar_empty = bar_full + 8 * STAGES, bar_acc = bar_empty + 8 * STAGES;
    const uint32_t bar_recv = bar_acc + 8, tmem_slot = bar_recv + 8;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + S::BAR_OFFSET + (2 * STAGES + 2) * 8);
    const bool push = g.cluster && g.splits > 1;
    __shared__ int s_abort, s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, split = blockIdx.z;
    const int kblocks = (g.K + BK - 1) / BK;
    const int chunk = (kblocks + g.splits - 1) / g.splits;
    const int kb0 = split * chunk, kb1 = min(kblocks, kb0 + chunk);

    if (tid == 0) {
        s_abort = 0;
        s_last = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_recv, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (push) {
            // what the peers will send: from each of the splits, per accumulator and row of this CTA's share, the
            // valid tokens rounded up to whole 16-byte pieces
            const int sent = (min(BN, g.T - n0) + 3) & ~3;
            mbar_expect_tx(bar_recv, (uint32_t)(g.splits * ACCS * (BM / g.splits) * sent * 4));
        }
    }
    // The peers may write into this CTA's own buffer as soon as its barrier stands: arrive now, wait just before the
    // first push.  (Without a buffer of its own a CTA arrives when its ring is idle.)
    if (push && S::OWN_RECV) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;

    // The weight does not depend on any earlier kernel of the step, so its first STAGES k-blocks are
    // requested before the grid dependency resolves: while the predecessor is still running, this
    // CTA's share of the weight is already on its way into shared memory.
    const int prefetched = min(STAGES, kb1 - kb0);
    if (warp == 0 && lane == 0) {
#ifdef LLB_TEST_STALL
        if (*(volatile int*)g.err == TEST_STALL_ARMED)       // sixteen bytes that nothing will ever bring (no arrival)
            asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar_full), "r"(16u) : "memory");
#endif
        for (int i = 0; i < prefetched; ++i) {
            uint32_t dst = base + i * S::STAGE_BYTES;
            mbar_expect_tx(bar_full + 8 * i, S::STAGE_BYTES);
            tma_load_2d(dst, &map_w, bar_full + 8 * i, (kb0 + i) * BK, m0, HINT_EVICT_FIRST);
            if (DUAL) tma_load_2d(dst + S::A_BYTES, &map_w, bar_full + 8 * i, (kb0 + i) * BK, m0 + g.dual_offset, HINT_EVICT_FIRST);
        }
    }
    // The peers of a cluster start together and arrived before this point in their own code: the wait that must
    // precede the first push into a buffer of its own is done here, where the block waits for its input anyway (even
    // satisfied it costs some hundred cycles, which behind the grid dependency would be on the step's critical path).
    if (push && S::OWN_RECV) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid == 64) LLB_STAMP(0);      // stamps: 0 set up, 1 input ready (grid dependency), 2 first stage full, 3 all products issued,
    llb_grid_dependency_sync();      // from here on memory written by earlier kernels is touched
    if (tid == 64) LLB_STAMP(1);      //         4 accumulator ready, 5 epilogue's own part done, 6 peers' partial rows received, 7 end

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: the activations of the prefetched k-blocks, then whole k-blocks into the ring
            for (int i = 0; i < prefetched; ++i)
                tma_load_2d(base + i * S::STAGE_BYTES + ACCS * S::A_BYTES, &map_x, bar_full + 8 * i, (kb0 + i) * BK, n0,
                            HINT_EVICT_LAST);
            int issued = prefetched;
            for (int kb = kb0 + prefetched; kb < kb1; ++kb, ++issued) {
                int s = issued % STAGES;
                uint32_t round = issued / STAGES;
                if (!mbar_wait(bar_empty + 8 * s, (round - 1) & 1, &s_abort)) {
                    if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_EMPTY); }
                    break;
                }
                uint32_t dst = base + s * S::STAGE_BYTES;
                mbar_expect_tx(bar_full + 8 * s, S::STAGE_BYTES);
                tma_load_2d(dst, &map_w, bar_full + 8 * s, kb * BK, m0, HINT_EVICT_FIRST);
                if (DUAL) tma_load_2d(dst + S::A_BYTES, &map_w, bar_full + 8 * s, kb * BK, m0 + g.dual_offset, HINT_EVICT_FIRST);
                tma_load_2d(dst + ACCS * S::A_BYTES, &map_x, bar_full + 8 * s, kb * BK, n0, HINT_EVICT_LAST);
            }
            if (s_abort) {
                // copies in flight must land before this CTA's shared memory is given up
                int first = issued > STAGES ? issued - STAGES : 0;
                for (int i = first; i < issued; ++i)
                    for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try(bar_full + 8 * (i % STAGES), (i / STAGES) & 1); ++t) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- tensor-core issue.  The whole warp waits (see warp_wait), one elected lane issues; the operand
        // descriptors are made once and an instruction's own differs from them by a constant: built per instruction,
        // the address arithmetic of the single issuing thread cost more than the products of a short K range
        // (measured: 1.0 us for twelve products, of a kernel that takes 2.6 us behind its input).
        const uint32_t idesc = umma_idesc(BN);
        const uint64_t a_desc0 = umma_desc(base), b_desc0 = umma_desc(base + ACCS * S::A_BYTES);
        int s = 0;
        uint32_t ph = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
            if (!warp_wait(bar_full + 8 * s, ph, &s_abort)) {
                if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_FULL); }
                break;
            }
            if (elect_one()) {
                if (kb == kb0) LLB_STAMP(2);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t so = (uint64_t)(s * (S::STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
                    const uint64_t bd = b_desc0 + so + (uint64_t)((k * UMMA_K * 2) >> 4);
                    umma(tmem, a_desc0 + so + (uint64_t)((k * UMMA_K * 2) >> 4), bd, idesc, acc);
                    if (DUAL) umma(tmem + BN, a_desc0 + so + (uint64_t)((S::A_BYTES + k * UMMA_K * 2) >> 4), bd, idesc, acc);
                }
                umma_commit(bar_empty + 8 * s);      // the stage is free once these MMAs have read it
            }
            __syncwarp();
            if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (elect_one()) {
            LLB_STAMP(3);
            umma_commit(bar_acc);                    // accumulator complete (arrives even after an early stop)
        }
        __syncwarp();
    }

    // ---- epilogue: all four warps; warp w owns tensor-memory lanes 32w..32w+31 = weight rows m0+32w..
    bool ok = mbar_wait(bar_acc, 0, &s_abort);
    if (!ok && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_ACC); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (tid == 64) LLB_STAMP(4);
    __syncthreads();
    const bool aborted = s_abort != 0;
    const int m = m0 + tid;                                   // this thread's weight row (output column)
    const int n_valid = min(BN, g.T - n0);
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    const bool row_ok = m < (DUAL ? g.dual_offset : g.N);

    // A row's bias is fetched once, before the first store of the row (a store may alias it as far as the compiler
    // can tell, so a load after a store is not moved ahead of it).
    auto bias_of = [&](int row) -> float {
        if (!g.bias) return 0.f;
        return g.bias_dtype == LLB_F32 ? ((const float*)g.bias)[row] : to_f32(((const bf16*)g.bias)[row]);
    };
    auto finish_at = [&](float acc0, float acc1, int j, int row, float bias_v) {
        float v = acc0;
        if (DUAL) v = acc1 * __fdividef(acc0, 1.0f + __expf(-acc0));
        v += bias_v;
        size_t o = (size_t)(n0 + j) * g.ldy + row;
        if (g.y_dtype == LLB_F32) ((float*)g.Y)[o] = v;
        else ((bf16*)g.Y)[o] = __float2bfloat16_rn(v);
    };
    // (the own row's bias is fetched inside the branches that finish whole rows: a load issued before the push
    // branch's cluster barrier would be waited for there)
    auto finish = [&](float acc0, float acc1, int j, float bias_v) { finish_at(acc0, acc1, j, m, bias_v); };

    if (INTO) {
        if (!aborted) {
            float* stg = reinterpret_cast<float*>(gen_base);              // [BN tokens][128 rows] float32 in the idle ring
            const float bias_v = (split == 0 && row_ok) ? bias_of(m) : 0.f;      // the bias goes in with the first K range
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v0[16];
                tmem_ld16(lane_addr + c, v0);
#pragma unroll
                for (int j = 0; j < 16; ++j) stg[(c + j) * BM + tid] = v0[j] + bias_v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                // what lies beyond the step's tokens or the matrix's rows is clipped by the copy engine
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&map_out), "r"(m0), "r"(n0), "r"(smem_u32(stg)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");         // before the shared memory is given up
            }
            __syncwarp();                      // (that thread's warp goes to the block's last barrier together)
        }
    } else if (!aborted) {
        if (g.splits == 1 && g.y_dtype == LLB_BF16 && m0 + BM <= (DUAL ? g.dual_offset : g.N) &&
            g.ldy % 8 == 0 && ((uintptr_t)g.Y & 15) == 0) {
            // Whole tile of bfloat16 outputs: a thread holds one weight row, i.e. one output COLUMN, so storing
            // straight from registers writes 2 bytes per thread per token (measured: 21,600 cycles for a
            // 128x256 tile, more than its 24 k-block main loop).  Instead the tile is transposed through the
            // now idle ring in shared memory and leaves as 16-byte stores along the output rows.
            bf16* stg = reinterpret_cast<bf16*>(gen_base);             // [token][128 rows]
            float bias_v = 0.f;
            if (g.bias) bias_v = g.bias_dtype == LLB_F32 ? ((const float*)g.bias)[m] : to_f32(((const bf16*)g.bias)[m]);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v0[16], v1[16];
                tmem_ld16(lane_addr + c, v0);                 // warp-collective: every lane takes part
                if (DUAL) tmem_ld16(lane_addr + BN + c, v1);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v = v0[j];
                    if (DUAL) v = v1[j] * __fdividef(v, 1.0f + __expf(-v));      // fast division: the result is rounded to bfloat16
                    stg[(c + j) * BM + tid] = __float2bfloat16_rn(v + bias_v);
                }
            }
            __syncthreads();
            // 16 threads move one token's 128 outputs (256 bytes); 8 tokens per pass
            const int sub = tid & 15;
            for (int j = tid >> 4; j < n_valid; j += THREADS / 16) {
                uint4 v = *reinterpret_cast<const uint4*>(stg + j * BM + sub * 8);
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.Y) + (size_t)(n0 + j) * g.ldy + m0 + sub * 8) = v;
            }
        } else if (g.splits == 1) {
            const float own_bias = row_ok ? bias_of(m) : 0.f;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v0[16], v1[16];
                tmem_ld16(lane_addr + c, v0);                 // warp-collective: every lane takes part
                if (DUAL) tmem_ld16(lane_addr + BN + c, v1);
                if (row_ok)
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c + j < n_valid) finish(v0[j], DUAL ? v1[j] : 0.f, c + j, own_bias);
            }
        } else if (push) {
            // Each thread holds one row of the partial tile; the row belongs to the share of CTA `dest`, which
            // gets it as 16-byte pieces of four tokens, counted on its receive barrier.
            const int S_ = g.splits, R = BM / S_;
            uint32_t rank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
            const uint32_t dest = (uint32_t)(tid / R), row = (uint32_t)(tid % R);
            uint32_t rbar, rbuf;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar_recv), "r"(dest));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbuf) : "r"(base + (uint32_t)(S::OWN_RECV ? S::RECV_OFFSET : 0)), "r"(dest));
            if (!S::OWN_RECV) {       // this ring is idle; every peer's must be before anything is written into it
                asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
                asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            }
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v0[16], v1[16];
                tmem_ld16(lane_addr + c, v0);
                if (DUAL) tmem_ld16(lane_addr + BN + c, v1);
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    if (c + j < n_valid) {
                        const uint32_t piece = (((rank * ACCS) * (BN / 4) + (uint32_t)((c + j) / 4)) * R + row) * 16;
                        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                                     ::"r"(rbuf + piece), "f"(v0[j]), "f"(v0[j + 1]), "f"(v0[j + 2]), "f"(v0[j + 3]), "r"(rbar) : "memory");
                        if (DUAL)
                            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                                         ::"r"(rbuf + piece + (uint32_t)((BN / 4) * R * 16)), "f"(v1[j]), "f"(v1[j + 1]), "f"(v1[j + 2]),
                                           "f"(v1[j + 3]), "r"(rbar) : "memory");
                    }
            }
        } else {
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
            float* mine = g.scratch + ((size_t)tile * g.splits + split) * (ACCS * BN * BM);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v0[16], v1[16];
                tmem_ld16(lane_addr + c, v0);
                if (DUAL) tmem_ld16(lane_addr + BN + c, v1);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c + j < n_valid) {
                        mine[(c + j) * BM + tid] = v0[j];
                        if (DUAL) mine[(BN + c + j) * BM + tid] = v1[j];
                    }
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) s_last = (atomicAdd(&g.counters[tile], 1) == g.splits - 1);
            __syncthreads();
            if (s_last) {
                __threadfence();
                const float* all = g.scratch + (size_t)tile * g.splits * (ACCS * BN * BM);
                // eight tokens at a time and four splits ahead, so that the loads overlap instead of
                // each waiting for the one before; the sums still run in split order
                const float own_bias = row_ok ? bias_of(m) : 0.f;
                if (row_ok)
                    for (int j0 = 0; j0 < n_valid; j0 += 8) {
                        float a0[8], a1[8];
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) a0[jj] = a1[jj] = 0.f;
#pragma unroll 4
                        for (int s = 0; s < g.splits; ++s) {
                            const float* p = all + (size_t)s * (ACCS * BN * BM);
                            float v0[8], v1[8];
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                bool in = j0 + jj < n_valid;
                                v0[jj] = in ? __ldcg(p + (j0 + jj) * BM + tid) : 0.f;
                                v1[jj] = (DUAL && in) ? __ldcg(p + (BN + j0 + jj) * BM + tid) : 0.f;
                            }
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                a0[jj] += v0[jj];
                                a1[jj] += v1[jj];
                            }
                        }
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj)
                            if (j0 + jj < n_valid) finish(a0[jj], a1[jj], j0 + jj, own_bias);
                    }
                if (tid == 0) g.counters[tile] = 0;
            }
        }
    }
    if (!INTO && aborted && g.splits > 1 && !push && tid == 0) {
        // A block that gave up still arrives at its tile's counter, so that the counter is back at zero when the
        // launch is over whatever happened (the tile's output is not valid; the error word says so).
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        if (atomicAdd(&g.counters[tile], 1) == g.splits - 1) g.counters[tile] = 0;
    }
    if (push) {
        if (aborted && !S::OWN_RECV) {      // pairs with the arrivals of the peers
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        // All the peers' pieces (bounded wait: a peer that gave up sends none), then this CTA's share of the rows:
        // the partial sums are added in split order.
        const int S_ = g.splits, R = BM / S_, groups = (n_valid + 3) / 4;
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        const int limit = DUAL ? g.dual_offset : g.N;
        // the bias of this thread's first output piece is asked for before the wait for the peers
        float bias_first = 0.f;
        if (!aborted && tid < R * groups && m0 + (int)rank * R + tid % R < limit) bias_first = bias_of(m0 + (int)rank * R + tid % R);
        if (tid == 64) LLB_STAMP(5);
        bool got = mbar_wait(bar_recv, 0, &s_abort);
        if (tid == 64) LLB_STAMP(6);
        if (!got && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_RECV); }
        if (got && !aborted) {
            const float4* rb = reinterpret_cast<const float4*>(gen_base + (S::OWN_RECV ? S::RECV_OFFSET : 0));
            // one piece: four tokens of one row of this CTA's share
            auto piece = [&](int item, float bias_v) {
                const int row = item % R, jg = item / R, mm = m0 + (int)rank * R + row, j = jg * 4;
                if (mm >= limit) return;
                float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
                for (int sp = 0; sp < S_; ++sp) {
                    const float4 p0 = rb[((sp * ACCS) * (BN / 4) + jg) * R + row];
                    a0.x += p0.x; a0.y += p0.y; a0.z += p0.z; a0.w += p0.w;
                    if (DUAL) {
                        const float4 p1 = rb[((sp * ACCS + 1) * (BN / 4) + jg) * R + row];
                        a1.x += p1.x; a1.y += p1.y; a1.z += p1.z; a1.w += p1.w;
                    }
                }
                finish_at(a0.x, a1.x, j, mm, bias_v);
                if (j + 1 < n_valid) finish_at(a0.y, a1.y, j + 1, mm, bias_v);
                if (j + 2 < n_valid) finish_at(a0.z, a1.z, j + 2, mm, bias_v);
                if (j + 3 < n_valid) finish_at(a0.w, a1.w, j + 3, mm, bias_v);
            };
            if (tid < R * groups) piece(tid, bias_first);
            for (int item = tid + THREADS; item < R * groups; item += THREADS) {      // tiles of 64 tokens and more
                const int mm = m0 + (int)rank * R + item % R;
                piece(item, mm < limit ? bias_of(mm) : 0.f);
            }
        }
    }
    if (tid == 64) LLB_STAMP(7);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
template <int BN, int STAGES, bool DUAL, bool INTO = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, dim3 grid, cudaStream_t stream,
           const CUtensorMap* mo = nullptr) {
    auto k = gemm_tc_kernel<BN, STAGES, DUAL, INTO>;
    constexpr int smem = Smem<BN, STAGES, DUAL>::TOTAL;
    // function attributes belong to a device's copy of the kernel: set them once on every device that launches it
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -2000 - (int)e;       // shared-memory opt-in refused: -(2000 + cudaError)
        cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);      // clusters of sixteen
        configured[dev] = true;
    }
    llb_prefer_max_shared((const void*)k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
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
    if (g.cluster && g.splits > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = (unsigned)g.splits;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaLaunchKernelEx(&cfg, k, mw, mx, mo ? *mo : mw, g);
    return llb_status();
}


// ------------------------------------------------------------------ gate/up for 17 to 64 tokens, rows side by side
// The fused gate/up product  Y[T, I] = up * gate / (1 + exp(-gate))  as DUAL above computes it, for the case where
// tiles of 128 gate rows would leave half of the SMs without a block (I / 128 tiles and no K split: 70 blocks for
// I = 8960).  A block's operand tile holds 64 gate rows followed by the 64 up rows of the same outputs (two TMA
// boxes), so the one accumulator has gate values in lanes 0-63 and up values in lanes 64-127 and there are I / 64
// blocks.  The upper lanes' threads pass their values through the idle ring to the lower lanes' threads, which
// compute and stage bfloat16 rows; all threads store them as 16-byte pieces along the output rows.  Whole K range
// per block, bfloat16 output, I and ldy multiples of 8.  Waits are bounded as in gemm_tc_kernel (same error codes).
// Measured for I = 8960, K = 1536 inside CUDA graphs: 11.4 against 12.7 us at 32 tokens, 12.8 against 13.1 at 64; a
// decode step of batch 64 1.813 against 1.84 ms.  At 128 tokens it lost (15.4 against 14.8 us), at 256 it was even.
template <int BN, int STAGES>
struct SmemGU {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;     // + slack to align the base
    static constexpr int XCH_BYTES = BN * (BM / 2) * 4, STG_BYTES = BN * (BM / 2) * 2;
    static_assert(XCH_BYTES + STG_BYTES <= BAR_OFFSET, "the epilogue's buffers fit the idle ring");
    static_assert(TOTAL <= 232448, "a block's shared memory");
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gateup_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmArgs g) {
    using S = SmemGU<BN, STAGES>;
    constexpr int HALF = BM / 2;
    constexpr int TMEM_COLS = BN <= 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = base + S::BAR_OFFSET, bar_empty = bar_full + 8 * STAGES, bar_acc = bar_empty + 8 * STAGES;
    const uint32_t tmem_slot = bar_acc + 8;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(gen_base + S::BAR_OFFSET + (2 * STAGES + 1) * 8);
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * HALF, n0 = blockIdx.y * BN;            // first gate row (= output column), first token
    const int kblocks = (g.K + BK - 1) / BK;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;

    // the weight depends on no earlier kernel of the step: its first k-blocks are requested before the dependency resolves
    const int prefetched = min(STAGES, kblocks);
    auto load_w = [&](uint32_t dst, uint32_t bar, int kb) {
        tma_load_2d(dst, &map_w, bar, kb * BK, m0, HINT_EVICT_FIRST);                                   // 64 gate rows
        tma_load_2d(dst + S::A_BYTES / 2, &map_w, bar, kb * BK, m0 + g.dual_offset, HINT_EVICT_FIRST);  // their 64 up rows
    };
    if (warp == 0 && lane == 0) {
        for (int i = 0; i < prefetched; ++i) {
            mbar_expect_tx(bar_full + 8 * i, S::STAGE_BYTES);
            load_w(base + i * S::STAGE_BYTES, bar_full + 8 * i, i);
        }
    }
    llb_grid_dependency_sync();      // from here on memory written by earlier kernels is touched

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < prefetched; ++i)
                tma_load_2d(base + i * S::STAGE_BYTES + S::A_BYTES, &map_x, bar_full + 8 * i, i * BK, n0, HINT_EVICT_LAST);
            int issued = prefetched;
            for (int kb = prefetched; kb < kblocks; ++kb, ++issued) {
                const int s = issued % STAGES;
                const uint32_t round = issued / STAGES;
                if (!mbar_wait(bar_empty + 8 * s, (round - 1) & 1, &s_abort)) {
                    if (!s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_EMPTY); }
                    break;
                }
                const uint32_t dst = base + s * S::STAGE_BYTES;
                mbar_expect_tx(bar_full + 8 * s, S::STAGE_BYTES);
                load_w(dst, bar_full + 8 * s, kb);
                tma_load_2d(dst + S::A_BYTES, &map_x, bar_full + 8 * s, kb * BK, n0, HINT_EVICT_LAST);
            }
            if (s_abort) {
                // copies in flight must land before this CTA's shared memory is given up
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int i = first; i < issued; ++i)
                    for (uint32_t t = 0; t < WAIT_LIMIT && !mbar_try(bar_full + 8 * (i % STAGES), (i / STAGES) & 1); ++t) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = umma_idesc(BN);
        const uint64_t a_desc0 = umma_desc(base), b_desc0 = umma_desc(base + S::A_BYTES);
        int s = 0;
        uint32_t ph = 0;
        for (int kb = 0; kb < kblocks; ++kb) {
            if (!warp_wait(bar_full + 8 * s, ph, &s_abort)) {
                if (lane == 0 && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_FULL); }
                break;
            }
            if (elect_one()) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t so = (uint64_t)(s * (S::STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                    umma(tmem, a_desc0 + so + step, b_desc0 + so + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar_empty + 8 * s);      // the stage is free once these MMAs have read it
            }
            __syncwarp();
            if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (elect_one()) umma_commit(bar_acc);       // accumulator complete (arrives even after an early stop)
        __syncwarp();
    }

    // ---- epilogue: all four warps; warp w owns tensor-memory lanes 32w .. 32w + 31
    const bool ok = mbar_wait(bar_acc, 0, &s_abort);
    if (!ok && !s_abort) { s_abort = 1; atomicExch(g.err, ERR_TC_WAIT_ACC); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();                                              // the ring is idle: every product has read it
    const bool aborted = s_abort != 0;
    const int n_valid = min(BN, g.T - n0);
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    float* xch = reinterpret_cast<float*>(gen_base);              // [token][64 rows] up values
    bf16* stg = reinterpret_cast<bf16*>(gen_base + S::XCH_BYTES); // [token][64 rows] outputs
    if (!aborted && tid >= HALF) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
            float v[16];
            tmem_ld16(lane_addr + c, v);                          // warp-collective: every lane takes part
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[(c + j) * HALF + tid - HALF] = v[j];
        }
    }
    __syncthreads();
    if (!aborted && tid < HALF) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
            float v[16];
            tmem_ld16(lane_addr + c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float gate = v[j], up = xch[(c + j) * HALF + tid];
                stg[(c + j) * HALF + tid] = __float2bfloat16_rn(up * __fdividef(gate, 1.0f + __expf(-gate)));   // fast division: the result is rounded to bfloat16
            }
        }
    }
    __syncthreads();
    if (!aborted) {
        // 8 threads move one token's 64 outputs (128 bytes); 16 tokens per pass
        const int sub = tid & 7;
        if (m0 + sub * 8 < g.dual_offset)
            for (int j = tid >> 3; j < n_valid; j += THREADS / 8)
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.Y) + (size_t)(n0 + j) * g.ldy + m0 + sub * 8) =
                    *reinterpret_cast<const uint4*>(stg + j * HALF + sub * 8);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
}

template <int BN, int STAGES>
int launch_gateup(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, dim3 grid, cudaStream_t stream) {
    auto k = gateup_tc_kernel<BN, STAGES>;
    constexpr int smem = SmemGU<BN, STAGES>::TOTAL;
    static bool configured[64] = {};          // function attributes belong to a device's copy of the kernel
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -2000 - (int)e;
        configured[dev] = true;
    }
    llb_prefer_max_shared((const void*)k);
    llb_launch(k, grid, dim3(THREADS), (size_t)smem, stream, mw, mx, g);
    return llb_status();
}

}  // namespace

LLB_DEFINE_SET_STAMPS

// float32 elements of scratch a launch needs (0 when splits == 1).
static long long llb_gemm_tc_scratch_elems(int T, int N, int bn, int splits, int dual) {
    if (splits <= 1) return 0;
    long long tiles = (long long)((N + BM - 1) / BM) * ((T + bn - 1) / bn);
    return tiles * splits * (dual ? 2 : 1) * bn * BM;
}

// X [T, K] bf16 with row stride ldx; W [N, K] bf16 dense ([2 * dual_offset, K] when dual_offset > 0,
// giving Y [T, dual_offset]); bias bf16/f32 or null; Y bf16 or f32 with row stride ldy.
// bn: tokens per tile (16, 32, 64, 128, 256).  cluster: reduce the splits through a thread-block cluster where
// that applies (splits 2, 4, 8 or 16 and bn <= 128), else through `scratch`.  Requirements: K and ldx multiples of 8, X and W 16-byte
// aligned.  Returns 0, a cudaError, or cudaErrorInvalidValue for a shape it does not take.
LLB_API int llb_gemm_tc(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                        int T, int N, int K, int ldx, int ldy, int bn, int splits, int cluster, int dual_offset,
                        float* scratch, long long scratch_elems, int* counters, int n_counters, int* err,
                        cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (y_dtype != LLB_F32 && y_dtype != LLB_BF16) return (int)cudaErrorInvalidValue;
    const bool dual = dual_offset > 0;
    if (dual && (N != 2 * dual_offset || bias)) return (int)cudaErrorInvalidValue;
    const int rows_out = dual ? dual_offset : N;
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kblocks) splits = kblocks;
    {   // no split may be empty
        int chunk = (kblocks + splits - 1) / splits;
        splits = (kblocks + chunk - 1) / chunk;
    }
    dim3 grid((rows_out + BM - 1) / BM, (T + bn - 1) / bn, splits);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    if (cluster && !(splits == 2 || splits == 4 || splits == 8 || splits == 16)) cluster = 0;
    if (cluster && bn > 128) cluster = 0;
    if (splits > 1 && !cluster) {
        long long need = llb_gemm_tc_scratch_elems(T, rows_out, bn, splits, dual);
        if (!scratch || !counters || need > scratch_elems || (long long)grid.x * grid.y > n_counters)
            return (int)cudaErrorInvalidValue;
    }
    CUtensorMap mw, mx;
    int rc = llb_tma::bf16_map_64(W, N, K, K, BM, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, K, ldx, bn, &mx);
    if (rc) return rc;
    GemmArgs g{bias, bias_dtype, Y, y_dtype, T, N, K, ldy, dual_offset, splits, cluster, scratch, counters, err};
#define LLB_TC(BN_, ST_, STD_) \
    case BN_: return dual ? launch<BN_, STD_, true>(mw, mx, g, grid, stream) : launch<BN_, ST_, false>(mw, mx, g, grid, stream)
    switch (bn) {
        LLB_TC(16, 5, 3);       // 99 KB / 102 KB of shared memory (ring + receive buffer): two CTAs per SM
        LLB_TC(32, 4, 3);       // 97 KB / 108 KB
        LLB_TC(64, 4, 4);       //  96 KB / 160 KB
        LLB_TC(128, 6, 4);      // 192 KB / 192 KB
        LLB_TC(256, 4, 3);      // 192 KB / 192 KB
        default: return (int)cudaErrorInvalidValue;
    }
#undef LLB_TC
}

// The fused gate/up product for 17 to 64 tokens with a block per 64 outputs (gateup_tc_kernel): X [T, K] bf16 with
// row stride ldx, W [2 I, K] bf16 dense (gate rows first), Y [T, I] bf16 with row stride ldy.  bn: tokens per tile
// (32 or 64; with larger tiles the kernel above was measured as fast or faster).  K, ldx, ldy and I multiples of 8,
// all three 16-byte aligned; cudaErrorInvalidValue otherwise.
LLB_API int llb_gemm_tc_gateup(const void* X, const void* W, void* Y, int T, int I, int K, int ldx, int ldy, int bn,
                               int* err, cudaStream_t stream) {
    if (T <= 0 || I <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldy % 8 || I % 8 || (((uintptr_t)X | (uintptr_t)W | (uintptr_t)Y) & 15))
        return (int)cudaErrorInvalidValue;
    dim3 grid((I + BM / 2 - 1) / (BM / 2), (T + bn - 1) / bn, 1);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    CUtensorMap mw, mx;
    int rc = llb_tma::bf16_map_64(W, 2 * I, K, K, BM / 2, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, K, ldx, bn, &mx);
    if (rc) return rc;
    GemmArgs g{nullptr, 0, Y, LLB_BF16, T, 2 * I, K, ldy, I, 1, 0, nullptr, nullptr, err};
    switch (bn) {
        case 32: return launch_gateup<32, 8>(mw, mx, g, grid, stream);        // 160 KB of ring
        case 64: return launch_gateup<64, 8>(mw, mx, g, grid, stream);        // 192 KB (with 96 KB, two blocks to an SM: slower)
        default: return (int)cudaErrorInvalidValue;
    }
}

// stream[T, N] (float32, row stride lds a multiple of 4, 16-byte aligned) += X W^T + bias for up to 256 tokens: the K
// range divided over `splits` blocks (any number up to the k-blocks), every block adding its partial tile to the
// stream by a TMA reduction.  bn: tokens per tile (16, 32, 64, 128, 256).  The sums meet in the L2 in no fixed order.
LLB_API int llb_gemm_tc_into(const void* X, const void* W, const void* bias, int bias_dtype, float* stream_, int T, int N, int K,
                             int ldx, int lds, int bn, int splits, int* err, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || lds % 4 || !stream_ || (((uintptr_t)X | (uintptr_t)W | (uintptr_t)stream_) & 15))
        return (int)cudaErrorInvalidValue;
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kblocks) splits = kblocks;
    {   // no split may be empty
        int chunk = (kblocks + splits - 1) / splits;
        splits = (kblocks + chunk - 1) / chunk;
    }
    dim3 grid((N + BM - 1) / BM, (T + bn - 1) / bn, splits);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    CUtensorMap mw, mx, mo;
    int rc = llb_tma::bf16_map_64(W, N, K, K, BM, &mw);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(X, T, K, ldx, bn, &mx);
    if (rc) return rc;
    rc = llb_tma::f32_map_plain(stream_, T, N, lds, BM, bn, &mo);
    if (rc) return rc;
    GemmArgs g{bias, bias_dtype, nullptr, LLB_F32, T, N, K, lds, 0, splits, 0, nullptr, nullptr, err};
    switch (bn) {
        case 16: return launch<16, 5, false, true>(mw, mx, g, grid, stream, &mo);
        case 32: return launch<32, 4, false, true>(mw, mx, g, grid, stream, &mo);
        case 64: return launch<64, 4, false, true>(mw, mx, g, grid, stream, &mo);
        case 128: return launch<128, 6, false, true>(mw, mx, g, grid, stream, &mo);
        case 256: return launch<256, 4, false, true>(mw, mx, g, grid, stream, &mo);
        default: return (int)cudaErrorInvalidValue;
    }
}

// ------------------------------------------------------------------ allocation-free entry point
// See gemm_tc_noalloc.h.  The scratch of the split launches lives in the device image.  In host
// code the names below are host-side stand-ins, not device addresses, so the addresses are
// looked up once per device with cudaGetSymbolAddress and passed to the kernel.
#include "gemm_tc_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[LLB_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_counters[LLB_NOALLOC_TILES];
static __device__ __align__(256) int g_noalloc_err[64];

namespace {

struct NoAllocPtrs { float* scratch; int* counters; int* err; bool ready; };
constexpr int NOALLOC_MAX_DEVICES = 64;
NoAllocPtrs g_noalloc_ptrs[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mutex;

// Device addresses of the built-in arrays on the current device; looked up on the first call there.
int noalloc_setup(NoAllocPtrs* out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return LLB_NOALLOC_SETUP_FAILED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocPtrs& p = g_noalloc_ptrs[dev];
    if (!p.ready) {
        void *s = nullptr, *c = nullptr, *e = nullptr;
        if (cudaGetSymbolAddress(&s, g_noalloc_scratch) != cudaSuccess || cudaGetSymbolAddress(&c, g_noalloc_counters) != cudaSuccess ||
            cudaGetSymbolAddress(&e, g_noalloc_err) != cudaSuccess || !s || !c || !e) {
            cudaGetLastError();
            return LLB_NOALLOC_SETUP_FAILED;
        }
        p.scratch = (float*)s;
        p.counters = (int*)c;
        p.err = (int*)e;
        p.ready = true;
    }
    *out = p;
    return 0;
}

}  // namespace

int llb_gemm_tc_noalloc_status(cudaStream_t stream) {
    NoAllocPtrs ptrs;
    int rc = noalloc_setup(&ptrs);
    if (rc) return rc;
    int code = 0;                                   // caller-side storage on the stack: nothing is allocated
    if (cudaMemcpyAsync(&code, ptrs.err, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaGetLastError();
        return LLB_NOALLOC_SETUP_FAILED;
    }
    if (code != 0) {
        // a block gave up a wait: clear the word, and the tile counters in case a launch was cut short
        cudaMemsetAsync(ptrs.err, 0, sizeof(int), stream);
        cudaMemsetAsync(ptrs.counters, 0, sizeof(int) * LLB_NOALLOC_TILES, stream);
    }
    return code;
}

int llb_gemm_tc_noalloc(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                        int T, int N, int K, int ldx, int ldy, int bn, int splits, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (y_dtype != LLB_F32 && y_dtype != LLB_BF16) return (int)cudaErrorInvalidValue;
    if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return (int)cudaErrorInvalidValue;
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kblocks) splits = kblocks;
    {
        int chunk = (kblocks + splits - 1) / splits;
        splits = (kblocks + chunk - 1) / chunk;
    }
    dim3 grid((N + BM - 1) / BM, (T + bn - 1) / bn, splits);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    const long long tiles = (long long)grid.x * grid.y;
    if (splits > 1 && (tiles * splits * bn * BM > (long long)LLB_NOALLOC_SCRATCH_FLOATS || tiles > LLB_NOALLOC_TILES))
        return LLB_NOALLOC_TOO_LARGE;
    NoAllocPtrs ptrs;
    int rc = noalloc_setup(&ptrs);
    if (rc) return rc;
    CUtensorMap mw, mx;
    rc = llb_tma::encode_bf16_map_64(W, N, K, K, BM, &mw);
    if (rc) return rc;
    rc = llb_tma::encode_bf16_map_64(X, T, K, ldx, bn, &mx);
    if (rc) return rc;
    GemmArgs g{bias, bias_dtype, Y, y_dtype, T, N, K, ldy, 0, splits, 0, ptrs.scratch, ptrs.counters, ptrs.err};
    switch (bn) {
        case 16: return launch<16, 5, false>(mw, mx, g, grid, stream);
        case 32: return launch<32, 4, false>(mw, mx, g, grid, stream);
        case 64: return launch<64, 4, false>(mw, mx, g, grid, stream);
        case 128: return launch<128, 6, false>(mw, mx, g, grid, stream);
        default: return launch<256, 4, false>(mw, mx, g, grid, stream);
    }
}
