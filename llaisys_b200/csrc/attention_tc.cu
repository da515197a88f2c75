// bfloat16 prefill attention over the paged cache on the 5th-generation tensor cores (tcgen05),
// for head sizes 64 and 128.  Same formula and masks as attention_simt.cu (xsmccc/llaisys
// src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112, plus the window).  All keys, those of
// the step included, are read from the cache: the caller appends before it attends.
//
// A CTA owns 128 consecutive new tokens of one query head.  Warps 0-3 are the softmax warps:
// thread r owns query row r (and lane r of tensor memory).  Warp 4 issues every copy and every
// matrix product, so the softmax warps never leave their arithmetic.  Per tile of one cache page
// (64 keys):
//
//   warp 4   TMA            K and V pages -> shared memory (128-byte swizzle), two stages each
//   warp 4   tcgen05.mma    S[128, 64] = Q K^T into one of two score buffers in tensor memory, two tiles
//                           ahead of the softmax (Q, K both K-major)
//   rows     tcgen05.ld of the own row of S: mask, maximum, exponentials (float32, no cross-thread
//            reduction: a row is one thread's), P as bfloat16 into shared memory
//   warp 4   tcgen05.mma    O[128, dh] += P V  (P K-major, V MN-major as it lies in the cache); the
//                           accumulator stays in tensor memory over all tiles
//
// The exponent base of a row is its running maximum, but it moves only when the maximum has grown
// by more than 8 (a factor 256, far inside the range of bfloat16 and float32): then the row's sum
// and its accumulator in tensor memory are scaled by exp2(old base - new base) (tcgen05.ld, multiply,
// tcgen05.st) before the next product is added.  After the first tiles that is rare, and the result
// is the same quotient O / l.  With the accumulator out of the registers the compiler has room to
// interleave the independent chains of a row, which a warp alone on its scheduler needs.
// Two CTAs share an SM (112 KB of shared memory and 256 tensor-memory columns each).
//
// With few row blocks (a prompt of some thousand tokens) the launch is as long as its longest CTA, the last row
// block, which walks every key tile.  n_split = 2 or 4 then gives each row block to a cluster of CTAs that take even
// shares of its key tiles; at the end they exchange their rows' (base, sum) pairs, scale their accumulators to the
// pairs and their accumulators, column share by column share, with the CTA that owns the share (staged in shared
// memory that is idle by then, sent by bulk copies between two cluster barriers), which scales the shares to the
// common base, adds them up, divides and stores.
// Every mbarrier wait is bounded; a wait that runs out sets *err and the CTA leaves in order.
#include "common.cuh"
#include "tma_map.cuh"

#ifndef LLB_HEAD_DIM
#error "compile with -DLLB_HEAD_DIM=<64 or 128>"
#endif

namespace {

constexpr int DH = LLB_HEAD_DIM;
static_assert(DH == 64 || DH == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int BQ = 128;                    // query rows of a CTA (UMMA M)
constexpr int BKV = LLB_PAGE;              // keys of a tile (UMMA N of Q K^T, K of P V)
constexpr int NBLK = DH / 64;              // 64-column (128-byte) blocks of a head
constexpr int ROW_THREADS = 128;           // warps 0-3: one query row each
constexpr int THREADS = 160;               // warp 4: copies and matrix products
constexpr int Q_BYTES = BQ * DH * 2;       // [NBLK][128 rows][128 B]
constexpr int KV_BYTES = BKV * DH * 2;     // [NBLK][64 rows][128 B]
constexpr int KV_STAGES = 2;               // value stages (and score buffers)
constexpr int K_STAGES = 3;                // key stages
constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + K_STAGES * KV_BYTES;
constexpr int OFF_BAR = OFF_V + KV_STAGES * KV_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 96;
// merge buffers of a split row block, in the shared memory that is idle by then (Q and the ring): staged shares for
// up to three peers, received shares from up to three peers, the rows' (base, sum) pairs staged and received
constexpr int OFF_STG = 0, OFF_RECV = 3 * BQ * (DH / 4) * 4, OFF_ML_STG = 2 * OFF_RECV, OFF_ML_RECV = OFF_ML_STG + BQ * 8;
constexpr int TMEM_COLS = 256;             // S: two buffers at columns [0, 64) and [64, 128); O: columns [128, 128 + DH)
constexpr int O_COL = 128;
constexpr float BASE_STEP = 8.f;           // the exponent base follows the maximum in steps larger than this (log2)
constexpr uint32_t WAIT_LIMIT = 1u << 22;
enum { ERR_ATTN_TC_WAIT = 121, ERR_ATTN_TC_ALIGN = 122 };
static_assert(OFF_ML_RECV + 4 * BQ * 8 <= OFF_BAR, "the merge buffers fit the idle shared memory");

struct TcAttnParams {
    bf16* out;                  // [T, nh * DH]
    const int* page_table;      // [B, table_stride]
    int table_stride;
    const int* seq_start;
    const int* seq_len_before;
    int nh, nkvh, window;
    float scale;
    int* err;
    int n_split;                // 1, 2 or 4: CTAs (a thread-block cluster) that share the key range of a row block
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait of a whole (converged) warp: every lane polls and the vote keeps the control flow uniform, so
// either every lane goes on or none does and the warp-wide instructions that follow never run with lanes
// missing.  Gives up early when another warp of the CTA has already given up.  (Measured: a satisfied wait
// costs 60 cycles this way and 300 when one lane polls in a divergent branch and a shuffle spreads the result.)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return true;
        if ((i & 255u) == 255u && __any_sync(0xffffffffu, *abort_flag != 0)) return false;
    }
    *abort_flag = 1;
    return false;
}
// True in exactly one lane of a converged warp.  The compiler knows that the code under it runs in one
// thread, which lets it feed the tensor-core and copy instructions from uniform registers directly.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand tile (V as it lies in the cache: a row per key, the head dimension contiguous): 64-element
// column blocks `lbo` bytes apart, groups of 8 keys 1024 bytes apart, 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__host__ __device__ constexpr uint32_t idesc_f16(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BQ >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (row r in lane r, two 16-bit elements to a 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One row of 16 accumulator columns; several loads can be in flight before one tmem_wait().
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two float32 multiply-adds in one instruction
__device__ __forceinline__ void fma2(float& lo, float& hi, float a_lo, float a_hi, uint64_t b, uint64_t c) {
    uint64_t a, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a_lo), "f"(a_hi));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(d));
}
// acc += both bfloat16 halves of w (float32 accumulation)
__device__ __forceinline__ void add_bf16_pair(float& acc, uint32_t w) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %0, hi, %0;\n\t}" : "+f"(acc) : "r"(w));
}
__device__ __forceinline__ uint64_t twice(float v) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 2)
attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    // barriers: Q landed; the first two key tiles landed; score buffer written; P V done; tile ready (one per score
    // buffer, the rows may be a tile ahead of the issuing warp): P stored by all 128 rows, the tile's values landed,
    // the keys of the tile two ahead landed, so that one wait of the issuing warp covers all that its two products
    // need; the last P V done.
    // A waiter must never be a whole phase behind or ahead of its barrier, or the parity would lie: hence the
    // pairs, and a barrier of its own for the end.
    const uint32_t bar_q = base + OFF_BAR, bar_k01 = bar_q + 8, bar_s = bar_k01 + 8, bar_o = bar_s + 16, bar_p = bar_o + 16,
                   bar_done = bar_p + 16, bar_merge = bar_done + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + 88);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_BAR + 92);
    const int S = p.n_split;
    const int tid = threadIdx.x, warp = tid >> 5;

    if (tid == 0) {
        *s_abort = (base & 1023u) ? 1 : 0;          // the swizzled tiles need a 1024-byte aligned base
        if (*s_abort) atomicExch(p.err, ERR_ATTN_TC_ALIGN);
        mbar_init(bar_q, 1);
        mbar_init(bar_k01, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(bar_s + 8 * s, 1);
            mbar_init(bar_p + 8 * s, ROW_THREADS + 2);          // the rows, the value copy, the key copy
            mbar_init(bar_o + 8 * s, 1);
        }
        mbar_init(bar_done, 1);
        mbar_init(bar_merge, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (S > 1) mbar_expect_tx(bar_merge, (uint32_t)((S - 1) * (BQ * (DH / S) * 4 + BQ * 8)));    // what the peers will send
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + OFF_BAR + 88), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    // ---- which rows, which keys.  The step's index arrays (sequence starts and lengths, page tables) reach the device
    // by a copy that has ended before the step's first kernel starts, so they are read here, while the kernel before
    // this one may still be running; its output (queries, and the keys and values it appended) only behind the dependency.
    const int b = blockIdx.z, head = blockIdx.x;
    const int tok0 = p.seq_start[b], n_new = p.seq_start[b + 1] - tok0, len_before = p.seq_len_before[b];
    uint32_t rank = 0;
    if (S > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    // Row blocks along y, heads along x: CTAs are handed out x first, so the row blocks with the most key tiles (the
    // last ones, which get the first y) start first for every head, and the short ones fill the end of the launch.
    const int t0 = ((int)(gridDim.y - 1 - blockIdx.y) / S) * BQ;
    const bool active = t0 < n_new && !*s_abort;
    const int kvh = head / (p.nh / p.nkvh);
    const int n_rows = min(BQ, n_new - t0);
    const int first_pos = len_before + t0, last_pos = first_pos + n_rows - 1;
    const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    int tile_lo = key_lo / BKV, n_tiles = active ? last_pos / BKV + 1 - tile_lo : 0;
    if (S > 1) {          // this CTA's even share of the row block's tiles
        const int q = n_tiles / S, r = n_tiles - q * S;
        tile_lo += (int)rank * q + min((int)rank, r);
        n_tiles = q + ((int)rank < r ? 1 : 0);
    }
    const int* table = p.page_table + (size_t)b * p.table_stride;
    auto page_row = [&](int i) { return i < n_tiles ? (table[tile_lo + i] * p.nkvh + kvh) * BKV : 0; };
    int r0 = 0, r1 = 0, r2 = 0, r3 = 0;                             // the issuing warp: page rows of its first four tiles
    if (warp == 4) { r0 = page_row(0); r1 = page_row(1); r2 = page_row(2); r3 = page_row(3); }
    llb_grid_dependency_sync();
    bool failed = false;
    float m = -INFINITY, l = 0.f;                                   // row threads: the exponent base of the row, its sum
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    if (warp == 4) {
        // ================================================= copies and matrix products (one elected lane issues)
        // Descriptors are made once; an instruction's own differs from them by a constant.  (Built per
        // instruction, the address arithmetic of the single issuing thread cost more than the products.)
        const uint64_t q_desc = desc_kmajor(base), k_desc0 = desc_kmajor(base + OFF_K),
                       v_desc0 = desc_mnmajor(base + OFF_V, BKV * 128);
        constexpr uint32_t IDESC_S = idesc_f16(BKV, false), IDESC_O = idesc_f16(DH, true);
        // keys / values of one tile into `stage`; the bytes count on `bar`, which also gets one arrival
        auto issue_k = [&](int stage, int row, uint32_t bar) {
            mbar_expect_tx(bar, KV_BYTES);
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk)
                tma_load_2d(base + OFF_K + stage * KV_BYTES + blk * (BKV * 128), &map_k, bar, blk * 64, row);
        };
        auto issue_v = [&](int stage, int row, uint32_t bar) {
            mbar_expect_tx(bar, KV_BYTES);
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk)
                tma_load_2d(base + OFF_V + stage * KV_BYTES + blk * (BKV * 128), &map_v, bar, blk * 64, row);
        };
        // S = Q K^T of the keys in `stage` into score buffer `buf`
        auto issue_qk = [&](int stage, int buf) {
            const uint64_t kd = k_desc0 + (uint64_t)(stage * (KV_BYTES >> 4));
            const uint32_t d = tmem + buf * BKV;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < DH / 16; ++ks)
                umma(d, q_desc + (uint64_t)(((ks / 4) * (BQ * 128) + (ks % 4) * 32) >> 4),
                     kd + (uint64_t)(((ks / 4) * (BKV * 128) + (ks % 4) * 32) >> 4), IDESC_S, ks > 0 ? 1u : 0u);
            umma_commit(bar_s + 8 * buf);
        };
        // r1, r2, r3: page rows of tiles i + 1, i + 2, i + 3
        if (n_tiles > 0) {
            if (elect_one()) {
                mbar_expect_tx(bar_q, Q_BYTES);
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk)
                    tma_load_2d(base + blk * (BQ * 128), &map_q, bar_q, head * DH + blk * 64, tok0 + t0);
                // the first two key tiles have a barrier of their own (one arrival, the bytes of both)
                mbar_expect_tx(bar_k01, KV_BYTES * min(2, n_tiles));
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk) {
                    tma_load_2d(base + OFF_K + blk * (BKV * 128), &map_k, bar_k01, blk * 64, r0);
                    if (n_tiles > 1) tma_load_2d(base + OFF_K + KV_BYTES + blk * (BKV * 128), &map_k, bar_k01, blk * 64, r1);
                }
                // tile 0: its values and the keys of tile 2; tile 1: its values (the keys of tile 3 follow at the first tile)
                issue_v(0, r0, bar_p);
                if (n_tiles > 2) issue_k(2, r2, bar_p); else mbar_arrive(bar_p);
                if (n_tiles > 1) issue_v(1, r1, bar_p + 8);
            }
            failed = !warp_wait(bar_q, 0, s_abort) || !warp_wait(bar_k01, 0, s_abort);
            if (!failed && elect_one()) {
                issue_qk(0, 0);
                if (n_tiles > 1) issue_qk(1, 1);
            }
            __syncwarp();
        }
        int k_stage = 0;                                // key stage of tile i; tile i + 2 sits in stage k2
        for (int i = 0; i < n_tiles && !failed; ++i) {
            const int s = i & 1;                        // score buffer and value stage of tile i
            const uint32_t ph = (i >> 1) & 1;
            const int k2 = k_stage == 0 ? 2 : k_stage - 1;
            const int r4 = page_row(i + 4);             // for the next round; its latency hides behind the wait
            // every row has read S(i), brought O to its base and stored P(i); V(i) and K(i + 2) have landed.  The
            // key stage of tile i is free as well (the rows saw S(i), so Q K^T of tile i is done).
            if (!warp_wait(bar_p + 8 * s, ph, s_abort)) { failed = true; break; }
            // rows of the last page beyond the last position of this block were never written for this sequence:
            // a zero probability must meet a finite value
            const int p0 = (tile_lo + i) * BKV;
            if (p0 + BKV - 1 > last_pos) {
                const int j0 = last_pos - p0 + 1;
                for (int idx = tid - ROW_THREADS; idx < (BKV - j0) * NBLK * 8; idx += 32) {
                    int j = j0 + idx / (NBLK * 8), rest = idx % (NBLK * 8);
                    *reinterpret_cast<uint4*>(smem + OFF_V + s * KV_BYTES + (rest / 8) * (BKV * 128) + j * 128 + (rest % 8) * 16) =
                        make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // before the tensor core reads them
                __syncwarp();
            }
            if (elect_one()) {
                const uint64_t vd = v_desc0 + (uint64_t)(s * (KV_BYTES >> 4));
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < BKV / 16; ++ks)
                    umma_ts(tmem + O_COL, tmem + s * BKV + ks * 8, vd + (uint64_t)((ks * 16 * 128) >> 4), IDESC_O,
                            (i > 0 || ks > 0) ? 1u : 0u);
                umma_commit(bar_o + 8 * s);
                if (i == n_tiles - 1) umma_commit(bar_done);
                if (i + 2 < n_tiles) issue_qk(k2, s);
                // ---- refill for tile i + 1: the keys of tile i + 3 into the stage of tile i
                if (i + 1 < n_tiles) {
                    if (i + 3 < n_tiles) issue_k(k_stage, r3, bar_p + 8 * (s ^ 1)); else mbar_arrive(bar_p + 8 * (s ^ 1));
                }
            }
            __syncwarp();
            // ---- and its values, once P V of tile i - 1 has left their stage (tile 1's were sent at the start)
            if (i > 0 && i + 1 < n_tiles) {
                if (!warp_wait(bar_o + 8 * (s ^ 1), ((i - 1) >> 1) & 1, s_abort)) { failed = true; break; }
                if (elect_one()) issue_v(s ^ 1, r1, bar_p + 8 * (s ^ 1));
                __syncwarp();
            }
            r1 = r2; r2 = r3; r3 = r4;
            if (++k_stage == K_STAGES) k_stage = 0;
        }
    } else {
        // ================================================= softmax: thread r owns query row r
        const int qpos = first_pos + min(tid, n_rows - 1);          // rows past the end behave like the last row
        const int qlo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
        const float scale_log2 = p.scale * 1.4426950408889634f;
        const uint64_t scale2 = twice(scale_log2);

        for (int i = 0; i < n_tiles && !failed; ++i) {
            const int s = i % KV_STAGES;
            const int p0 = (tile_lo + i) * BKV;
            if (!warp_wait(bar_s + 8 * s, (i / KV_STAGES) & 1, s_abort)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sr[BKV];
#pragma unroll
            for (int c = 0; c < BKV; c += 16) tmem_ld16_nowait(lane_addr + s * BKV + c, sr + c);
            tmem_wait();

            // ---- mask (only tiles that some row of the block sees in part), maximum
            if (!(p0 + BKV - 1 <= first_pos && (p.window <= 0 || p0 >= last_pos - p.window + 1))) {
#pragma unroll
                for (int j = 0; j < BKV; ++j)
                    if (!(p0 + j >= qlo && p0 + j <= qpos)) sr[j] = 0xff800000u;       // -inf
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BKV; j += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx[c] = fmax3(mx[c], __uint_as_float(sr[j + 2 * c]), __uint_as_float(sr[j + 2 * c + 1]));
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;      // the scale is positive
            // ---- the base follows the maximum in large steps only
            const bool move = mt > m + BASE_STEP;                    // false while both are -inf
            const float alpha = move ? fast_exp2(m - mt) : 1.f;      // 0 at the row's first visible key
            if (move) m = mt;
            const float nbase = m == -INFINITY ? 0.f : -m;
            const uint64_t nbase2 = twice(nbase);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < BKV; j += 2) {
                float pa, pb;
                fma2(pa, pb, __uint_as_float(sr[j]), __uint_as_float(sr[j + 1]), scale2, nbase2);
                pa = fast_exp2(pa);
                pb = fast_exp2(pb);
                sr[j / 2] = pack_bf16(pa, pb);                       // packed in place: sr[0..31] hold P
                // the row sum is that of the rounded values, the same weights the product with V uses: their
                // rounding errors then cancel in O / l (a single dominant key gives exactly its value)
                add_bf16_pair(sum[(j / 2) % 4], sr[j / 2]);
            }
            l = l * alpha + (sum[0] + sum[1]) + (sum[2] + sum[3]);

            // ---- a row's base moved: once P V of tile i - 1 is done, its accumulator is scaled to the new base
            if (i > 0 && __any_sync(0xffffffffu, move)) {
                if (!warp_wait(bar_o + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, s_abort)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < DH; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld16_nowait(lane_addr + O_COL + c0, v);
                    tmem_ld16_nowait(lane_addr + O_COL + c0 + 16, v + 16);
                    tmem_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                    tmem_st16(lane_addr + O_COL + c0, v);
                    tmem_st16(lane_addr + O_COL + c0 + 16, v + 16);
                }
            }
            // ---- P(i) takes the place of the row's scores in tensor memory: 64 keys in 32 columns
            tmem_st16(lane_addr + s * BKV, sr);
            tmem_st16(lane_addr + s * BKV + 16, sr + 16);
            tmem_wait_st();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p + 8 * s);
        }
        if (!failed && n_tiles > 0) failed = !warp_wait(bar_done, 0, s_abort);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    // Every thread of every CTA of a cluster passes this barrier, whatever happened before: behind it nobody reads or
    // fills its ring any more, so the peers may write into it.
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp < 4 && S == 1) {
        if (n_tiles > 0 && !__any_sync(0xffffffffu, failed)) {
            const float inv = 1.0f / l;
            bf16* dst = p.out + (size_t)(tok0 + t0 + tid) * p.nh * DH + (size_t)head * DH;
#pragma unroll
            for (int c0 = 0; c0 < DH; c0 += 32) {
                uint32_t v[32];
                tmem_ld16_nowait(lane_addr + O_COL + c0, v);
                tmem_ld16_nowait(lane_addr + O_COL + c0 + 16, v + 16);
                tmem_wait();
                if (tid < n_rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[d + 4]) * inv, __uint_as_float(v[d + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[d + 6]) * inv, __uint_as_float(v[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + d) = w;
                    }
                }
            }
        }
    }
    if (S > 1) {
        // ================================================= merge of a split row block
        // Each CTA stages, per peer, the column share of its accumulator that the peer owns, and its rows' (base, sum)
        // pairs; after the cluster barrier above one thread sends each block with one bulk copy into the peer's
        // shared memory, counted on the peer's merge barrier.  (Storing the pieces remotely one by one was measured:
        // four thousand 16-byte stores per CTA took 10 us, with an mbarrier count on each 12 us.)
        const int COLS = DH / S, PCS = COLS / 4, SWZ = PCS >= 8 ? 7 : PCS - 1;       // this CTA's columns; 16-byte pieces of a row
        const uint32_t share_bytes = (uint32_t)(BQ * COLS * 4);
        const bool take_part = warp < 4 && active && !__any_sync(0xffffffffu, failed);
        float2* ml_recv = reinterpret_cast<float2*>(smem + OFF_ML_RECV);
        if (take_part) {
            reinterpret_cast<float2*>(smem + OFF_ML_STG)[tid] = make_float2(m, l);
            ml_recv[rank * BQ + tid] = make_float2(m, l);
#pragma unroll 1
            for (int c0 = 0; c0 < DH; c0 += 32) {
                const int owner = c0 / COLS;
                if (owner == (int)rank) continue;
                uint32_t v[32];
                if (n_tiles > 0) {
                    tmem_ld16_nowait(lane_addr + O_COL + c0, v);
                    tmem_ld16_nowait(lane_addr + O_COL + c0 + 16, v + 16);
                    tmem_wait();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0u;
                }
                uint8_t* row = smem + OFF_STG + (size_t)(owner < (int)rank ? owner : owner - 1) * share_bytes + (size_t)tid * (COLS * 4);
                const int pc0 = (c0 % COLS) / 4;
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    *reinterpret_cast<uint4*>(row + (((pc0 + e / 4) ^ (tid & SWZ)) * 16)) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");         // the staged blocks before the bulk copies read them
        }
        // every thread of the cluster: all blocks are staged (and every ring is idle)
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (take_part && tid == 0) {
            for (int o = 0; o < S; ++o) {
                if (o == (int)rank) continue;
                const uint32_t slot = (uint32_t)(o < (int)rank ? o : o - 1);          // where this CTA staged the peer's share
                const uint32_t mine = rank < (uint32_t)o ? rank : rank - 1;           // this CTA's place among the peer's sources
                const uint32_t rbar = mapa(bar_merge, (uint32_t)o);
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(mapa(base + OFF_RECV + mine * share_bytes, (uint32_t)o)), "r"(base + OFF_STG + slot * share_bytes),
                               "r"(share_bytes), "r"(rbar) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(mapa(base + OFF_ML_RECV + rank * (uint32_t)(BQ * 8), (uint32_t)o)), "r"(base + OFF_ML_STG),
                               "r"((uint32_t)(BQ * 8)), "r"(rbar) : "memory");
            }
        }
        bool got = true;
        if (take_part) got = warp_wait(bar_merge, 0, s_abort);
        if (take_part && !__any_sync(0xffffffffu, !got)) {
            // ---- this CTA's columns of the row (every lane takes part in the tensor-memory loads; rows past the end store nothing): every source scaled to the common base, added, divided, stored
            float M = -INFINITY, L = 0.f, f[4] = {0.f, 0.f, 0.f, 0.f};
            for (int sp = 0; sp < S; ++sp) M = fmaxf(M, ml_recv[sp * BQ + tid].x);
            for (int sp = 0; sp < S; ++sp) {
                const float2 v = ml_recv[sp * BQ + tid];
                f[sp] = v.x == -INFINITY ? 0.f : fast_exp2(v.x - M);
                L += v.y * f[sp];
            }
            const float inv = 1.0f / L;
            bf16* dst = p.out + (size_t)(tok0 + t0 + tid) * p.nh * DH + (size_t)head * DH + rank * COLS;
#pragma unroll 1
            for (int c0 = 0; c0 < COLS; c0 += 32) {
                float acc[32];
                if (n_tiles > 0) {
                    uint32_t v[32];
                    tmem_ld16_nowait(lane_addr + O_COL + rank * COLS + c0, v);
                    tmem_ld16_nowait(lane_addr + O_COL + rank * COLS + c0 + 16, v + 16);
                    tmem_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = __uint_as_float(v[e]) * f[rank];
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = 0.f;
                }
                for (int sp = 0; sp < S; ++sp) {
                    if (sp == (int)rank) continue;
                    const uint8_t* row = smem + OFF_RECV + (size_t)(sp < (int)rank ? sp : sp - 1) * share_bytes + (size_t)tid * (COLS * 4);
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        const float4 x = *reinterpret_cast<const float4*>(row + (((c0 / 4 + e / 4) ^ (tid & SWZ)) * 16));
                        acc[e] += x.x * f[sp]; acc[e + 1] += x.y * f[sp]; acc[e + 2] += x.z * f[sp]; acc[e + 3] += x.w * f[sp];
                    }
                }
#pragma unroll
                for (int d = 0; d < 32; d += 8) {
                    uint4 w;
                    w.x = pack_bf16(acc[d] * inv, acc[d + 1] * inv);
                    w.y = pack_bf16(acc[d + 2] * inv, acc[d + 3] * inv);
                    w.z = pack_bf16(acc[d + 4] * inv, acc[d + 5] * inv);
                    w.w = pack_bf16(acc[d + 6] * inv, acc[d + 7] * inv);
                    if (tid < n_rows) *reinterpret_cast<uint4*>(dst + c0 + d) = w;
                }
            }
        }
        if (take_part && !got) failed = true;
        // no CTA may leave while a bulk copy still reads its shared memory: all have received what was sent to them
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (failed) {
        *s_abort = 1;
        atomicExch(p.err, ERR_ATTN_TC_WAIT);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);       // copies that may still be in flight get a bounded time to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*s_abort && !failed)                                     // a CTA that gave up leaves together, after the same bounded time
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

}  // namespace

// q: the packed projections [T, row_stride] (query heads first, already rotated); kpool / vpool: one call's pages
// [n_pages, nkvh, 64, DH], already holding the step's keys and values.  max_new: most new tokens of a sequence.
LLB_API int llb_attn_tc_prefill(const void* q, int T, int row_stride, const void* kpool, const void* vpool, int n_pages,
                                TcAttnParams p, int B, int max_new, cudaStream_t stream) {
    if (B == 0 || max_new == 0) return 0;
    if (p.nkvh <= 0 || p.nh % p.nkvh || !(p.scale > 0.f) || row_stride % 8 || (((uintptr_t)q | (uintptr_t)kpool | (uintptr_t)vpool | (uintptr_t)p.out) & 15))
        return (int)cudaErrorInvalidValue;
    if (p.n_split != 1 && p.n_split != 2 && p.n_split != 4) return (int)cudaErrorInvalidValue;
    if (DH / p.n_split < 32) return (int)cudaErrorInvalidValue;          // a column share is whole 32-column pieces
    dim3 grid(p.nh, ((max_new + BQ - 1) / BQ) * p.n_split, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    int rc = llb_tma::bf16_map_64(q, T, p.nh * DH, row_stride, BQ, &mq);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(kpool, (long long)n_pages * p.nkvh * BKV, DH, DH, BKV, &mk);
    if (rc) return rc;
    rc = llb_tma::bf16_map_64(vpool, (long long)n_pages * p.nkvh * BKV, DH, DH, BKV, &mv);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return -2000 - (int)e;
        configured = true;
    }
    if (p.n_split == 1) {
        llb_launch(attn_tc_prefill_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mq, mk, mv, p);
        return llb_status();
    }
    llb_prefer_max_shared((const void*)attn_tc_prefill_kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (llb_pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = (unsigned)p.n_split;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaLaunchKernelEx(&cfg, attn_tc_prefill_kernel, mq, mk, mv, p);
    return llb_status();
}
