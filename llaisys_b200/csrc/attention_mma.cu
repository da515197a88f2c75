// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32
// accumulation), for prefill and for decode.  Compiled per head size:
// -DLLB_HEAD_DIM=<multiple of 16, at most 128>.  Same formula and masks as attention_simt.cu
// (xsmccc/llaisys src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112, plus the window).
//
// Keys and values are walked in tiles of one cache page (64 keys).  A tile's rows are fetched
// with 16-byte cp.async copies by all threads into a ring of shared-memory stages whose rows are
// padded by 16 bytes (so that ldmatrix reads them without bank conflicts).  (One bulk copy per
// row was measured first: the copy engine takes them one after another, about 36 ns each, which
// made a tile cost 4.6 us.)  A row comes from the cache page of its position or, for positions
// of the step itself in prefill, from the packed projection output.  Scores, the running
// maximum, the exponentials and the normaliser are float32; the probabilities are rounded to
// bfloat16 only as the tensor-core operand of P*V.
//
//  * decode: a block owns up to 16 query heads that share one kv head, for one sequence and one
//    slice of its key range; its four warps take 16 keys each of every tile and are merged at the
//    end.  Up to eight slices form a thread-block cluster and are merged through distributed
//    shared memory; more slices go through global memory and a second kernel.  The kernel can
//    also do what would otherwise take a kernel before it: rotate the query heads and the new key
//    (half-split rotary encoding) and append the new key and value to the cache.
//  * prefill: a block owns 64 consecutive new tokens of one query head; each warp 16 of them.
//
// The only waits are cp.async.wait_group and __syncthreads, which cannot outlast the copies.
#include "common.cuh"

#ifndef LLB_HEAD_DIM
#error "compile with -DLLB_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int DH = LLB_HEAD_DIM;
static_assert(DH % 16 == 0 && DH <= 128, "head size must be a multiple of 16, at most 128");
constexpr int TILE = LLB_PAGE;                 // keys of a tile
constexpr int ROW_BYTES = DH * 2;
constexpr int ROW_STRIDE = ROW_BYTES + 16;     // padded shared-memory row
constexpr int TILE_BYTES = TILE * ROW_STRIDE;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;    // keys, then values
constexpr int STAGES_PREFILL = 2;   // prefill: two stages leave room for three blocks per SM (twelve warps to hide latency)
constexpr int STAGES = 3;     // ring depth of decode.  (A deeper ring for decode was measured: its blocks fill an SM's shared memory,
                              // the next kernel's blocks can no longer start early and stream their weights, and the step slows.)
constexpr int THREADS = 128;
constexpr int KSTEPS = DH / 16;
constexpr int DTILES = DH / 8;

struct MmaAttnParams {
    const bf16* q;          // packed projections [T, row_stride]; query head h at column h * DH
    const bf16* k_new;      // the same buffer at its first key column
    const bf16* v_new;      // the same buffer at its first value column
    int row_stride;
    bf16* out;              // [T, nh * DH]
    const bf16* kpool;      // [pages, nkvh, TILE, DH]
    const bf16* vpool;
    const int* page_table;  // [B, table_stride]
    int table_stride;
    int ring;
    const int* seq_start;
    const int* seq_len_before;
    int nh, nkvh, window;
    float scale;
    int all_from_cache;     // prefill: read the step's own keys from the cache too
    int n_splits;           // decode
    float* part_o;          // decode: [B, nh, n_splits, DH]
    float* part_ml;         // decode: [B, nh, n_splits, 2]
    // decode, optional fusions (null / 0 when not used)
    const float* rope_cos;  // [rope_rows, DH/2]: rotate the query heads and the new key here (half-split pairs) and
    const float* rope_sin;  //   append the new key and value to the cache, instead of in a kernel before this one
    int rope_rows;
    int append_new;         // the new token's key/value are not in the cache yet: take them from the packed projections
                            // (rotating the key when rope_cos is set), use them, and write them to the cache
    int cluster;            // the n_splits (<= 8) blocks of a (sequence, head group) are a thread-block cluster and merge
                            // their key slices through distributed shared memory; part_o / part_ml are not used
    int* err;               // decode, cluster merge: set when the bounded wait for the peers' partial sums runs out
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (relative error about 2^-22; exp2(-inf) = 0).  The results feed
// bfloat16 probabilities and float32 sums whose other terms carry the same error.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// What a block needs to fetch tiles: where each key position of the sequence lives.
struct Source {
    const bf16 *kpool, *vpool, *k_new, *v_new;
    const int* table;
    int ring, nkvh, kvh, row_stride, tok0, len_before;
    bool use_new;           // positions >= len_before come from k_new / v_new
};

// Starts the copies of tile `tile` (key positions tile*TILE ...) restricted to [key_lo, key_hi] into
// stage memory at `stage`; all threads of the block take part.  The caller commits the group.
__device__ __forceinline__ void issue_tile(const Source& s, int tile, int key_lo, int key_hi, uint32_t stage, int tid) {
    constexpr int CH = ROW_BYTES / 16;                     // 16-byte chunks of a row
    const int p0 = tile * TILE;
    const int j_lo = max(0, key_lo - p0), j_hi = min(TILE, key_hi - p0 + 1);       // valid rows [j_lo, j_hi)
    const size_t page_off = paged_row(s.table, s.ring, p0, s.kvh, s.nkvh, DH);      // one page per tile
    for (int i = tid; i < TILE * CH; i += THREADS) {
        int j = i / CH, c = i - j * CH;
        if (j < j_lo || j >= j_hi) continue;
        int pos = p0 + j;
        const bf16 *ks, *vs;
        if (s.use_new && pos >= s.len_before) {
            size_t off = (size_t)(s.tok0 + pos - s.len_before) * s.row_stride + (size_t)s.kvh * DH;
            ks = s.k_new + off;
            vs = s.v_new + off;
        } else {
            size_t off = page_off + (size_t)j * DH;
            ks = s.kpool + off;
            vs = s.vpool + off;
        }
        uint32_t d = stage + j * ROW_STRIDE + c * 16;
        cp_async16(d, ks + c * 8);
        cp_async16(d + TILE_BYTES, vs + c * 8);
    }
}

// Zeroes the value rows of a tile outside [key_lo, key_hi] (they were not fetched; a zero
// probability must meet a finite value).  All threads of the block; block-uniform condition.
__device__ __forceinline__ void zero_unfetched(uint8_t* stage_ptr, int tile, int key_lo, int key_hi, int tid) {
    int p0 = tile * TILE;
    int j_lo = max(0, key_lo - p0), j_hi = min(TILE, key_hi - p0 + 1);
    if (j_lo == 0 && j_hi == TILE) return;
    constexpr int CH = ROW_BYTES / 16;
    for (int i = tid; i < TILE * CH; i += THREADS) {
        int j = i / CH, c = i - j * CH;
        if (j < j_lo || j >= j_hi)
            *reinterpret_cast<uint4*>(stage_ptr + TILE_BYTES + j * ROW_STRIDE + c * 16) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
}

// The same two for the decode kernel, in which warp w owns the key rows [16 w, 16 w + 16) of every tile: it requests
// them, multiplies with them and requests their successors itself, so its pace depends on no other warp's and the
// walk over the tiles needs no barrier of the whole block.  (With one barrier in front of and one behind every tile
// and the requests for a tile shared by all threads, the pass that re-requested a stage took 1,300 cycles longer.)
// page_off: where the tile's page begins in the pools (paged_row of its first position), which the caller looks up a
// pass ahead: the entry comes from global memory, and read here its latency would stand in front of the requests.
__device__ __forceinline__ void issue_tile_rows(const Source& s, int tile, int key_lo, int key_hi, uint32_t stage, int warp, int lane,
                                                size_t page_off) {
    constexpr int CH = ROW_BYTES / 16;
    const int p0 = tile * TILE;
    const int j_lo = max(0, key_lo - p0), j_hi = min(TILE, key_hi - p0 + 1);
    for (int it = lane; it < 16 * CH; it += 32) {
        const int j = warp * 16 + it / CH, c = it % CH;
        if (j < j_lo || j >= j_hi) continue;
        const size_t off = page_off + (size_t)j * DH;
        const uint32_t d = stage + j * ROW_STRIDE + c * 16;
        cp_async16(d, s.kpool + off + c * 8);
        cp_async16(d + TILE_BYTES, s.vpool + off + c * 8);
    }
}
__device__ __forceinline__ void zero_unfetched_rows(uint8_t* stage_ptr, int tile, int key_lo, int key_hi, int warp, int lane) {
    const int p0 = tile * TILE;
    const int j_lo = max(0, key_lo - p0), j_hi = min(TILE, key_hi - p0 + 1);
    if (j_lo == 0 && j_hi == TILE) return;
    constexpr int CH = ROW_BYTES / 16;
    for (int it = lane; it < 16 * CH; it += 32) {
        const int j = warp * 16 + it / CH, c = it % CH;
        if (j < j_lo || j >= j_hi)
            *reinterpret_cast<uint4*>(stage_ptr + TILE_BYTES + j * ROW_STRIDE + c * 16) = make_uint4(0, 0, 0, 0);
    }
    __syncwarp();
}

// Elements d, d+1 of a head's vector after the half-split rotation by the angles of one position
// (cs, sn: that position's DH/2 cosines and sines), rounded to bfloat16 like the separate kernel does.
__device__ __forceinline__ uint32_t rotated_pair(const bf16* x, int d, const float* cs, const float* sn) {
    constexpr int HALF = DH / 2;
    float r[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        int i = d + e;
        if (i < HALF) r[e] = to_f32(x[i]) * cs[i] - to_f32(x[i + HALF]) * sn[i];
        else r[e] = to_f32(x[i]) * cs[i - HALF] + to_f32(x[i - HALF]) * sn[i - HALF];
    }
    return pack_bf16(r[0], r[1]);
}

// Query rows as A fragments: q_of(row) gives the pointer to that row's DH elements or nullptr.
template <typename F>
__device__ __forceinline__ void load_q(uint32_t (&qf)[KSTEPS][4], F q_of, int lane, const float* cs = nullptr,
                                       const float* sn = nullptr) {
    const bf16* r0 = q_of(lane >> 2);
    const bf16* r1 = q_of((lane >> 2) + 8);
    int c = (lane & 3) * 2;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        if (cs) {
            qf[kk][0] = r0 ? rotated_pair(r0, kk * 16 + c, cs, sn) : 0u;
            qf[kk][1] = r1 ? rotated_pair(r1, kk * 16 + c, cs, sn) : 0u;
            qf[kk][2] = r0 ? rotated_pair(r0, kk * 16 + 8 + c, cs, sn) : 0u;
            qf[kk][3] = r1 ? rotated_pair(r1, kk * 16 + 8 + c, cs, sn) : 0u;
        } else {
            qf[kk][0] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c) : 0u;
            qf[kk][1] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c) : 0u;
            qf[kk][2] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + 8 + c) : 0u;
            qf[kk][3] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + 8 + c) : 0u;
        }
    }
}

// One warp: scores of its 16 rows against NT*8 keys starting at row `key0` of the tile in `stage`,
// masking, online softmax update, and O += P V.  lo0/hi0 and lo1/hi1: visible key positions of
// the thread's two rows (lane/4 and lane/4 + 8).
template <int NT, bool MASKED = true>
__device__ __forceinline__ void tile_step(const uint32_t (&qf)[KSTEPS][4], float (&o)[DTILES][4], float (&m)[2],
                                          float (&l)[2], uint32_t stage, int key0, int pos0, int lo0, int hi0, int lo1,
                                          int hi1, float scale_log2, int lane) {
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    const int mid = lane >> 3, mr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
            uint32_t b[4];
            uint32_t addr = stage + (key0 + n2 * 16 + (mid >> 1) * 8 + mr) * ROW_STRIDE + (kk * 16 + (mid & 1) * 8) * 2;
            ldsm_x4(b, addr);
            mma16816(s[2 * n2], qf[kk], b[0], b[1]);
            mma16816(s[2 * n2 + 1], qf[kk], b[2], b[3]);
        }
    }
    // mask and row maxima (MASKED = false: the caller knows every key of the tile is visible to every row)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        if (MASKED) {
            int kp = pos0 + key0 + n * 8 + (lane & 3) * 2;
            s[n][0] = (kp >= lo0 && kp <= hi0) ? s[n][0] * scale_log2 : -INFINITY;
            s[n][1] = (kp + 1 >= lo0 && kp + 1 <= hi0) ? s[n][1] * scale_log2 : -INFINITY;
            s[n][2] = (kp >= lo1 && kp <= hi1) ? s[n][2] * scale_log2 : -INFINITY;
            s[n][3] = (kp + 1 >= lo1 && kp + 1 <= hi1) ? s[n][3] * scale_log2 : -INFINITY;
        } else {
            s[n][0] *= scale_log2;
            s[n][1] *= scale_log2;
            s[n][2] *= scale_log2;
            s[n][3] *= scale_log2;
        }
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    // a row that has seen no visible key yet keeps m = -inf; use 0 as the exponent base then so that
    // exp2(-inf - 0) = 0 and no inf - inf arises
    float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
    float a0 = fast_exp2(m[0] - b0), a1 = fast_exp2(m[1] - b1);
    m[0] = mn0;
    m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[NT][2];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float p0 = fast_exp2(s[n][0] - b0), p1 = fast_exp2(s[n][1] - b0), p2 = fast_exp2(s[n][2] - b1), p3 = fast_exp2(s[n][3] - b1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pf[n][0] = pack_bf16(p0, p1);
        pf[n][1] = pack_bf16(p2, p3);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l[0] = l[0] * a0 + sum0;
    l[1] = l[1] * a1 + sum1;
#pragma unroll
    for (int d = 0; d < DTILES; ++d) {
        o[d][0] *= a0;
        o[d][1] *= a0;
        o[d][2] *= a1;
        o[d][3] *= a1;
    }
    // O += P V: 16 keys per k-step
    const uint32_t vbase = stage + TILE_BYTES;
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
        uint32_t a[4] = {pf[2 * n2][0], pf[2 * n2][1], pf[2 * n2 + 1][0], pf[2 * n2 + 1][1]};
#pragma unroll
        for (int d2 = 0; d2 < DTILES / 2; ++d2) {
            uint32_t b[4];
            uint32_t addr = vbase + (key0 + n2 * 16 + (mid & 1) * 8 + mr) * ROW_STRIDE + (d2 * 16 + (mid >> 1) * 8) * 2;
            ldsm_x4_trans(b, addr);
            mma16816(o[2 * d2], a, b[0], b[1]);
            mma16816(o[2 * d2 + 1], a, b[2], b[3]);
        }
    }
}

template <int NST>
struct Ring {
    uint32_t base;
    uint8_t* ptr;
    __device__ uint32_t stage(int i) const { return base + (i % NST) * STAGE_BYTES; }
    __device__ uint8_t* stage_ptr(int i) const { return ptr + (i % NST) * STAGE_BYTES; }
};

template <int NST>
__device__ __forceinline__ Ring<NST> make_ring(uint8_t* smem_raw) {
    Ring<NST> r;
    uint32_t raw = smem_u32(smem_raw);
    r.base = (raw + 127u) & ~127u;
    r.ptr = smem_raw + (r.base - raw);
    return r;
}
constexpr int MAX_CLUSTER = 16;            // key slices that merge inside a thread-block cluster (16 needs the non-portable size)
constexpr int QS_BYTES = 16 * (DH + 8) * 2;
// What a block receives in the cluster merge by pushing: from each block its share of the heads' sums (n_heads * DH * 4
// bytes over all sources) and 16 (maximum, sum) pairs.  A region of its own, so that a peer may push whenever it is done,
// without asking whether this block still needs the memory; 6 KB, which two blocks of the largest head size still fit an
// SM with (ten heads of 128 to a kv head and eight slices; beyond that the slices merge by loads from the peers).
constexpr int MERGE_RECV_BYTES = 6144;
constexpr int smem_bytes(int nst) { return nst * STAGE_BYTES + QS_BYTES + 16 + 128; }     // ring, staged queries, a barrier, alignment slack
constexpr int smem_bytes_decode(int nst) { return smem_bytes(nst) + MERGE_RECV_BYTES; }
constexpr uint32_t MERGE_WAIT_LIMIT = 1u << 22;
enum { ERR_ATTN_MERGE_WAIT = 141 };

// Block `rank` of a cluster of S (<= MAXS) blocks merges its share of the n_heads * DH outputs from the partial
// results every block keeps in shared memory (ml: [16][2] maximum and sum, o: [16][DH]) and writes them to out.
template <int MAXS>
__device__ __forceinline__ void cluster_merge(int S, int n_heads, uint32_t ml_addr, uint32_t o_addr, bf16* out, int tid) {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int total = n_heads * DH, share = (total + S - 1) / S;
    for (int i = (int)rank * share + tid; i < min(total, ((int)rank + 1) * share); i += THREADS) {
        int r = i / DH, d = i - r * DH;
        float ms[MAXS], ls[MAXS], os[MAXS];
#pragma unroll
        for (int sp = 0; sp < MAXS; ++sp) {
            ms[sp] = -INFINITY;
            ls[sp] = os[sp] = 0.f;
            if (sp < S) {
                uint32_t ra;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(ml_addr + (uint32_t)(r * 8)), "r"(sp));
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ms[sp]) : "r"(ra) : "memory");
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ls[sp]) : "r"(ra + 4) : "memory");
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(o_addr + (uint32_t)((r * DH + d) * 4)), "r"(sp));
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(os[sp]) : "r"(ra) : "memory");
            }
        }
        float M = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < MAXS; ++sp) M = fmaxf(M, ms[sp]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int sp = 0; sp < MAXS; ++sp) {
            float f = ms[sp] == -INFINITY ? 0.f : fast_exp2(ms[sp] - M);
            L += ls[sp] * f;
            acc += os[sp] * f;
        }
        out[(size_t)r * DH + d] = __float2bfloat16_rn(acc / L);
    }
}

// ------------------------------------------------------------------ decode
template <int NST>
__global__ void __launch_bounds__(THREADS) attn_mma_decode_kernel(MmaAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    Ring<NST> ring = make_ring<NST>(smem_raw);
    LLB_STAMPS_BEGIN();
    // The key slices of a cluster merge by pushing (below) when every block's share of the outputs is whole 16-byte
    // pieces and what it receives fits the receive region.
    const int G_ = p.nh / p.nkvh, chunks_ = (G_ + 15) / 16;
    const int nh_blk = min(16, G_ - (int)(blockIdx.y % chunks_) * 16);
    const int share4 = p.n_splits > 0 ? nh_blk * (DH / 4) / p.n_splits : 0;               // 16-byte pieces a block owns
    const bool push_merge = p.cluster && p.n_splits > 1 && (nh_blk * (DH / 4)) % p.n_splits == 0 &&
                            p.n_splits * (share4 * 16 + 16 * 8) <= MERGE_RECV_BYTES;
    const uint32_t bar_merge = ring.base + NST * STAGE_BYTES + QS_BYTES;
    if (push_merge && tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_merge));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // from each block of the cluster: its partial sums of this block's share, and every head's maximum and sum
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                     ::"r"(bar_merge), "r"((uint32_t)(p.n_splits * (share4 * 16 + nh_blk * 8))) : "memory");
    }
    if (push_merge) {
        // The peers may push as soon as this barrier stands: arrive now, long before anyone has anything to push; the
        // wait that precedes a block's first push then costs nothing.  (With the receive region in the memory of the
        // staged queries the arrival had to follow their last use, behind the grid dependency: 2,600 cycles.)
        __syncthreads();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    }
    // With append_new nothing this kernel fetches from the cache was written by the kernels just before it
    // (the new token's row comes from the projections), and the step's description was copied before the
    // step's first kernel: the first tiles are requested before the grid dependency resolves.
    if (!p.append_new) llb_grid_dependency_sync();

    const int b = blockIdx.z;
    const int G = p.nh / p.nkvh;
    const int chunks = (G + 15) / 16;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
    const int head0 = kvh * G + chunk * 16, n_heads = min(16, G - chunk * 16);
    const int tok = p.seq_start[b];
    const int pos = p.seq_len_before[b];                 // the new token's position
    const int key_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    // with append_new the new token's key and value are not in the cache: tiles are fetched up to pos - 1 and
    // the block that owns the last tile puts the new row there itself
    const int fetch_hi = p.append_new ? pos - 1 : pos;
    const float* cs = p.rope_cos ? p.rope_cos + (size_t)min(pos, p.rope_rows - 1) * (DH / 2) : nullptr;
    const float* sn = p.rope_cos ? p.rope_sin + (size_t)min(pos, p.rope_rows - 1) * (DH / 2) : nullptr;
    int tile_lo = key_lo / TILE, tile_hi = pos / TILE + 1;
    {   // as even a share of the tiles as there is: the slowest block of a sequence sets the time of all
        const int n = tile_hi - tile_lo, q = n / p.n_splits, r = n - q * p.n_splits, x = blockIdx.x;
        tile_lo += x * q + min(x, r);
        tile_hi = tile_lo + q + (x < r ? 1 : 0);
    }
    const int n_tiles = max(0, tile_hi - tile_lo);

    Source src{p.kpool, p.vpool, nullptr, nullptr, p.page_table + (size_t)b * p.table_stride,
               p.ring, p.nkvh, kvh, 0, 0, 0, false};
    for (int i = 0; i < NST; ++i) {
        if (i < n_tiles)
            issue_tile_rows(src, tile_lo + i, key_lo, fetch_hi, ring.stage(i), warp, lane,
                            paged_row(src.table, p.ring, (tile_lo + i) * TILE, kvh, p.nkvh, DH));
        cp_async_commit();                                 // one group per stage, empty or not
    }
    // The ring holds NST tiles; the pages of the block's next two tiles are asked into L2 now, so that their
    // copies, which can start only when a stage is free, find them there (a page is contiguous per kv head).
    // Only two: a block with a long walk (large batches) streams at full rate anyway, and asking for all its
    // pages at once was measured to cost 5 % at batch 64.
    size_t off_ahead = NST < n_tiles ? paged_row(src.table, p.ring, (tile_lo + NST) * TILE, kvh, p.nkvh, DH) : 0;      // page of the first re-request
    for (int i = NST; i < min(n_tiles, NST + 2); ++i) {
        const size_t off = i == NST ? off_ahead : paged_row(src.table, p.ring, (tile_lo + i) * TILE, kvh, p.nkvh, DH);
        for (int c = tid * 64; c < TILE * DH; c += THREADS * 64) {          // 64 elements = one 128-byte line
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.kpool + off + c));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.vpool + off + c));
        }
    }
    // The query staging below gives each thread one pair index j of the rotation: its angle is fetched now.
    constexpr int HALF = DH / 2, Q_ROWS_PER_PASS = THREADS / HALF, Q_PASSES = (16 + Q_ROWS_PER_PASS - 1) / Q_ROWS_PER_PASS;
    const int qj = tid % HALF, qr0 = tid / HALF;
    float q_co = 1.f, q_si = 0.f;
    if (cs) { q_co = cs[qj]; q_si = sn[qj]; }
    // every peer's barrier stands (they arrived at their start, as this block did; a cluster's blocks start together):
    // waited for here, where the block is waiting for the projections anyway, and not in front of the first push
    if (push_merge) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid == 0) LLB_STAMP(0);       // stamps: 0 set up, 1 projections ready (grid dependency), 2 queries staged, 3 tiles walked,
    if (p.append_new) llb_grid_dependency_sync();          // the projections are read from here on
    if (tid == 0) LLB_STAMP(1);       //         4 warps' sums in shared memory, 5 merged pieces pushed, 6 peers' pieces received, 7 stored

    // the new token's key and value (for the block that owns the last tile): loaded now, used at that tile
    const bool owns_new = p.append_new && n_tiles > 0 && tile_hi - 1 == pos / TILE;
    uint32_t new_k = 0, new_v = 0;
    if (owns_new && tid * 2 < DH) {
        const bf16* kn = p.k_new + (size_t)tok * p.row_stride + (size_t)kvh * DH;
        const bf16* vn = p.v_new + (size_t)tok * p.row_stride + (size_t)kvh * DH;
        new_k = cs ? rotated_pair(kn, tid * 2, cs, sn) : *reinterpret_cast<const uint32_t*>(kn + tid * 2);
        new_v = *reinterpret_cast<const uint32_t*>(vn + tid * 2);
    }
    // the query heads of this block, rotated if asked for, staged in shared memory behind the ring: all loads
    // of a thread are in flight together
    bf16* qs = reinterpret_cast<bf16*>(ring.ptr + NST * STAGE_BYTES);       // [16][DH + 8]
    {
        const bf16* qg = p.q + (size_t)tok * p.row_stride + (size_t)head0 * DH;
        float qa[Q_PASSES], qb[Q_PASSES];
#pragma unroll
        for (int k = 0; k < Q_PASSES; ++k) {
            const int r = qr0 + k * Q_ROWS_PER_PASS;
            const bool in = qr0 < Q_ROWS_PER_PASS && r < n_heads;
            qa[k] = in ? to_f32(qg[r * DH + qj]) : 0.f;
            qb[k] = in ? to_f32(qg[r * DH + qj + HALF]) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < Q_PASSES; ++k) {
            const int r = qr0 + k * Q_ROWS_PER_PASS;
            if (qr0 < Q_ROWS_PER_PASS && r < 16) {
                qs[r * (DH + 8) + qj] = __float2bfloat16_rn(qa[k] * q_co - qb[k] * q_si);
                qs[r * (DH + 8) + qj + HALF] = __float2bfloat16_rn(qb[k] * q_co + qa[k] * q_si);
            }
        }
    }
    __syncthreads();
    if (tid == 0) LLB_STAMP(2);
    uint32_t qf[KSTEPS][4];
    load_q(qf, [&](int r) -> const bf16* { return qs + r * (DH + 8); }, lane);
    float o[DTILES][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    const float scale_log2 = p.scale * 1.4426950408889634f;

    for (int i = 0; i < n_tiles; ++i) {
        const size_t off_now = off_ahead;                  // page of tile i + NST, looked up a pass ago
        if (i + 1 + NST < n_tiles) off_ahead = paged_row(src.table, p.ring, (tile_lo + i + 1 + NST) * TILE, kvh, p.nkvh, DH);
        cp_async_wait<NST - 1>();                       // this thread's copies of tile i have landed
        __syncwarp();                                      // ... and those of the warp's other lanes: the warp's rows are there
        if (owns_new && tile_lo + i == pos / TILE) {
            // the new token's row into this tile (and, once per kv head, into the cache).  The one place where the warps
            // meet: every warp is in this pass, so none still reads what the stage held three passes ago.
            __syncthreads();
            uint8_t* krow = ring.stage_ptr(i) + (pos % TILE) * ROW_STRIDE;
            const int d = tid * 2;
            if (d < DH) {
                *reinterpret_cast<uint32_t*>(krow + d * 2) = new_k;
                *reinterpret_cast<uint32_t*>(krow + TILE_BYTES + d * 2) = new_v;
                if (chunk == 0) {
                    size_t goff = paged_row(src.table, p.ring, pos, kvh, p.nkvh, DH);
                    *reinterpret_cast<uint32_t*>(const_cast<bf16*>(p.kpool) + goff + d) = new_k;
                    *reinterpret_cast<uint32_t*>(const_cast<bf16*>(p.vpool) + goff + d) = new_v;
                }
            }
            __syncthreads();
        }
        zero_unfetched_rows(ring.stage_ptr(i), tile_lo + i, key_lo, pos, warp, lane);
        tile_step<2>(qf, o, m, l, ring.stage(i), warp * 16, (tile_lo + i) * TILE, key_lo, pos, key_lo, pos, scale_log2, lane);
        __syncwarp();                                      // the warp's rows of the stage are free
        if (i + NST < n_tiles) issue_tile_rows(src, tile_lo + i + NST, key_lo, fetch_hi, ring.stage(i + NST), warp, lane, off_now);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    if (tid == 0) LLB_STAMP(3);

    // ---- merge the four warps (each saw a quarter of the keys) through shared memory
    float* sm_ml = reinterpret_cast<float*>(ring.ptr);               // [4][16][2]
    float* sm_o = sm_ml + 4 * 16 * 2;                                 // [4][16][SO]; SO = DH + 8 keeps the rows' 8-byte
    constexpr int SO = DH + 8;                                        // stores of a half-warp on distinct banks
    {
        int r0 = lane >> 2, c = (lane & 3) * 2;
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + r0) * 2] = m[0];
            sm_ml[(warp * 16 + r0) * 2 + 1] = l[0];
            sm_ml[(warp * 16 + r0 + 8) * 2] = m[1];
            sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l[1];
        }
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            float* w0 = sm_o + (size_t)(warp * 16 + r0) * SO + d * 8 + c;
            float* w1 = sm_o + (size_t)(warp * 16 + r0 + 8) * SO + d * 8 + c;
            *reinterpret_cast<float2*>(w0) = make_float2(o[d][0], o[d][1]);
            *reinterpret_cast<float2*>(w1) = make_float2(o[d][2], o[d][3]);
        }
    }
    __syncthreads();
    if (tid == 0) LLB_STAMP(4);
    if (push_merge) {
        // ---- merge of the key slices by pushing.  The four warps' partial sums are merged 16 bytes at a time and each
        // piece goes straight from the registers to the block that owns it (block q owns the q-th share of the
        // [head][column] outputs), counted on the owner's barrier, with the head's (maximum, sum) to every owner.  The
        // owner scales the S sources to a common base, adds, divides and stores.  Nobody loads from another block's
        // memory, and there is no barrier at the end: nobody reads this block's memory, and everything written into it
        // has arrived when its own barrier completes.  (Before: every block merged its warps value by value, a cluster
        // barrier, loads from all peers, a second barrier; 7,600 of the kernel's 16,300 cycles at batch 8 lay behind
        // the last tile.  Pushing the warps' sums unmerged, 1,500 eight-byte stores a block, was slower still.)
        const int S = p.n_splits;
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        const uint32_t recv = ring.base + NST * STAGE_BYTES + QS_BYTES + 16;     // [S][share4] float4, then [S][16] (maximum, sum)
        const uint32_t ml_off = (uint32_t)(S * share4 * 16);
        for (int i4 = tid; i4 < n_heads * (DH / 4); i4 += THREADS) {
            const int r = i4 / (DH / 4), d4 = i4 - r * (DH / 4);
            float mw[4], M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                mw[w] = sm_ml[(w * 16 + r) * 2];
                M = fmaxf(M, mw[w]);
            }
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = mw[w] == -INFINITY ? 0.f : fast_exp2(mw[w] - M);
                const float4 v = *reinterpret_cast<const float4*>(sm_o + (size_t)(w * 16 + r) * SO + d4 * 4);
                L += sm_ml[(w * 16 + r) * 2 + 1] * f;
                acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
            }
            const int owner = i4 / share4, slot = i4 - owner * share4;
            uint32_t rbuf, rbar;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbuf) : "r"(recv + (uint32_t)((rank * share4 + slot) * 16)), "r"(owner));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar_merge), "r"(owner));
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                         ::"r"(rbuf), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w), "r"(rbar) : "memory");
            if (d4 == 0) {
                for (int q = 0; q < S; ++q) {
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbuf) : "r"(recv + ml_off + (uint32_t)((rank * 16 + r) * 8)), "r"(q));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar_merge), "r"(q));
                    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                                 ::"r"(rbuf), "f"(M), "f"(L), "r"(rbar) : "memory");
                }
            }
        }
        if (tid == 0) LLB_STAMP(5);
        // ---- all blocks' pieces (bounded wait)
        bool got = false;
        for (uint32_t t = 0; t < MERGE_WAIT_LIMIT && !got; ++t) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(bar_merge), "r"(0u) : "memory");
            got = done != 0;
        }
        if (!got) {
            if (p.err) atomicExch(p.err, ERR_ATTN_MERGE_WAIT);
            return;
        }
        if (tid == 0) LLB_STAMP(6);
        // ---- this block's share: every source scaled to the common base, added, divided, stored
        const uint8_t* rp = ring.ptr + NST * STAGE_BYTES + QS_BYTES + 16;
        const float2* rml = reinterpret_cast<const float2*>(rp + ml_off);
        bf16* out_tok = p.out + (size_t)tok * p.nh * DH + (size_t)head0 * DH;
        for (int j = tid; j < share4 * 4; j += THREADS) {
            const int idx = (int)rank * share4 * 4 + j, r = idx / DH;           // index among the [head][column] outputs
            float M = -INFINITY;
            for (int sp = 0; sp < S; ++sp) M = fmaxf(M, rml[sp * 16 + r].x);
            float L = 0.f, acc = 0.f;
            for (int sp = 0; sp < S; ++sp) {
                const float2 ml2 = rml[sp * 16 + r];
                const float f = ml2.x == -INFINITY ? 0.f : fast_exp2(ml2.x - M);
                L += ml2.y * f;
                acc += reinterpret_cast<const float*>(rp)[(size_t)(sp * share4) * 4 + j] * f;
            }
            out_tok[idx] = __float2bfloat16_rn(acc / L);
        }
        if (tid == 0) LLB_STAMP(7);
        return;
    }
    // merged over the four warps: fin_ml [16][2], fin_o [16][DH] (kept in shared memory for the cluster merge)
    float* fin_ml = sm_o + 4 * 16 * SO;
    float* fin_o = fin_ml + 16 * 2;
    for (int i = tid; i < n_heads * DH; i += THREADS) {
        int r = i / DH, d = i - r * DH;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float mw = sm_ml[(w * 16 + r) * 2];
            if (mw != -INFINITY) {
                float f = fast_exp2(mw - M);
                L += sm_ml[(w * 16 + r) * 2 + 1] * f;
                acc += sm_o[(size_t)(w * 16 + r) * SO + d] * f;
            }
        }
        int head = head0 + r;
        if (p.n_splits == 1) {
            p.out[(size_t)tok * p.nh * DH + (size_t)head * DH + d] = __float2bfloat16_rn(acc / L);
        } else if (p.cluster) {
            fin_o[r * DH + d] = acc;
            if (d == 0) {
                fin_ml[r * 2] = M;                    // base-2 logarithmic scale
                fin_ml[r * 2 + 1] = L;
            }
        } else {
            size_t slot = ((size_t)b * p.nh + head) * p.n_splits + blockIdx.x;
            p.part_o[slot * DH + d] = acc;
            if (d == 0) {
                p.part_ml[slot * 2] = M;
                p.part_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (p.n_splits == 1 || !p.cluster) return;

    // ---- cluster merge of the key slices: block `rank` produces one share of the (head, dim) outputs
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    {
        // Two instances of the same code: the common one for up to eight slices stays as short as it was (a block
        // runs this part once, so its time is the time to fetch its instructions).
        const uint32_t ml_addr = smem_u32(fin_ml), o_addr = smem_u32(fin_o);
        bf16* out_tok = p.out + (size_t)tok * p.nh * DH + (size_t)head0 * DH;
        if (p.n_splits <= 8) cluster_merge<8>(p.n_splits, n_heads, ml_addr, o_addr, out_tok, tid);
        else cluster_merge<MAX_CLUSTER>(p.n_splits, n_heads, ml_addr, o_addr, out_tok, tid);
    }
    // no block may leave while another still reads its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void attn_mma_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                        const float* __restrict__ part_ml, const int* __restrict__ seq_start, int nh,
                                        int n_splits) {
    llb_grid_dependency_sync();
    int head = blockIdx.x, b = blockIdx.y;
    size_t base = ((size_t)b * nh + head) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float ms = part_ml[(base + s) * 2];
        if (ms != -INFINITY) L += part_ml[(base + s) * 2 + 1] * exp2f(ms - M);
    }
    int tok = seq_start[b];
    for (int d = threadIdx.x; d < DH; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ms = part_ml[(base + s) * 2];
            if (ms != -INFINITY) acc += part_o[(base + s) * DH + d] * exp2f(ms - M);
        }
        out[(size_t)tok * nh * DH + (size_t)head * DH + d] = __float2bfloat16_rn(acc / L);
    }
}

// ------------------------------------------------------------------ prefill
__global__ void __launch_bounds__(THREADS, 3) attn_mma_prefill_kernel(MmaAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Heads along x, row blocks along y with the last (longest) ones first: blocks are handed out x first, so the
    // long blocks of every head start first and the short ones fill the end of the launch.
    const int b = blockIdx.z, head = blockIdx.x;
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b], n_new = p.seq_start[b + 1] - tok0, len_before = p.seq_len_before[b];
    const int t0 = (int)(gridDim.y - 1 - blockIdx.y) * 64;
    if (t0 >= n_new) return;
    Ring<STAGES_PREFILL> ring = make_ring<STAGES_PREFILL>(smem_raw);
    const int kvh = head / (p.nh / p.nkvh);
    const int n_rows = min(64, n_new - t0);
    const int first_pos = len_before + t0, last_pos = first_pos + n_rows - 1;
    const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    const int tile_lo = key_lo / TILE, n_tiles = last_pos / TILE + 1 - tile_lo;

    Source src{p.kpool, p.vpool, p.k_new, p.v_new, p.page_table + (size_t)b * p.table_stride,
               p.ring, p.nkvh, kvh, p.row_stride, tok0, len_before, !p.all_from_cache};
    for (int i = 0; i < STAGES_PREFILL; ++i) {
        if (i < n_tiles) issue_tile(src, tile_lo + i, key_lo, last_pos, ring.stage(i), tid);
        cp_async_commit();
    }

    // this thread's two query rows
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    uint32_t qf[KSTEPS][4];
    load_q(qf, [&](int r) -> const bf16* {
        int row = warp * 16 + r;
        return row < n_rows ? p.q + (size_t)(tok0 + t0 + row) * p.row_stride + (size_t)head * DH : nullptr; }, lane);
    const int hi0 = first_pos + r0, hi1 = first_pos + r1;          // causal: keys up to the row's own position
    const int lo0 = p.window > 0 ? max(0, hi0 - p.window + 1) : 0, lo1 = p.window > 0 ? max(0, hi1 - p.window + 1) : 0;
    const int warp_hi = first_pos + warp * 16 + 15;                  // last position any row of this warp sees
    const int warp_lo = p.window > 0 ? max(0, first_pos + warp * 16 - p.window + 1) : 0;
    float o[DTILES][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    const float scale_log2 = p.scale * 1.4426950408889634f;

    for (int i = 0; i < n_tiles; ++i) {
        cp_async_wait<STAGES_PREFILL - 1>();
        __syncthreads();
        zero_unfetched(ring.stage_ptr(i), tile_lo + i, key_lo, last_pos, tid);
        int p0 = (tile_lo + i) * TILE;
        if (p0 <= warp_hi && p0 + TILE - 1 >= warp_lo) {             // the tile holds a key some row of the warp sees
            // every key of the tile visible to every row of the warp (most tiles of a causal prompt): no masks
            const bool all_visible = p0 + TILE - 1 <= first_pos + warp * 16 &&
                                     (p.window <= 0 || p0 >= first_pos + warp * 16 + 15 - p.window + 1);
            if (all_visible) tile_step<8, false>(qf, o, m, l, ring.stage(i), 0, p0, lo0, hi0, lo1, hi1, scale_log2, lane);
            else tile_step<8, true>(qf, o, m, l, ring.stage(i), 0, p0, lo0, hi0, lo1, hi1, scale_log2, lane);
        }
        __syncthreads();
        if (i + STAGES_PREFILL < n_tiles) issue_tile(src, tile_lo + i + STAGES_PREFILL, key_lo, last_pos, ring.stage(i + STAGES_PREFILL), tid);
        cp_async_commit();
    }
    cp_async_wait<0>();
    const int c = (lane & 3) * 2;
    if (r0 < n_rows) {
        float inv = 1.0f / l[0];
        bf16* dst = p.out + (size_t)(tok0 + t0 + r0) * p.nh * DH + (size_t)head * DH + c;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][0] * inv, o[d][1] * inv);
    }
    if (r1 < n_rows) {
        float inv = 1.0f / l[1];
        bf16* dst = p.out + (size_t)(tok0 + t0 + r1) * p.nh * DH + (size_t)head * DH + c;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2] * inv, o[d][3] * inv);
    }
}

template <int WHICH, typename K>       // WHICH tells the kernels apart: they share one function type
int configure(K kernel, int smem) {
    static bool done = false;
    if (!done && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    done = true;
    return 0;
}

bool aligned_ok(const MmaAttnParams& p) {
    return !(((uintptr_t)p.q | (uintptr_t)p.kpool | (uintptr_t)p.vpool | (uintptr_t)p.out) & 15) && p.row_stride % 8 == 0 &&
           p.nkvh > 0 && p.nh % p.nkvh == 0;
}

}  // namespace

LLB_API int llb_attn_mma_prefill(MmaAttnParams p, int B, int max_new, cudaStream_t stream) {
    if (B == 0 || max_new == 0) return 0;
    if (!aligned_ok(p)) return (int)cudaErrorInvalidValue;
    dim3 grid(p.nh, (max_new + 63) / 64, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    int rc = configure<0>(attn_mma_prefill_kernel, smem_bytes(STAGES_PREFILL));
    if (rc) return rc;
    llb_launch(attn_mma_prefill_kernel, grid, dim3(THREADS), smem_bytes(STAGES_PREFILL), stream, p);
    return llb_status();
}

// How many clusters of `size` blocks of the decode kernel the device can hold at once (0: that size cannot be launched).
LLB_API int llb_attn_mma_decode_max_clusters(int size) {
    auto kernel = attn_mma_decode_kernel<STAGES>;
    const int smem = smem_bytes_decode(STAGES);
    if (configure<1>(kernel, smem)) return 0;
    if (size > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    llb_prefer_max_shared((const void*)kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size, 1, 1);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

LLB_DEFINE_SET_STAMPS

LLB_API int llb_attn_mma_decode(MmaAttnParams p, int B, cudaStream_t stream) {
    if (B == 0) return 0;
    if (!aligned_ok(p) || p.n_splits < 1 || p.n_splits > 64) return (int)cudaErrorInvalidValue;
    if (p.cluster && p.n_splits > MAX_CLUSTER) return (int)cudaErrorInvalidValue;
    int G = p.nh / p.nkvh;
    dim3 grid(p.n_splits, p.nkvh * ((G + 15) / 16), B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    auto kernel = attn_mma_decode_kernel<STAGES>;
    const int smem = smem_bytes_decode(STAGES);
    int rc = configure<1>(kernel, smem);
    if (rc) return rc;
    if (p.cluster && p.n_splits > 8) {
        static bool allowed = false;
        if (!allowed) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return (int)e;
            allowed = true;
        }
    }
    if (p.cluster && p.n_splits > 1) {
        llb_prefer_max_shared((const void*)kernel);
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
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = (unsigned)p.n_splits;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        cudaLaunchKernelEx(&cfg, kernel, p);
    } else {
        llb_launch(kernel, grid, dim3(THREADS), smem, stream, p);
    }
    rc = llb_status();
    if (rc == 0 && p.n_splits > 1 && !p.cluster) {
        llb_launch(attn_mma_combine_kernel, dim3(p.nh, B), dim3(128), 0, stream, p.out, p.part_o, p.part_ml, p.seq_start, p.nh, p.n_splits);
        rc = llb_status();
    }
    return rc;
}
