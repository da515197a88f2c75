// Causal grouped-query attention over the paged cache on the CUDA cores, float32 arithmetic.
// It serves the true 32-bit path in both phases and is the reference the tensor-core kernels
// are checked against.  Compiled per head size: -DLLB_HEAD_DIM=<multiple of 2, at most 256>.
//
// Formula (src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112 of xsmccc/llaisys): for a
// query at absolute position p of head h, scores s_t = (q . k_t) * scale over the keys t of kv
// head h / (nh / nkvh) with t <= p; softmax with the maximum subtracted; out = sum_t p_t v_t.
// A window W > 0 (not in that project) further restricts the keys to p - W < t <= p.
//
// Keys are walked in tiles of one cache page with an online softmax, so nothing of size
// [queries, keys] is ever stored.
//
//  * prefill: a block owns 32 consecutive new tokens of one head of one sequence.  Keys at
//    positions before the step come from the cache pages, keys of the step itself from the
//    packed projection output (the cache is appended to afterwards, which lets a window layer
//    keep a ring of pages shorter than the prompt).
//  * decode: one new token per sequence, already appended.  A block owns the query heads that
//    share one kv head and one slice of the key range; slices are merged by llb_attn_combine.
#include "common.cuh"

#ifndef LLB_HEAD_DIM
#error "compile with -DLLB_HEAD_DIM=<head size>"
#endif

constexpr int DH = LLB_HEAD_DIM;
constexpr int ROWS = 32;            // query rows of a block
constexpr int WARPS = 4;
constexpr int RPW = ROWS / WARPS;   // rows of a warp
constexpr int DPL = (DH + 31) / 32; // output dims of a lane

struct AttnParams {
    const void* q;        // packed projections [T, row_stride]; query head h at column h * DH
    const void* k_new;    // the same buffer at its first key column
    const void* v_new;    // the same buffer at its first value column
    int row_stride;
    void* out;            // [T, nh * DH]
    const void* kpool;    // [pages, nkvh, LLB_PAGE, DH]
    const void* vpool;
    const int* page_table;  // [B, table_stride]
    int table_stride;
    int ring;
    const int* seq_start;       // [B + 1] first packed token of each sequence
    const int* seq_len_before;  // [B] tokens in the cache before this step
    int nh, nkvh, window;
    float scale;
    int all_from_cache;   // prefill only: the step's own keys are already in the cache (a call that
                          // reads another call's cache); read nothing from k_new / v_new
    int n_splits;         // decode only
    float* part_o;        // decode only: [B, nh, n_splits, DH]
    float* part_ml;       // decode only: [B, nh, n_splits, 2]
};

template <typename T, bool DECODE>
__global__ void __launch_bounds__(WARPS * 32) attn_kernel(AttnParams p) {
    extern __shared__ float smem[];
    float* Qs = smem;                        // [ROWS][DH]
    float* Ks = Qs + ROWS * DH;              // [LLB_PAGE][DH + 1]
    float* Vs = Ks + LLB_PAGE * (DH + 1);    // [LLB_PAGE][DH]
    float* Ps = Vs + LLB_PAGE * DH;          // [WARPS][LLB_PAGE]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z;
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b];
    const int n_new = p.seq_start[b + 1] - tok0;
    const int len_before = p.seq_len_before[b];
    const int G = p.nh / p.nkvh;
    const int* table = p.page_table + (size_t)b * p.table_stride;

    // ---- the rows of this block: (token, head, position) per row
    int kvh, n_rows, first_pos, last_pos;
    int row_tok0, row_head0;                 // row r: token row_tok0 + (DECODE ? 0 : r), head row_head0 + (DECODE ? r : 0)
    if (DECODE) {
        int chunks = (G + ROWS - 1) / ROWS;
        kvh = blockIdx.y / chunks;
        int c = blockIdx.y - kvh * chunks;
        n_rows = min(ROWS, G - c * ROWS);
        row_head0 = kvh * G + c * ROWS;
        row_tok0 = tok0;
        first_pos = last_pos = len_before;   // n_new == 1
    } else {
        int t0 = blockIdx.x * ROWS;
        if (t0 >= n_new) return;
        n_rows = min(ROWS, n_new - t0);
        row_head0 = blockIdx.y;
        kvh = row_head0 / G;
        row_tok0 = tok0 + t0;
        first_pos = len_before + t0;
        last_pos = first_pos + n_rows - 1;
    }
    const T* qbase = (const T*)p.q;
    for (int i = tid; i < n_rows * DH; i += WARPS * 32) {
        int r = i / DH, d = i - r * DH;
        int tok = row_tok0 + (DECODE ? 0 : r), head = row_head0 + (DECODE ? r : 0);
        Qs[r * DH + d] = to_f32(qbase[(size_t)tok * p.row_stride + head * DH + d]);
    }

    // ---- key tiles of this block
    int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    int tile_lo = key_lo / LLB_PAGE, tile_hi = last_pos / LLB_PAGE + 1;
    if (DECODE) {
        int n_tiles = tile_hi - tile_lo;
        int chunk = (n_tiles + p.n_splits - 1) / p.n_splits;
        tile_lo = tile_lo + blockIdx.x * chunk;
        tile_hi = min(tile_hi, tile_lo + chunk);
    }

    float m[RPW], l[RPW], o[RPW][DPL];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[i][e] = 0.f;
    }

    const T* kpool = (const T*)p.kpool;
    const T* vpool = (const T*)p.vpool;
    const T* knew = (const T*)p.k_new;
    const T* vnew = (const T*)p.v_new;

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        __syncthreads();                     // previous tile fully consumed (and Qs written)
        for (int i = tid; i < LLB_PAGE * DH; i += WARPS * 32) {
            int j = i / DH, d = i - j * DH;
            int kp = tile * LLB_PAGE + j;
            float kv = 0.f, vv = 0.f;
            if (kp >= key_lo && kp <= last_pos) {
                if (!DECODE && !p.all_from_cache && kp >= len_before) {
                    size_t off = (size_t)(tok0 + kp - len_before) * p.row_stride + kvh * DH + d;
                    kv = to_f32(knew[off]);
                    vv = to_f32(vnew[off]);
                } else {
                    size_t off = paged_row(table, p.ring, kp, kvh, p.nkvh, DH) + d;
                    kv = to_f32(kpool[off]);
                    vv = to_f32(vpool[off]);
                }
            }
            Ks[j * (DH + 1) + d] = kv;
            Vs[j * DH + d] = vv;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            int r = warp + i * WARPS;
            if (r >= n_rows) continue;       // uniform within the warp
            int pos = DECODE ? first_pos : first_pos + r;
            int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const float* qr = Qs + r * DH;
            const float* k0 = Ks + lane * (DH + 1);
            const float* k1 = Ks + (lane + 32) * (DH + 1);
            float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
            for (int d = 0; d < DH; ++d) {
                float qv = qr[d];
                s0 = fmaf(qv, k0[d], s0);
                s1 = fmaf(qv, k1[d], s1);
            }
            int kp0 = tile * LLB_PAGE + lane, kp1 = kp0 + 32;
            bool v0 = kp0 >= lo && kp0 <= pos, v1 = kp1 >= lo && kp1 <= pos;
            s0 = v0 ? s0 * p.scale : -INFINITY;
            s1 = v1 ? s1 * p.scale : -INFINITY;
            float m_new = fmaxf(m[i], warp_max(fmaxf(s0, s1)));
            if (m_new == -INFINITY) continue;          // no visible key yet (uniform)
            float alpha = expf(m[i] - m_new);           // exp(-inf) = 0 on the first visible tile
            float p0 = v0 ? expf(s0 - m_new) : 0.f, p1 = v1 ? expf(s1 - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(p0 + p1);
            m[i] = m_new;
            float* ps = Ps + warp * LLB_PAGE;
            __syncwarp();
            ps[lane] = p0;
            ps[lane + 32] = p1;
            __syncwarp();
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int d = lane + e * 32;
                if (d < DH) {
                    float acc = o[i][e] * alpha;
#pragma unroll 8
                    for (int j = 0; j < LLB_PAGE; ++j) acc = fmaf(ps[j], Vs[j * DH + d], acc);
                    o[i][e] = acc;
                }
            }
        }
    }

    // ---- write out
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        int r = warp + i * WARPS;
        if (r >= n_rows) continue;
        int tok = row_tok0 + (DECODE ? 0 : r), head = row_head0 + (DECODE ? r : 0);
        if (!DECODE || p.n_splits == 1) {
            T* out = (T*)p.out + (size_t)tok * p.nh * DH + head * DH;
            float inv = 1.0f / l[i];
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int d = lane + e * 32;
                if (d < DH) out[d] = from_f32<T>(o[i][e] * inv);
            }
        } else {
            size_t slot = ((size_t)b * p.nh + head) * p.n_splits + blockIdx.x;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int d = lane + e * 32;
                if (d < DH) p.part_o[slot * DH + d] = o[i][e];
            }
            if (lane == 0) {
                p.part_ml[slot * 2] = m[i];
                p.part_ml[slot * 2 + 1] = l[i];
            }
        }
    }
}

// Merges the key slices of decode: out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M).
template <typename T>
__global__ void attn_combine_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, const int* __restrict__ seq_start,
                                    int nh, int n_splits) {
    llb_grid_dependency_sync();
    int head = blockIdx.x, b = blockIdx.y;
    size_t base = ((size_t)b * nh + head) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float ms = part_ml[(base + s) * 2];
        if (ms != -INFINITY) L += part_ml[(base + s) * 2 + 1] * expf(ms - M);
    }
    int tok = seq_start[b];
    for (int d = threadIdx.x; d < DH; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ms = part_ml[(base + s) * 2];
            if (ms != -INFINITY) acc += part_o[(base + s) * DH + d] * expf(ms - M);
        }
        out[(size_t)tok * nh * DH + head * DH + d] = from_f32<T>(acc / L);
    }
}

static size_t attn_smem_bytes() {
    return (size_t)(ROWS * DH + LLB_PAGE * (DH + 1) + LLB_PAGE * DH + WARPS * LLB_PAGE) * sizeof(float);
}

template <typename T, bool DECODE>
static int launch_attn(const AttnParams& p, dim3 grid, cudaStream_t stream) {
    auto k = attn_kernel<T, DECODE>;
    size_t smem = attn_smem_bytes();
    static bool configured = false;          // once per instantiation: not repeated inside a graph capture
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    configured = true;
    llb_launch(k, grid, dim3(WARPS * 32), smem, stream, p);
    return llb_status();
}

// Prefill and any step with more than one new token in some sequence.  max_new is the largest
// number of new tokens of a sequence in the batch.
LLB_API int llb_attn_prefill(AttnParams p, int dtype, int B, int max_new, cudaStream_t stream) {
    if (B == 0 || max_new == 0) return 0;
    if (p.nkvh <= 0 || p.nh % p.nkvh) return (int)cudaErrorInvalidValue;
    dim3 grid((max_new + ROWS - 1) / ROWS, p.nh, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, T, return launch_attn<T, false>(p, grid, stream));
    return 0;
}

// Decode: every sequence has exactly one new token, already in the cache.
LLB_API int llb_attn_decode(AttnParams p, int dtype, int B, cudaStream_t stream) {
    if (B == 0) return 0;
    if (p.nkvh <= 0 || p.nh % p.nkvh || p.n_splits < 1) return (int)cudaErrorInvalidValue;
    int G = p.nh / p.nkvh;
    dim3 grid(p.n_splits, p.nkvh * ((G + ROWS - 1) / ROWS), B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    int rc;
    LLB_DISPATCH_DTYPE(dtype, T, {
        rc = launch_attn<T, true>(p, grid, stream);
        if (rc == 0 && p.n_splits > 1) {
            llb_launch(attn_combine_kernel<T>, dim3(p.nh, B), dim3(128), 0, stream,
                       (T*)p.out, (const float*)p.part_o, (const float*)p.part_ml, p.seq_start, p.nh, p.n_splits);
            rc = llb_status();
        }
        return rc;
    });
    return 0;
}
