// Row-wise and element-wise kernels of the decoder: embedding gather, residual add fused with
// RMSNorm, half-split rotary encoding fused with the append to the paged cache, SwiGLU.
//
// Conventions: the residual stream is float32 in both precisions; activations that feed a
// matrix product have the model's activation dtype; sums of squares, the reciprocal root, the
// rotation and the residual sum are float32.  Formulas follow xsmccc/llaisys' CPU operators
// (src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34, src/ops/rope/cpu/rope_cpu.cpp:16-46,
// src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21, src/ops/embedding/cpu/embedding_cpu.cpp:16-22).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V, int* err) {
    llb_grid_dependency_sync();
    int t = blockIdx.x;
    int id = ids[t];
    bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicExch(err, 1);
    const TW* row = table + (size_t)(ok ? id : 0) * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x)
        out[(size_t)t * H + j] = ok ? to_f32(row[j]) : 0.f;
}

LLB_API int llb_embedding(float* out, const void* table, int table_dtype, const int* ids, int T,
                          int H, int V, int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_DISPATCH_DTYPE(table_dtype, TW,
        llb_launch(embedding_kernel<TW>, dim3(T), dim3(256), 0, stream, out, (const TW*)table, ids, H, V, err));
    return llb_status();
}

// ------------------------------------------------------------------ token ids that stay on the device
// dst[i] = src[idx[i]] and dst[idx[i]] = src[i]: the last sampled token of every cache slot is kept in a table
// on the device, written after sampling and read by the next step, so that the next step can be launched
// before the host has seen the tokens.
__global__ void gather_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ idx, int n) {
    llb_grid_dependency_sync();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[idx[i]];
}
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ src, int n) {
    llb_grid_dependency_sync();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[idx[i]] = src[i];
}
LLB_API int llb_gather_i32(int* dst, const int* src, const int* idx, int n, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(gather_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, dst, src, idx, n);
    return llb_status();
}
LLB_API int llb_scatter_i32(int* dst, const int* idx, const int* src, int n, cudaStream_t stream) {
    if (n == 0) return 0;
    llb_launch(scatter_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, dst, idx, src, n);
    return llb_status();
}

// ------------------------------------------------------------------ residual add + RMSNorm
// Row r of the output is norm(residual[src] + sum_p delta[p][src]) with src = rows ? rows[r] : r.
// When write_back is set the summed row replaces residual[src] (never together with `rows`).
template <typename TD, typename TW, typename TO, int PER>     // PER > 0: H <= PER * 256 and the row lives in registers
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_part, size_t part_stride,
                   const TW* __restrict__ weight, TO* __restrict__ out, const int* __restrict__ rows, int H,
                   float eps, int write_back) {
    extern __shared__ float rowbuf[];          // H floats when PER == 0
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x;
    float x[PER > 0 ? PER : 1], w[PER > 0 ? PER : 1];
    if (PER > 0) {                             // the norm weight depends on no earlier kernel: fetch it first
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            w[i] = (j < H && out) ? to_f32(weight[j]) : 0.f;
        }
    }
    llb_grid_dependency_sync();
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * H;
    float ss = 0.f;
    if (PER > 0) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            x[i] = j < H ? res[j] : 0.f;
        }
        if (delta) {
            // the partial sums are added to one another first, then to the residual, as in the general path
            float d[PER > 0 ? PER : 1];
#pragma unroll
            for (int i = 0; i < PER; ++i) d[i] = 0.f;
            for (int p = 0; p < n_part; ++p) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    int j = tid + i * 256;
                    if (j < H) d[i] += to_f32(delta[p * part_stride + src * H + j]);
                }
            }
#pragma unroll
            for (int i = 0; i < PER; ++i) x[i] += d[i];
            if (write_back) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    int j = tid + i * 256;
                    if (j < H) res[j] = x[i];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) ss += x[i] * x[i];
    } else {
        for (int j = tid; j < H; j += 256) {
            float v = res[j];
            if (delta) {
                float d = 0.f;
                for (int p = 0; p < n_part; ++p) d += to_f32(delta[p * part_stride + src * H + j]);
                v += d;
                if (write_back) res[j] = v;
            }
            rowbuf[j] = v;
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    const int lane = tid & 31, wp = tid >> 5;
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    if (!out) return;
    if (PER > 0) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int j = tid + i * 256;
            if (j < H) out[(size_t)r * H + j] = from_f32<TO>(x[i] * w[i] * inv);
        }
    } else {
        for (int j = tid; j < H; j += 256)
            out[(size_t)r * H + j] = from_f32<TO>(rowbuf[j] * to_f32(weight[j]) * inv);
    }
}

// The same for the common case of the bfloat16 path (bfloat16 delta, weight and output, a width that is a multiple
// of 8 up to 8192, 16-byte aligned rows): a thread owns groups of eight consecutive columns, so that every access is a
// 16-byte one (two for the float32 residual).  Sums are formed in the same order as above.
template <int GROUPS>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ delta, int n_part, size_t part_stride,
                       const bf16* __restrict__ weight, bf16* __restrict__ out, const int* __restrict__ rows, int H,
                       float eps, int write_back) {
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, n_groups = H >> 3;
    uint4 w[GROUPS];
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {         // the norm weight depends on no earlier kernel: fetch it first
        const int gidx = tid + i * 256;
        w[i] = (gidx < n_groups && out) ? *reinterpret_cast<const uint4*>(weight + gidx * 8) : make_uint4(0, 0, 0, 0);
    }
    llb_grid_dependency_sync();
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * H;
    float x[GROUPS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {
        const int gidx = tid + i * 256;
        if (gidx < n_groups) {
            const float4 a = *reinterpret_cast<const float4*>(res + gidx * 8), b = *reinterpret_cast<const float4*>(res + gidx * 8 + 4);
            x[i][0] = a.x; x[i][1] = a.y; x[i][2] = a.z; x[i][3] = a.w; x[i][4] = b.x; x[i][5] = b.y; x[i][6] = b.z; x[i][7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] = 0.f;
        }
    }
    if (delta) {
#pragma unroll
        for (int i = 0; i < GROUPS; ++i) {
            const int gidx = tid + i * 256;
            if (gidx >= n_groups) continue;
            float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < n_part; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(delta + q * part_stride + src * H + gidx * 8);
                const bf16* e8 = reinterpret_cast<const bf16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) d[e] += to_f32(e8[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] += d[e];
            if (write_back) {
                *reinterpret_cast<float4*>(res + gidx * 8) = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
                *reinterpret_cast<float4*>(res + gidx * 8 + 4) = make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < GROUPS; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[i][e] * x[i][e];
    ss = warp_sum(ss);
    const int lane = tid & 31, wp = tid >> 5;
    if (lane == 0) red[wp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    if (!out) return;
#pragma unroll
    for (int i = 0; i < GROUPS; ++i) {
        const int gidx = tid + i * 256;
        if (gidx >= n_groups) continue;
        const bf16* w8 = reinterpret_cast<const bf16*>(&w[i]);
        uint4 o;
        bf16* o8 = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = from_f32<bf16>(x[i][e] * to_f32(w8[e]) * inv);
        *reinterpret_cast<uint4*>(out + (size_t)r * H + gidx * 8) = o;
    }
}

// The same once more for many rows (prefill): a warp owns a row, a lane G groups of eight columns 256 columns apart, so
// a row needs no barrier of the block and no shared memory, every load of a lane is in flight at once, and eight rows
// share a block (a block per row is 2,048 blocks of which a quarter run as a second, partial wave).
template <int G>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ residual, const bf16* __restrict__ delta, int n_part, size_t part_stride,
                        const bf16* __restrict__ weight, bf16* __restrict__ out, int R, int H, float eps) {
    const int lane = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
    uint4 w[G];
#pragma unroll
    for (int i = 0; i < G; ++i) w[i] = *reinterpret_cast<const uint4*>(weight + (lane + i * 32) * 8);      // depends on no earlier kernel
    llb_grid_dependency_sync();
    if (r >= R) return;
    float* res = residual + (size_t)r * H;
    float x[G][8];
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int c = (lane + i * 32) * 8;
        const float4 a = *reinterpret_cast<const float4*>(res + c), b = *reinterpret_cast<const float4*>(res + c + 4);
        x[i][0] = a.x; x[i][1] = a.y; x[i][2] = a.z; x[i][3] = a.w; x[i][4] = b.x; x[i][5] = b.y; x[i][6] = b.z; x[i][7] = b.w;
    }
    if (delta) {
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const int c = (lane + i * 32) * 8;
            float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < n_part; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(delta + q * part_stride + (size_t)r * H + c);
                const bf16* e8 = reinterpret_cast<const bf16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) d[e] += to_f32(e8[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[i][e] += d[e];
            *reinterpret_cast<float4*>(res + c) = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
            *reinterpret_cast<float4*>(res + c + 4) = make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[i][e] * x[i][e];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const bf16* w8 = reinterpret_cast<const bf16*>(&w[i]);
        uint4 o;
        bf16* o8 = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = from_f32<bf16>(x[i][e] * to_f32(w8[e]) * inv);
        *reinterpret_cast<uint4*>(out + (size_t)r * H + (lane + i * 32) * 8) = o;
    }
}

template <typename TD, typename TW>
static int add_rmsnorm_out(float* residual, const void* delta, int n_part, size_t part_stride,
                           const void* weight, void* out, int out_dtype, const int* rows, int R,
                           int H, float eps, int write_back, cudaStream_t stream) {
    size_t smem = (size_t)H * sizeof(float);
    LLB_DISPATCH_DTYPE(out_dtype, TO, {
        if (H <= 8 * 256) {
            llb_launch(add_rmsnorm_kernel<TD, TW, TO, 8>, dim3(R), dim3(256), 0, stream, residual, (const TD*)delta,
                       n_part, part_stride, (const TW*)weight, (TO*)out, rows, H, eps, write_back);
        } else {
            auto k = add_rmsnorm_kernel<TD, TW, TO, 0>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            llb_launch(k, dim3(R), dim3(256), smem, stream, residual, (const TD*)delta, n_part, part_stride,
                       (const TW*)weight, (TO*)out, rows, H, eps, write_back);
        }
    });
    return llb_status();
}

LLB_API int llb_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_part,
                            long long part_stride, const void* weight, int weight_dtype, void* out,
                            int out_dtype, const int* rows, int R, int H, float eps,
                            int write_back, cudaStream_t stream) {
    if (R == 0) return 0;
    if ((size_t)H * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (rows && write_back) return (int)cudaErrorInvalidValue;
    // the bfloat16 case with 16-byte accesses
    if ((!delta || delta_dtype == LLB_BF16) && weight_dtype == LLB_BF16 && (!out || out_dtype == LLB_BF16) && H % 8 == 0 &&
        H <= 8192 && part_stride % 8 == 0 &&
        !(((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15)) {
        // many whole rows, a width of G * 256 columns: a warp per row
        if (R >= 256 && !rows && out && write_back && H % 256 == 0 && H <= 4096) {
#define LLB_NW(G) case G: llb_launch(add_rmsnorm_warp_kernel<G>, dim3((R + 7) / 8), dim3(256), 0, stream, residual, (const bf16*)delta, \
                                     n_part, (size_t)part_stride, (const bf16*)weight, (bf16*)out, R, H, eps); return llb_status()
            switch (H / 256) {
                LLB_NW(1); LLB_NW(2); LLB_NW(3); LLB_NW(4); LLB_NW(5); LLB_NW(6); LLB_NW(7); LLB_NW(8);
                LLB_NW(9); LLB_NW(10); LLB_NW(11); LLB_NW(12); LLB_NW(13); LLB_NW(14); LLB_NW(15); LLB_NW(16);
            }
#undef LLB_NW
        }
#define LLB_NV(G) llb_launch(add_rmsnorm_vec_kernel<G>, dim3(R), dim3(256), 0, stream, residual, (const bf16*)delta, n_part, \
                             (size_t)part_stride, (const bf16*)weight, (bf16*)out, rows, H, eps, write_back)
        if (H <= 2048) LLB_NV(1);
        else if (H <= 4096) LLB_NV(2);
        else LLB_NV(4);
#undef LLB_NV
        return llb_status();
    }
    if (!delta) delta_dtype = LLB_F32;
    LLB_DISPATCH_DTYPE(delta_dtype, TD, {
        LLB_DISPATCH_DTYPE(weight_dtype, TW, {
            return add_rmsnorm_out<TD, TW>(residual, delta, n_part, (size_t)part_stride, weight, out,
                                           out_dtype, rows, R, H, eps, write_back, stream);
        });
    });
    return llb_status();
}

// ------------------------------------------------------------------ plain residual add
// residual[t] += sum_p delta[p][t]  (used where no norm follows).
template <typename TD>
__global__ void add_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_part,
                           size_t part_stride, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = 0.f;
    for (int p = 0; p < n_part; ++p) d += to_f32(delta[p * part_stride + i]);
    residual[i] += d;
}

LLB_API int llb_residual_add(float* residual, const void* delta, int delta_dtype, int n_part,
                             long long part_stride, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_DISPATCH_DTYPE(delta_dtype, TD,
        llb_launch(add_kernel<TD>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                   residual, (const TD*)delta, n_part, (size_t)part_stride, (size_t)n));
    return llb_status();
}

// ------------------------------------------------------------------ rotary + cache append
// qkv is the packed projection output [T, row_stride]: nh query heads, then nkvh key heads,
// then nkvh value heads, each of dh elements.  With ROPE the query and key heads are rotated in
// place (half-split pairs (j, j + dh/2), angle from the float32 cos/sin table built in double
// precision on the host).  With APPEND the (rotated) keys and the values of each token are
// written to the token's row of the paged cache.  A window layer keeps a ring of `ring` pages:
// tokens whose page would be overwritten within the same step are skipped.
template <typename T, bool ROPE, bool APPEND>
__global__ void rope_append_kernel(T* __restrict__ qkv, int row_stride, int nh, int nkvh, int dh,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   int table_rows, const int* __restrict__ tok_pos,
                                   const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_len_before,
                                   T* __restrict__ kpool, T* __restrict__ vpool,
                                   const int* __restrict__ page_table, int table_stride, int ring,
                                   int* err) {
    llb_grid_dependency_sync();
    int t = blockIdx.x;
    int pos = tok_pos[t];
    T* row = qkv + (size_t)t * row_stride;
    int half = dh >> 1;
    const int* table = nullptr;
    bool store = false;
    if (APPEND) {
        int s = tok_seq[t];
        table = page_table + (size_t)s * table_stride;
        int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = (pos / LLB_PAGE) + ring > (last / LLB_PAGE);
    }
    if (ROPE) {
        if (pos < 0 || pos >= table_rows) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            return;
        }
        int n_rot = (nh + nkvh) * half;
        for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
            int h = i / half, j = i - h * half;
            float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
            T* x = row + h * dh;
            float a = to_f32(x[j]), b = to_f32(x[j + half]);
            T ya = from_f32<T>(a * c - b * s), yb = from_f32<T>(b * c + a * s);
            x[j] = ya;
            x[j + half] = yb;
            if (APPEND && store && h >= nh) {
                size_t o = paged_row(table, ring, pos, h - nh, nkvh, dh);
                kpool[o + j] = ya;
                kpool[o + j + half] = yb;
            }
        }
    } else if (APPEND && store) {
        for (int i = threadIdx.x; i < nkvh * dh; i += blockDim.x) {
            int h = i / dh, j = i - h * dh;
            kpool[paged_row(table, ring, pos, h, nkvh, dh) + j] = row[(nh + h) * dh + j];
        }
    }
    if (APPEND && store) {
        for (int i = threadIdx.x; i < nkvh * dh; i += blockDim.x) {
            int h = i / dh, j = i - h * dh;
            vpool[paged_row(table, ring, pos, h, nkvh, dh) + j] = row[(nh + nkvh + h) * dh + j];
        }
    }
}

// The same for bfloat16 rows whose head size is a multiple of 16 and whose rows start on 16-byte boundaries: a
// thread handles eight consecutive pairs (two 16-byte pieces of a head), so every access is a 16-byte one.
template <bool ROPE, bool APPEND>
__global__ void __launch_bounds__(128)
rope_append_vec_kernel(bf16* __restrict__ qkv, int row_stride, int nh, int nkvh, int dh,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_len_before,
                       bf16* __restrict__ kpool, bf16* __restrict__ vpool, const int* __restrict__ page_table,
                       int table_stride, int ring, int* err) {
    // The step's index arrays reach the device by a copy that has ended before the step's first kernel starts, and the
    // rotation tables are older still, so they are read while the kernel before this one may still be running; its
    // output, the rows of qkv, only behind the dependency.
    const int t = blockIdx.x, pos = tok_pos[t], half = dh >> 1, vec_per_half = half >> 3;
    bf16* row = qkv + (size_t)t * row_stride;
    bool store = false;
    size_t page_base = 0;                     // element offset of the token's row of kv head 0 in the pools
    if (APPEND) {
        const int s = tok_seq[t];
        const int* table = page_table + (size_t)s * table_stride;
        const int last = seq_len_before[s] + (seq_start[s + 1] - seq_start[s]) - 1;
        store = (pos / LLB_PAGE) + ring > (last / LLB_PAGE);
        if (store) page_base = paged_row(table, ring, pos, 0, nkvh, dh);
    }
    if (ROPE && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    const size_t head_step = (size_t)LLB_PAGE * dh;            // from one kv head's row to the next one's
    // the angles of this thread's first work item
    float4 pc0 = {}, pc1 = {}, ps0 = {}, ps1 = {};
    if (ROPE && (int)threadIdx.x < (nh + nkvh) * vec_per_half) {
        const int j = ((int)threadIdx.x % vec_per_half) * 8;
        pc0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
        pc1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
        ps0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
        ps1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
    }
    llb_grid_dependency_sync();
    // work items: (nh + nkvh) heads x vec_per_half pieces of rotation (or key copy), then nkvh x 2 vec_per_half of values
    const int n_rot = (nh + nkvh) * vec_per_half, n_val = APPEND && store ? nkvh * 2 * vec_per_half : 0;
    for (int i = threadIdx.x; i < n_rot + n_val; i += blockDim.x) {
        if (i < n_rot) {
            const int h = i / vec_per_half, j = (i - h * vec_per_half) * 8;
            if (!ROPE && !(APPEND && store && h >= nh)) continue;
            bf16* x = row + h * dh;
            uint4 lo = *reinterpret_cast<const uint4*>(x + j), hi = *reinterpret_cast<const uint4*>(x + j + half);
            if (ROPE) {
                float4 c0 = pc0, c1 = pc1, s0 = ps0, s1 = ps1;
                if (i != (int)threadIdx.x) {
                    c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
                    c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
                    s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
                    s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
                }
                const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                bf16* a = reinterpret_cast<bf16*>(&lo);
                bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float av = to_f32(a[e]), bv = to_f32(b[e]);
                    a[e] = from_f32<bf16>(av * c[e] - bv * sn[e]);
                    b[e] = from_f32<bf16>(bv * c[e] + av * sn[e]);
                }
                *reinterpret_cast<uint4*>(x + j) = lo;
                *reinterpret_cast<uint4*>(x + j + half) = hi;
            }
            if (APPEND && store && h >= nh) {
                const size_t o = page_base + (size_t)(h - nh) * head_step;
                *reinterpret_cast<uint4*>(kpool + o + j) = lo;
                *reinterpret_cast<uint4*>(kpool + o + j + half) = hi;
            }
        } else {
            const int v = i - n_rot, h = v / (2 * vec_per_half), j = (v - h * 2 * vec_per_half) * 8;
            *reinterpret_cast<uint4*>(vpool + page_base + (size_t)h * head_step + j) =
                *reinterpret_cast<const uint4*>(row + (nh + nkvh + h) * dh + j);
        }
    }
}

template <typename TT>
static void launch_rope_append(TT* qkv, int T, int row_stride, int nh, int nkvh, int dh, int do_rope,
                               const float* cos_t, const float* sin_t, int table_rows,
                               const int* tok_pos, int do_append, const int* tok_seq,
                               const int* seq_start, const int* seq_len_before, TT* kpool, TT* vpool,
                               const int* page_table, int table_stride, int ring, int* err,
                               cudaStream_t stream) {
#define LLB_RA(R, A)                                                                          \
    llb_launch(rope_append_kernel<TT, R, A>, dim3(T), dim3(128), 0, stream,                   \
        qkv, row_stride, nh, nkvh, dh, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, \
        seq_len_before, kpool, vpool, page_table, table_stride, ring, err)
    if (do_rope && do_append) LLB_RA(true, true);
    else if (do_rope) LLB_RA(true, false);
    else if (do_append) LLB_RA(false, true);
#undef LLB_RA
}

// bfloat16 with 16-byte pieces where sizes and addresses allow it
static bool rope_vec_ok(const void* qkv, int row_stride, int dh, const void* cos_t, const void* sin_t, const void* kpool,
                        const void* vpool) {
    return dh % 16 == 0 && row_stride % 8 == 0 &&
           !(((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)kpool | (uintptr_t)vpool) & 15);
}
static void launch_rope_append_vec(bf16* qkv, int T, int row_stride, int nh, int nkvh, int dh, int do_rope,
                                   const float* cos_t, const float* sin_t, int table_rows, const int* tok_pos,
                                   int do_append, const int* tok_seq, const int* seq_start, const int* seq_len_before,
                                   bf16* kpool, bf16* vpool, const int* page_table, int table_stride, int ring, int* err,
                                   cudaStream_t stream) {
#define LLB_RAV(R, A)                                                                         \
    llb_launch(rope_append_vec_kernel<R, A>, dim3(T), dim3(128), 0, stream,                   \
        qkv, row_stride, nh, nkvh, dh, cos_t, sin_t, table_rows, tok_pos, tok_seq, seq_start, \
        seq_len_before, kpool, vpool, page_table, table_stride, ring, err)
    if (do_rope && do_append) LLB_RAV(true, true);
    else if (do_rope) LLB_RAV(true, false);
    else if (do_append) LLB_RAV(false, true);
#undef LLB_RAV
}

LLB_API int llb_rope_append(void* qkv, int dtype, int T, int row_stride, int nh, int nkvh, int dh,
                            int do_rope, const float* cos_t, const float* sin_t, int table_rows,
                            const int* tok_pos, int do_append, const int* tok_seq,
                            const int* seq_start, const int* seq_len_before, void* kpool,
                            void* vpool, const int* page_table, int table_stride, int ring,
                            int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    if (dh % 2) return (int)cudaErrorInvalidValue;
    if (dtype == LLB_BF16 && rope_vec_ok(qkv, row_stride, dh, cos_t, sin_t, kpool, vpool)) {
        launch_rope_append_vec((bf16*)qkv, T, row_stride, nh, nkvh, dh, do_rope, cos_t, sin_t, table_rows, tok_pos,
                               do_append, tok_seq, seq_start, seq_len_before, (bf16*)kpool, (bf16*)vpool, page_table,
                               table_stride, ring, err, stream);
        return llb_status();
    }
    LLB_DISPATCH_DTYPE(dtype, TT,
        launch_rope_append<TT>((TT*)qkv, T, row_stride, nh, nkvh, dh, do_rope, cos_t, sin_t,
                               table_rows, tok_pos, do_append, tok_seq, seq_start, seq_len_before,
                               (TT*)kpool, (TT*)vpool, page_table, table_stride, ring, err, stream));
    return llb_status();
}

// ------------------------------------------------------------------ SwiGLU
// gate_up is [T, 2I] with the gate columns first; out[t, i] = up * gate / (1 + exp(-gate)).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int I, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t t = i / I;
    int c = (int)(i - t * I);
    float g = to_f32(gate_up[t * 2 * I + c]);
    float u = to_f32(gate_up[t * 2 * I + I + c]);
    out[i] = from_f32<T>(u * (g / (1.0f + expf(-g))));
}

LLB_API int llb_swiglu(void* out, const void* gate_up, int dtype, int T, int I, cudaStream_t stream) {
    size_t n = (size_t)T * I;
    if (n == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT,
        llb_launch(swiglu_kernel<TT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TT*)out, (const TT*)gate_up, I, n));
    return llb_status();
}

// ------------------------------------------------------------------ the same on dense operands
// out = up * gate / (1 + exp(-gate)) and c = a + b on dense tensors of one dtype: the operators
// swiglu and add of xsmccc/llaisys (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21, src/ops/add/cpu/add_cpu.cpp:8-16)
// as the op-level interface exposes them; float32 arithmetic, one rounding at the output.
template <typename T, bool SWIGLU>
__global__ void dense_binary_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n) {
    llb_grid_dependency_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x = to_f32(a[i]), y = to_f32(b[i]);
    out[i] = from_f32<T>(SWIGLU ? y * (x / (1.0f + expf(-x))) : x + y);
}

// op 0: out = a + b;  op 1: out = b * a / (1 + exp(-a))  (a the gate, b the up projection)
LLB_API int llb_dense_binary(void* out, const void* a, const void* b, int dtype, long long n, int op, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (op != 0 && op != 1) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    LLB_DISPATCH_DTYPE(dtype, TT, {
        if (op == 0) llb_launch(dense_binary_kernel<TT, false>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const TT*)a, (const TT*)b, (size_t)n);
        else llb_launch(dense_binary_kernel<TT, true>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const TT*)a, (const TT*)b, (size_t)n);
    });
    return llb_status();
}

// ------------------------------------------------------------------ misc
LLB_API const char* llb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
