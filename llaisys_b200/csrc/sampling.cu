// Next-token choice on the device: arg-max, and temperature / top-k / top-p sampling.
//
// xsmccc/llaisys chooses by arg-max only (src/ops/argmax/cpu/argmax_cpu.cpp:14-27: the first
// maximum wins, compared in float32); its generate() takes top_k, top_p and temperature and
// ignores them (python/llaisys/models/qwen2.py:212-219).  The sampling rule here:
//   top_k == 1 or temperature == 0  ->  arg-max;
//   p_i = exp((l_i - max) / temperature);
//   keep the top_k largest (ties: lower index first; top_k <= 0 or >= V keeps all);
//   of these, in descending order (ties: lower index first), keep while the mass before an
//   element is below top_p times the kept mass;
//   draw by inverse CDF over the kept elements in index order with u = uniform(seed, key, step).
// Masses are summed as 40-bit fixed point integers, so every sum is exact and the result does
// not depend on the order in which threads add.
#include "common.cuh"
#include <limits.h>

constexpr int SB = 1024;   // threads of a block; one block per row

__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// splitmix64 finaliser: the uniform of (seed, key, step) is the top 53 bits of
// mix(mix(seed + GOLDEN * (key + 1)) + GOLDEN * (step + 1)).
__host__ __device__ inline uint64_t llb_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline double llb_uniform(uint64_t seed, uint64_t key, uint64_t step) {
    const uint64_t G = 0x9E3779B97F4A7C15ull;
    uint64_t z = llb_mix64(llb_mix64(seed + G * (key + 1)) + G * (step + 1));
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// the best of the block's threads' candidates, in every thread
__device__ ArgMax block_best(ArgMax best, ArgMax* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) red[w] = best;
    __syncthreads();
    if (w == 0) {
        best = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0) red[0] = best;
    }
    __syncthreads();
    best = red[0];
    __syncthreads();
    return best;
}

__device__ ArgMax block_argmax(const float* row, int V, ArgMax* red) {
    ArgMax best = {-INFINITY, INT_MAX};
    for (int i = threadIdx.x; i < V; i += SB) {
        float v = row[i];
        if (v > best.v || best.i == INT_MAX) best = {v, i};     // increasing i: first maximum stays
    }
    return block_best(best, red);
}

__global__ void __launch_bounds__(SB) argmax_kernel(const float* __restrict__ logits, long long ld,
                                                    int V, int* __restrict__ out) {
    __shared__ ArgMax red[32];
    llb_grid_dependency_sync();
    ArgMax b = block_argmax(logits + (size_t)blockIdx.x * ld, V, red);
    if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// Few rows of a wide vocabulary (a decode step: 8 rows of 151,936 logits) leave most SMs without a block when a block
// takes a whole row: 11 us for 4.9 MB.  Here gridDim.x blocks share a row; each leaves its part's first maximum in
// `part`, and the block that finds itself the last of its row (a counter per row, back at zero afterwards) takes the
// best of the parts.  The order in which the blocks finish does not change the result: ties go to the lower index.
constexpr int SPLIT_THREADS = 256, MAX_PARTS = 64;
__global__ void __launch_bounds__(SPLIT_THREADS)
argmax_split_kernel(const float* __restrict__ logits, long long ld, int V, int chunk, ArgMax* __restrict__ part,
                    int* __restrict__ counters, int* __restrict__ out) {
    __shared__ ArgMax red[32];
    __shared__ int s_last;
    llb_grid_dependency_sync();
    const int r = blockIdx.y, c = blockIdx.x, C = gridDim.x, tid = threadIdx.x;
    const int lo = min(V, c * chunk), hi = min(V, lo + chunk);
    const float* row = logits + (size_t)r * ld;
    ArgMax best = {-INFINITY, INT_MAX};
    auto take = [&](float v, int i) { if (v > best.v || best.i == INT_MAX) best = {v, i}; };      // increasing i: first maximum stays
    int done = lo;
    if ((reinterpret_cast<uintptr_t>(row + lo) & 15) == 0) {
        const int n4 = (hi - lo) >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row + lo);
        for (int i = tid; i < n4; i += SPLIT_THREADS) {
            const float4 v = row4[i];
            const int at = lo + 4 * i;
            take(v.x, at); take(v.y, at + 1); take(v.z, at + 2); take(v.w, at + 3);
        }
        done = lo + 4 * n4;
    }
    for (int i = done + tid; i < hi; i += SPLIT_THREADS) take(row[i], i);      // (a thread's indices still increase)
    // block_best() reduces over 32 warps' places: the places of the warps this block does not have stay neutral
    if (tid < 32) red[tid] = {-INFINITY, INT_MAX};
    __syncthreads();
    best = block_best(best, red);
    if (tid == 0) {
        part[(size_t)r * C + c] = best;
        __threadfence();
        s_last = atomicAdd(counters + r, 1) == C - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid < 32) {
        ArgMax b = {-INFINITY, INT_MAX};
        for (int k = tid; k < C; k += 32) {
            const volatile ArgMax* q = part + (size_t)r * C + k;
            ArgMax o = {q->v, q->i};
            if (o.i != INT_MAX) b = b.i == INT_MAX ? o : better(b, o);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other = {__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
            if (other.i != INT_MAX) b = b.i == INT_MAX ? other : better(b, other);
        }
        if (tid == 0) {
            out[r] = b.i;
            counters[r] = 0;
        }
    }
}

LLB_API int llb_argmax(const float* logits, long long ld, int R, int V, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    if (V <= 0) return (int)cudaErrorInvalidValue;
    llb_launch(argmax_kernel, dim3(R), dim3(SB), 0, stream, logits, ld, V, out);
    return llb_status();
}

// The same with `parts` blocks per row (2 to 64): part [R * parts] pairs of (float, int) of scratch, counters [R] ints
// that are zero before the call and zero again after it.
LLB_API int llb_argmax_split(const float* logits, long long ld, int R, int V, int parts, void* part, int* counters, int* out,
                             cudaStream_t stream) {
    if (R == 0) return 0;
    if (V <= 0 || parts < 2 || parts > MAX_PARTS || R > 65535 || !part || !counters) return (int)cudaErrorInvalidValue;
    const int chunk = (((V + parts - 1) / parts) + 3) & ~3;            // whole 16-byte pieces
    llb_launch(argmax_split_kernel, dim3(parts, R), dim3(SPLIT_THREADS), 0, stream, logits, ld, V, chunk, (ArgMax*)part, counters, out);
    return llb_status();
}

// exclusive prefix sum over the block's threads; total returned through *total
__device__ unsigned long long block_excl_scan(unsigned long long v, unsigned long long* sh,
                                              unsigned long long* total) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned long long n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) sh[w] = inc;
    __syncthreads();
    if (w == 0) {
        unsigned long long x = sh[lane], xi = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned long long n = __shfl_up_sync(0xffffffffu, xi, o);
            if (lane >= o) xi += n;
        }
        sh[lane] = xi - x;
        if (lane == 31) sh[32] = xi;
    }
    __syncthreads();
    unsigned long long r = sh[w] + inc - v;
    *total = sh[32];
    __syncthreads();
    return r;
}

__device__ __forceinline__ unsigned long long mass_fp(float logit, float mx, float inv_t) {
    float e = expf((logit - mx) * inv_t);
    if (!(e >= 0.f)) return 0;                                            // NaN
    return (unsigned long long)((double)fminf(e, 1.0f) * 1099511627776.0);   // 2^40
}

__global__ void __launch_bounds__(SB)
sample_kernel(const float* __restrict__ logits, long long ld, int V, int* __restrict__ out,
              float temperature, int top_k, float top_p, unsigned long long seed,
              const int* __restrict__ keys, const int* __restrict__ steps) {
    __shared__ ArgMax red[32];
    __shared__ unsigned int cnt[256];
    __shared__ unsigned long long mass[256];
    __shared__ unsigned long long scan_sh[33];
    __shared__ unsigned int sh_prefix, sh_krem;
    __shared__ unsigned long long sh_acc;
    const float* row = logits + (size_t)blockIdx.x * ld;
    const int tid = threadIdx.x;
    llb_grid_dependency_sync();

    ArgMax top = block_argmax(row, V, red);
    if (top_k == 1 || temperature == 0.f) {
        if (tid == 0) out[blockIdx.x] = top.i;
        return;
    }
    const float mx = top.v, inv_t = 1.0f / temperature;

    // ---- top-k: the k-th largest key and how many of its equals are admitted
    uint32_t kth_key = 0;
    unsigned int ties_k = UINT_MAX;
    if (top_k > 0 && top_k < V) {
        if (tid == 0) { sh_prefix = 0; sh_krem = (unsigned)top_k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) cnt[tid] = 0;
            __syncthreads();
            uint32_t prefix = sh_prefix;
            for (int i = tid; i < V; i += SB) {
                uint32_t k = order_key(row[i]);
                if (shift == 24 || (k >> (shift + 8)) == prefix) atomicAdd(&cnt[(k >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int rem = sh_krem, above = 0;
                int d = 255;
                for (; d > 0; --d) {
                    if (above + cnt[d] >= rem) break;
                    above += cnt[d];
                }
                sh_krem = rem - above;
                sh_prefix = (prefix << 8) | (unsigned)d;
            }
            __syncthreads();
        }
        kth_key = sh_prefix;
        ties_k = sh_krem;
    }

    // ---- kept mass after top-k
    uint32_t cut_key = kth_key;
    unsigned int ties = ties_k;
    unsigned long long kth_mass = mass_fp(key_value(kth_key), mx, inv_t);
    if (top_p < 1.0f) {
        unsigned long long part = 0;
        for (int i = tid; i < V; i += SB) {
            float v = row[i];
            if (order_key(v) > kth_key) part += mass_fp(v, mx, inv_t);
        }
        unsigned long long zk;
        block_excl_scan(part, scan_sh, &zk);
        unsigned int n_eq_kept = ties_k;
        if (ties_k == UINT_MAX) {             // no top-k: every element equal to the minimum key counts
            unsigned long long c = 0;
            for (int i = tid; i < V; i += SB) c += order_key(row[i]) == kth_key;
            unsigned long long tot;
            block_excl_scan(c, scan_sh, &tot);
            n_eq_kept = (unsigned)tot;
        }
        zk += (unsigned long long)n_eq_kept * kth_mass;
        unsigned long long target = (unsigned long long)ceil((double)top_p * (double)zk);
        if (target < 1) target = 1;

        // radix descent by mass: the lowest key whose mass of greater kept keys is below target
        if (tid == 0) { sh_prefix = 0; sh_acc = 0; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) { cnt[tid] = 0; mass[tid] = 0; }
            __syncthreads();
            uint32_t prefix = sh_prefix;
            for (int i = tid; i < V; i += SB) {
                float v = row[i];
                uint32_t k = order_key(v);
                if (k > kth_key && (shift == 24 || (k >> (shift + 8)) == prefix)) {
                    atomicAdd(&cnt[(k >> shift) & 255u], 1u);
                    atomicAdd(&mass[(k >> shift) & 255u], mass_fp(v, mx, inv_t));
                }
            }
            if (tid == 0 && n_eq_kept > 0 && (shift == 24 || (kth_key >> (shift + 8)) == prefix)) {
                atomicAdd(&cnt[(kth_key >> shift) & 255u], n_eq_kept);
                atomicAdd(&mass[(kth_key >> shift) & 255u], (unsigned long long)n_eq_kept * kth_mass);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long running = sh_acc, chosen_acc = sh_acc;
                int chosen = -1;
                for (int d = 255; d >= 0; --d) {
                    if (running >= target) break;
                    if (cnt[d] > 0) { chosen = d; chosen_acc = running; }
                    running += mass[d];
                }
                if (chosen < 0) chosen = 255;
                sh_prefix = (prefix << 8) | (unsigned)chosen;
                sh_acc = chosen_acc;
            }
            __syncthreads();
        }
        cut_key = sh_prefix;
        unsigned long long acc = sh_acc;
        unsigned long long cm = mass_fp(key_value(cut_key), mx, inv_t);
        unsigned long long need = target > acc ? target - acc : 1;
        unsigned long long n_ties_p = cm > 0 ? (need + cm - 1) / cm : (unsigned long long)UINT_MAX;
        if (n_ties_p > UINT_MAX) n_ties_p = UINT_MAX;
        ties = (unsigned)n_ties_p;
        if (cut_key == kth_key && ties > ties_k) ties = ties_k;
        if (ties < 1) ties = 1;
    }
    const unsigned long long cut_mass = mass_fp(key_value(cut_key), mx, inv_t);

    // ---- draw over the kept set in index order; thread t owns one contiguous segment
    const int seg = (V + SB - 1) / SB;
    const int lo = min(V, tid * seg), hi = min(V, lo + seg);
    unsigned long long eq = 0;
    for (int i = lo; i < hi; ++i) eq += order_key(row[i]) == cut_key;
    unsigned long long eq_total;
    unsigned long long eq_base = block_excl_scan(eq, scan_sh, &eq_total);
    unsigned long long seg_mass = 0, rank = eq_base;
    for (int i = lo; i < hi; ++i) {
        float v = row[i];
        uint32_t k = order_key(v);
        if (k > cut_key) seg_mass += mass_fp(v, mx, inv_t);
        else if (k == cut_key) { if (rank < ties) seg_mass += cut_mass; ++rank; }
    }
    unsigned long long total;
    unsigned long long before = block_excl_scan(seg_mass, scan_sh, &total);
    if (total == 0) {                      // every kept mass underflowed: fall back to the maximum
        if (tid == 0) out[blockIdx.x] = top.i;
        return;
    }
    double u = llb_uniform(seed, (unsigned long long)(keys ? keys[blockIdx.x] : blockIdx.x),
                           (unsigned long long)(steps ? steps[blockIdx.x] : 0));
    unsigned long long target = (unsigned long long)(u * (double)total);
    if (target >= total) target = total - 1;
    if (target >= before && target < before + seg_mass) {
        unsigned long long run = before, rk = eq_base;
        int pick = lo;
        for (int i = lo; i < hi; ++i) {
            float v = row[i];
            uint32_t k = order_key(v);
            unsigned long long mfp = 0;
            if (k > cut_key) mfp = mass_fp(v, mx, inv_t);
            else if (k == cut_key) { if (rk < ties) mfp = cut_mass; ++rk; }
            if (mfp > 0 && target < run + mfp) { pick = i; break; }
            run += mfp;
        }
        out[blockIdx.x] = pick;
    }
}

// keys[r], steps[r]: the request number and the count of tokens already drawn for row r; they
// and the seed fix the uniform, so a request's draws do not depend on what else is in the batch.
LLB_API int llb_sample(const float* logits, long long ld, int R, int V, int* out, float temperature,
                       int top_k, float top_p, unsigned long long seed, const int* keys,
                       const int* steps, cudaStream_t stream) {
    if (R == 0) return 0;
    if (V <= 0 || temperature < 0.f || !(top_p > 0.f)) return (int)cudaErrorInvalidValue;
    llb_launch(sample_kernel, dim3(R), dim3(SB), 0, stream, logits, ld, V, out, temperature, top_k, top_p, seed, keys, steps);
    return llb_status();
}

LLB_API double llb_uniform_host(unsigned long long seed, unsigned long long key, unsigned long long step) {
    return llb_uniform(seed, key, step);
}
