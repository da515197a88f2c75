// Shared declarations of the CUDA modules: dtype codes, conversions, the paged key/value
// cache addressing, and the launch-status convention of the C entry points.
//
// Every exported function is `extern "C" int llb_*(..., cudaStream_t stream)`; it returns 0 or
// the cudaError_t of the launch, never allocates, and works on the stream it is given.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define LLB_API extern "C" __attribute__((visibility("default")))

enum { LLB_F32 = 0, LLB_BF16 = 1 };

// Tokens of a cache page.  Attention kernels walk keys in tiles of one page.
constexpr int LLB_PAGE = 64;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- cycle stamps: a build with -DLLB_STAMPS=1 records clock64() at a few places of a kernel, per block, so that
// the inside of a short kernel can be read while it runs in its real place in a step (python bench.py --stamps ...).
// llb_set_stamps(buffer, blocks) switches them on for launches of exactly `blocks` blocks (a module's kernels are
// launched with several grids in a step; 0: every launch; the buffer holds LLB_STAMP_SLOTS values for every block of the
// largest launch that stamps); a null buffer switches them off.  Without the definition the macro is empty and the kernels are what they are without it.
#ifdef LLB_STAMPS
constexpr int LLB_STAMP_SLOTS = 16;
static __device__ long long* llb_stamps_buf = nullptr;
static __device__ unsigned int llb_stamps_blocks = 0;
// at the top of a kernel: where this block's stamps go (null: nowhere), read once so that a stamp is a clock read and a store
#define LLB_STAMPS_BEGIN()                                                                                            \
    long long* llb_sp = nullptr;                                                                                      \
    {                                                                                                                 \
        long long* const llb_b = llb_stamps_buf;                                                                      \
        const unsigned int llb_n = llb_stamps_blocks;                                                                 \
        if (llb_b && (llb_n == 0 || gridDim.x * gridDim.y * gridDim.z == llb_n))                                      \
            llb_sp = llb_b + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * LLB_STAMP_SLOTS; \
    }
// (the clock is read by an instruction that the compiler may not move across the memory operations and barriers around it)
#define LLB_STAMP(i)                                                                                                  \
    do {                                                                                                              \
        if (llb_sp) {                                                                                                 \
            long long llb_t;                                                                                          \
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(llb_t) : : "memory");                                       \
            llb_sp[i] = llb_t;                                                                                        \
        }                                                                                                             \
    } while (0)
#define LLB_DEFINE_SET_STAMPS                                                                                         \
    LLB_API int llb_set_stamps(long long* buf, unsigned int blocks) {                                                  \
        cudaError_t e = cudaMemcpyToSymbol(llb_stamps_blocks, &blocks, sizeof(blocks));                               \
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(llb_stamps_buf, &buf, sizeof(buf));                              \
        return (int)e;                                                                                                \
    }
#else
#define LLB_STAMPS_BEGIN() do { } while (0)
#define LLB_STAMP(i) do { } while (0)
#define LLB_DEFINE_SET_STAMPS
#endif

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// One layer's keys or values live in pages of LLB_PAGE tokens: pool[page][kv_head][token][dim].
// A sequence's page table lists its physical pages; logical page lp sits at entry lp % ring
// (ring is the table length for layers that keep every key, and the ring length for layers
// that keep a window).
__device__ __forceinline__ size_t paged_row(const int* table, int ring, int pos, int kvh,
                                            int n_kv_heads, int head_dim) {
    int lp = pos / LLB_PAGE;
    int page = table[lp % ring];
    return (((size_t)page * n_kv_heads + kvh) * LLB_PAGE + (pos % LLB_PAGE)) * (size_t)head_dim;
}

static inline int llb_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch
// Kernels of a step follow one another on one stream, each a few microseconds long, so the gap
// between them matters.  Every kernel is launched with programmatic stream serialization: it may
// start (be scheduled, set up its shared memory, barriers and tensor memory) while its
// predecessor is still running, and calls llb_grid_dependency_sync() before it first touches
// global memory; that call returns when the predecessor has completed and its writes are
// visible.  The same call lets this kernel's successor start early in turn.  LLAISYS_PDL=0 in
// the environment launches the plain way (the device-side call is then a no-op).
__device__ __forceinline__ void llb_grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

#include <stdlib.h>
static inline bool llb_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("LLAISYS_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// All kernels ask for the same split of the SM's L1/shared memory (all of it as shared memory), so
// that an SM never has to drain and reconfigure between two kernels of a step.
static inline void llb_prefer_max_shared(const void* kernel) {
    static const void* seen[256];
    static int n_seen = 0;
    for (int i = 0; i < n_seen; ++i)
        if (seen[i] == kernel) return;
    if (getenv("LLAISYS_CARVEOUT") && getenv("LLAISYS_CARVEOUT")[0] == '0') return;
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (n_seen < 256) seen[n_seen++] = kernel;
}

template <typename... P, typename... A>
static inline void llb_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
    llb_prefer_max_shared((const void*)kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = llb_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

#define LLB_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                   \
        if ((code) == LLB_F32) { typedef float T; __VA_ARGS__; }           \
        else if ((code) == LLB_BF16) { typedef bf16 T; __VA_ARGS__; }      \
        else return (int)cudaErrorInvalidValue;                            \
    } while (0)
