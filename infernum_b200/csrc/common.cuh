// Shared device helpers for the sm_100a kernels of this package.
//
// Conventions used by every exported function:
//   * plain C ABI, pointers are device pointers, `stream` is a cudaStream_t
//     passed as void*;
//   * the return value is 0 on success, a positive cudaError_t from the
//     launch, or a negative IB_ERR_* code when the arguments are refused;
//   * nothing is allocated and nothing synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IB_OK 0
#define IB_ERR_BAD_ARG (-1)       // a size or pointer the kernel cannot take
#define IB_ERR_UNSUPPORTED (-2)   // a configuration this build does not cover
#define IB_ERR_TOO_LARGE (-3)     // beyond a stated maximum
#define IB_ERR_NOALLOC_SETUP (-4) // ib_argmax_noalloc: the per-device look-up of its scratch array failed

// Bits of the device-side error word that kernels may set (never trap).
#define IB_FLAG_BAD_TOKEN 1u      // token id outside the vocabulary
#define IB_FLAG_BAD_PAGE 2u       // block-table entry outside the pool
#define IB_FLAG_WAIT_TIMEOUT 4u   // a bounded wait on a barrier gave up
// Which wait gave up: bit 8 + site is set beside IB_FLAG_WAIT_TIMEOUT.
#define IB_SITE_GEMM_PRODUCER 0      // gemm_tcgen05: TMA producer
#define IB_SITE_GEMM_MMA 1           // gemm_tcgen05: MMA issuer
#define IB_SITE_GEMM_EPILOGUE 2      // gemm_tcgen05: epilogue
#define IB_SITE_PAIR_PRODUCER 3      // gemm_tcgen05_2cta: TMA producer
#define IB_SITE_PAIR_MMA 4           // gemm_tcgen05_2cta: MMA issuer
#define IB_SITE_PAIR_EPILOGUE 5      // gemm_tcgen05_2cta: epilogue
#define IB_SITE_ATTN_TC_PRODUCER 6   // attention_tcgen05: TMA producer
#define IB_SITE_ATTN_TC_MMA 7        // attention_tcgen05: MMA issuer
#define IB_SITE_ATTN_TC_SOFTMAX 8    // attention_tcgen05: softmax warps
#define IB_SITE_ATTN_TC_LAYOUT 9     // attention_tcgen05: shared memory window not where the budget assumes
#define IB_SITE_SPLIT_PRODUCER 10    // attention_mma split mode: TMA producer
#define IB_SITE_SPLIT_COMPUTE 11     // attention_mma split mode: computing warps
#define IB_TIMEOUT_AT(site) (IB_FLAG_WAIT_TIMEOUT | (1u << (8 + (site))))

#define IB_EXPORT extern "C" __attribute__((visibility("default")))

#define IB_LAUNCH_CHECK()                         \
    do {                                          \
        cudaError_t e__ = cudaGetLastError();     \
        if (e__ != cudaSuccess) return (int)e__;  \
    } while (0)

namespace ib {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with launch_kernel() may
// begin while the kernel before it in the stream still runs.  It must call
// pdl_wait() before it touches anything an earlier kernel wrote (and before
// it writes anything an earlier kernel may read); what it does before that -
// setting up barriers, fetching weights, which no kernel writes - overlaps
// with its predecessor.  pdl_trigger() lets the next kernel in the stream do
// the same with this one.  Without the launch attribute both are no-ops.
// Every thread of such a kernel calls pdl_wait() at some point, also warps that
// touch nothing a predecessor wrote (an MMA issuer that only polls a barrier,
// lanes that idle): with some threads left out, steps of the product on pairs of
// SMs stalled for good now and then, and with all threads waiting they did not.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// ---------------------------------------------------------------------------
// Bounded wait on an mbarrier in this CTA's shared memory: polls until the phase
// with the given parity is complete, gives up after IB_WAIT_LIMIT_NS of wall
// time (read from %globaltimer once in a while, not on the fast path) and
// returns false then.  `cluster`: arrivals may come from other CTAs of the
// cluster, so the successful poll acquires at cluster scope.
// ---------------------------------------------------------------------------
constexpr unsigned long long IB_WAIT_LIMIT_NS = 2000000000ull;  // two seconds

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait_bounded(unsigned bar_addr, unsigned parity,
                                                  unsigned long long limit_ns = IB_WAIT_LIMIT_NS) {
    unsigned long long t0 = 0;
    for (;;) {
        for (int i = 0; i < 2048; ++i) {
            unsigned done;
            if (CLUSTER)
                asm volatile(
                    "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}\n"
                    : "=r"(done) : "r"(bar_addr), "r"(parity) : "memory");
            else
                asm volatile(
                    "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}\n"
                    : "=r"(done) : "r"(bar_addr), "r"(parity) : "memory");
            if (done) return true;
        }
        const unsigned long long now = global_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit_ns) return false;
    }
}

inline int& pdl_flag() {
    static int enabled = 1;
    return enabled;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_flag() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same without the attribute: the kernel starts when everything before it in
// the stream is complete (its pdl_wait() is then a no-op), while its own
// pdl_trigger() still lets the kernel after it begin early.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_in_order(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` must hold 33 floats of shared memory.  The order of the additions
// depends only on blockDim, never on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace ib

// Turns programmatic dependent launch on or off for this library (default on).
extern "C" __attribute__((visibility("default"), weak)) int ib_set_pdl(int on) {
    ib::pdl_flag() = on ? 1 : 0;
    return 0;
}
