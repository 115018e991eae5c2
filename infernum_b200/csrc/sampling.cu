// Token selection from 32-bit logits, one block per row.
//
//  ib_argmax   greedy: the largest logit, the lowest index among equals.
//              (the reference: infernum-cuda/kernels/argmax.cu:64-136)
//  ib_sample   the reference's sampler (infernum-cuda/src/inner/cuda/ops/sample.rs:86-160),
//              which runs on the host there, as one device kernel:
//                1. repetition penalty over the recent tokens, applied once per
//                   occurrence: logit > 0 ? logit / r : logit * r
//                2. divide by the temperature, softmax with max subtraction
//                3. nucleus: keep the most probable tokens whose mass first
//                   reaches top_p (all tokens as probable as the last one kept)
//                4. inverse CDF over the kept tokens with a uniform number u
//              The reference walks the kept tokens in order of probability; this
//              kernel walks them in order of index, which gives the same
//              distribution without a sort.  u is supplied by the caller.
#include "common.cuh"

using namespace ib;

__global__ void argmax_kernel(const float* __restrict__ logits, int ld, int V,
                              int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* x = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int bi = V;  // "none yet": any real index is lower
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : V;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (lane == 0) out[blockIdx.x] = bi < V ? bi : 0;
    }
}

// Wide rows are cut in slices so that more than one CTA per row reads memory:
// first the best (value, index) of every slice, then the best of those.
__global__ void argmax_slice_kernel(const float* __restrict__ logits, int ld, int V, int slice,
                                    float* __restrict__ part_val, int* __restrict__ part_idx) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* x = logits + (size_t)blockIdx.x * ld;
    const int begin = blockIdx.y * slice, end = min(V, begin + slice);
    float best = -INFINITY;
    int bi = V;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : V;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            part_val[blockIdx.x * gridDim.y + blockIdx.y] = best;
            part_idx[blockIdx.x * gridDim.y + blockIdx.y] = bi;
        }
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ part_val,
                                    const int* __restrict__ part_idx, int n_slices, int V,
                                    int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    // one warp per row
    const int row = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    int bi = V;
    for (int i = lane; i < n_slices; i += 32) {
        const float v = part_val[row * n_slices + i];
        const int idx = part_idx[row * n_slices + i];
        if (v > best || (v == best && idx < bi)) {
            best = v;
            bi = idx;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    if (lane == 0) out[row] = bi < V ? bi : 0;
}

#define IB_ARGMAX_MAX_SLICES 64

// `scratch` (optional) holds n_rows * 64 floats followed by n_rows * 64 ints;
// with it, wide rows are read by several CTAs each.
IB_EXPORT int ib_argmax(const float* logits, int ld, int n_rows, int V, int* out, void* scratch,
                        long long scratch_bytes, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !out || V <= 0 || ld < V) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int slices = 1;
    if (scratch && V >= 16384) {
        slices = (V + 4095) / 4096;
        if (slices > IB_ARGMAX_MAX_SLICES) slices = IB_ARGMAX_MAX_SLICES;
        while (slices > 1 && (long long)n_rows * slices > 4096) slices /= 2;
        if (scratch_bytes < (long long)n_rows * slices * 8) slices = 1;
    }
    if (slices <= 1) {
        const int threads = V >= 8192 ? 1024 : 256;
        cudaError_t le = launch_kernel(argmax_kernel, dim3(n_rows), dim3(threads), 0, s, logits, ld, V, out);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    const int slice = (V + slices - 1) / slices;
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (size_t)n_rows * slices);
    cudaError_t le = launch_kernel(argmax_slice_kernel, dim3(n_rows, slices), dim3(256), 0, s, logits, ld, V,
                                   slice, pv, pi);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    le = launch_kernel(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)pv, (const int*)pi,
                       slices, V, out);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// ib_argmax_noalloc: greedy selection for callers that cannot allocate.
//
// Who that is: code that is handed its input and output buffers by a host
// application and nothing else - a sampling plug-in inside someone else's
// serving loop, say - and that must stay off cudaMalloc on its hot path,
// because cudaMalloc synchronises the whole device, and because an engine
// like this one gives nearly all free memory to cache pages, so a late
// allocation can simply fail.  ib_argmax needs a scratch buffer from its
// caller to spread a wide row over several CTAs; this variant keeps that
// scratch inside the library instead.
//
// The scratch is the file-scope device array below: 128 KiB, enough for
// IB_NOALLOC_MAX_ROWS rows of 64 partial results.  Every GPU that loads this
// library holds those 128 KiB until the process exits.  All calls share the
// array and it keeps whatever the last call left; nothing in it has to start
// at zero, because every partial result that is read was written by the same
// call.  Two calls that overlap on the GPU (different streams, or different
// host threads on one device) race on it: keep calls on one stream, or
// serialise them.
//
// The first call on a device looks the array's address up (in host code the
// array's name is only a stand-in for the symbol, not a device address) and
// remembers it per device; that first call should come before any stream
// capture begins.  Two host threads that make their first call on one device
// at the same moment both do the look-up and store the same address, which
// is harmless (the store is one aligned pointer).  The function calls no
// cudaMalloc, cudaFree or other allocating routine.  It has no counterpart in
// the reference.
// ---------------------------------------------------------------------------
#define IB_NOALLOC_MAX_ROWS 256
#define IB_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char
    g_argmax_noalloc_scratch[IB_NOALLOC_MAX_ROWS * IB_ARGMAX_MAX_SLICES * 8];

static void* g_argmax_noalloc_ptr[IB_NOALLOC_MAX_DEVICES] = {nullptr};

IB_EXPORT int ib_argmax_noalloc_max_rows() { return IB_NOALLOC_MAX_ROWS; }

IB_EXPORT int ib_argmax_noalloc(const float* logits, int ld, int n_rows, int V, int* out,
                                void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !out || V <= 0 || ld < V) return IB_ERR_BAD_ARG;
    if (n_rows > IB_NOALLOC_MAX_ROWS) return IB_ERR_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= IB_NOALLOC_MAX_DEVICES) return IB_ERR_NOALLOC_SETUP;
    if (!g_argmax_noalloc_ptr[dev]) {
        // set-up, once per device, with that device current
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_argmax_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!ptr) return IB_ERR_NOALLOC_SETUP;
        g_argmax_noalloc_ptr[dev] = ptr;
    }
    cudaStream_t s = (cudaStream_t)stream;
    int slices = (V + 4095) / 4096;
    if (slices > IB_ARGMAX_MAX_SLICES) slices = IB_ARGMAX_MAX_SLICES;
    if (slices < 1) slices = 1;
    const int slice = (V + slices - 1) / slices;
    float* pv = (float*)g_argmax_noalloc_ptr[dev];
    int* pi = (int*)(pv + (size_t)n_rows * slices);
    argmax_slice_kernel<<<dim3(n_rows, slices), 256, 0, s>>>(logits, ld, V, slice, pv, pi);
    IB_LAUNCH_CHECK();
    argmax_merge_kernel<<<n_rows, 32, 0, s>>>(pv, pi, slices, V, out);
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// Per-row parameters of ib_sample (one struct per row, in device memory).
struct SampleParams {
    float temperature;  // > 0
    float top_p;        // in (0, 1]; >= 1 keeps every token
    float penalty;      // repetition penalty, 1 = off
    float u;            // uniform number in [0, 1)
    int n_recent;       // how many entries of this row's recent-token list count
    int pad;
};

__global__ void sample_kernel(float* __restrict__ logits, int ld, int V,
                              const SampleParams* __restrict__ params,
                              const int* __restrict__ recent, int recent_ld,
                              int* __restrict__ out) {
    __shared__ float scratch[33];
    __shared__ float chunk_sum[1024];
    __shared__ int chosen;
    const int row = blockIdx.x;
    float* x = logits + (size_t)row * ld;
    const SampleParams pr = params[row];
    const int nt = blockDim.x;

    // 1. repetition penalty, in place, once per occurrence, in list order.
    if (threadIdx.x == 0 && pr.penalty != 1.f) {
        const int* rt = recent + (size_t)row * recent_ld;
        for (int i = 0; i < pr.n_recent; ++i) {
            const int t = rt[i];
            if (t >= 0 && t < V) {
                const float v = x[t];
                x[t] = v > 0.f ? v / pr.penalty : v * pr.penalty;
            }
        }
    }
    __syncthreads();

    // 2. softmax statistics of logits / temperature.
    const float inv_t = 1.f / pr.temperature;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += nt) mx = fmaxf(mx, x[i] * inv_t);
    mx = block_max(mx, scratch);
    float sum = 0.f;
    for (int i = threadIdx.x; i < V; i += nt) sum += expf(x[i] * inv_t - mx);
    sum = block_sum(sum, scratch);
    const float inv_sum = 1.f / sum;

    // 3. nucleus threshold: the largest probability t with mass{p >= t} >= top_p,
    //    found by bisection on the bit pattern of t (positive floats order like
    //    their bits), so t ends exactly on the probability of the last token kept.
    float thresh = 0.f;
    if (pr.top_p < 1.f) {
        unsigned lo = 0u, hi = __float_as_uint(1.0f);  // mass(lo) >= top_p always
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            const float t = __uint_as_float(mid);
            float mass = 0.f;
            for (int i = threadIdx.x; i < V; i += nt) {
                const float p = expf(x[i] * inv_t - mx) * inv_sum;
                mass += p >= t ? p : 0.f;
            }
            mass = block_sum(mass, scratch);
            if (mass >= pr.top_p) lo = mid; else hi = mid - 1u;
        }
        thresh = __uint_as_float(lo);
    }

    // 4. inverse CDF over kept tokens in index order.  Thread k owns the
    //    contiguous range [k*per, (k+1)*per).
    const int per = (V + nt - 1) / nt;
    const int begin = min(V, threadIdx.x * per), end = min(V, begin + per);
    float mine = 0.f;
    for (int i = begin; i < end; ++i) {
        const float p = expf(x[i] * inv_t - mx) * inv_sum;
        mine += p >= thresh ? p : 0.f;
    }
    chunk_sum[threadIdx.x] = mine;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int k = 0; k < nt; ++k) total += chunk_sum[k];
        const float target = pr.u * total;
        float run = 0.f, excl = 0.f;
        int owner = -1;
        for (int k = 0; k < nt; ++k) {
            if (chunk_sum[k] > 0.f) {
                owner = k;  // the last non-empty chunk is the fallback
                excl = run;
                if (target < run + chunk_sum[k]) break;
            }
            run += chunk_sum[k];
        }
        scratch[0] = excl;
        scratch[1] = target;
        chosen = owner;
    }
    __syncthreads();
    if (threadIdx.x == chosen) {
        float run = scratch[0];
        const float target = scratch[1];
        int pick = -1, last_kept = -1;
        for (int i = begin; i < end; ++i) {
            const float p = expf(x[i] * inv_t - mx) * inv_sum;
            if (p >= thresh) {
                last_kept = i;
                run += p;
                if (target < run) {
                    pick = i;
                    break;
                }
            }
        }
        out[row] = pick >= 0 ? pick : (last_kept >= 0 ? last_kept : 0);
    }
    if (chosen < 0 && threadIdx.x == 0) out[row] = 0;
}

IB_EXPORT int ib_sample(float* logits, int ld, int n_rows, int V, const void* params,
                        const int* recent, int recent_ld, int* out, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !params || !out || V <= 0 || ld < V) return IB_ERR_BAD_ARG;
    if (recent_ld > 0 && !recent) return IB_ERR_BAD_ARG;
    sample_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(
        logits, ld, V, (const SampleParams*)params, recent, recent_ld, out);
    IB_LAUNCH_CHECK();
    return IB_OK;
}
