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
//              Two kernels: a row over the CTAs of a cluster with the probabilities in
//              registers (vocabularies up to 262,144), and one CTA a row for wider ones.
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

// The repetition penalty over a row's recent tokens, by all threads of a CTA: a
// token that occurs k times is penalised k times (logit > 0 ? logit / r : logit * r
// never changes the sign, so the order of the occurrences does not matter); the
// thread that holds a token's first occurrence applies them all.
__device__ __forceinline__ void apply_penalty(float* __restrict__ x, int V, const int* __restrict__ rt,
                                              int n_recent, float penalty) {
    for (int i = threadIdx.x; i < n_recent; i += blockDim.x) {
        const int t = rt[i];
        if (t < 0 || t >= V) continue;
        int k = 0;
        bool first = true;
        for (int j = 0; j < n_recent; ++j) {
            if (rt[j] == t) {
                if (j < i) {
                    first = false;
                    break;
                }
                ++k;
            }
        }
        if (!first) continue;
        float v = x[t];
        for (int q = 0; q < k; ++q) v = v > 0.f ? v / penalty : v * penalty;
        x[t] = v;
    }
}

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

    // 1. repetition penalty, in place, once per occurrence.
    if (pr.penalty != 1.f) apply_penalty(x, V, recent + (size_t)row * recent_ld, pr.n_recent, pr.penalty);
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

// ---------------------------------------------------------------------------
// The same sampler for wide rows: a row is shared out over the CTAs of a
// cluster, every thread keeps its E consecutive probabilities in registers,
// and the passes of the threshold search touch no memory.  (One CTA per row
// reads its row from L2 once per pass - 30 passes of a 128k vocabulary take
// 0.8 ms.)  The search narrows the bit pattern of the threshold WAYS-fold per
// pass: WAYS - 1 candidate thresholds at a time, their masses summed per
// thread in index order, per CTA in warp order and over the cluster in rank
// order, so the result does not depend on timing.
// ---------------------------------------------------------------------------
namespace {

constexpr int SC_THREADS = 1024;
constexpr int SC_MAX_WAYS = 16;

__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned sc_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned sc_cluster_size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ float sc_ld_peer(const float* local, unsigned rank) {
    unsigned laddr = (unsigned)__cvta_generic_to_shared(local), raddr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(laddr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

// Sums (IS_MAX: maxima) of N values per thread over the whole cluster; every thread of every CTA
// gets the same N results.  `post` is this CTA's mailbox for this call (the caller alternates
// between two, so that a CTA that runs ahead does not overwrite what a peer still reads).
template <int N, bool IS_MAX>
__device__ __forceinline__ void sc_cluster_reduce(float (&v)[N], float (*warp_part)[SC_MAX_WAYS],
                                                  float* post, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < N; ++k) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, v[k], o);
            v[k] = IS_MAX ? fmaxf(v[k], other) : v[k] + other;
        }
        if (lane == 0) warp_part[warp][k] = v[k];
    }
    __syncthreads();
    if (threadIdx.x < N) {
        float acc = IS_MAX ? -INFINITY : 0.f;
        for (int w = 0; w < SC_THREADS / 32; ++w)
            acc = IS_MAX ? fmaxf(acc, warp_part[w][threadIdx.x]) : acc + warp_part[w][threadIdx.x];
        post[threadIdx.x] = acc;
    }
    sc_cluster_sync();
    if (threadIdx.x < N) {
        const unsigned n = sc_cluster_size();
        float acc = IS_MAX ? -INFINITY : 0.f;
        for (unsigned r = 0; r < n; ++r) {
            const float other = sc_ld_peer(post + threadIdx.x, r);
            acc = IS_MAX ? fmaxf(acc, other) : acc + other;
        }
        total[threadIdx.x] = acc;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = total[k];
}

template <int E, int WAYS>
__global__ void __launch_bounds__(SC_THREADS)
sample_cluster_kernel(float* __restrict__ logits, int ld, int V, const SampleParams* __restrict__ params,
                      const int* __restrict__ recent, int recent_ld, int* __restrict__ out, int slice) {
    __shared__ float warp_part[SC_THREADS / 32][SC_MAX_WAYS];
    __shared__ float post[2][SC_MAX_WAYS];
    __shared__ float total[SC_MAX_WAYS];
    __shared__ float warp_incl[SC_THREADS / 32];
    __shared__ int picked_thread, last_thread;
    const unsigned C = sc_cluster_size(), rank = sc_cluster_rank();
    const int row = blockIdx.x / C;
    float* x = logits + (size_t)row * ld;
    const SampleParams pr = params[row];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int turn = 0;

    // 1. repetition penalty, in place, once per occurrence (one CTA of the cluster).
    if (pr.penalty != 1.f) {
        if (rank == 0) {
            apply_penalty(x, V, recent + (size_t)row * recent_ld, pr.n_recent, pr.penalty);
            __threadfence();
        }
        sc_cluster_sync();
    }

    // 2. this thread's E consecutive logits over the temperature, then probabilities.
    const int begin = (int)rank * slice + threadIdx.x * E;
    const int limit = min(V, ((int)rank + 1) * slice);
    const float inv_t = 1.f / pr.temperature;
    float p[E];
    if (begin + E <= limit && ((reinterpret_cast<uintptr_t>(x + begin) & 15) == 0) && E % 4 == 0) {
#pragma unroll
        for (int j = 0; j < E; j += 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + begin + j);
            p[j] = v.x * inv_t;
            p[j + 1] = v.y * inv_t;
            p[j + 2] = v.z * inv_t;
            p[j + 3] = v.w * inv_t;
        }
    } else {
#pragma unroll
        for (int j = 0; j < E; ++j) p[j] = begin + j < limit ? x[begin + j] * inv_t : -INFINITY;
    }
    float one[1];
    one[0] = -INFINITY;
#pragma unroll
    for (int j = 0; j < E; ++j) one[0] = fmaxf(one[0], p[j]);
    sc_cluster_reduce<1, true>(one, warp_part, post[turn], total);
    turn ^= 1;
    const float mx = one[0];
    one[0] = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        p[j] = begin + j < limit ? expf(p[j] - mx) : 0.f;
        one[0] += p[j];
    }
    sc_cluster_reduce<1, false>(one, warp_part, post[turn], total);
    turn ^= 1;
    const float inv_sum = 1.f / one[0];
#pragma unroll
    for (int j = 0; j < E; ++j) p[j] *= inv_sum;

    // 3. nucleus threshold: the largest t with mass{p >= t} >= top_p, on the bit pattern of t.
    float thresh = 0.f;
    if (pr.top_p < 1.f) {
        unsigned lo = 0u, hi = __float_as_uint(1.0f);  // mass(lo) >= top_p always
        while (lo < hi) {
            // candidates lo + step, lo + 2 step, ... (those beyond hi count as hi + 1: never reached)
            const unsigned step = (hi - lo + (unsigned)WAYS - 1u) / (unsigned)WAYS;
            float mass[WAYS - 1];
            float cand[WAYS - 1];
#pragma unroll
            for (int k = 0; k < WAYS - 1; ++k) {
                const unsigned long long c = (unsigned long long)lo + (unsigned long long)(k + 1) * step;
                cand[k] = c <= hi ? __uint_as_float((unsigned)c) : INFINITY;
                mass[k] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < E; ++j) {
#pragma unroll
                for (int k = 0; k < WAYS - 1; ++k) mass[k] += p[j] >= cand[k] ? p[j] : 0.f;
            }
            sc_cluster_reduce<WAYS - 1, false>(mass, warp_part, post[turn], total);
            turn ^= 1;
            // the largest candidate that still holds top_p; the answer lies from there to just below the next
            int best = -1;
#pragma unroll
            for (int k = 0; k < WAYS - 1; ++k)
                if (cand[k] != INFINITY && mass[k] >= pr.top_p) best = k;
            // (the candidate after it, if there was one, did not hold top_p)
            const unsigned long long next = (unsigned long long)lo + (unsigned long long)(best + 2) * step;
            if (best + 1 <= WAYS - 2 && next <= hi) hi = (unsigned)next - 1u;
            if (best >= 0) lo = lo + (unsigned)(best + 1) * step;
        }
        thresh = __uint_as_float(lo);
    }

    // 4. inverse CDF over the kept tokens in index order.
    float mine = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) mine += p[j] >= thresh ? p[j] : 0.f;
    // inclusive sums over the CTA's threads: within a warp, then over the warps
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float below = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += below;
    }
    if (lane == 31) warp_incl[warp] = incl;
    if (threadIdx.x == 0) {
        picked_thread = SC_THREADS;
        last_thread = -1;
    }
    __syncthreads();
    if (warp == 0) {
        float w = warp_incl[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float below = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += below;
        }
        warp_incl[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const float warp_base = warp > 0 ? warp_incl[warp - 1] : 0.f;
    incl += warp_base;
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = warp_base;
    // the CTAs' totals, then this CTA's base and the whole mass
    if (threadIdx.x == 0) post[turn][0] = warp_incl[SC_THREADS / 32 - 1];
    sc_cluster_sync();
    float base = 0.f, all = 0.f;
    for (unsigned r = 0; r < C; ++r) {
        const float t = sc_ld_peer(&post[turn][0], r);
        if (r < rank) base += t;
        all += t;
    }
    turn ^= 1;
    const float target = pr.u * all;
    if (mine > 0.f) {
        atomicMax(&last_thread, (int)threadIdx.x);
        if (target < base + incl) atomicMin(&picked_thread, (int)threadIdx.x);
    }
    __syncthreads();
    // which CTA picks: the first that has a thread for the target; if rounding left none, the last
    // CTA that kept any token gives its last one
    if (threadIdx.x == 0) {
        post[turn][0] = picked_thread < SC_THREADS ? 1.f : 0.f;
        post[turn][1] = last_thread >= 0 ? 1.f : 0.f;
    }
    sc_cluster_sync();
    int first_with = -1, last_kept_cta = -1;
    for (unsigned r = 0; r < C; ++r) {
        if (first_with < 0 && sc_ld_peer(&post[turn][0], r) != 0.f) first_with = (int)r;
        if (sc_ld_peer(&post[turn][1], r) != 0.f) last_kept_cta = (int)r;
    }
    const bool normal = first_with >= 0;
    const int owner_cta = normal ? first_with : last_kept_cta;
    const int owner_thread = normal ? picked_thread : last_thread;
    if (owner_cta < 0) {
        if (rank == 0 && threadIdx.x == 0) out[row] = 0;
    } else if ((int)rank == owner_cta && (int)threadIdx.x == owner_thread) {
        float run = base + excl;
        int pick = -1, last_kept = -1;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            if (p[j] >= thresh && begin + j < limit && pick < 0) {
                last_kept = begin + j;
                run += p[j];
                if (normal && target < run) pick = begin + j;
            }
        }
        out[row] = pick >= 0 ? pick : (last_kept >= 0 ? last_kept : 0);
    }
    sc_cluster_sync();  // nobody leaves while a peer may still read its mailbox
}

template <int E, int WAYS>
int launch_sample_cluster(float* logits, int ld, int n_rows, int V, const SampleParams* params,
                          const int* recent, int recent_ld, int* out, int ctas, int slice, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_rows * ctas));
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel<E, WAYS>, logits, ld, V, params, recent,
                                       recent_ld, out, slice);
    return e == cudaSuccess ? IB_OK : (int)e;
}

}  // namespace

IB_EXPORT int ib_sample(float* logits, int ld, int n_rows, int V, const void* params,
                        const int* recent, int recent_ld, int* out, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !params || !out || V <= 0 || ld < V) return IB_ERR_BAD_ARG;
    if (recent_ld > 0 && !recent) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    // A row over up to 8 CTAs of a cluster, up to 32 probabilities a thread; wider rows (beyond
    // 262,144 tokens) go to the kernel that reads its row once per pass.
    int ctas = 1;
    while (ctas < 8 && (long long)ctas * SC_THREADS * 16 < V) ctas *= 2;
    int slice = ((V + ctas - 1) / ctas + 3) / 4 * 4;
    const int per_thread = (slice + SC_THREADS - 1) / SC_THREADS;
    const SampleParams* sp = (const SampleParams*)params;
    int rc;
    // Few rows: the search is a chain of cluster-wide sums, so it takes 16 candidates a pass (8
    // passes).  Many rows fill the machine and the candidates' arithmetic is what costs: 4 a pass.
    const bool wide = (long long)n_rows * ctas <= 72;
#define IB_SAMPLE_LAUNCH(E) \
    (wide ? launch_sample_cluster<E, 16>(logits, ld, n_rows, V, sp, recent, recent_ld, out, ctas, slice, s) \
          : launch_sample_cluster<E, 4>(logits, ld, n_rows, V, sp, recent, recent_ld, out, ctas, slice, s))
    if (per_thread <= 4) rc = IB_SAMPLE_LAUNCH(4);
    else if (per_thread <= 8) rc = IB_SAMPLE_LAUNCH(8);
    else if (per_thread <= 16) rc = IB_SAMPLE_LAUNCH(16);
    else if (per_thread <= 32) rc = launch_sample_cluster<32, 4>(logits, ld, n_rows, V, sp, recent, recent_ld, out, ctas, slice, s);
#undef IB_SAMPLE_LAUNCH
    else {
        sample_kernel<<<n_rows, 1024, 0, s>>>(logits, ld, V, sp, recent, recent_ld, out);
        rc = IB_OK;
    }
    if (rc != IB_OK) return rc;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
