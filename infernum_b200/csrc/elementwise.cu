// Bandwidth-bound kernels of the decoder step: token embedding, residual add
// fused with RMSNorm, rotary embedding fused with the write of K and V into
// the paged cache, and SiLU(gate) * up.  All arithmetic is done in 32-bit and
// rounded once at the store.
//
// What each computes follows the reference's kernels:
//   embedding  out[t,:] = table[ids[t],:]            infernum-cuda/kernels/embed.cu:36-50
//   rmsnorm    y = x * rsqrt(mean(x^2)+eps) * w      infernum-cuda/kernels/rmsnorm.cu:64-94
//   add+norm   s = r + x; y = rmsnorm(s)             infernum-cuda/kernels/add_rmsnorm.cu:78-108
//   rope       half-rotation pairs (j, j+rd/2)       infernum-cuda/kernels/rope.cu:25-41
//   kv append  pool[table[p/bs]][p%bs] = k, v        infernum-cuda/kernels/append_kv_paged.cu:110-192
//   silu*mul   g/(1+exp(-g)) * u                     infernum-cuda/kernels/silu.cu:105-116
// Unlike the reference the residual stream stays in 32-bit between layers, and
// rotation angles are computed in 32-bit from the position and the inverse
// frequency (the reference rounds its tables to bf16).
#include "common.cuh"

using namespace ib;

// ---------------------------------------------------------------------------
// Embedding: residual[t, :] = table[ids[t], :] widened to 32-bit.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int V, unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* o = out + (size_t)row * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(src[i]);
}

IB_EXPORT int ib_embed(const int* ids, const void* table, int table_dtype, float* out, int n_rows,
                       int H, int V, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || V <= 0 || !ids || !table || !out || !err) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == 0)
        { cudaError_t le__ = launch_kernel(embed_kernel<float>, dim3(n_rows), dim3(threads), 0, s, ids, (const float*)table, out, H, V, err); if (le__ != cudaSuccess) return (int)le__; }
    else if (table_dtype == 1)
        { cudaError_t le__ = launch_kernel(embed_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, ids, (const bf16*)table, out, H, V, err); if (le__ != cudaSuccess) return (int)le__; }
    else
        return IB_ERR_UNSUPPORTED;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm.
//   s = residual[src] (+ delta[src]);  if write_residual: residual[src] = s
//   out[row] = s * rsqrt(mean(s^2) + eps) * weight
// `row_idx` (optional) selects source rows, the output is then compact; it is
// how the final norm runs only on the rows whose logits are wanted.
// One block per row; the reduction order depends on H and blockDim only.
// ---------------------------------------------------------------------------
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const TW* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ row_idx, int H, float eps,
                                   int write_residual) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x;
    const int src = row_idx ? row_idx[row] : row;
    float* r = residual + (size_t)src * H;
    const TD* d = delta ? delta + (size_t)src * H : nullptr;
    TO* o = out + (size_t)row * H;

    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (d) {
            v += to_f32(d[i]);
            if (write_residual) r[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (d && !write_residual) v += to_f32(d[i]);
        o[i] = from_f32<TO>((v * inv) * to_f32(weight[i]));
    }
}

// Vectorised variant for H % 4 == 0: each thread owns up to NV groups of four
// consecutive elements, keeps them in registers, and the row is read once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&a);
        raw.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TD, typename TW, typename TO, int NV>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                       const TW* __restrict__ weight, TO* __restrict__ out,
                                       const int* __restrict__ row_idx, int H, float eps,
                                       int write_residual) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int row = blockIdx.x;
    const int src = row_idx ? row_idx[row] : row;
    float* r = residual + (size_t)src * H;
    const TD* d = delta ? delta + (size_t)src * H : nullptr;
    TO* o = out + (size_t)row * H;
    const int groups = H >> 2;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int gidx = threadIdx.x + k * blockDim.x;
        if (gidx < groups) {
            v[k] = Vec4<float>::load(r + 4 * gidx);
            if (d) {
                const float4 dv = Vec4<TD>::load(d + 4 * gidx);
                v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
                if (write_residual) Vec4<float>::store(r + 4 * gidx, v[k]);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int gidx = threadIdx.x + k * blockDim.x;
        if (gidx < groups) {
            const float4 w = Vec4<TW>::load(weight + 4 * gidx);
            Vec4<TO>::store(o + 4 * gidx, make_float4((v[k].x * inv) * w.x, (v[k].y * inv) * w.y,
                                                      (v[k].z * inv) * w.z, (v[k].w * inv) * w.w));
        }
    }
}

template <typename TD, typename TW, typename TO>
static bool try_launch_vec(float* residual, const void* delta, const void* weight, void* out,
                           const int* row_idx, int n_rows, int H, float eps, int write_residual,
                           cudaStream_t s) {
    if (H % 4) return false;
    if (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) return false;
    const int groups = H / 4;
    int threads = ((groups + 31) / 32) * 32;
    int nv = 1;
    while (threads > 1024 || (threads > 256 && nv < 2 && groups >= 2048)) {
        nv *= 2;
        threads = (((groups + nv - 1) / nv + 31) / 32) * 32;
        if (nv > 8) return false;
    }
#define IB_VEC_LAUNCH(NV)                                                                   \
    launch_kernel(add_rmsnorm_vec_kernel<TD, TW, TO, NV>, dim3(n_rows), dim3(threads), 0, s, \
                  residual, (const TD*)delta, (const TW*)weight, (TO*)out, row_idx, H, eps,  \
                  write_residual)
    // a failed launch is picked up by cudaGetLastError in the caller
    switch (nv) {
        case 1: IB_VEC_LAUNCH(1); break;
        case 2: IB_VEC_LAUNCH(2); break;
        case 4: IB_VEC_LAUNCH(4); break;
        case 8: IB_VEC_LAUNCH(8); break;
        default: return false;
    }
#undef IB_VEC_LAUNCH
    return true;
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* residual, const void* delta, const void* weight,
                              int weight_dtype, void* out, const int* row_idx, int n_rows, int H,
                              float eps, int write_residual, cudaStream_t s) {
    if (weight_dtype == 0 && try_launch_vec<TD, float, TO>(residual, delta, weight, out, row_idx, n_rows,
                                                            H, eps, write_residual, s)) {
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    if (weight_dtype == 1 && try_launch_vec<TD, bf16, TO>(residual, delta, weight, out, row_idx, n_rows,
                                                           H, eps, write_residual, s)) {
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    int threads = 256;
    if (H >= 8192) threads = 1024;
    else if (H >= 2048) threads = 512;
    else if (H <= 256) threads = 64;
    if (weight_dtype == 0)
        { cudaError_t le__ = launch_kernel(add_rmsnorm_kernel<TD, float, TO>, dim3(n_rows), dim3(threads), 0, s, 
            residual, (const TD*)delta, (const float*)weight, (TO*)out, row_idx, H, eps,
            write_residual); if (le__ != cudaSuccess) return (int)le__; }
    else if (weight_dtype == 1)
        { cudaError_t le__ = launch_kernel(add_rmsnorm_kernel<TD, bf16, TO>, dim3(n_rows), dim3(threads), 0, s, 
            residual, (const TD*)delta, (const bf16*)weight, (TO*)out, row_idx, H, eps,
            write_residual); if (le__ != cudaSuccess) return (int)le__; }
    else
        return IB_ERR_UNSUPPORTED;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// act_dtype is the type of `delta` and of `out` (0 = f32, 1 = bf16).
IB_EXPORT int ib_add_rmsnorm(float* residual, const void* delta, const void* weight,
                             int weight_dtype, void* out, int act_dtype, const int* row_idx,
                             int n_rows, int H, float eps, int write_residual, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || !residual || !weight || !out || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == 0)
        return launch_add_rmsnorm<float, float>(residual, delta, weight, weight_dtype, out, row_idx,
                                                n_rows, H, eps, write_residual, s);
    if (act_dtype == 1)
        return launch_add_rmsnorm<bf16, bf16>(residual, delta, weight, weight_dtype, out, row_idx,
                                              n_rows, H, eps, write_residual, s);
    return IB_ERR_UNSUPPORTED;
}

// residual[row] += delta[row] with no norm (used when a stream ends without one).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                    size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) residual[i] += to_f32(delta[i]);
}

IB_EXPORT int ib_residual_add(float* residual, const void* delta, int act_dtype, long long n,
                              void* stream) {
    if (n <= 0) return IB_OK;
    if (!residual || !delta) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == 0)
        { cudaError_t le__ = launch_kernel(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, s, residual, (const float*)delta, (size_t)n); if (le__ != cudaSuccess) return (int)le__; }
    else if (act_dtype == 1)
        { cudaError_t le__ = launch_kernel(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, s, residual, (const bf16*)delta, (size_t)n); if (le__ != cudaSuccess) return (int)le__; }
    else
        return IB_ERR_UNSUPPORTED;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// Rotary embedding of q and k (in 32-bit), and the write of rotated k and of
// v into the pages of the cache.
//   qkv row layout: [ q: nh*hd | k: nkv*hd | v: nkv*hd ], row stride qkv_stride.
//   q is rotated in place; k is rotated in place too (so the row can be
//   checked) and copied to the pool; v is copied.
//   pools: [num_pages, nkv, page_size, hd].
//   A pair item p < rd/2 rotates elements (p, p + rd/2); items beyond cover
//   the dims [rd, hd) that are not rotated.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, int qkv_stride,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ row_entry,
                                   const int* __restrict__ block_tables, int max_blocks,
                                   const float* __restrict__ inv_freq, T* __restrict__ k_pool,
                                   T* __restrict__ v_pool, int nh, int nkv, int hd, int rd,
                                   int page_size, int num_pages, int write_kv,
                                   unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int half = hd / 2;
    const int rhalf = rd / 2;
    const int items_qk = (nh + nkv) * half;
    const int items = items_qk + (write_kv ? nkv * half : 0);
    const int pos = positions[row];
    T* base = qkv + (size_t)row * qkv_stride;

    long long slot_base = -1;  // element offset of (page, kv head 0, slot, 0)
    if (write_kv) {
        const int e = row_entry[row];
        // (a position beyond the row of the table is reported like a bad entry, not followed)
        const int slot_idx = pos / page_size;
        const int page = (pos >= 0 && slot_idx < max_blocks) ? block_tables[(size_t)e * max_blocks + slot_idx] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
        } else {
            slot_base = ((long long)page * nkv * page_size + (pos % page_size)) * hd;
        }
    }
    const long long head_step = (long long)page_size * hd;

    for (int it = blockIdx.y * blockDim.x + threadIdx.x; it < items; it += gridDim.y * blockDim.x) {
        if (it < items_qk) {
            const int head = it / half, p = it % half;
            T* x = base + (size_t)head * hd;
            int d0, d1;
            float y0, y1;
            if (p < rhalf) {
                d0 = p;
                d1 = p + rhalf;
                const float angle = (float)pos * inv_freq[p];
                float sn, cs;
                sincosf(angle, &sn, &cs);
                const float x0 = to_f32(x[d0]), x1 = to_f32(x[d1]);
                y0 = x0 * cs - x1 * sn;
                y1 = x0 * sn + x1 * cs;
                x[d0] = from_f32<T>(y0);
                x[d1] = from_f32<T>(y1);
            } else {
                d0 = rd + 2 * (p - rhalf);
                d1 = d0 + 1;
                y0 = to_f32(x[d0]);
                y1 = to_f32(x[d1]);
            }
            if (head >= nh && slot_base >= 0) {
                T* dst = k_pool + slot_base + (long long)(head - nh) * head_step;
                dst[d0] = from_f32<T>(y0);
                dst[d1] = from_f32<T>(y1);
            }
        } else if (slot_base >= 0) {
            const int vi = it - items_qk;
            const int g = vi / half, p = vi % half;
            const T* x = base + (size_t)(nh + nkv + g) * hd;
            T* dst = v_pool + slot_base + (long long)g * head_step;
            dst[2 * p] = x[2 * p];
            dst[2 * p + 1] = x[2 * p + 1];
        }
    }
}

// bf16 variant that moves 16 bytes at a time: an item is 8 consecutive pairs
// (elements j..j+7 and j+rd/2..j+rd/2+7 of one head), 8 unrotated elements, or
// 8 elements of v.  Needs rd % 16 == 0, hd % 8 == 0 and 16-byte aligned rows.
constexpr int ROPE_VEC8_MAX_PAIRS = 256;  // rotated pairs of a head the vectorised kernel takes (rd <= 512)
__global__ void rope_append_vec8_kernel(bf16* __restrict__ qkv, int qkv_stride,
                                        const int* __restrict__ positions,
                                        const int* __restrict__ row_entry,
                                        const int* __restrict__ block_tables, int max_blocks,
                                        const float* __restrict__ inv_freq, bf16* __restrict__ k_pool,
                                        bf16* __restrict__ v_pool, int nh, int nkv, int hd, int rd,
                                        int page_size, int num_pages, int write_kv,
                                        unsigned* __restrict__ err) {
    pdl_trigger();
    // Positions, block tables and frequencies were complete before this chain of
    // kernels began: the page look-up and the row's sines and cosines are done
    // while the product before this kernel still runs, and only then is its
    // result waited for.  The angles depend on the position and the pair, not on
    // the head: the block works them out once (a pair per thread) and every head's
    // items read them from shared memory.
    __shared__ __align__(16) float sn_s[ROPE_VEC8_MAX_PAIRS];
    __shared__ __align__(16) float cs_s[ROPE_VEC8_MAX_PAIRS];
    const int row = blockIdx.x;
    const int rot_items = rd >> 4;             // per head: items of 8 pairs
    const int pass_items = (hd - rd) >> 3;     // per head: items of 8 unrotated elements
    const int per_head = rot_items + pass_items;
    const int items_qk = (nh + nkv) * per_head;
    const int v_items = write_kv ? nkv * (hd >> 3) : 0;
    const int items = items_qk + v_items;
    const int pos = positions[row];
    bf16* base = qkv + (size_t)row * qkv_stride;

    long long slot_base = -1;
    if (write_kv) {
        const int e = row_entry[row];
        // (a position beyond the row of the table is reported like a bad entry, not followed)
        const int slot_idx = pos / page_size;
        const int page = (pos >= 0 && slot_idx < max_blocks) ? block_tables[(size_t)e * max_blocks + slot_idx] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
        } else {
            slot_base = ((long long)page * nkv * page_size + (pos % page_size)) * hd;
        }
    }
    const long long head_step = (long long)page_size * hd;
    const int half = rd >> 1;

    const int first_it = blockIdx.y * blockDim.x + threadIdx.x;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sn_s[j], &cs_s[j]);
    __syncthreads();
    pdl_wait();

    for (int it = first_it; it < items; it += gridDim.y * blockDim.x) {
        if (it < items_qk) {
            const int head = it / per_head, p = it % per_head;
            bf16* x = base + (size_t)head * hd;
            bf16* dst = (head >= nh && slot_base >= 0)
                            ? k_pool + slot_base + (long long)(head - nh) * head_step : nullptr;
            if (p < rot_items) {
                const int j = p << 3;
                uint4 a4 = *reinterpret_cast<const uint4*>(x + j);
                uint4 b4 = *reinterpret_cast<const uint4*>(x + j + half);
                __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a4);
                __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b4);
                float sn[8], cs[8];
                *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sn_s + j);
                *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sn_s + j + 4);
                *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(cs_s + j);
                *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(cs_s + j + 4);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 xa = __bfloat1622float2(a2[k]), xb = __bfloat1622float2(b2[k]);
                    const float s0 = sn[2 * k], c0 = cs[2 * k], s1 = sn[2 * k + 1], c1 = cs[2 * k + 1];
                    a2[k] = __floats2bfloat162_rn(xa.x * c0 - xb.x * s0, xa.y * c1 - xb.y * s1);
                    b2[k] = __floats2bfloat162_rn(xa.x * s0 + xb.x * c0, xa.y * s1 + xb.y * c1);
                }
                *reinterpret_cast<uint4*>(x + j) = a4;
                *reinterpret_cast<uint4*>(x + j + half) = b4;
                if (dst) {
                    *reinterpret_cast<uint4*>(dst + j) = a4;
                    *reinterpret_cast<uint4*>(dst + j + half) = b4;
                }
            } else if (dst) {
                const int d0 = rd + ((p - rot_items) << 3);
                *reinterpret_cast<uint4*>(dst + d0) = *reinterpret_cast<const uint4*>(x + d0);
            }
        } else if (slot_base >= 0) {
            const int vi = it - items_qk;
            const int g = vi / (hd >> 3), d0 = (vi % (hd >> 3)) << 3;
            *reinterpret_cast<uint4*>(v_pool + slot_base + (long long)g * head_step + d0) =
                *reinterpret_cast<const uint4*>(base + (size_t)(nh + nkv + g) * hd + d0);
        }
    }
}

IB_EXPORT int ib_rope_append(void* qkv, int act_dtype, int qkv_stride, const int* positions,
                             const int* row_entry, const int* block_tables, int max_blocks,
                             const float* inv_freq, void* k_pool, void* v_pool, int n_rows, int nh,
                             int nkv, int hd, int rd, int page_size, int num_pages, int write_kv,
                             unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!qkv || !positions || !err || nh <= 0 || nkv < 0 || hd <= 0 || (hd & 1) || rd < 0 ||
        rd > hd || (rd & 1))
        return IB_ERR_BAD_ARG;
    if (rd > 0 && !inv_freq) return IB_ERR_BAD_ARG;
    if (write_kv && (!row_entry || !block_tables || !k_pool || !v_pool || page_size <= 0 ||
                     max_blocks <= 0 || num_pages <= 0))
        return IB_ERR_BAD_ARG;
    if (qkv_stride < (nh + 2 * nkv) * hd && write_kv) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int items = (nh + nkv) * (hd / 2) + (write_kv ? nkv * (hd / 2) : 0);
    const int threads = 128;
    int by = (items + threads - 1) / threads;
    if (by > 16) by = 16;
    if (act_dtype == 1 && rd % 16 == 0 && rd / 2 <= ROPE_VEC8_MAX_PAIRS && hd % 8 == 0 && qkv_stride % 8 == 0 &&
        !(((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15)) {
        const int vitems = (nh + nkv) * ((rd >> 4) + ((hd - rd) >> 3)) + (write_kv ? nkv * (hd >> 3) : 0);
        int vby = (vitems + threads - 1) / threads;
        if (vby > 8) vby = 8;
        cudaError_t le = launch_kernel(rope_append_vec8_kernel, dim3(n_rows, vby), dim3(threads), 0, s,
                                       (bf16*)qkv, qkv_stride, positions, row_entry, block_tables,
                                       max_blocks, inv_freq, (bf16*)k_pool, (bf16*)v_pool, nh, nkv, hd,
                                       rd, page_size, num_pages, write_kv, err);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    dim3 grid(n_rows, by);
    if (act_dtype == 0)
        { cudaError_t le__ = launch_kernel(rope_append_kernel<float>, dim3(grid), dim3(threads), 0, s, 
            (float*)qkv, qkv_stride, positions, row_entry, block_tables, max_blocks, inv_freq,
            (float*)k_pool, (float*)v_pool, nh, nkv, hd, rd, page_size, num_pages, write_kv, err); if (le__ != cudaSuccess) return (int)le__; }
    else if (act_dtype == 1)
        { cudaError_t le__ = launch_kernel(rope_append_kernel<bf16>, dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, qkv_stride, positions, row_entry, block_tables, max_blocks, inv_freq,
            (bf16*)k_pool, (bf16*)v_pool, nh, nkv, hd, rd, page_size, num_pages, write_kv, err); if (le__ != cudaSuccess) return (int)le__; }
    else
        return IB_ERR_UNSUPPORTED;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// SwiGLU activation: out[t, i] = silu(gate_i) * up_i, x is [N, 2I].
// Where gate and up sit in a row of x is given by `blk`: the row is cut in
// pieces of 2*blk values, each blk gates followed by their blk ups.  blk = I is
// the plain layout [all gates | all ups]; blk = 64 is the layout of a product
// whose weight rows were interleaved 64 by 64 (so that one 128-row tile of the
// tcgen05 product holds gates and their ups).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int I, int blk,
                                size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / I;
    const int i = (int)(idx % I);
    const size_t gi = row * 2 * I + (size_t)(i / blk) * 2 * blk + (i % blk);
    const float g = to_f32(x[gi]);
    const float u = to_f32(x[gi + blk]);
    const float act = g / (1.f + expf(-g));
    out[idx] = from_f32<T>(act * u);
}

// Eight outputs per thread with 16-byte loads and stores (I and blk multiples of 8).
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int I,
                                     int blk, size_t total_vec) {
    pdl_trigger();
    pdl_wait();
    const size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= total_vec) return;
    const int per_row = I >> 3;
    const size_t row = v / per_row;
    const int i = (int)(v % per_row) << 3;
    const size_t gi = row * 2 * I + (size_t)(i / blk) * 2 * blk + (i % blk);
    const uint4 g4 = *reinterpret_cast<const uint4*>(x + gi);
    const uint4 u4 = *reinterpret_cast<const uint4*>(x + gi + blk);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + row * I + i) = o4;
}

IB_EXPORT int ib_silu_mul(const void* x, void* out, int act_dtype, int n_rows, int I, int blk,
                          void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !out || I <= 0 || blk <= 0 || I % blk) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)n_rows * I;
    if (act_dtype == 1 && I % 8 == 0 && blk % 8 == 0 && !(((uintptr_t)x | (uintptr_t)out) & 15)) {
        const size_t total_vec = total / 8;
        cudaError_t le = launch_kernel(silu_mul_vec8_kernel, dim3((unsigned)((total_vec + 255) / 256)),
                                       dim3(256), 0, s, (const bf16*)x, (bf16*)out, I, blk, total_vec);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
        return IB_OK;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_dtype == 0) {
        cudaError_t le = launch_kernel(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s,
                                       (const float*)x, (float*)out, I, blk, total);
        if (le != cudaSuccess) return (int)le;
    } else if (act_dtype == 1) {
        cudaError_t le = launch_kernel(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s,
                                       (const bf16*)x, (bf16*)out, I, blk, total);
        if (le != cudaSuccess) return (int)le;
    } else {
        return IB_ERR_UNSUPPORTED;
    }
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// After a decode step whose inputs live on the device: every request moves one
// position on, and (optionally) the token just selected becomes the next input.
// ---------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ tokens, const int* __restrict__ selected,
                                      int* __restrict__ positions, int* __restrict__ kv_len,
                                      const int* __restrict__ slot_ids, int pad_slot, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // a row that only fills up a batch bucket stays where it is: at position 0 of the spare page
    if (slot_ids && slot_ids[i] == pad_slot) return;
    positions[i] += 1;
    kv_len[i] += 1;
    if (selected) tokens[i] = selected[i];
}

// ---------------------------------------------------------------------------
// Input tokens of a step that is launched while the step before it still runs:
// row i takes the token that step selected for its row src[i]; a row with
// src[i] < 0 keeps the token the host put there.  Launched the ordinary way,
// behind the copy that brought `src`.
// ---------------------------------------------------------------------------
// The same token also goes into the row's list of recent tokens (for its
// repetition penalty) at place recent_pos[i], where that is not negative.
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                   const int* __restrict__ selected, int n_selected, int n,
                                   int* __restrict__ recent, int recent_ld,
                                   const int* __restrict__ recent_pos) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int s = src[i];
    if (s < 0 || s >= n_selected) return;
    const int tok = selected[s];
    tokens[i] = tok;
    if (recent && recent_pos) {
        const int at = recent_pos[i];
        if (at >= 0 && at < recent_ld) recent[(size_t)i * recent_ld + at] = tok;
    }
}

IB_EXPORT int ib_feed_tokens(int* tokens, const int* src, const int* selected, int n_selected, int n,
                             int* recent, int recent_ld, const int* recent_pos, void* stream) {
    if (n <= 0) return IB_OK;
    if (!tokens || !src || !selected || n_selected <= 0) return IB_ERR_BAD_ARG;
    if (recent && (!recent_pos || recent_ld <= 0)) return IB_ERR_BAD_ARG;
    feed_tokens_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(tokens, src, selected, n_selected, n,
                                                                           recent, recent_ld, recent_pos);
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// The first launch of every step.  The kernels of this package start under the
// tail of their predecessor (programmatic dependent launch) and some read what
// describes the step - positions, block tables, row offsets - before they wait
// for it.  Those must be complete by then, whoever wrote them (a copy from the
// host, or the advance kernel of the step before).  This kernel is launched
// the ordinary way, so it starts only when everything before it in the stream
// is complete, and the kernels after it cannot start before it does.
// ---------------------------------------------------------------------------
__global__ void step_fence_kernel() {}

IB_EXPORT int ib_step_fence(void* stream) {
    step_fence_kernel<<<1, 1, 0, (cudaStream_t)stream>>>();
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// ---------------------------------------------------------------------------
// A wait that nothing ends, for testing the bounded wait itself: one thread
// waits `limit_ns` for a barrier on which nobody arrives, sets the time-out
// flag (with the site bit `site`) and returns.  Nothing faults and nothing
// hangs; the context stays usable.
// ---------------------------------------------------------------------------
__global__ void wait_probe_kernel(unsigned* __restrict__ err, unsigned long long limit_ns, int site) {
    __shared__ __align__(8) unsigned long long bar;
    const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(addr));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (!mbar_wait_bounded<false>(addr, 0, limit_ns)) atomicOr(err, IB_TIMEOUT_AT(site));
}

IB_EXPORT int ib_wait_probe(unsigned* err, long long limit_ns, int site, void* stream) {
    if (!err || limit_ns <= 0 || limit_ns > 1000000000ll || site < 0 || site > 20) return IB_ERR_BAD_ARG;
    wait_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(err, (unsigned long long)limit_ns, site);
    IB_LAUNCH_CHECK();
    return IB_OK;
}

IB_EXPORT int ib_decode_advance(int* tokens, const int* selected, int* positions, int* kv_len,
                                const int* slot_ids, int pad_slot, int n, void* stream) {
    if (n <= 0) return IB_OK;
    if (!tokens || !positions || !kv_len) return IB_ERR_BAD_ARG;
    { cudaError_t le__ = launch_kernel(decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tokens, selected,
                                                                             positions, kv_len, slot_ids, pad_slot, n); if (le__ != cudaSuccess) return (int)le__; }
    IB_LAUNCH_CHECK();
    return IB_OK;
}
