// Plain attention over the paged cache: one warp per (query row, head), keys
// visited one by one in order, online softmax, everything in 32-bit.  It takes
// any head size, page size, head grouping and window.  It is the attention of
// the 32-bit path and the yardstick the faster kernels are checked against.
//
// For query head a the key/value head is a / (nh / nkv); scores are
// (q . k) * scale; the query at absolute position p sees keys j with
// max(0, p - window + 1) <= j <= p (window <= 0: all keys 0..p); softmax with
// max subtraction and expf; output sum_j P_j v_j.  This restates
// infernum-cuda/kernels/paged_decode_attention.cu:540-644 (decode) and
// infernum-cuda/kernels/flash_prefill_attention_v2.cu:82-95,149-192 (prefill)
// as one kernel over a batch of rows that each carry their own position.
#include "common.cuh"

using namespace ib;

#define PLAIN_MAX_REGS 8  // head sizes up to 256

template <typename T>
__global__ void attention_plain_kernel(const T* __restrict__ q, int q_stride,
                                       const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                       T* __restrict__ out, int out_stride,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ row_entry,
                                       const int* __restrict__ block_tables, int max_blocks,
                                       int nh, int nkv, int hd, int page_size, int num_pages,
                                       int window, float scale, unsigned* __restrict__ err) {
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (head >= nh) return;
    const int g = head / (nh / nkv);
    const int pos = positions[row];
    const int e = row_entry[row];
    const int* table = block_tables + (size_t)e * max_blocks;

    float qr[PLAIN_MAX_REGS], acc[PLAIN_MAX_REGS];
    const T* qp = q + (size_t)row * q_stride + (size_t)head * hd;
#pragma unroll
    for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
        const int d = lane + 32 * i;
        qr[i] = d < hd ? to_f32(qp[d]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j = lo; j <= pos; ++j) {
        const int page = j / page_size < max_blocks ? table[j / page_size] : -1;  // beyond the row: reported, not read
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(err, IB_FLAG_BAD_PAGE);
            continue;
        }
        const size_t off = (((size_t)page * nkv + g) * page_size + (j % page_size)) * hd;
        const T* kp = k_pool + off;
        const T* vp = v_pool + off;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) part += qr[i] * to_f32(kp[d]);
        }
        const float s = warp_sum(part) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) acc[i] = acc[i] * corr + p * to_f32(vp[d]);
        }
        m = m_new;
    }
    T* op = out + (size_t)row * out_stride + (size_t)head * hd;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < PLAIN_MAX_REGS; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) op[d] = from_f32<T>(acc[i] * inv);
    }
}

IB_EXPORT int ib_attention_plain(const void* q, int q_stride, const void* k_pool,
                                 const void* v_pool, void* out, int out_stride, int act_dtype,
                                 const int* positions, const int* row_entry,
                                 const int* block_tables, int max_blocks, int n_rows, int nh,
                                 int nkv, int hd, int page_size, int num_pages, int window,
                                 float scale, unsigned* err, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !row_entry || !block_tables || !err)
        return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0 ||
        num_pages <= 0)
        return IB_ERR_BAD_ARG;
    if (hd > 32 * PLAIN_MAX_REGS) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    dim3 grid(n_rows, (nh + warps - 1) / warps);
    if (act_dtype == 0)
        attention_plain_kernel<float><<<grid, warps * 32, 0, s>>>(
            (const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, (float*)out,
            out_stride, positions, row_entry, block_tables, max_blocks, nh, nkv, hd, page_size,
            num_pages, window, scale, err);
    else if (act_dtype == 1)
        attention_plain_kernel<bf16><<<grid, warps * 32, 0, s>>>(
            (const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out,
            out_stride, positions, row_entry, block_tables, max_blocks, nh, nkv, hd, page_size,
            num_pages, window, scale, err);
    else
        return IB_ERR_UNSUPPORTED;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
