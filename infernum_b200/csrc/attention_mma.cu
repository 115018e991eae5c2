// Tensor-core attention over the paged cache for bfloat16, one head size per
// build (-DIB_HD=<multiple of 16, at most 256>).
//
// One kernel body, two ways of spreading the work:
//   * tile mode (prompt portions): a CTA owns 64 "packed rows" - query rows of
//     one request times the query heads that share one key/value head - and
//     walks the keys in tiles of 64; each of its 4 warps owns 16 packed rows.
//   * split mode (decoded tokens and very short portions): a CTA owns the
//     (at most 8) packed rows of one request and one slice of its keys.  The
//     product is turned around so that the many keys, not the few queries,
//     ride on the 16-wide side of the MMA: S^T = K Q^T (keys x queries) and
//     O^T = V^T P^T (head dims x queries), with the queries on the 8-wide side.
//     The 4 warps each take 16 keys of every tile and are merged at the end.
//     Up to 8 slices of one request are the CTAs of one thread-block cluster
//     and are merged through distributed shared memory; more slices are merged
//     by a second small kernel through scratch memory.
// Keys and values are fetched page by page through the request's block table:
// in split mode by TMA, one bulk copy per page into swizzled shared memory,
// issued by a fifth warp (head sizes that are multiples of 64, pages of a power
// of two of at least 8 tokens); otherwise with 16-byte cp.async copies into
// padded shared-memory rows.  Two tiles are in flight while a third is used.  Scores, the running maximum, the running sum and the output
// accumulator are 32-bit; exponentials are 2^x (ex2.approx, 32-bit) of scores
// pre-multiplied by log2(e).  Key tiles start at absolute multiples of 64, so the order of the
// additions for a query does not depend on how its prompt was cut.
//
// Same mathematics as attention_plain.cu (which restates
// infernum-cuda/kernels/flash_prefill_attention_v2.cu:82-95,149-192 and
// infernum-cuda/kernels/paged_decode_attention.cu:540-644); the reference has
// no tensor-core attention (its bf16 prefill loops cuBLAS per head over a
// materialised score matrix: infernum-cuda/src/inner/cuda/ops/fused_attention.rs:265-473).
#include "common.cuh"

#include <cuda.h>

#ifndef IB_HD
#define IB_HD 128
#endif

using namespace ib;

namespace {

constexpr int HD = IB_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16, at most 256");
constexpr int BN = 64;            // keys per tile
constexpr int LDS = HD + 8;       // padded row length (elements): conflict-free ldmatrix
constexpr int CH = HD / 8;        // 16-byte chunks per row
constexpr int NTHREADS = 128;
constexpr int TILE_ELEMS = BN * LDS;
constexpr int SMEM_BYTES = 4 * TILE_ELEMS * 2;  // tile mode: K and V, two stages
constexpr int SPLIT_STAGES = 3;
constexpr int SPLIT_SMEM_BYTES = SPLIT_STAGES * 2 * TILE_ELEMS * 2;

struct Params {
    const bf16* q;
    const bf16* k_pool;
    const bf16* v_pool;
    bf16* out;
    const int* cu_rows;
    const int* q_start;
    const int* block_tables;
    float* part_o;    // [splits][n_rows][nh][HD]
    float* part_ml;   // [splits][n_rows][nh][2]
    unsigned* err;
    int q_stride, out_stride, max_blocks, nh, nkv, page_size, num_pages, window;
    int gs;           // tile mode: query heads of one kv head handled together (<= 16)
    int n_hsub;       // tile mode: ceil((nh / nkv) / gs)
    int gs_split;     // split mode: the same with at most 8
    int n_hsub_split;
    int splits;       // split mode: slices of keys per request
    int page_shift;   // log2(page_size) when it is a power of two, else -1
    int n_rows;       // rows of the whole step
    int small_rows;   // an entry with rows * gs <= small_rows belongs to split mode
    int cluster_merge;  // split mode: the slices of a request are the CTAs of one cluster
    float scale_log2;
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                            const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2,
                                                  unsigned& r3, const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Reads a float from the shared memory of CTA `rank` of this cluster, at the
// address `local` has in this CTA.
__device__ __forceinline__ float ld_peer_smem(const float* local, unsigned rank) {
    unsigned laddr = (unsigned)__cvta_generic_to_shared(local), raddr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(laddr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}
// 2^x in 32-bit with the hardware approximation (relative error about 2^-22).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Transposes an 8x8 matrix of 16-bit values held one row per 4 lanes.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// How a tile's 64 x CH chunks of 16 bytes are dealt to the 128 threads: chunk
// c = tid + 128 * i, i < LOAD_ITERS, is row c / CH, column c % CH.
constexpr int LOAD_ITERS = (BN * CH + NTHREADS - 1) / NTHREADS;

// Where this thread's rows of a tile live: the raw block-table entries.  The
// loads are issued here and first used by copy_tile one iteration later, so
// their latency is off the critical path.  (Nothing here may depend on the
// loaded value, or the wait for it would move here.)
struct TileRows {
    int page[LOAD_ITERS];   // block-table entry of the row's page (unchecked)
    int tile_start;
};

__device__ __forceinline__ void locate_tile(TileRows& tr, const Params& p, const int* table,
                                            int tile_start) {
    tr.tile_start = tile_start;
#pragma unroll
    for (int i = 0; i < LOAD_ITERS; ++i) {
        const int c = threadIdx.x + NTHREADS * i;
        const int j = tile_start + c / CH;
        int pi = p.page_shift >= 0 ? (j >> p.page_shift) : (j / p.page_size);
        pi = min(pi, p.max_blocks - 1);
        tr.page[i] = table[pi];
    }
}

// Copies one tile into a stage.  Rows outside [kv_min, kv_hi) - pages below
// kv_min may already have been given back by a window - and rows whose
// block-table entry is not a page of the pool are zero-filled.
__device__ __forceinline__ void copy_tile(bf16* ks, bf16* vs, const Params& p, const TileRows& tr,
                                          int g, int kv_min, int kv_hi) {
#pragma unroll
    for (int i = 0; i < LOAD_ITERS; ++i) {
        const int c = threadIdx.x + NTHREADS * i;
        if (c >= BN * CH) break;
        const int row = c / CH, ch = c % CH;
        const int j = tr.tile_start + row;
        const int slot = p.page_shift >= 0 ? (j & (p.page_size - 1)) : (j % p.page_size);
        const int page = tr.page[i];
        const bool in_range = j >= kv_min && j < kv_hi;
        const bool ok = in_range && page >= 0 && page < p.num_pages;
        if (in_range && !ok) atomicOr(p.err, IB_FLAG_BAD_PAGE);
        const size_t src =
            ok ? ((((size_t)page * p.nkv + g) * p.page_size + slot) * HD + ch * 8) : 0;
        cp_async_16(ks + row * LDS + ch * 8, p.k_pool + src, ok ? 16 : 0);
        cp_async_16(vs + row * LDS + ch * 8, p.v_pool + src, ok ? 16 : 0);
    }
}

// Tile mode.
__global__ void __launch_bounds__(NTHREADS) attention_tile_kernel(const Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    pdl_wait();  // queries, keys and values come from the kernels before this one
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_s[2] = {smem, smem + TILE_ELEMS};
    bf16* v_s[2] = {smem + 2 * TILE_ELEMS, smem + 3 * TILE_ELEMS};

    const int e = blockIdx.y;
    const int g = blockIdx.z / p.n_hsub;        // kv head
    const int hsub = blockIdx.z % p.n_hsub;     // which block of the group's query heads
    const int G = p.nh / p.nkv;
    const int row0 = p.cu_rows[e];
    const int rows_e = p.cu_rows[e + 1] - row0;
    const int pos0 = p.q_start[e];
    if (rows_e * p.gs_split <= p.small_rows) return;  // split mode takes this entry

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int* table = p.block_tables + (size_t)e * p.max_blocks;

    // ---- which packed rows are mine ----------------------------------------
    const int rq = BN / p.gs;  // query rows (within the entry) per CTA: 64 packed rows
    // the last rows of a prompt see the most keys: their CTAs go first, so the
    // long ones do not straggle at the end of the grid
    const int r_begin = ((int)gridDim.x - 1 - (int)blockIdx.x) * rq;
    if (r_begin >= rows_e) return;
    const int r_count = min(rq, rows_e - r_begin);
    const int m_base = warp * 16;
    int my_row[2], my_head[2], my_pos[2];  // for packed rows gid and gid + 8 of my 16
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int m = m_base + gid + 8 * h;
        const int r = r_begin + m / p.gs;
        const int hh = hsub * p.gs + m % p.gs;
        const bool ok = (m / p.gs) < r_count && hh < G;
        my_row[h] = ok ? row0 + r : -1;
        my_head[h] = g * G + hh;
        my_pos[h] = ok ? pos0 + r : -1;
    }

    // ---- key range -----------------------------------------------------------
    const int kv_hi = pos0 + r_begin + r_count;  // exclusive
    const int kv_min = p.window > 0 ? max(0, pos0 + r_begin - p.window + 1) : 0;
    const int kv_lo = (kv_min / BN) * BN;
    const int n_tiles = (kv_hi - kv_lo + BN - 1) / BN;
    const int t_begin = 0, t_end = n_tiles;

    // ---- queries as A fragments, straight from global memory -------------------
    unsigned qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = i & 1;
            const int col = ks * 16 + tig * 2 + (i >> 1) * 8;
            qf[ks][i] = my_row[h] >= 0
                ? *reinterpret_cast<const unsigned*>(p.q + (size_t)my_row[h] * p.q_stride +
                                                     (size_t)my_head[h] * HD + col)
                : 0u;
        }
    }

    constexpr int NT = 8;       // score tiles of 8 keys per warp
    constexpr int key_base = 0;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // The copies of tile t+1 are issued while tile t is computed, and the
    // block-table reads for tile t+2 are issued before that, so neither latency
    // sits on the critical path.
    TileRows tr;
    if (t_begin < t_end) {
        locate_tile(tr, p, table, kv_lo + t_begin * BN);
        copy_tile(k_s[0], v_s[0], p, tr, g, kv_min, kv_hi);
    }
    cp_async_commit();
    if (t_begin + 1 < t_end) locate_tile(tr, p, table, kv_lo + (t_begin + 1) * BN);

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t + 1 < t_end) copy_tile(k_s[stage ^ 1], v_s[stage ^ 1], p, tr, g, kv_min, kv_hi);
        cp_async_commit();
        if (t + 2 < t_end) locate_tile(tr, p, table, kv_lo + (t + 2) * BN);
        cp_async_wait<1>();
        __syncthreads();

        const int tile_start = kv_lo + t * BN;
        const bf16* ks_ = k_s[stage];
        const bf16* vs_ = v_s[stage];

        // S = Q K^T
        float s[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                unsigned b0, b1, b2, b3;
                const int key = key_base + n2 * 16 + (lane & 7) + 8 * (lane >> 4);
                const int dim = ks * 16 + 8 * ((lane >> 3) & 1);
                ldmatrix_x4(b0, b1, b2, b3, ks_ + key * LDS + dim);
                mma_bf16(s[2 * n2], qf[ks], b0, b1);
                mma_bf16(s[2 * n2 + 1], qf[ks], b2, b3);
            }
        }

        // mask, scale, online softmax (per thread: rows gid and gid + 8).  Tiles
        // wholly below the diagonal of every row of this CTA need no mask.
        float m_new[2] = {m_run[0], m_run[1]};
        const bool need_mask = p.window > 0 || tile_start + BN - 1 > pos0 + r_begin;
        if (need_mask) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int h = i >> 1;
                    const int key = tile_start + key_base + n * 8 + tig * 2 + (i & 1);
                    const bool ok = key <= my_pos[h] && (p.window <= 0 || key > my_pos[h] - p.window);
                    const float v = ok ? s[n][i] * p.scale_log2 : -INFINITY;
                    s[n][i] = v;
                    m_new[h] = fmaxf(m_new[h], v);
                }
            }
        } else {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[n][i] *= p.scale_log2;
                    m_new[i >> 1] = fmaxf(m_new[i >> 1], s[n][i]);
                }
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
            m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h];
            corr[h] = fast_exp2(m_run[h] - m_use[h]);  // 0 when nothing was seen before
            m_run[h] = m_new[h];
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const float pv = fast_exp2(s[n][i] - m_use[h]);
                s[n][i] = pv;
                l_run[h] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }

        // O += P V
#pragma unroll
        for (int kb = 0; kb < NT / 2; ++kb) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
            a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
            a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
            a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                unsigned b0, b1, b2, b3;
                const int key = key_base + kb * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int dim = nt * 8 + 8 * (lane >> 4);
                ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + key * LDS + dim);
                mma_bf16(o[nt], a, b0, b1);
                mma_bf16(o[nt + 1], a, b2, b3);
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (my_row[h] < 0) continue;
        const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
        bf16* dst = p.out + (size_t)my_row[h] * p.out_stride + (size_t)my_head[h] * HD;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8 + tig * 2) =
                __floats2bfloat162_rn(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
        }
    }
}

// The end of split mode: the 4 warps of a CTA, each of which saw different keys,
// are merged through shared memory (every thread of the block takes part, also
// those of a warp that computed nothing), and then the slices of the request:
// within a cluster through distributed shared memory, else through scratch.
__device__ __forceinline__ void split_merge(const Params& p, unsigned char* smem_raw, const float (&o)[HD / 16][4],
                                            const float (&m_run)[2], const float (&l_run)[2], int g, int hsub,
                                            int row0, int rows_e) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = p.nh / p.nkv;
    const int gs = p.gs_split;
    // ---- merge the 4 warps (each saw different keys) -----------------------------
    __syncthreads();
    float* so = reinterpret_cast<float*>(smem_raw);   // [4][8][HD]
    float* sml = so + 4 * 8 * HD;                     // [4][8][2]
    float* fin = sml + 4 * 8 * 2;                     // [8][HD]   this CTA's result (cluster merge)
    float* finml = fin + 8 * HD;                      // [8][2]
    if (warp < 4) {
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int n = tig * 2 + (i & 1);
                const int d = mt * 16 + gid + 8 * (i >> 1);
                so[((size_t)warp * 8 + n) * HD + d] = o[mt][i];
            }
        }
    }
    if (warp < 4 && gid == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sml[(warp * 8 + tig * 2 + h) * 2] = m_run[h];
            sml[(warp * 8 + tig * 2 + h) * 2 + 1] = l_run[h];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 8 * HD; idx += (int)blockDim.x) {
        const int n = idx / HD, d = idx % HD;
        const int r = n / gs, hh = hsub * gs + n % gs;
        if (r >= rows_e || hh >= G) continue;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, sml[(w * 8 + n) * 2]);
        float acc = 0.f, l = 0.f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(sml[(w * 8 + n) * 2] - mx);
                acc += f * so[((size_t)w * 8 + n) * HD + d];
                l += f * sml[(w * 8 + n) * 2 + 1];
            }
        }
        const int grow = row0 + r, head = g * G + hh;
        if (p.splits == 1) {
            p.out[(size_t)grow * p.out_stride + (size_t)head * HD + d] =
                __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else if (p.cluster_merge) {
            fin[n * HD + d] = acc;
            if (d == 0) {
                finml[n * 2] = mx;
                finml[n * 2 + 1] = l;
            }
        } else {
            const size_t base = ((size_t)blockIdx.x * p.n_rows + grow) * p.nh + head;
            p.part_o[base * HD + d] = acc;
            if (d == 0) {
                p.part_ml[base * 2] = mx;
                p.part_ml[base * 2 + 1] = l;
            }
        }
    }
    if (p.splits > 1 && p.cluster_merge) {
        // The slices of this request are the CTAs of my cluster.  Each has its
        // result in its own shared memory; after a cluster barrier each CTA merges
        // a share of the (column, dim) elements over all slices, in slice order,
        // reading the peers' shared memory directly.
        cluster_sync_all();
        const int total = 8 * HD;
        const int share = (total + p.splits - 1) / p.splits;
        const int begin = (int)blockIdx.x * share, end = min(total, begin + share);
        for (int idx = begin + threadIdx.x; idx < end; idx += (int)blockDim.x) {
            const int n = idx / HD, d = idx % HD;
            const int r = n / gs, hh = hsub * gs + n % gs;
            if (r >= rows_e || hh >= G) continue;
            float mx = -INFINITY;
            for (int sidx = 0; sidx < p.splits; ++sidx)
                mx = fmaxf(mx, ld_peer_smem(finml + n * 2, (unsigned)sidx));
            float acc = 0.f, l = 0.f;
            if (mx > -INFINITY) {
                for (int sidx = 0; sidx < p.splits; ++sidx) {
                    const float f = fast_exp2(ld_peer_smem(finml + n * 2, (unsigned)sidx) - mx);
                    acc += f * ld_peer_smem(fin + n * HD + d, (unsigned)sidx);
                    l += f * ld_peer_smem(finml + n * 2 + 1, (unsigned)sidx);
                }
            }
            p.out[(size_t)(row0 + r) * p.out_stride + (size_t)(g * G + hh) * HD + d] =
                __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        }
        cluster_sync_all();  // nobody leaves while a peer may still read its result
    }
}

// ---------------------------------------------------------------------------
// Split mode.  Packed query columns n in [0, 8): n = r * gs + hh (query row r of
// the entry, head hh of the kv head's group, gs = min(group, 8)).
//   S^T[key, n]  = sum_d K[key, d] Q[n, d]          M = 16 keys of this warp, N = 8, K = HD
//   O^T[d, n]   += sum_key V[key, d] P[key, n]      M = HD, N = 8, K = 16 keys
// K rows feed the A operand through ldmatrix, V rows through ldmatrix.trans,
// Q sits in registers as the B operand, and P goes from the accumulator layout
// to the B layout with two movmatrix transposes.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS) attention_split_kernel(const Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    pdl_wait();  // queries, keys and values come from the kernels before this one
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    // a ring of SPLIT_STAGES stages, each one K tile followed by one V tile
    auto k_stage = [&](int st) { return smem + (size_t)st * 2 * TILE_ELEMS; };
    auto v_stage = [&](int st) { return smem + (size_t)st * 2 * TILE_ELEMS + TILE_ELEMS; };

    const int e = blockIdx.y;
    const int g = blockIdx.z / p.n_hsub_split;
    const int hsub = blockIdx.z % p.n_hsub_split;
    const int G = p.nh / p.nkv;
    const int gs = p.gs_split;
    const int row0 = p.cu_rows[e];
    const int rows_e = p.cu_rows[e + 1] - row0;
    const int pos0 = p.q_start[e];
    if (rows_e * gs > p.small_rows) return;  // tile mode takes this entry

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int* table = p.block_tables + (size_t)e * p.max_blocks;

    // ---- key range of this slice -------------------------------------------------
    const int kv_hi = pos0 + rows_e;
    const int kv_min = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int kv_lo = (kv_min / BN) * BN;
    const int n_tiles = (kv_hi - kv_lo + BN - 1) / BN;
    const int per = (n_tiles + p.splits - 1) / p.splits;
    const int t_begin = blockIdx.x * per;
    const int t_end = min(n_tiles, t_begin + per);

    // Two tiles are in flight while a third is computed: with little arithmetic
    // per byte, what limits this kernel is how many bytes each SM has under way.
    TileRows tr;
#pragma unroll
    for (int pre = 0; pre < SPLIT_STAGES - 1; ++pre) {
        if (t_begin + pre < t_end) {
            locate_tile(tr, p, table, kv_lo + (t_begin + pre) * BN);
            copy_tile(k_stage(pre), v_stage(pre), p, tr, g, kv_min, kv_hi);
        }
        cp_async_commit();
    }
    if (t_begin + SPLIT_STAGES - 1 < t_end)
        locate_tile(tr, p, table, kv_lo + (t_begin + SPLIT_STAGES - 1) * BN);

    // ---- queries as B fragments (column n = gid), while the first tile flies ----------
    unsigned qf[HD / 16][2];
    {
        const int r = gid / gs, hh = hsub * gs + gid % gs;
        const bool ok = r < rows_e && hh < G;
        const bf16* qp = p.q + (size_t)(row0 + (ok ? r : 0)) * p.q_stride + (size_t)(g * G + (ok ? hh : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qf[ks][0] = ok ? *reinterpret_cast<const unsigned*>(qp + ks * 16 + tig * 2) : 0u;
            qf[ks][1] = ok ? *reinterpret_cast<const unsigned*>(qp + ks * 16 + 8 + tig * 2) : 0u;
        }
    }
    // positions of my two score columns (n = tig*2, tig*2 + 1); -1: not a query
    int col_pos[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int n = tig * 2 + h;
        const int r = n / gs, hh = hsub * gs + n % gs;
        col_pos[h] = (r < rows_e && hh < G) ? pos0 + r : -1;
    }

    float o[HD / 16][4];  // O^T: rows = head dims, my columns tig*2, tig*2 + 1
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int key_base = warp * 16;

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) % SPLIT_STAGES;
        cp_async_wait<SPLIT_STAGES - 2>();  // tile t has landed
        __syncthreads();                    // and everyone is done with tile t - 1
        if (t + SPLIT_STAGES - 1 < t_end) {
            const int nst = (t - t_begin + SPLIT_STAGES - 1) % SPLIT_STAGES;  // the stage of tile t - 1
            copy_tile(k_stage(nst), v_stage(nst), p, tr, g, kv_min, kv_hi);
        }
        cp_async_commit();
        if (t + SPLIT_STAGES < t_end) locate_tile(tr, p, table, kv_lo + (t + SPLIT_STAGES) * BN);

        const int tile_start = kv_lo + t * BN;
        const bf16* ks_ = k_stage(stage);
        const bf16* vs_ = v_stage(stage);

        // S^T for my 16 keys
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            unsigned a[4];
            const int key = key_base + (lane & 7) + 8 * ((lane >> 3) & 1);
            const int dim = ks * 16 + 8 * (lane >> 4);
            ldmatrix_x4(a[0], a[1], a[2], a[3], ks_ + key * LDS + dim);
            mma_bf16(sc, a, qf[ks][0], qf[ks][1]);
        }
        // mask and scale: sc[0], sc[1] belong to key gid, sc[2], sc[3] to key gid + 8
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = i & 1;
            const int key = tile_start + key_base + gid + 8 * (i >> 1);
            const bool ok = key <= col_pos[h] && (p.window <= 0 || key > col_pos[h] - p.window);
            sc[i] = ok ? sc[i] * p.scale_log2 : -INFINITY;
            m_new[h] = fmaxf(m_new[h], sc[i]);
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // the keys of a column are spread over the lanes with the same tig
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 4));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 8));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 16));
            m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h];
            corr[h] = fast_exp2(m_run[h] - m_use[h]);
            m_run[h] = m_new[h];
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sc[i] = fast_exp2(sc[i] - m_use[i & 1]);
            l_run[i & 1] += sc[i];
        }
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[1];
            o[i][2] *= corr[0];
            o[i][3] *= corr[1];
        }
        // P^T as the B operand: (keys tig*2, tig*2+1 ; column gid), then keys + 8
        const unsigned b0 = movmatrix_trans(pack_bf16(sc[0], sc[1]));
        const unsigned b1 = movmatrix_trans(pack_bf16(sc[2], sc[3]));
        // O^T += V^T P^T
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) {
            unsigned a[4];
            const int mi = lane >> 3;
            const int key = key_base + (lane & 7) + 8 * (mi >> 1);
            const int dim = mt * 16 + 8 * (mi & 1);
            ldmatrix_x4_trans(a[0], a[1], a[2], a[3], vs_ + key * LDS + dim);
            mma_bf16(o[mt], a, b0, b1);
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }

    split_merge(p, smem_raw, o, m_run, l_run, g, hsub, row0, rows_e);
}

#if IB_HD % 64 == 0
// ---------------------------------------------------------------------------
// Split mode with keys and values fetched by TMA: the same mathematics, but a
// fifth warp brings whole pages into 128-byte-swizzled shared memory with one
// bulk copy each, so that the four computing warps spend no instructions on
// addresses and copies and need no block-wide barrier per tile (each stage has
// a "full" and an "empty" mbarrier; every wait is bounded).  For head sizes
// that are multiples of 64 and pages of 8, 16, 32, 64, 128, ... tokens.
//
// A stage holds a K tile and a V tile, each as HD / 64 blocks of 64 rows x
// 128 bytes: element (row, dim) of a tile lies at block dim / 64, row `row`,
// 16-byte chunk ((dim % 64) / 8) ^ (row % 8).
//
// Whole pages are copied, so rows outside the request's keys hold whatever the
// page held: their scores are masked, and the warp that owns them clears their
// V rows in shared memory first (0 x anything must be 0).  Pages outside the
// key range are not looked up (a window may have given them back); page 0 is
// fetched in their place.
// ---------------------------------------------------------------------------
constexpr int TMA_KB = HD / 64;
constexpr int TMA_BLOCK_BYTES = BN * 128;                   // 64 rows x 128 bytes
constexpr int TMA_TILE_BYTES = TMA_KB * TMA_BLOCK_BYTES;
constexpr int TMA_STAGE_BYTES = 2 * TMA_TILE_BYTES;         // K and V
constexpr int TMA_STAGES = 3;
constexpr int TMA_SMEM_BYTES = TMA_STAGES * TMA_STAGE_BYTES + 1024;
constexpr int TMA_THREADS = 160;
static_assert(4 * 8 * HD * 4 + 4 * 8 * 2 * 4 + 8 * HD * 4 + 8 * 2 * 4 <= TMA_STAGES * TMA_STAGE_BYTES,
              "the merge buffers reuse the stages");

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    return mbar_wait_bounded<false>(smem_u32(bar), parity);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, void* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Element (row, dim) of a swizzled tile; dim a multiple of 8.
__device__ __forceinline__ const bf16* swz(const bf16* tile, int row, int dim) {
    return tile + (dim >> 6) * (TMA_BLOCK_BYTES / 2) + row * 64 + ((((dim & 63) >> 3) ^ (row & 7)) << 3);
}

__global__ void __launch_bounds__(TMA_THREADS, 2)
attention_split_tma_kernel(const Params p, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[TMA_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[TMA_STAGES];
    pdl_trigger();
    unsigned char* smem_raw = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    auto k_stage = [&](int st) { return reinterpret_cast<bf16*>(smem_raw + (size_t)st * TMA_STAGE_BYTES); };
    auto v_stage = [&](int st) {
        return reinterpret_cast<bf16*>(smem_raw + (size_t)st * TMA_STAGE_BYTES + TMA_TILE_BYTES);
    };
    if (threadIdx.x == 0) {
#pragma unroll
        for (int st = 0; st < TMA_STAGES; ++st) {
            mbar_init(&full_bar[st], 1);
            mbar_init(&empty_bar[st], 4);   // the four computing warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    // What the kernel before this one wrote - the queries, and the keys and values
    // of this step's tokens - is waited for where it is first needed: the computing
    // warps wait before they read the queries, the producer before the first tile
    // that holds a token of this step.  Older keys and values, the block tables
    // and the step's positions were complete before this chain of kernels began,
    // so the first tiles are under way while the predecessor finishes.

    const int e = blockIdx.y;
    const int g = blockIdx.z / p.n_hsub_split;
    const int hsub = blockIdx.z % p.n_hsub_split;
    const int G = p.nh / p.nkv;
    const int gs = p.gs_split;
    const int row0 = p.cu_rows[e];
    const int rows_e = p.cu_rows[e + 1] - row0;
    const int pos0 = p.q_start[e];
    if (rows_e * gs > p.small_rows) return;  // tile mode takes this entry (the whole block leaves)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;

    const int kv_hi = pos0 + rows_e;
    const int kv_min = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int kv_lo = (kv_min / BN) * BN;
    const int n_tiles = (kv_hi - kv_lo + BN - 1) / BN;
    const int per = (n_tiles + p.splits - 1) / p.splits;
    const int t_begin = blockIdx.x * per;
    const int t_end = min(n_tiles, t_begin + per);

    float o[HD / 16][4];  // O^T: rows = head dims, my columns tig*2, tig*2 + 1
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (warp == 4) {
        // ---- producer ---------------------------------------------------------------
        // Lane i fetches the i-th page of a tile (one lane when a page holds the
        // whole tile).  The block-table entry of the next tile is read while this
        // tile's copies are issued, so no copy waits for a dependent load.
        const int* table = p.block_tables + (size_t)e * p.max_blocks;
        const int box_rows = p.page_size < BN ? p.page_size : BN;
        const int ppt = BN / box_rows;
        const int first_page = kv_min >> p.page_shift, last_page = (kv_hi - 1) >> p.page_shift;
        auto lookup = [&](int t) -> int {
            const int pi = (kv_lo + t * BN + lane * box_rows) >> p.page_shift;
            return (lane < ppt && t < t_end && pi >= first_page && pi <= last_page && pi < p.max_blocks)
                       ? table[pi] : 0;
        };
        int page_next = lookup(t_begin);
        bool ok = true;
        const int t_wait = (pos0 - kv_lo) / BN;  // the first tile with a token of this step
        bool waited = false;
        for (int t = t_begin; t < t_end; ++t) {
            const int i = t - t_begin, st = i % TMA_STAGES;
            int page = page_next;
            page_next = lookup(t + 1);
            if (!waited && t >= t_wait) {
                pdl_wait();
                waited = true;
            }
            if (i >= TMA_STAGES && !mbar_wait(&empty_bar[st], ((i / TMA_STAGES) - 1) & 1)) { ok = false; break; }
            if (lane == 0) mbar_expect_tx(&full_bar[st], TMA_STAGE_BYTES);
            __syncwarp();
            if (lane < ppt) {
                if (page < 0 || page >= p.num_pages) {
                    atomicOr(p.err, IB_FLAG_BAD_PAGE);
                    page = 0;
                }
                const int key0 = kv_lo + t * BN + lane * box_rows;
                const int y = (page * p.nkv + g) * p.page_size + (key0 & (p.page_size - 1));
                unsigned char* kd = reinterpret_cast<unsigned char*>(k_stage(st)) + lane * box_rows * 128;
                unsigned char* vd = reinterpret_cast<unsigned char*>(v_stage(st)) + lane * box_rows * 128;
#pragma unroll
                for (int kb = 0; kb < TMA_KB; ++kb) {
                    tma_load_2d(kd + kb * TMA_BLOCK_BYTES, &map_k, &full_bar[st], kb * 64, y);
                    tma_load_2d(vd + kb * TMA_BLOCK_BYTES, &map_v, &full_bar[st], kb * 64, y);
                }
            }
        }
        if (!ok && lane == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_SPLIT_PRODUCER));
        if (!waited) pdl_wait();  // this warp helps to write the result, which a predecessor may still read
    } else {
        // ---- the four computing warps -----------------------------------------------------
        pdl_wait();
        unsigned qf[HD / 16][2];
        {
            const int r = gid / gs, hh = hsub * gs + gid % gs;
            const bool okq = r < rows_e && hh < G;
            const bf16* qp =
                p.q + (size_t)(row0 + (okq ? r : 0)) * p.q_stride + (size_t)(g * G + (okq ? hh : 0)) * HD;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                qf[ks][0] = okq ? *reinterpret_cast<const unsigned*>(qp + ks * 16 + tig * 2) : 0u;
                qf[ks][1] = okq ? *reinterpret_cast<const unsigned*>(qp + ks * 16 + 8 + tig * 2) : 0u;
            }
        }
        int col_pos[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = tig * 2 + h;
            const int r = n / gs, hh = hsub * gs + n % gs;
            col_pos[h] = (r < rows_e && hh < G) ? pos0 + r : -1;
        }
        const int key_base = warp * 16;
        bool ok = true;
        for (int t = t_begin; t < t_end; ++t) {
            const int i = t - t_begin, st = i % TMA_STAGES;
            if (!mbar_wait(&full_bar[st], (i / TMA_STAGES) & 1)) { ok = false; break; }
            const int tile_start = kv_lo + t * BN;
            const bf16* ks_ = k_stage(st);
            bf16* vs_ = v_stage(st);
            if (tile_start < kv_min || tile_start + BN > kv_hi) {
                // clear the V rows of my keys that are not the request's
                for (int c = lane; c < 16 * CH; c += 32) {
                    const int row = key_base + c / CH, key = tile_start + row;
                    if (key < kv_min || key >= kv_hi)
                        *reinterpret_cast<uint4*>(const_cast<bf16*>(swz(vs_, row, (c % CH) * 8))) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
                // these ordinary stores come before the bulk copy that refills the stage later
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
            }

            // S^T for my 16 keys
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                unsigned a[4];
                const int key = key_base + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int dim = ks * 16 + 8 * (lane >> 4);
                ldmatrix_x4(a[0], a[1], a[2], a[3], swz(ks_, key, dim));
                mma_bf16(sc, a, qf[ks][0], qf[ks][1]);
            }
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int h = q & 1;
                const int key = tile_start + key_base + gid + 8 * (q >> 1);
                const bool in = key <= col_pos[h] && (p.window <= 0 || key > col_pos[h] - p.window);
                sc[q] = in ? sc[q] * p.scale_log2 : -INFINITY;
                m_new[h] = fmaxf(m_new[h], sc[q]);
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 4));
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 8));
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 16));
                m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h];
                corr[h] = fast_exp2(m_run[h] - m_use[h]);
                m_run[h] = m_new[h];
                l_run[h] *= corr[h];
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                sc[q] = fast_exp2(sc[q] - m_use[q & 1]);
                l_run[q & 1] += sc[q];
            }
#pragma unroll
            for (int q = 0; q < HD / 16; ++q) {
                o[q][0] *= corr[0];
                o[q][1] *= corr[1];
                o[q][2] *= corr[0];
                o[q][3] *= corr[1];
            }
            const unsigned b0 = movmatrix_trans(pack_bf16(sc[0], sc[1]));
            const unsigned b1 = movmatrix_trans(pack_bf16(sc[2], sc[3]));
#pragma unroll
            for (int mt = 0; mt < HD / 16; ++mt) {
                unsigned a[4];
                const int mi = lane >> 3;
                const int key = key_base + (lane & 7) + 8 * (mi >> 1);
                const int dim = mt * 16 + 8 * (mi & 1);
                ldmatrix_x4_trans(a[0], a[1], a[2], a[3], swz(vs_, key, dim));
                mma_bf16(o[mt], a, b0, b1);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);   // my warp is done with this stage
        }
        if (!ok && lane == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_SPLIT_COMPUTE));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
        }
    }
    split_merge(p, smem_raw, o, m_run, l_run, g, hsub, row0, rows_e);
}
#endif  // IB_HD % 64 == 0

// Merges the slices of split mode: one block per (row, head).
__global__ void attention_combine_kernel(const Params p) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y;
    float mx = -INFINITY;
    for (int s = 0; s < p.splits; ++s)
        mx = fmaxf(mx, p.part_ml[(((size_t)s * p.n_rows + row) * p.nh + head) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f, l = 0.f;
        if (mx > -INFINITY) {
            for (int s = 0; s < p.splits; ++s) {
                const size_t base = ((size_t)s * p.n_rows + row) * p.nh + head;
                const float f = exp2f(p.part_ml[base * 2] - mx);
                acc += f * p.part_o[base * HD + d];
                l += f * p.part_ml[base * 2 + 1];
            }
        }
        p.out[(size_t)row * p.out_stride + (size_t)head * HD + d] =
            __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
}

#if IB_HD % 64 == 0
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A pool [pages][kv heads][page_size][HD] as rows of HD values; a box is 64 values
// of up to 64 consecutive rows (one page, or the tile's part of a larger page).
bool make_pool_map(CUtensorMap* map, const void* pool, long long rows, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
#endif

}  // namespace

IB_EXPORT int ib_attention_mma_head_dim() { return HD; }

// Bytes of scratch that `splits` slices need: partial outputs and statistics.
IB_EXPORT long long ib_attention_mma_scratch_bytes(int n_rows, int nh, int splits) {
    if (splits <= 1) return 0;
    return (long long)splits * n_rows * nh * (HD + 2) * (long long)sizeof(float);
}

// mode bits: 1 = launch tile mode, 2 = launch split mode.  With both, an entry
// whose rows times min(group, 8) is at most 8 goes to split mode and the rest
// to tile mode; with one bit every entry is taken by that mode, except that
// split mode can never take an entry with more than 8 packed rows.  Bit 4 with
// bit 2: the tile-mode entries were computed by another kernel; only the small
// entries are taken here.  Bit 8: split mode fetches keys and values with cp.async
// also where it could use TMA (head size a multiple of 64, pages of a power of
// two of at least 8 tokens).
IB_EXPORT int ib_attention_mma(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                               void* out, int out_stride, const int* cu_rows, const int* q_start,
                               const int* block_tables, int max_blocks, int n_entries, int n_rows,
                               int max_rows_per_entry, int nh, int nkv, int page_size,
                               int num_pages, int window, float scale, int mode, int splits,
                               void* scratch, long long scratch_bytes, unsigned* err,
                               void* stream) {
    if (n_entries <= 0 || n_rows <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !cu_rows || !q_start || !block_tables || !err)
        return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 || num_pages <= 0 ||
        (q_stride & 1) || (out_stride & 1) || !(mode & 3) || splits < 1)
        return IB_ERR_BAD_ARG;
    if (((uintptr_t)q & 3) || ((uintptr_t)out & 3) || ((uintptr_t)k_pool & 15) ||
        ((uintptr_t)v_pool & 15))
        return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    Params p;
    p.q = (const bf16*)q;
    p.k_pool = (const bf16*)k_pool;
    p.v_pool = (const bf16*)v_pool;
    p.out = (bf16*)out;
    p.cu_rows = cu_rows;
    p.q_start = q_start;
    p.block_tables = block_tables;
    p.err = err;
    p.q_stride = q_stride;
    p.out_stride = out_stride;
    p.max_blocks = max_blocks;
    p.nh = nh;
    p.nkv = nkv;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.window = window;
    p.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if ((1 << b) == page_size) p.page_shift = b;
    const int G = nh / nkv;
    p.gs = G < 16 ? G : 16;
    p.n_hsub = (G + p.gs - 1) / p.gs;
    p.gs_split = G < 8 ? G : 8;
    p.n_hsub_split = (G + p.gs_split - 1) / p.gs_split;
    p.splits = splits;
    p.n_rows = n_rows;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.part_o = nullptr;
    p.part_ml = nullptr;
    p.cluster_merge = 0;
    // which entries each mode takes
    const bool no_tma = (mode & 8) != 0;
    (void)no_tma;
    mode &= 7;
    const bool tiles_done_elsewhere = (mode & 4) != 0;  // another kernel took the tile-mode entries
    if (tiles_done_elsewhere) mode = 2;
    if ((mode & 3) == 3 || tiles_done_elsewhere) p.small_rows = 8;
    else if (mode & 2) p.small_rows = 1 << 30;   // everything is "small"
    else p.small_rows = -1;                      // nothing is "small"
    if ((mode & 2) && !(mode & 1) && !tiles_done_elsewhere && max_rows_per_entry * p.gs_split > 8)
        return IB_ERR_BAD_ARG;
    if (n_entries > 65535 || nkv * p.n_hsub > 65535) return IB_ERR_TOO_LARGE;

    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e1 = cudaFuncSetAttribute(attention_tile_kernel,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaError_t e2 = cudaFuncSetAttribute(attention_split_kernel,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, SPLIT_SMEM_BYTES);
        if (e1 != cudaSuccess) return (int)e1;
        if (e2 != cudaSuccess) return (int)e2;
        attr_done = true;
    }
    if (mode & 1) {
        const int rq = BN / p.gs;
        dim3 grid((max_rows_per_entry + rq - 1) / rq, n_entries, nkv * p.n_hsub);
        cudaError_t le = launch_kernel(attention_tile_kernel, grid, dim3(NTHREADS), SMEM_BYTES, s, p);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
    }
    if (mode & 2) {
        // only rows that split mode handled could be merged: with both modes in
        // one step the caller keeps splits at 1
        if (splits > 1 && (mode & 1)) return IB_ERR_BAD_ARG;
        if (splits > 8) {
            const long long need = ib_attention_mma_scratch_bytes(n_rows, nh, splits);
            if (!scratch || scratch_bytes < need || ((uintptr_t)scratch & 15)) return IB_ERR_BAD_ARG;
            p.part_o = (float*)scratch;
            p.part_ml = p.part_o + (size_t)splits * n_rows * nh * HD;
        }
        dim3 grid(splits, n_entries, nkv * p.n_hsub_split);
        p.cluster_merge = (splits > 1 && splits <= 8) ? 1 : 0;
        bool use_tma = false;
#if IB_HD % 64 == 0
        CUtensorMap map_k, map_v;
        const long long pool_rows = (long long)num_pages * nkv * page_size;
        if (!no_tma && p.page_shift >= 3 && pool_rows < 0x7fffffffLL) {
            const int box_rows = page_size < BN ? page_size : BN;
            use_tma = make_pool_map(&map_k, k_pool, pool_rows, box_rows) &&
                      make_pool_map(&map_v, v_pool, pool_rows, box_rows);
        }
        if (use_tma) {
            static bool tma_attr_done = false;
            if (!tma_attr_done) {
                cudaError_t e3 = cudaFuncSetAttribute(attention_split_tma_kernel,
                                                      cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_SMEM_BYTES);
                if (e3 != cudaSuccess) return (int)e3;
                tma_attr_done = true;
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(TMA_THREADS);
            cfg.dynamicSmemBytes = TMA_SMEM_BYTES;
            cfg.stream = s;
            cudaLaunchAttribute attr[2];
            int n_attr = 0;
            if (p.cluster_merge) {
                attr[n_attr].id = cudaLaunchAttributeClusterDimension;
                attr[n_attr].val.clusterDim.x = splits;
                attr[n_attr].val.clusterDim.y = 1;
                attr[n_attr].val.clusterDim.z = 1;
                ++n_attr;
            }
            if (pdl_flag()) {
                attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
                ++n_attr;
            }
            cfg.attrs = attr;
            cfg.numAttrs = n_attr;
            cudaError_t le = cudaLaunchKernelEx(&cfg, attention_split_tma_kernel, p, map_k, map_v);
            if (le != cudaSuccess) return (int)le;
            IB_LAUNCH_CHECK();
        }
#endif
        if (use_tma) {
            // launched above
        } else if (p.cluster_merge) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(NTHREADS);
            cfg.dynamicSmemBytes = SPLIT_SMEM_BYTES;
            cfg.stream = s;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = splits;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl_flag() ? 2 : 1;
            cudaError_t le = cudaLaunchKernelEx(&cfg, attention_split_kernel, p);
            if (le != cudaSuccess) return (int)le;
            IB_LAUNCH_CHECK();
        } else {
            cudaError_t le =
                launch_kernel(attention_split_kernel, grid, dim3(NTHREADS), SPLIT_SMEM_BYTES, s, p);
            if (le != cudaSuccess) return (int)le;
            IB_LAUNCH_CHECK();
        }
        if (splits > 1 && !p.cluster_merge) {
            dim3 cgrid(n_rows, nh);
            cudaError_t le = launch_kernel(attention_combine_kernel, cgrid, dim3(HD >= 128 ? 128 : 64), 0, s, p);
            if (le != cudaSuccess) return (int)le;
            IB_LAUNCH_CHECK();
        }
    }
    return IB_OK;
}
