// Prompt attention over the paged cache on the tcgen05 tensor cores (bf16),
// one head size per build (-DIB_HD=64 or 128).
//
// A CTA owns 128 packed rows - query rows of one request times the query heads
// that share one key/value head - and walks the keys in tiles of 64:
//
//   producer warp   TMA: the query tile once (a 3-D box: dims x heads x rows,
//                   which lands in packed-row order), then per tile the pages
//                   of K and of V through the request's block table (2-D
//                   boxes of page_size x 64, 128-byte swizzle)
//   MMA warp        S = Q K^T into tensor memory (8 MMAs of 128 x 64 x 16),
//                   then O += P V (4 MMAs of 128 x HD x 16, P from tensor
//                   memory, V as an N-major operand straight from its
//                   [key][dim] rows)
//   4 softmax warps one thread per packed row = one TMEM lane: read the
//                   scores with tcgen05.ld, mask, running maximum and sum in
//                   32-bit, write P as bf16 back into tensor memory
//                   (tcgen05.st), and rescale the output accumulator there
//                   when a maximum moved.  (Two threads per row, one for each
//                   half of a tile's keys, were slower: 560 against 521 us
//                   for 8,192 tokens.)
//
// Scores, K and V are double-buffered: while the softmax warps work on tile t the
// tensor cores already compute the scores of tile t+1, and K of tile t+2 and V of
// tile t+1 load.  P goes back into tensor memory, over the scores it came from.  The exponents refer to a
// reference maximum that follows the true one only when that rose by more than
// 2^8, so the accumulator is rescaled seldom.  Two CTAs share an SM and fill
// each other's gaps.  Every wait is bounded.
//
// The grid has the kv head on x, the request on y and the row tile on z, the
// last rows first: blocks start in that order, so every long CTA starts before
// any short one.  For a portion after a long cached prefix, whose few row
// tiles would leave the SMs idle, the key tiles of a row tile are shared out
// over 2 or 4 CTAs of one cluster (consecutive in x), which merge their
// unnormalised outputs, maxima and sums through distributed shared memory.
//
// Same mathematics as attention_plain.cu; what it restates of the reference is
// cited there.  The reference has no tensor-core attention kernel.
#include "common.cuh"

#include <cuda.h>

#ifndef IB_HD
#define IB_HD 128
#endif

using namespace ib;

namespace {

constexpr int HD = IB_HD;
static_assert(HD == 64 || HD == 128, "this kernel is built for head sizes 64 and 128");
constexpr int BM = 128;                 // packed rows per CTA
constexpr int BN = 64;                  // keys per tile
constexpr int KB = HD / 64;             // 64-wide blocks of the head dimension
constexpr int SOFTMAX_WARPS = 4;        // one thread per packed row = TMEM lane
constexpr int SOFTMAX_THREADS = SOFTMAX_WARPS * 32;
constexpr int PRODUCER_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int NUM_THREADS = SOFTMAX_THREADS + 64;
constexpr int Q_BYTES = BM * HD * 2;
constexpr int K_BYTES = BN * HD * 2;
constexpr int V_BYTES = BN * HD * 2;
constexpr int TILE_BYTES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES;  // K and V are double-buffered
constexpr int BAR_BYTES = 128;  // the mbarriers and the TMEM address, behind the tiles
// (1 KB more than is used: the tiles start on the next 1 KB boundary of the window)
constexpr int SMEM_BYTES = TILE_BYTES + BAR_BYTES + 1024;
static_assert(2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs must fit an SM (228 KB, 1 KB of it taken per CTA)");
static_assert(HD * BM * 4 + 2 * BM * 4 <= TILE_BYTES, "the merge of key slices reuses the tiles' shared memory");
constexpr unsigned TMEM_COLS = 256;     // two score tiles in columns [0, 64) and [64, 128), output from 128
constexpr unsigned O_COL = 128;

struct Params {
    bf16* out;
    const int* cu_rows;
    const int* q_start;
    const int* block_tables;
    unsigned* err;
    int out_stride, max_blocks, nh, nkv, page_size, num_pages;
    int small_rows;     // entries with rows * min(group, 8) <= small_rows belong to split mode
    int splits;         // CTAs (one cluster) that share the keys of a row tile: 1, 2 or 4
    int entry_offset;   // the grid's y starts at this entry (those before it are all split mode's)
    float scale_log2;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool elect_one() {
    unsigned pred = 0;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}
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
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, void* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A float from the shared memory of CTA `rank` of this cluster, at the address `local` has here.
__device__ __forceinline__ float ld_peer_smem(const float* local, unsigned rank) {
    unsigned raddr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory: row i in lane i, two bf16 of
// consecutive k per 32-bit column (k even in the low half), 8 columns per MMA.
__device__ __forceinline__ void umma_bf16_a_tmem(unsigned tmem_d, unsigned tmem_a, uint64_t bdesc, unsigned idesc,
                                                 unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned addr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_st16(unsigned addr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// Sixty-four consecutive columns of this thread's lane and the wait for them, as
// one statement: the values may be used as soon as it returns, and the four
// loads are in flight together.
__device__ __forceinline__ void tmem_ld64_wait(unsigned addr, float (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%65];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47}, [%66];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%67];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
          "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
          "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
          "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31]),
          "=f"(r[32]), "=f"(r[33]), "=f"(r[34]), "=f"(r[35]), "=f"(r[36]), "=f"(r[37]), "=f"(r[38]), "=f"(r[39]),
          "=f"(r[40]), "=f"(r[41]), "=f"(r[42]), "=f"(r[43]), "=f"(r[44]), "=f"(r[45]), "=f"(r[46]), "=f"(r[47]),
          "=f"(r[48]), "=f"(r[49]), "=f"(r[50]), "=f"(r[51]), "=f"(r[52]), "=f"(r[53]), "=f"(r[54]), "=f"(r[55]),
          "=f"(r[56]), "=f"(r[57]), "=f"(r[58]), "=f"(r[59]), "=f"(r[60]), "=f"(r[61]), "=f"(r[62]), "=f"(r[63])
        : "r"(addr), "r"(addr + 16), "r"(addr + 32), "r"(addr + 48)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 in one 64-bit register, for the packed arithmetic of sm_100 (one
// instruction, two results): the softmax warps are bound by the instructions
// they issue, not by any arithmetic unit.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
// (d0, d1) = (a0, a1) * b + c, b and c packed pairs
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, unsigned long long b,
                                     unsigned long long c) {
    asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tfma.rn.f32x2 rd, ra, %4, %5;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}\n"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "l"(b), "l"(c));
}
// acc += (a0, a1), acc a packed pair
__device__ __forceinline__ void add2(unsigned long long& acc, float a0, float a1) {
    asm("{\n\t.reg .b64 ra;\n\tmov.b64 ra, {%1, %2};\n\tadd.rn.f32x2 %0, %0, ra;\n\t}\n"
        : "+l"(acc) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float sum2(unsigned long long v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// K-major operand tile with 128-byte rows and the 128-byte swizzle: groups of 8
// rows are 1024 bytes apart.  (Addresses and offsets in units of 16 bytes;
// version 1; layout type 2 = SWIZZLE_128B.)
__device__ __forceinline__ uint64_t desc_k_major(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// N-major operand (V as [key][dim] rows of 128 bytes, swizzled): along K, groups
// of 8 keys are 1024 bytes apart (stride byte offset); along N, the next block
// of 64 dims starts `block_bytes` further on (leading byte offset).
__device__ __forceinline__ uint64_t desc_n_major(const void* tile, unsigned block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)((block_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// float32 accumulator, bf16 operands, A K-major; B K-major or N-major (bit 16).
__host__ __device__ constexpr unsigned make_idesc(int n, bool b_n_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_n_major ? (1u << 16) : 0u) |
           ((unsigned)(n >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}

// SPLIT: the variant whose CTAs share a row tile's keys and merge at the end.
template <bool SPLIT>
__device__ __forceinline__ void attention_body(const CUtensorMap& map_q, const CUtensorMap& map_k,
                                               const CUtensorMap& map_v, const Params& p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    if (smem + TILE_BYTES + BAR_BYTES > smem_dyn + SMEM_BYTES) {
        // the window does not start where the budget assumes: refuse rather than overrun
        if (threadIdx.x == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_ATTN_TC_LAYOUT));
        return;
    }
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + Q_BYTES;
    unsigned char* v_s = k_s + 2 * K_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(v_s + 2 * V_BYTES);
    unsigned long long& q_full = bars[0];
    unsigned long long* k_full = bars + 1;
    unsigned long long* k_empty = bars + 3;
    unsigned long long* v_full = bars + 5;
    unsigned long long* v_empty = bars + 7;
    unsigned long long* s_full = bars + 9;
    // p_full: P of tile t is written (phase t).  o_done: the output update of tile t
    // is complete (phase t).  One barrier each is enough, because every waiter
    // follows every phase: the MMA thread waits for p_full of every tile in turn
    // (and P of tile t + 1 needs scores that it issues itself); every softmax thread
    // waits for o_done of tile t - 1 before it hands over P of tile t, without
    // which the update of tile t cannot begin.  A thread that skipped phases could
    // not tell by the parity whether the one it waits for has come.
    unsigned long long& p_full = bars[11];
    unsigned long long& o_done = bars[12];
    unsigned& tmem_slot = *reinterpret_cast<unsigned*>(bars + 13);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks start in the order x, then y, then z.  The row tile is on z, the last rows
    // (which see the most keys) first, so that the long CTAs of every kv head and
    // entry start before any short one; the kv head and the slice of keys are on x.
    const int e = blockIdx.y + p.entry_offset;
    const int G = p.nh / p.nkv;
    const int rq = BM / G;  // query rows per CTA
    const int row0 = p.cu_rows[e];
    const int rows_e = p.cu_rows[e + 1] - row0;
    const int pos0 = p.q_start[e];
    const int gs_split = G < 8 ? G : 8;
    if (rows_e * gs_split <= p.small_rows) return;  // split mode takes this entry
    // The CTAs of a cluster (p.splits of them, consecutive in x) share one row tile
    // and take a slice of its key tiles each; they are merged at the end.
    const int S = SPLIT ? p.splits : 1;
    const int rank = (int)blockIdx.x % S;
    const int g = (int)blockIdx.x / S;
    const int r_begin = ((int)gridDim.z - 1 - (int)blockIdx.z) * rq;
    if (r_begin >= rows_e) return;  // (the whole cluster leaves)
    const int r_count = min(rq, rows_e - r_begin);
    const int kv_hi = pos0 + r_begin + r_count;
    const int all_tiles = (kv_hi + BN - 1) / BN;
    const int per = (all_tiles + S - 1) / S;
    const int t_off = rank * per;                            // my first key tile
    const int n_tiles = max(0, min(all_tiles, t_off + per) - t_off);  // and how many are mine

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        mbar_init(&p_full, SOFTMAX_THREADS);
        mbar_init(&o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_slot;
    pdl_wait();  // queries, keys and values come from the kernels before this one
    // what a softmax thread carries to the merge of the slices
    float m_keep = -INFINITY, l_keep = 0.f;
    bool sm_ok = true;

    if (warp == PRODUCER_WARP) {
        // ---- producer: the whole warp ------------------------------------------------
        // Block-table entries are fetched 32 at a time (one per lane) and handed
        // round with shuffles, so that no TMA copy waits for a dependent load; the
        // pages of a tile are issued by as many lanes in parallel.
        const int* table = p.block_tables + (size_t)e * p.max_blocks;
        const int ppt = BN / p.page_size;                       // pages per tile
        const int total_pages = (kv_hi + p.page_size - 1) / p.page_size;
        if (lane == 0) {
            mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                tma_load_3d(q_s + kb * (BM * 128), &map_q, &q_full, kb * 64, g * G, row0 + r_begin);
        }
        struct Window { int base, page; };
        auto refill = [&](Window& w, int base) {
            w.base = base;
            const int pi = base + lane;
            int page = pi < total_pages ? table[pi] : 0;
            if (page < 0 || page >= p.num_pages) {
                atomicOr(p.err, IB_FLAG_BAD_PAGE);
                page = 0;
            }
            w.page = page;
        };
        Window wk, wv;
        refill(wk, t_off * ppt);
        wv = wk;
        auto load = [&](unsigned char* dst, const CUtensorMap* map, void* full, int t, Window& w) {
            const int pi0 = t * ppt;
            if (pi0 + ppt > w.base + 32) refill(w, pi0);
            if (lane == 0) mbar_expect_tx(full, K_BYTES);
            __syncwarp();
            const int page = __shfl_sync(0xffffffffu, w.page, (pi0 - w.base + lane) & 31);
            if (lane < ppt) {
                const int y = (page * p.nkv + g) * p.page_size;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(dst + kb * (BN * 128) + lane * p.page_size * 128, map, full, kb * 64, y);
            }
        };
        // K of tile t goes to K buffer t % 2 (free once the scores of tile t - 2 are
        // computed), V of tile t to V buffer t % 2 (free once tile t - 2's output
        // update is done), so that a tile's fetch has the time of a whole tile: with
        // one V buffer every output update waited out the latency of its V, which
        // could start only when the update before had ended.  K runs one tile ahead.
        bool ok = true;
        for (int t = 0; t < n_tiles + 1 && ok; ++t) {
            if (t < n_tiles) {
                const int b = t & 1;
                if (t >= 2 && !mbar_wait(&k_empty[b], ((t - 2) >> 1) & 1)) { ok = false; break; }
                load(k_s + b * K_BYTES, &map_k, &k_full[b], t_off + t, wk);
            }
            if (t >= 1) {
                const int tv = t - 1;
                if (tv >= 2 && !mbar_wait(&v_empty[tv & 1], ((tv - 2) >> 1) & 1)) { ok = false; break; }
                load(v_s + (tv & 1) * V_BYTES, &map_v, &v_full[tv & 1], t_off + tv, wv);
            }
        }
        if (!ok && lane == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_ATTN_TC_PRODUCER));
    } else if (warp == MMA_WARP) {
        // ---- MMA issuer -------------------------------------------------------------
        if (elect_one()) {
            constexpr unsigned idesc_s = make_idesc(BN, false);
            constexpr unsigned idesc_o = make_idesc(HD, true);
            bool ok = mbar_wait(&q_full, 0);
            // scores of tile t into score buffer t % 2
            auto issue_scores = [&](int t) -> bool {
                const int b = t & 1;
                if (!mbar_wait(&k_full[b], (t >> 1) & 1)) return false;
                tc_fence_after();
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const uint64_t a = desc_k_major(q_s + kb * (BM * 128));
                    const uint64_t bd = desc_k_major(k_s + b * K_BYTES + kb * (BN * 128));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_bf16(tmem + b * BN, a + 2 * kk, bd + 2 * kk, idesc_s, (kb > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&k_empty[b]);
                umma_commit(&s_full[b]);
                return true;
            };
            if (ok && n_tiles > 0) ok = issue_scores(0);
            for (int t = 0; t < n_tiles && ok; ++t) {
                // The scores of tile t + 1 are computed while the softmax warps work on
                // tile t.  Their buffer held the scores and then P of tile t - 1, which
                // the output update issued in the last round read; MMAs run in order.
                if (t + 1 < n_tiles && !issue_scores(t + 1)) { ok = false; break; }
                // O += P V once the softmax warps have written P (and rescaled O)
                if (!mbar_wait(&p_full, t & 1) || !mbar_wait(&v_full[t & 1], (t >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
                // P lies over the first 32 columns of the tile's score buffer
                const unsigned a = tmem + (unsigned)((t & 1) * BN);
                const uint64_t b = desc_n_major(v_s + (t & 1) * V_BYTES, BN * 128);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)
                    umma_bf16_a_tmem(tmem + O_COL, a + 8 * kk, b + (uint64_t)(kk * ((16 * 128) >> 4)), idesc_o,
                                     (t > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&v_empty[t & 1]);
                umma_commit(&o_done);
            }
            if (!ok) {
                atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_ATTN_TC_MMA));
                // let the softmax warps run out of their waits quickly
            }
        }
    } else {
        // ---- softmax: thread m owns packed row m = TMEM lane m ---------------------
        const int m = threadIdx.x;  // 0..127
        const int r = m / G, h = m % G;
        const bool valid = r < r_count;
        const int my_pos = valid ? pos0 + r_begin + r : -1;
        const unsigned lane_addr = tmem + ((unsigned)(warp * 32) << 16);
        float m_run = -INFINITY, l_run = 0.f;   // the row's reference maximum and its sum
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            if (ok && !mbar_wait(&s_full[t & 1], (t >> 1) & 1)) ok = false;
            tc_fence_after();
            static_assert(BN == 64, "the score tile is read 64 columns at a time");
            float s[BN];
            tmem_ld64_wait(lane_addr + (t & 1) * BN, s);
            // The maxima are kept in raw scores (the scale is positive); the scale and
            // the reference enter the exponent in one multiply-add.
            const int key0 = (t_off + t) * BN;
            if (key0 + BN - 1 > pos0 + r_begin || !valid) {
#pragma unroll
                for (int c = 0; c < BN; ++c) s[c] = (key0 + c <= my_pos) ? s[c] : -INFINITY;
            }
            // the tile's maximum: four chains of three-input maxima over 15 values each,
            // then the chains, the running maximum and the four values left over
            float ch[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                ch[q] = max3(s[16 * q], s[16 * q + 1], s[16 * q + 2]);
#pragma unroll
                for (int i = 3; i < 15; i += 2) ch[q] = max3(ch[q], s[16 * q + i], s[16 * q + i + 1]);
            }
            float m_new = max3(max3(m_run, ch[0], ch[1]), ch[2], ch[3]);
            m_new = max3(max3(m_new, s[15], s[31]), s[47], s[63]);
            // The exponents refer to m_run, which follows the true maximum only when
            // that has risen by more than 2^8 in the exponent: softmax does not depend
            // on the reference, P stays below 256 (fine in bfloat16, the sum is 32-bit),
            // and the output accumulator is rescaled seldom instead of at most tiles.
            float corr = 1.f;
            if (m_new > -INFINITY && (m_run == -INFINITY || (m_new - m_run) * p.scale_log2 > 8.f)) {
                corr = fast_exp2((m_run - m_new) * p.scale_log2);  // 0 from a reference of -inf
                m_run = m_new;
            }
            const float m_scaled = m_run == -INFINITY ? 0.f : m_run * p.scale_log2;
            // exponent = score * scale - reference, two scores per instruction; the sums in
            // four packed accumulators (eight chains of additions)
            const unsigned long long scale2 = pack2(p.scale_log2, p.scale_log2);
            const unsigned long long ref2 = pack2(-m_scaled, -m_scaled);
            unsigned long long acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                fma2(s[c], s[c + 1], s[c], s[c + 1], scale2, ref2);
                s[c] = fast_exp2(s[c]);
                s[c + 1] = fast_exp2(s[c + 1]);
                add2(acc[(c >> 1) & 3], s[c], s[c + 1]);
            }
            const float sum0 = sum2(acc[0]) + sum2(acc[1]), sum1 = sum2(acc[2]) + sum2(acc[3]);
            l_run = l_run * corr + (sum0 + sum1);
            // The update of tile t - 1 began when the exponentials of this tile did and is
            // long complete; the wait is there to follow the barrier's phases, and for the
            // rescaling below.
            if (t > 0 && ok && !mbar_wait(&o_done, (t - 1) & 1)) ok = false;
            // the output accumulator holds tiles 0..t-1: rescale it if any row of
            // this warp moved its reference
            if (t > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 16) {
                    unsigned v[16];
                    tmem_ld16(lane_addr + O_COL + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                    tmem_st16(lane_addr + O_COL + c, v);
                }
            }
            // P (bf16) into tensor memory, where the output update reads it as its A
            // operand: 32 columns of two keys each, over the first half of this tile's
            // score buffer (this lane's scores are in registers).  Through shared memory,
            // P cost a store and a read of 16 KB a tile on the path that also feeds K, V
            // and Q to the tensor core, and that path was the busiest unit of the kernel.
#pragma unroll
            for (int i = 0; i < BN / 32; ++i) {
                unsigned pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 two = __floats2bfloat162_rn(s[32 * i + 2 * j], s[32 * i + 2 * j + 1]);
                    pk[j] = *reinterpret_cast<unsigned*>(&two);
                }
                tmem_st16(lane_addr + (t & 1) * BN + 16 * i, pk);
            }
            tmem_st_wait();
            if (t == n_tiles - 1 && t_off + t == all_tiles - 1 && key0 + BN > kv_hi) {
                // The last tile of the row tile ends beyond the request's keys: what lies
                // there in the page (left by whoever held it before) or in the page that
                // stands in for a missing table entry may be anything, and 0 x Inf or
                // 0 x NaN is NaN in the product P V.  The rows of V from key kv_hi on are
                // cleared in shared memory once the tile has landed (whole 128-byte rows,
                // which the swizzle permutes only within themselves).
                if (ok && !mbar_wait(&v_full[t & 1], (t >> 1) & 1)) ok = false;
                const int first = kv_hi - key0;  // 1..63
                unsigned char* vt = v_s + (t & 1) * V_BYTES;
                for (int i = m; i < (BN - first) * KB * 8; i += SOFTMAX_THREADS) {
                    const int chunk = i & 7, row = first + (i >> 3) % (BN - first), kb = (i >> 3) / (BN - first);
                    *reinterpret_cast<uint4*>(vt + kb * (BN * 128) + row * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(&p_full);
        }
        // ---- epilogue: O / l -------------------------------------------------------
        if (n_tiles > 0) {
            if (ok && !mbar_wait(&o_done, (n_tiles - 1) & 1)) ok = false;
            tc_fence_after();
        }
        if (!ok && lane == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_ATTN_TC_SOFTMAX));
        if (SPLIT) {
            sm_ok = ok;
            m_keep = m_run;
            l_keep = l_run;
        }
        if (S == 1) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = valid ? p.out + (size_t)(row0 + r_begin + r) * p.out_stride + (size_t)(g * G + h) * HD : nullptr;
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                unsigned v[16];
                tmem_ld16(lane_addr + O_COL + c, v);
                tmem_ld_wait();
                if (valid && ok) {
                    uint4 lo, hi;
                    __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        l2[j] = __floats2bfloat162_rn(__uint_as_float(v[2 * j]) * inv, __uint_as_float(v[2 * j + 1]) * inv);
                        h2[j] = __floats2bfloat162_rn(__uint_as_float(v[8 + 2 * j]) * inv,
                                                      __uint_as_float(v[8 + 2 * j + 1]) * inv);
                    }
                    *reinterpret_cast<uint4*>(dst + c) = lo;
                    *reinterpret_cast<uint4*>(dst + c + 8) = hi;
                }
            }
        } else if (rank != 0) {
            // My slice's unnormalised output row, its reference maximum and its sum go to
            // shared memory (the tiles are done with), value c of row m at [c][m] so that
            // neither these stores nor the leader's loads meet in a bank.
            float* mo = reinterpret_cast<float*>(smem);
            float* mm = mo + HD * BM;
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                unsigned v[16];
                if (n_tiles > 0) {
                    tmem_ld16(lane_addr + O_COL + c, v);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) mo[(c + j) * BM + m] = n_tiles > 0 ? __uint_as_float(v[j]) : 0.f;
            }
            mm[m] = m_run;
            mm[BM + m] = l_run;
        }
        tc_fence_before();
    }
    __syncwarp();  // the elected lane is back with its warp before the aligned barriers
    if (S > 1) {
        // ---- merge of the slices: the leader adds the others' rows to its own ----------
        cluster_sync_all();
        if (warp < SOFTMAX_WARPS && rank == 0) {
            tc_fence_after();
            const int m = threadIdx.x;
            const int r = m / G, h = m % G;
            const bool valid = r < r_count;
            const unsigned lane_addr = tmem + ((unsigned)(warp * 32) << 16);
            const float* mo = reinterpret_cast<const float*>(smem);
            const float* mm = mo + HD * BM;
            float m_all = m_keep;
            float m_peer[3], l_peer[3];
            for (int q = 1; q < S; ++q) {
                m_peer[q - 1] = ld_peer_smem(mm + m, (unsigned)q);
                l_peer[q - 1] = ld_peer_smem(mm + BM + m, (unsigned)q);
                m_all = fmaxf(m_all, m_peer[q - 1]);
            }
            // weights 2^((m_i - m_all) * scale); a slice that saw no key of this row weighs nothing
            const float base = m_all == -INFINITY ? 0.f : m_all * p.scale_log2;
            const float w0 = (n_tiles > 0 && m_keep > -INFINITY) ? fast_exp2(fmaf(m_keep, p.scale_log2, -base)) : 0.f;
            float w[3], l_all = w0 * l_keep;
            for (int q = 1; q < S; ++q) {
                w[q - 1] = m_peer[q - 1] > -INFINITY ? fast_exp2(fmaf(m_peer[q - 1], p.scale_log2, -base)) : 0.f;
                l_all += w[q - 1] * l_peer[q - 1];
            }
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            bf16* dst = valid ? p.out + (size_t)(row0 + r_begin + r) * p.out_stride + (size_t)(g * G + h) * HD : nullptr;
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
                unsigned v[16];
                float acc[16];
                if (n_tiles > 0) {
                    tmem_ld16(lane_addr + O_COL + c, v);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = n_tiles > 0 ? w0 * __uint_as_float(v[j]) : 0.f;
                for (int q = 1; q < S; ++q) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] += w[q - 1] * ld_peer_smem(mo + (c + j) * BM + m, (unsigned)q);
                }
                if (valid && sm_ok) {
                    uint4 lo, hi;
                    __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        l2[j] = __floats2bfloat162_rn(acc[2 * j] * inv, acc[2 * j + 1] * inv);
                        h2[j] = __floats2bfloat162_rn(acc[8 + 2 * j] * inv, acc[8 + 2 * j + 1] * inv);
                    }
                    *reinterpret_cast<uint4*>(dst + c) = lo;
                    *reinterpret_cast<uint4*>(dst + c + 8) = hi;
                }
            }
            tc_fence_before();
        }
        cluster_sync_all();  // nobody leaves while the leader may still read its rows
    }
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// Left alone the compiler settles at 96 registers with spills, as if for three CTAs per
// SM; tensor memory allows two, so it may as well use the registers of two.
__global__ void __maxnreg__(128)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const Params p) {
    attention_body<false>(map_q, map_k, map_v, p);
}

__global__ void __launch_bounds__(NUM_THREADS, 2)
attention_tcgen05_split_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_v, const Params p) {
    attention_body<true>(map_q, map_k, map_v, p);
}

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

}  // namespace

IB_EXPORT int ib_attention_tc_head_dim() { return HD; }

// Tile-mode attention for every entry with more rows than split mode takes.
// `splits` (1, 2 or 4): the key tiles of a row tile are shared out over so many
// CTAs of one cluster, which merge their results through distributed shared
// memory; for prompt portions with a long cached prefix, whose row tiles alone
// would leave most SMs idle.  `entry_offset`: the first entry the grid covers (a
// step lists its decoded tokens first; no CTA is launched for them here).
// Needs: bf16, head size 64 or 128, (heads / kv_heads) a divisor of 128,
// page_size a multiple of 8 that divides 64, no window, 16-byte aligned q rows.
IB_EXPORT int ib_attention_tc(const void* q, int q_stride, const void* k_pool, const void* v_pool, void* out,
                              int out_stride, const int* cu_rows, const int* q_start, const int* block_tables,
                              int max_blocks, int n_entries, int n_rows, int max_rows_per_entry, int nh, int nkv,
                              int page_size, int num_pages, float scale, int small_rows, int splits,
                              int entry_offset, unsigned* err, void* stream) {
    if (n_entries <= 0 || n_rows <= 0) return IB_OK;
    if (!q || !k_pool || !v_pool || !out || !cu_rows || !q_start || !block_tables || !err) return IB_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || (splits != 1 && splits != 2 && splits != 4) || entry_offset < 0 ||
        entry_offset >= n_entries)
        return IB_ERR_BAD_ARG;
    const int G = nh / nkv;
    if (BM % G || page_size % 8 || BN % page_size || (q_stride % 8) || (out_stride % 8) ||
        ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
        return IB_ERR_UNSUPPORTED;
    if (n_entries > 65535 || nkv > 65535) return IB_ERR_TOO_LARGE;
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return IB_ERR_UNSUPPORTED;
    const int rq = BM / G;
    CUtensorMap mq, mk, mv;
    {
        // queries as [row][head][dim]; a box of 64 dims x G heads x rq rows lands in
        // packed-row order (row-major over (row, head))
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)n_rows};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)rq};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB_ERR_BAD_ARG;
    }
    for (int which = 0; which < 2; ++which) {
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * nkv * page_size};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        cuuint32_t es[2] = {1, 1};
        if (enc(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                const_cast<void*>(which ? v_pool : k_pool), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB_ERR_BAD_ARG;
    }
    Params p;
    p.out = (bf16*)out;
    p.cu_rows = cu_rows;
    p.q_start = q_start;
    p.block_tables = block_tables;
    p.err = err;
    p.out_stride = out_stride;
    p.max_blocks = max_blocks;
    p.nh = nh;
    p.nkv = nkv;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.small_rows = small_rows;
    p.splits = splits;
    p.entry_offset = entry_offset;
    p.scale_log2 = scale * 1.4426950408889634f;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e1 = cudaFuncSetAttribute(attention_tcgen05_kernel,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e1 != cudaSuccess) return (int)e1;
        e1 = cudaFuncSetAttribute(attention_tcgen05_split_kernel,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e1 != cudaSuccess) return (int)e1;
        attr_done = true;
    }
    const int row_tiles = (max_rows_per_entry + rq - 1) / rq;
    if (row_tiles > 65535) return IB_ERR_TOO_LARGE;
    dim3 grid(nkv * splits, n_entries - entry_offset, row_tiles);
    cudaError_t le;
    if (splits == 1) {
        le = launch_kernel(attention_tcgen05_kernel, grid, dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                           (cudaStream_t)stream, mq, mk, mv, p);
    } else {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_flag() ? 2 : 1;
        le = cudaLaunchKernelEx(&cfg, attention_tcgen05_split_kernel, mq, mk, mv, p);
    }
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
