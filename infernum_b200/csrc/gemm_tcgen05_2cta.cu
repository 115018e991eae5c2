// bf16 matrix product for many tokens (prompts) on pairs of SMs:
//
//     out[t, n] = sum_k X[t, k] * W[n, k]          X: [T, K] tokens, W: [N, K] weights
//
// Two CTAs of a cluster work as one on a tile of 256 tokens x 256 weight rows
// with tcgen05.mma.cta_group::2: each CTA holds 128 of the tokens (its half of
// the M side and of the accumulator, in its own tensor memory) and 128 of the
// weight rows (its half of the N side, which the tensor core of the other CTA
// reads from here too).  So each SM fetches only half of the weight tile from
// shared memory per MMA, which is what lets the pair run at the tensor cores'
// rate; one CTA alone is bound by its shared-memory bandwidth at 128 x 256.
//
// The kernel is persistent: one pair per two SMs walks over the tiles, and the
// accumulator is double-buffered in tensor memory (2 x 256 columns), so that
// the epilogue of a tile runs under the MMAs of the next.
//
//   warp 0      TMA producer: its CTA's token and weight boxes of every k block,
//               completing on the leader CTA's "full" barrier
//   warp 1      allocates tensor memory (both CTAs); in the leader CTA one lane
//               issues the MMAs and commits to the barriers of both CTAs
//   warps 2..9  epilogue (two warps per 32 TMEM lanes, half of the columns each):
//               TMEM -> registers -> bf16 -> 32-byte pieces of a token's row of
//               `out`; with `swiglu`, W holds per 128 rows 64 gate rows and their
//               64 up rows, and silu(gate) * up is written to out[T, N/2]
//
// The weight rows are cut into columns of tiles in two regions: `cols_a` columns
// of `bn_a` rows, then the rest in columns of `bn_b` rows.  The caller picks them
// so that the last round of tiles, which seldom fills all pairs, is a narrow one.
//
// Every wait on an mbarrier is bounded; on a time-out the CTA sets
// IB_FLAG_WAIT_TIMEOUT, stops, frees its tensor memory and returns.
// The kernel is launched in order (see launch_pair), so its griddepcontrol.wait
// returns at once; its launch_dependents still lets the next kernel begin early.
//
// The reference computes these products with cuBLAS GemmEx
// (infernum-cuda/src/inner/cuda/ops/matmul.rs:68-116) and SwiGLU in a kernel of
// its own (infernum-cuda/src/inner/cuda/ops/swiglu.rs).
#include "common.cuh"

#include <cuda.h>

using namespace ib;

namespace {

constexpr int BT = 128;        // tokens per CTA (256 per pair): the M side
constexpr int BNH = 128;       // most weight rows per CTA (256 per pair): the N side
constexpr int TILE = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int X_BYTES = BT * BK * 2;
constexpr int STAGE_BYTES = X_BYTES + BNH * BK * 2;   // 32 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 320;   // producer, MMA and eight epilogue warps
constexpr unsigned TMEM_COLS = 512;   // two accumulators of 256 columns
constexpr unsigned PEER_BIT_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool elect_one() {
    unsigned pred = 0;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One arrival on the barrier at this offset in the leader CTA's shared memory.
__device__ __forceinline__ void mbar_arrive_leader(void* bar) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(bar)), "r"(0u));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    return mbar_wait_bounded<false>(smem_u32(bar), parity);
}
// The same, when arrivals come from the other CTA of the pair too.
__device__ __forceinline__ bool mbar_wait_cluster(void* bar, unsigned parity) {
    return mbar_wait_bounded<true>(smem_u32(bar), parity);
}
// A box into this CTA's shared memory; the bytes are counted on the barrier at
// the same offset in the leader CTA (rank bit cleared).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, void* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc,
                                               unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the MMAs issued so far are done, on the barrier at this offset in
// both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(void* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
        ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned addr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ uint64_t desc_k_major(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// float32 accumulator, bf16 operands, both K-major, M = 256 (the pair), N = bn.
__device__ __forceinline__ unsigned instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(TILE >> 4) << 24);
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// The formula of the other SwiGLU kernels of this package, in float32.
__device__ __forceinline__ float silu_times(float g, float u) { return g / (1.f + expf(-g)) * u; }

// Sixteen values of a token's row, bf16, at out[col .. col+16); `limit` ends the row.
__device__ __forceinline__ void store16(bf16* row, int col, int limit, const float (&v)[16]) {
    if (col + 16 <= limit) {
        uint4 a, b;
        a.x = pack_bf16(v[0], v[1]);   a.y = pack_bf16(v[2], v[3]);
        a.z = pack_bf16(v[4], v[5]);   a.w = pack_bf16(v[6], v[7]);
        b.x = pack_bf16(v[8], v[9]);   b.y = pack_bf16(v[10], v[11]);
        b.z = pack_bf16(v[12], v[13]); b.w = pack_bf16(v[14], v[15]);
        uint4* dst = reinterpret_cast<uint4*>(row + col);
        dst[0] = a;
        dst[1] = b;
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (col + j < limit) row[col + j] = __float2bfloat16_rn(v[j]);
    }
}

struct Params {
    bf16* out;
    unsigned* err;
    int T, N, K, ldo;
    int t_tiles;   // token tiles of 256
    int t_group;   // token tiles of a group: the first region is walked group by group
    int tiles;     // all tiles
    int tiles_a;   // those of the first region
    int bn_a;      // weight rows of a tile (the pair's) there: a multiple of 16, at most 256
    int n_split;   // first weight row of the second region
    int bn_b;      // weight rows of a tile in the second region
};

struct TilePlace {
    int t0;      // first token of the pair's tile
    int n0;      // first weight row
    int bn;      // weight rows
    bool second; // in the second region
};
__device__ __forceinline__ TilePlace locate(const Params& p, int tile) {
    // Neighbours in the list share weights and differ in their tokens.  The first
    // region takes the tokens in groups: all its weight columns for the first
    // `t_group` token tiles, then for the next, so that the tokens which a round of
    // tiles reads stay in L2 however many there are; the weights are then read once
    // per group.  The second region, the list's last round, runs over all tokens.
    TilePlace at;
    at.second = tile >= p.tiles_a;
    if (!at.second) {
        const int cols_a = p.tiles_a / p.t_tiles;
        const int per_group = p.t_group * cols_a;
        const int g = tile / per_group, r = tile - g * per_group;
        const int left = p.t_tiles - g * p.t_group;
        const int tg = left < p.t_group ? left : p.t_group;
        at.bn = p.bn_a;
        at.t0 = (g * p.t_group + r % tg) * TILE;
        at.n0 = (r / tg) * p.bn_a;
    } else {
        const int r = tile - p.tiles_a;
        at.bn = p.bn_b;
        at.t0 = (r % p.t_tiles) * TILE;
        at.n0 = p.n_split + (r / p.t_tiles) * p.bn_b;
    }
    return at;
}

template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_w2, const Params p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_full[2];    // MMAs of a tile are done (both CTAs)
    __shared__ __align__(8) unsigned long long acc_empty[2];   // leader: both epilogues have read it
    __shared__ unsigned tmem_slot;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();           // 0 = leader
    const int n_pairs = gridDim.x >> 1;
    const int first = blockIdx.x >> 1;
    const int n_kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16);   // eight epilogue warps in each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals them
    tc_fence_after();
    const unsigned tmem = tmem_slot;

    if (warp == 0) {
        // ---- producer (both CTAs) ---------------------------------------------------
        if (elect_one()) {
            bool ok = true;
            unsigned it = 0;   // k blocks loaded so far, over all tiles
            pdl_wait();        // the tokens come from the kernel before this one
            for (int tile = first; tile < p.tiles && ok; tile += n_pairs) {
                const TilePlace at = locate(p, tile);
                const int bnh = at.bn >> 1;
                const int t0 = at.t0 + (int)rank * BT, n0 = at.n0 + (int)rank * bnh;
                const CUtensorMap* mw = at.second ? &map_w2 : &map_w;
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % STAGES;
                    const unsigned round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) { ok = false; break; }
                    unsigned char* xs = smem + (size_t)s * STAGE_BYTES;
                    // the leader's barrier counts the bytes of both CTAs
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * (X_BYTES + bnh * BK * 2));
                    tma_load_2d_pair(xs, &map_x, &full_bar[s], i * BK, t0);
                    tma_load_2d_pair(xs + X_BYTES, mw, &full_bar[s], i * BK, n0);
                }
            }
            if (!ok) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_PAIR_PRODUCER));
        } else {
            pdl_wait();  // every thread of a dependent waits for the grid before (see common.cuh)
        }
    } else if (warp == 1) {
        // ---- MMA issuer (leader CTA only) -----------------------------------------------
        pdl_wait();
        if (rank == 0 && elect_one()) {
            bool ok = true;
            unsigned it = 0, j = 0;
            for (int tile = first; tile < p.tiles && ok; tile += n_pairs, ++j) {
                const unsigned buf = j & 1;
                const unsigned idesc = instr_desc(tile < p.tiles_a ? p.bn_a : p.bn_b);
                if (j >= 2 && !mbar_wait_cluster(&acc_empty[buf], ((j >> 1) - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * TILE;
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) { ok = false; break; }
                    tc_fence_after();
                    unsigned char* xs = smem + (size_t)s * STAGE_BYTES;
                    const uint64_t adesc = desc_k_major(xs);
                    const uint64_t bdesc = desc_k_major(xs + X_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_bf16_pair(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[s]);
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
            if (!ok) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_PAIR_MMA));
        }
    } else {
        // ---- epilogue: my 128 tokens x the tile's weight rows, half of them per warp ------------
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int trow = quad * 32 + lane;   // token within my half = TMEM lane
        const int limit = SWIGLU ? p.N / 2 : p.N;
        bool ok = true;
        unsigned j = 0;
        pdl_wait();   // `out` may still be read by the kernel before this one
        for (int tile = first; tile < p.tiles && ok; tile += n_pairs, ++j) {
            const unsigned buf = j & 1;
            ok = mbar_wait(&acc_full[buf], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const TilePlace at = locate(p, tile);
            const int gt = at.t0 + (int)rank * BT + trow;
            const int n0 = at.n0, bn = at.bn;
            const unsigned taddr = tmem + buf * TILE + ((unsigned)(quad * 32) << 16);
            bf16* row = p.out + (size_t)(gt < p.T ? gt : 0) * p.ldo;
            const bool live = gt < p.T;
            if (SWIGLU) {
#pragma unroll 1
                for (int blk = 0; blk < bn / 128; ++blk) {
#pragma unroll
                    for (int c = half * 32; c < half * 32 + 32; c += 16) {
                        unsigned g[16], u[16];
                        tmem_ld16(taddr + blk * 128 + c, g);
                        tmem_ld16(taddr + blk * 128 + 64 + c, u);
                        tmem_ld_wait();
                        float v[16];
#pragma unroll
                        for (int q = 0; q < 16; ++q) v[q] = silu_times(__uint_as_float(g[q]), __uint_as_float(u[q]));
                        if (live) store16(row, n0 / 2 + blk * 64 + c, limit, v);
                    }
                }
            } else {
                const int split = ((bn >> 1) + 15) & ~15;
                const int c_end = half ? bn : split;
#pragma unroll 2
                for (int c = half ? split : 0; c < c_end; c += 32) {
                    const bool two = c + 16 < c_end;   // the same for the whole warp
                    unsigned a[16], b[16];
                    tmem_ld16(taddr + c, a);
                    if (two) tmem_ld16(taddr + c + 16, b);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(a[q]);
                    if (live) store16(row, n0 + c, limit, v);
                    if (two) {
#pragma unroll
                        for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(b[q]);
                        if (live) store16(row, n0 + c + 16, limit, v);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
        if (!ok && lane == 0) atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_PAIR_EPILOGUE));
    }
    __syncwarp();   // the elected lanes are back with their warps before the aligned instructions below
    tc_fence_before();
    cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
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

int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return IB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IB_OK : IB_ERR_BAD_ARG;
}

template <bool SWIGLU>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw2, const Params& p, int pairs,
                cudaStream_t stream) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    // In order, not as a programmatic dependent.  Begun under the tail of its
    // predecessor (where its CTAs, which fill an SM each, sit on the SMs that fall
    // free while the rest of the chain before them still runs), steps of whole
    // 2,048-token prompts at d = 5120 with 40 heads stopped for good now and then:
    // this kernel's MMA issuer, the one role that does not wait for the grid
    // before, reported its time-out, and producers and epilogues never came out of
    // griddepcontrol.wait.  Launched in order, with the same code, they never did
    // (the prologue that no longer overlaps is two or three microseconds a product).
    // In one binary with the variants chosen at run time, the dependent launch also
    // ran clean when every thread waited for the grid before (the MMA warp and the
    // idle lanes too, as they now do) or when the kernel let no successor begin
    // early, and stalled every time as it was.
    cudaError_t le = launch_kernel_in_order(gemm_pair_kernel<SWIGLU>, dim3((unsigned)(pairs * 2)),
                                            dim3(NUM_THREADS), (size_t)SMEM_BYTES, stream, mx, mw, mw2, p);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

}  // namespace

// out[T, N] (bf16) = X[T, K] . W[N, K]^T, bf16 operands; ldx, ldw, ldo in elements.
// With `swiglu`, W holds per 128 rows 64 gate rows followed by their 64 up rows
// (N a multiple of 128) and out[T, N/2] = silu(gate) * up.  Meant for many tokens:
// tiles of 256 tokens, one pair of SMs each; `sm_count` bounds the number of pairs
// that walk over them.  The weight rows are cut into `cols_a` columns of `bn_a`
// rows and the rest into columns of `bn_b` rows (multiples of 16 from 32 to 256; of
// 128 with `swiglu`).
IB_EXPORT int ib_gemm_pair(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int T, int N,
                           int K, int swiglu, int bn_a, int cols_a, int bn_b, int t_group, int sm_count,
                           unsigned* err, void* stream) {
    if (T <= 0 || N <= 0) return IB_OK;
    if (!x || !w || !out || !err || K <= 0 || sm_count < 2 || cols_a < 0) return IB_ERR_BAD_ARG;
    const int out_cols = swiglu ? N / 2 : N;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || (ldx % 8) || (ldw % 8) ||
        (ldo % 8) || ldx < K || ldw < K || ldo < out_cols || (swiglu && N % 128))
        return IB_ERR_UNSUPPORTED;
    const int step = swiglu ? 128 : 16;
    if (bn_a < 32 || bn_a > TILE || bn_a % step || bn_b < 32 || bn_b > TILE || bn_b % step) return IB_ERR_BAD_ARG;
    Params p;
    p.out = (bf16*)out;
    p.err = err;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.t_tiles = (T + TILE - 1) / TILE;
    p.t_group = t_group < 1 || t_group > p.t_tiles ? p.t_tiles : t_group;
    const long long all_a = (N + bn_a - 1) / bn_a;
    const long long a_cols = cols_a < all_a ? cols_a : all_a;
    p.bn_a = bn_a;
    p.bn_b = bn_b;
    p.n_split = (int)(a_cols * bn_a);
    const long long b_cols = p.n_split < N ? (N - p.n_split + bn_b - 1) / bn_b : 0;
    const long long tiles = (a_cols + b_cols) * p.t_tiles;
    if (tiles > 0x3fffffffLL) return IB_ERR_TOO_LARGE;
    p.tiles = (int)tiles;
    p.tiles_a = (int)(a_cols * p.t_tiles);
    const int pairs = (int)(tiles < sm_count / 2 ? tiles : sm_count / 2);
    CUtensorMap mx, mw, mw2;
    int rc = make_map(&mx, x, T, K, ldx, BT);
    if (rc != IB_OK) return rc;
    rc = make_map(&mw, w, N, K, ldw, bn_a / 2);
    if (rc != IB_OK) return rc;
    rc = make_map(&mw2, w, N, K, ldw, bn_b / 2);
    if (rc != IB_OK) return rc;
    return swiglu ? launch_pair<true>(mx, mw, mw2, p, pairs, (cudaStream_t)stream)
                  : launch_pair<false>(mx, mw, mw2, p, pairs, (cudaStream_t)stream);
}
