// bf16 matrix product on the 5th-generation tensor cores (tcgen05) of sm_100a:
//
//     out[t, n] = sum_k X[t, k] * W[n, k]          X: [T, K] tokens, W: [N, K] weights
//
// The weight rows ride on the 128-wide M side of the MMA and the tokens on its
// N side (16..256), so a decode step with a handful of tokens wastes no tensor
// work on padding and the kernel is, in effect, a weight streamer: one CTA owns
// 128 weight rows (and a slice of K when K is split) and pulls them through a
// ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte
// swizzle), a single thread issues tcgen05.mma from shared-memory descriptors
// into a float32 accumulator in tensor memory, and four warps read the
// accumulator back with tcgen05.ld and store it.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      allocates tensor memory; one elected lane issues the MMAs
//   warps 2..5  epilogue: TMEM -> registers -> global (lane = weight row)
//
// Split K: the CTAs that share an output tile form a thread-block cluster (up
// to 8).  Each leaves its float32 partial tile in its own shared memory; after
// a cluster barrier every CTA adds one share of the tile's columns over all
// slices - reading the peers' shared memory directly, in slice order, so the
// sum does not depend on timing - and stores it.  No scratch in global memory.
//
// Every wait on an mbarrier is bounded: when the limit is reached the CTA sets
// IB_FLAG_WAIT_TIMEOUT in the error word, stops issuing work, frees its tensor
// memory and returns.
//
// The reference computes these products with cuBLAS GemmEx
// (infernum-cuda/src/inner/cuda/ops/matmul.rs:68-116); it has no kernel of
// its own for them.
#include "common.cuh"

#include <cuda.h>

using namespace ib;

namespace {

constexpr int BM = 128;       // weight rows per CTA (MMA M)
constexpr int BK = 64;        // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;    // k elements per tcgen05.mma (bf16)
constexpr int NUM_THREADS = 192;

__host__ __device__ constexpr int stage_bytes(int bn) { return BM * BK * 2 + bn * BK * 2; }
__host__ __device__ constexpr int num_stages(int bn) {
    // small token tiles: half of the SM's shared memory, so two CTAs overlap;
    // large ones: as many stages as fit in one CTA
    return bn <= 64 ? (100 * 1024) / stage_bytes(bn) : (200 * 1024) / stage_bytes(bn);
}

// ---- PTX wrappers -------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ bool elect_one() {
    unsigned pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait: false when the limit was reached.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    return mbar_wait_bounded<false>(smem_u32(bar), parity);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, void* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(void* dst_smem, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(dst_smem)),
                 "r"(cols));
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
}
__device__ __forceinline__ void tmem_dealloc(unsigned addr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(cols));
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::
                     "r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 16 consecutive columns of 32-bit values: lane i of the warp gets
// TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld16(unsigned addr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void epilogue_bar_sync() {
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// Reads a float from the shared memory of CTA `rank` of this cluster, at the
// address that `local` has in this CTA.
__device__ __forceinline__ float ld_peer_smem(const float* local, unsigned rank) {
    unsigned raddr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

// The same for four consecutive floats (16-byte aligned).
__device__ __forceinline__ float4 ld_peer_smem4(const float* local, unsigned rank) {
    unsigned raddr;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(raddr) : "memory");
    return v;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 bf16) with the 128-byte swizzle TMA wrote: 8-row groups are 1024 bytes
// apart (stride byte offset), the leading byte offset is 1 (unused for
// swizzled K-major), descriptor version 1 (Blackwell), layout type 2
// (SWIZZLE_128B).  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: float32 accumulator (bits 4-5 = 1), A and B bf16
// (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 at bit 17,
// M >> 4 at bit 24.
__host__ __device__ constexpr unsigned make_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) |
           ((unsigned)(BM >> 4) << 24);
}

struct GemmParams {
    void* out;            // [T, N] bf16 or float32
    unsigned* err;
    int T, N, K;
    int ldo;              // row stride of out, elements
    int splits;           // slices of K = CTAs per cluster (1, 2, 4 or 8)
    int kblocks_per_split;
    int out_f32;
    int swiglu;           // 1: W rows are 64 gates then their 64 ups per tile; out is [T, N/2]
};

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    constexpr int STAGES = num_stages(BN);
    constexpr int STAGE_BYTES = stage_bytes(BN);
    constexpr int W_BYTES = BM * BK * 2;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    static_assert(STAGES >= 2, "too few pipeline stages");

    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long accum_bar;
    __shared__ unsigned tmem_base_slot;
    __shared__ unsigned gave_up;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t_tile = blockIdx.x;   // token tile: fastest, so neighbours share a weight tile
    const int n_tile = blockIdx.y;
    const int split = blockIdx.z;
    const int total_kblocks = (p.K + BK - 1) / BK;
    const int kb_begin = split * p.kblocks_per_split;
    const int kb_end = min(total_kblocks, kb_begin + p.kblocks_per_split);
    const int n_kblocks = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer ------------------------------------------------------
        if (elect_one()) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
            // Weights are written by no kernel, so the first ring of weight
            // tiles is fetched before waiting for the kernel that produces the
            // tokens; only the token tiles have to wait for it.
            const int first = min(STAGES, n_kblocks);
            for (int i = 0; i < first; ++i) {
                unsigned char* ws = smem + (size_t)i * STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], STAGE_BYTES);
                tma_load_2d(ws, &map_w, &full_bar[i], (kb_begin + i) * BK, n_tile * BM);
            }
            pdl_wait();
            for (int i = 0; i < first; ++i) {
                unsigned char* xs = smem + (size_t)i * STAGE_BYTES + W_BYTES;
                tma_load_2d(xs, &map_x, &full_bar[i], (kb_begin + i) * BK, t_tile * BN);
            }
            for (int i = first; i < n_kblocks; ++i) {
                const int s = i % STAGES;
                const unsigned round = i / STAGES;
                if (!mbar_wait(&empty_bar[s], (round - 1) & 1)) {
                    atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_GEMM_PRODUCER));
                    gave_up = 1;
                    break;
                }
                unsigned char* ws = smem + (size_t)s * STAGE_BYTES;
                unsigned char* xs = ws + W_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                const int k0 = (kb_begin + i) * BK;
                tma_load_2d(ws, &map_w, &full_bar[s], k0, n_tile * BM);
                tma_load_2d(xs, &map_x, &full_bar[s], k0, t_tile * BN);
            }
        } else {
            pdl_wait();  // every thread of a dependent waits for the grid before (see common.cuh)
        }
    } else if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------
        pdl_wait();  // (it could issue nothing earlier: every stage holds token tiles too)
        if (elect_one()) {
            constexpr unsigned idesc = make_idesc(BN);
            bool ok = true;
            for (int i = 0; i < n_kblocks && ok; ++i) {
                const int s = i % STAGES;
                const unsigned round = i / STAGES;
                if (!mbar_wait(&full_bar[s], round & 1)) {
                    atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_GEMM_MMA));
                    gave_up = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                unsigned char* ws = smem + (size_t)s * STAGE_BYTES;
                const uint64_t adesc = make_smem_desc(ws);
                const uint64_t bdesc = make_smem_desc(ws + W_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                    // 16 k elements further on: 32 bytes = 2 units of the address field
                    umma_bf16(tmem_base, adesc + 2 * kk, bdesc + 2 * kk, idesc,
                              (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);  // frees the stage when these MMAs are done
            }
            umma_commit(&accum_bar);  // arrives when every MMA above is done
        }
    } else {
        // ---- epilogue: warps 2..5, TMEM lanes 32 * (warp % 4) .. + 31 -------------
        const int quad = warp & 3;
        const int row = quad * 32 + lane;          // weight row within the tile
        const int n = n_tile * BM + row;
        pdl_wait();  // nothing is stored before the kernels ahead of this one are done
        bool ok = mbar_wait(&accum_bar, 0);
        if (!ok && lane == 0) {
            atomicOr(p.err, IB_TIMEOUT_AT(IB_SITE_GEMM_EPILOGUE));
            gave_up = 1;
        }
        tc_fence_after();
        const unsigned taddr = tmem_base + ((unsigned)(quad * 32) << 16);
        const int t0 = t_tile * BN;
        if (p.swiglu) {
            // Rows 0..63 of the tile are gates, rows 64..127 their ups (splits == 1).
            // The up lanes park their values in shared memory (the stages are free:
            // every MMA has completed), the gate lanes fetch them and store
            // silu(gate) * up.  out is [T, N / 2], column n_tile * 64 + row.
            float* xch = reinterpret_cast<float*>(smem);  // [BN][64]
            if (row >= 64 && ok && n_kblocks > 0) {
#pragma unroll
                for (int c = 0; c < BN; c += 16) {
                    unsigned v[16];
                    tmem_ld16(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) xch[(c + j) * 64 + (row - 64)] = __uint_as_float(v[j]);
                }
            }
            epilogue_bar_sync();
            const int col = n_tile * 64 + row;
            if (row < 64 && ok && n_kblocks > 0 && col < p.N / 2) {
#pragma unroll
                for (int c = 0; c < BN; c += 16) {
                    unsigned v[16];
                    tmem_ld16(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c + j;
                        if (t < p.T) {
                            const float g = __uint_as_float(v[j]);
                            const float u = xch[(c + j) * 64 + row];
                            ((bf16*)p.out)[(size_t)t * p.ldo + col] =
                                __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                        }
                    }
                }
            }
        } else if (p.splits == 1) {
            if (ok && n_kblocks > 0) {
#pragma unroll
                for (int c = 0; c < BN; c += 16) {
                    unsigned v[16];
                    tmem_ld16(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c + j;
                        if (t < p.T && n < p.N) {
                            const float f = __uint_as_float(v[j]);
                            if (p.out_f32) ((float*)p.out)[(size_t)t * p.ldo + n] = f;
                            else ((bf16*)p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(f);
                        }
                    }
                }
            }
        } else {
            // my slice's partial tile into my own shared memory: [col][row].
            // The pipeline stages are free by now (every MMA has completed).
            float* red = reinterpret_cast<float*>(smem);
#pragma unroll
            for (int c = 0; c < BN; c += 16) {
                unsigned v[16];
                if (ok && n_kblocks > 0) {
                    tmem_ld16(taddr + c, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(c + j) * BM + row] = __uint_as_float(v[j]);
            }
        }
        tc_fence_before();
    }
    __syncwarp();  // the elected lanes are back with their warps before the aligned barriers
    if (p.splits > 1) {
        cluster_sync_all();  // every slice's partial tile is in place
        if (warp >= 2) {
            const int quad = warp & 3;
            const int row = quad * 32 + lane;
            const int n = n_tile * BM + row;
            const int t0 = t_tile * BN;
            const float* red = reinterpret_cast<const float*>(smem);
            const unsigned rank = cluster_ctarank();
            const int cols_per = (BN + p.splits - 1) / p.splits;
            const int c_begin = (int)rank * cols_per;
            const int c_end = min(BN, c_begin + cols_per);
            // Where the output's rows allow 16-byte (float32) or 8-byte (bfloat16) stores, a
            // thread takes four consecutive weight rows of a token and a warp one token at a
            // time, two tokens a round: 16 loads of 16 bytes in flight instead of 8 of 4.
            const bool vec_ok = (p.N % 4 == 0) && (p.ldo % 4 == 0) && (((uintptr_t)p.out & 15) == 0);
            if (vec_ok) {
                const int r4 = lane * 4;
                const int n4 = n_tile * BM + r4;
                for (int cb = c_begin + quad; cb < c_end; cb += 8) {
                    float4 part[2][8];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int c = cb + 4 * u;
                        const bool live = c < c_end && t0 + c < p.T;
#pragma unroll
                        for (int sidx = 0; sidx < 8; ++sidx)
                            part[u][sidx] = (live && sidx < p.splits)
                                                ? ld_peer_smem4(red + c * BM + r4, (unsigned)sidx)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int c = cb + 4 * u;
                        const int t = t0 + c;
                        if (c >= c_end || t >= p.T || n4 >= p.N) continue;
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int sidx = 0; sidx < 8; ++sidx) {  // in slice order
                            acc.x += part[u][sidx].x;
                            acc.y += part[u][sidx].y;
                            acc.z += part[u][sidx].z;
                            acc.w += part[u][sidx].w;
                        }
                        if (p.out_f32) {
                            *reinterpret_cast<float4*>((float*)p.out + (size_t)t * p.ldo + n4) = acc;
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
                            uint2 packed;
                            packed.x = *reinterpret_cast<unsigned*>(&lo);
                            packed.y = *reinterpret_cast<unsigned*>(&hi);
                            *reinterpret_cast<uint2*>((bf16*)p.out + (size_t)t * p.ldo + n4) = packed;
                        }
                    }
                }
            }
            for (int c = c_begin; c < c_end && !vec_ok; ++c) {
                const int t = t0 + c;
                if (t >= p.T) break;
                // all loads first (they are independent), then the sum in slice order
                float part[8];
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx)
                    part[sidx] = sidx < p.splits ? ld_peer_smem(red + c * BM + row, (unsigned)sidx) : 0.f;
                float acc = 0.f;
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) acc += part[sidx];
                if (n < p.N) {
                    if (p.out_f32) ((float*)p.out)[(size_t)t * p.ldo + n] = acc;
                    else ((bf16*)p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(acc);
                }
            }
        }
        cluster_sync_all();  // nobody leaves while a peer may still read its tile
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side -------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A [rows, cols] bf16 row-major matrix with row stride ld (elements), fetched
// in boxes of box_rows x 64 with the 128-byte swizzle; out-of-range elements
// read as zero.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols,
                    long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return IB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IB_OK : IB_ERR_BAD_ARG;
}

template <int BN>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int t_tiles,
                  int n_tiles, cudaStream_t s) {
    constexpr int smem = num_stages(BN) * stage_bytes(BN) + 1024;
    static_assert(BN * BM * 4 <= num_stages(BN) * stage_bytes(BN), "partial tile must fit the stages");
    if (p.swiglu && BN > 64) return IB_ERR_UNSUPPORTED;  // the exchange buffer is sized for small token tiles
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(t_tiles, n_tiles, p.splits);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = p.splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_flag() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN>, mw, mx, p);
    if (e != cudaSuccess) return (int)e;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

}  // namespace

// The token tile the kernel would use for T tokens.
IB_EXPORT int ib_gemm_tc_token_tile(int T) {
    if (T <= 16) return 16;
    if (T <= 32) return 32;
    if (T <= 64) return 64;
    if (T <= 128) return 128;
    return 256;
}

// out[T, N] = X[T, K] . W[N, K]^T, bf16 operands, out bf16 (out_f32 = 0) or float32.
// ldx, ldw, ldo: row strides in elements.  `splits` (1..8) cuts K over the
// CTAs of a cluster.  swiglu = 1: W holds, per
// 128 rows, 64 gate rows followed by their 64 up rows; out is [T, N / 2] bf16 with
// out[t, 64 b + r] = silu(x . W[128 b + r]) * (x . W[128 b + 64 + r]); K is not split.
IB_EXPORT int ib_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* out, int ldo,
                         int out_f32, int T, int N, int K, int splits, int swiglu, unsigned* err,
                         void* stream) {
    if (T <= 0 || N <= 0) return IB_OK;
    if (!x || !w || !out || !err || K <= 0) return IB_ERR_BAD_ARG;
    // TMA: 16-byte aligned bases and row strides
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || (ldx % 8) || (ldw % 8) || ldx < K || ldw < K ||
        ldo < (swiglu ? N / 2 : N))
        return IB_ERR_UNSUPPORTED;
    if (swiglu && (N % 128 || out_f32)) return IB_ERR_UNSUPPORTED;
    const int bn = ib_gemm_tc_token_tile(T);
    const int t_tiles = (T + bn - 1) / bn, n_tiles = (N + BM - 1) / BM;
    const int kblocks = (K + BK - 1) / BK;
    int sp = splits < 1 ? 1 : (splits > 8 ? 8 : splits);  // a cluster holds at most 8 CTAs
    if (sp > kblocks) sp = kblocks;
    if (swiglu) sp = 1;
    if (n_tiles > 65535) return IB_ERR_TOO_LARGE;
    GemmParams p;
    p.out = out;
    p.err = err;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.kblocks_per_split = (kblocks + sp - 1) / sp;
    p.splits = (kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;  // no empty slice
    p.out_f32 = out_f32;
    p.swiglu = swiglu ? 1 : 0;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, ldw, BM);
    if (rc != IB_OK) return rc;
    rc = make_map(&mx, x, T, K, ldx, bn);
    if (rc != IB_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (bn) {
        case 16: return launch<16>(mw, mx, p, t_tiles, n_tiles, s);
        case 32: return launch<32>(mw, mx, p, t_tiles, n_tiles, s);
        case 64: return launch<64>(mw, mx, p, t_tiles, n_tiles, s);
        case 128: return launch<128>(mw, mx, p, t_tiles, n_tiles, s);
        default: return launch<256>(mw, mx, p, t_tiles, n_tiles, s);
    }
}
