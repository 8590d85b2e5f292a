#pragma once
// A persistent, warp-specialised bf16 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fp32
// accumulation in tensor memory. Either operand may instead be given with the contraction along
// its rows (A stored K x M, B stored K x N, "MN-major"): the weight gradient of a linear layer
// contracts over the tokens and reads dY and X as they lie in memory, without a transposed copy.
//
//   warp 0      TMA producer: A and B tiles (128B-swizzled, K-major) into a 4-stage shared-memory ring
//   warp 1      MMA issuer:   one elected thread issues tcgen05.mma 128x256x16, accumulators in TMEM
//   warps 2..5  epilogue:     tcgen05.ld the accumulator (each warp owns a 32-lane quarter) and apply
//                             the epilogue functor; double-buffered accumulators (2 x 256 TMEM
//                             columns) let the epilogue of tile i overlap the main loop of tile i+1
//
// One CTA per SM, tiles visited in bands of 16 M-tiles so that a wave of CTAs shares A and B tiles
// through L2. No TMA load is multicast; every CTA fetches its own tiles.
//
// The epilogue is a template parameter: a functor called by the four epilogue warps with the
// accumulator buffer of a finished tile. Kernels that write peers' memory from the epilogue run
// their handshake through `Epi::open` / `Epi::close`.
#include <cuda.h>
#include <cuda_bf16.h>

#include "handshake.cuh"
#include "ptx.cuh"

namespace fu {
namespace gemm {

constexpr int BM       = 128;
constexpr int BN       = 256;
constexpr int BK       = 64;   // one 128-byte swizzle atom of bf16
constexpr int UMMA_K   = 16;
constexpr int STAGES   = 4;
constexpr int A_BYTES  = BM * BK * 2;
constexpr int B_BYTES  = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES  = STAGES * STAGE_BYTES + 1024;  // + slack to align the ring to 1024 B
constexpr int THREADS  = 192;
constexpr int BAND     = 16;   // M-tiles per rasterisation band
constexpr int TMEM_COLS = 512;

enum : uint32_t {
    ERR_NONE = 0,
    ERR_PRODUCER_WAIT = 1,
    ERR_MMA_WAIT_FULL = 2,
    ERR_MMA_WAIT_TMEM = 3,
    ERR_EPI_WAIT      = 4,
};

struct Core {
    CUtensorMap map_a;
    CUtensorMap map_b;
    int         M, N, K;
    int         tiles_m, tiles_n;
    int         a_mn, b_mn;  // operand stored K x M (K x N): tiles are fetched as 64 x 64 blocks
    uint32_t*   err;
};

__device__ __forceinline__ void tile_coords(const Core& c, int t, int& mt, int& nt)
{
    const int band_tiles = BAND * c.tiles_n;
    const int band       = t / band_tiles;
    const int r          = t - band * band_tiles;
    const int rows       = min(BAND, c.tiles_m - band * BAND);
    nt                   = r / rows;
    mt                   = band * BAND + (r - nt * rows);
}

__device__ __forceinline__ void flag_error(const Core& c, uint32_t code)
{
    if (c.err) {
        atomicCAS(c.err, 0u, code);
    }
}

// Optional policies. `Src::ready(mt, kb)` runs in the producer thread before the loads of K-block
// `kb` of M-tile `mt` are issued and may wait (bounded) for that part of A to exist; it returns
// false to give up. `Aux::run(aux_warp, lane)` is executed by `Aux::kWarps` extra warps (warps 6..)
// alongside the GEMM, e.g. to pull A from peers' memory into the buffer the GEMM reads.
struct NoSrc {
    __device__ __forceinline__ bool ready(int, int) const { return true; }
};
struct NoAux {
    static constexpr int kWarps = 0;
    __device__ __forceinline__ void run(int, int) const {}
};

// Epi requirements:
//   __device__ void open(int epi_warp)                       once, before the first tile
//   __device__ void tile(uint32_t tmem_acc, int mt, int nt, int quarter, int lane)
//   __device__ void close(int epi_tid)                       once, after the last tile (all 128 threads)
template <class Epi, class Src = NoSrc, class Aux = NoAux>
__device__ __forceinline__ void run(const Core& core, Epi& epi, Src src = Src{}, Aux aux = Aux{})
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t       full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t       tmem_holder;

    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t*       ring = smem_raw + (base - ptx::smem_addr(smem_raw));
    const int      warp = threadIdx.x >> 5;
    const int      lane = threadIdx.x & 31;
    const int      total_tiles = core.tiles_m * core.tiles_n;
    const int      kblocks     = (core.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 4);
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&core.map_a);
        ptx::tma_prefetch_desc(&core.map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<TMEM_COLS>(&tmem_holder);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool     ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int mt, nt;
                tile_coords(core, t, mt, nt);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int      s      = it % STAGES;
                    const uint32_t parity = ((it / STAGES) & 1u) ^ 1u;
                    if (!ptx::mbar_wait(&empty[s], parity) || !src.ready(mt, kb)) {
                        flag_error(core, ERR_PRODUCER_WAIT);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = ring + s * STAGE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
                    if (!core.a_mn) {
                        ptx::tma_load_2d(sa, &core.map_a, kb * BK, mt * BM, &full[s]);
                    }
                    else {  // 64 (k) x 64 (m) blocks of 8 KiB, one per 64 columns of the tile
                        for (int j = 0; j < BM / 64; ++j) {
                            ptx::tma_load_2d(sa + j * 8192, &core.map_a, mt * BM + j * 64, kb * BK, &full[s]);
                        }
                    }
                    if (!core.b_mn) {
                        ptx::tma_load_2d(sb, &core.map_b, kb * BK, nt * BN, &full[s]);
                    }
                    else {
                        for (int j = 0; j < BN / 64; ++j) {
                            ptx::tma_load_2d(sb + j * 8192, &core.map_b, nt * BN + j * 64, kb * BK, &full[s]);
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = ptx::make_idesc(1, 1, BM, BN, core.a_mn ? 1 : 0, core.b_mn ? 1 : 0);
            // K-major: 16 bf16 along K are 32 bytes inside the swizzle atom (+2 in the descriptor's
            // 16-byte units). MN-major: 16 rows of K are 2048 bytes (+128), 64-column blocks 8 KiB apart.
            const uint32_t a_lbo = core.a_mn ? 8192u : 16u, a_step = core.a_mn ? 128u : 2u;
            const uint32_t b_lbo = core.b_mn ? 8192u : 16u, b_step = core.b_mn ? 128u : 2u;
            uint32_t       it    = 0;
            uint32_t           tcount = 0;
            bool               ok    = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tcount) {
                const uint32_t acc = tcount & 1u;
                if (!ptx::mbar_wait(&tmem_empty[acc], ((tcount >> 1) & 1u) ^ 1u)) {
                    flag_error(core, ERR_MMA_WAIT_TMEM);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!ptx::mbar_wait(&full[s], (it / STAGES) & 1u)) {
                        flag_error(core, ERR_MMA_WAIT_FULL);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa     = base + s * STAGE_BYTES;
                    const uint64_t a_desc = ptx::smem_desc_sw128(sa, a_lbo, 1024);
                    const uint64_t b_desc = ptx::smem_desc_sw128(sa + A_BYTES, b_lbo, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        ptx::mma_f16_ss(d_tmem, a_desc + a_step * k, b_desc + b_step * k, idesc, (kb | k) != 0);
                    }
                    ptx::mma_commit(&empty[s]);
                }
                if (ok) {
                    ptx::mma_commit(&tmem_full[acc]);
                }
            }
        }
        __syncwarp();
    }
    else if (warp >= 6) {
        aux.run(warp - 6, lane);
    }
    else {
        const int epi_warp = warp - 2;
        const int quarter  = warp & 3;  // the TMEM lane quarter this warp may access
        epi.open(epi_warp);
        uint32_t tcount = 0;
        bool     ok     = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tcount) {
            const uint32_t acc = tcount & 1u;
            if (!ptx::mbar_wait(&tmem_full[acc], (tcount >> 1) & 1u)) {
                flag_error(core, ERR_EPI_WAIT);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            int mt, nt;
            tile_coords(core, t, mt, nt);
            epi.tile(tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16), mt, nt, quarter, lane);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&tmem_empty[acc]);
            }
        }
        epi.close(threadIdx.x - 64);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

// ---- the same GEMM on CTA pairs ---------------------------------------------------------------------
// Two CTAs of a cluster share a 256 x 256 output tile: each loads its own 128 rows of A and its own
// 128 rows of B per K-block (32 KiB per stage instead of 48, so six stages fit), the even CTA
// issues tcgen05.mma.cta_group::2 (M = 256) over both CTAs' shared memory, and each CTA's 128
// accumulator lanes hold its own rows of the tile. Per 256 x 256 of output the pair moves 64 KiB
// per K-block from L2 into shared memory where two single CTAs move 96: operand delivery is what
// bounds the single-CTA kernel. Operand loads are ordinary per-CTA TMA loads; what crosses between
// the CTAs are completion signals only (the loads' byte counts land on the even CTA's mbarrier,
// the MMA's completion is signalled to both CTAs, the odd CTA's epilogue frees the accumulator
// with a remote arrival).
constexpr int PAIR_STAGES      = 6;
constexpr int PAIR_B_BYTES     = (BN / 2) * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES  = PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
constexpr int PAIR_BAND        = 8;  // 256-row tiles per rasterisation band

__device__ __forceinline__ void pair_tile_coords(const Core& c, int tiles_m2, int t, int& mt2, int& nt)
{
    const int band_tiles = PAIR_BAND * c.tiles_n;
    const int band       = t / band_tiles;
    const int r          = t - band * band_tiles;
    const int rows       = min(PAIR_BAND, tiles_m2 - band * PAIR_BAND);
    nt                   = r / rows;
    mt2                  = band * PAIR_BAND + (r - nt * rows);
}

// `core.map_b` must have been built with a box of BN / 2 rows. Launch with cluster dimension 2.
template <class Epi>
__device__ __forceinline__ void run_pair(const Core& core, Epi& epi)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t       full[PAIR_STAGES], empty[PAIR_STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t       tmem_holder;

    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t*       ring = smem_raw + (base - ptx::smem_addr(smem_raw));
    const int      warp = threadIdx.x >> 5;
    const int      lane = threadIdx.x & 31;
    const uint32_t half = ptx::cluster_ctarank();  // 0: issues the MMAs; 1: the other half of the tile
    const int      pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int      tiles_m2    = (core.tiles_m + 1) / 2;
    const int      total_tiles = tiles_m2 * core.tiles_n;
    const int      kblocks     = (core.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 8);  // four epilogue warps in each CTA
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&core.map_a);
        ptx::tma_prefetch_desc(&core.map_b);
    }
    ptx::cluster_sync();  // both CTAs' barriers exist before either signals the other's
    if (warp == 1) {
        ptx::tmem_alloc_pair<TMEM_COLS>(&tmem_holder);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool     ok = true;
            for (int t = pair; t < total_tiles && ok; t += npairs) {
                int mt2, nt;
                pair_tile_coords(core, tiles_m2, t, mt2, nt);
                const int m0 = (mt2 * 2 + static_cast<int>(half)) * BM;
                const int n0 = nt * BN + static_cast<int>(half) * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int      s      = it % PAIR_STAGES;
                    const uint32_t parity = ((it / PAIR_STAGES) & 1u) ^ 1u;
                    if (!ptx::mbar_wait(&empty[s], parity)) {
                        flag_error(core, ERR_PRODUCER_WAIT);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = ring + s * PAIR_STAGE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    if (half == 0) {
                        ptx::mbar_expect_tx(&full[s], 2 * PAIR_STAGE_BYTES);  // both CTAs' bytes
                    }
                    if (!core.a_mn) {
                        ptx::tma_load_2d_pair(sa, &core.map_a, kb * BK, m0, &full[s]);
                    }
                    else {
                        for (int j = 0; j < BM / 64; ++j) {
                            ptx::tma_load_2d_pair(sa + j * 8192, &core.map_a, m0 + j * 64, kb * BK, &full[s]);
                        }
                    }
                    if (!core.b_mn) {
                        ptx::tma_load_2d_pair(sb, &core.map_b, kb * BK, n0, &full[s]);
                    }
                    else {
                        for (int j = 0; j < BN / 128; ++j) {
                            ptx::tma_load_2d_pair(sb + j * 8192, &core.map_b, n0 + j * 64, kb * BK, &full[s]);
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        if (lane == 0 && half == 0) {
            const uint32_t idesc = ptx::make_idesc(1, 1, 2 * BM, BN, core.a_mn ? 1 : 0, core.b_mn ? 1 : 0);
            const uint32_t a_lbo = core.a_mn ? 8192u : 16u, a_step = core.a_mn ? 128u : 2u;
            const uint32_t b_lbo = core.b_mn ? 8192u : 16u, b_step = core.b_mn ? 128u : 2u;
            uint32_t       it    = 0;
            uint32_t       tcount = 0;
            bool           ok    = true;
            for (int t = pair; t < total_tiles && ok; t += npairs, ++tcount) {
                const uint32_t acc = tcount & 1u;
                if (!ptx::mbar_wait_cluster(&tmem_empty[acc], ((tcount >> 1) & 1u) ^ 1u)) {
                    flag_error(core, ERR_MMA_WAIT_TMEM);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    if (!ptx::mbar_wait(&full[s], (it / PAIR_STAGES) & 1u)) {
                        flag_error(core, ERR_MMA_WAIT_FULL);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa     = base + s * PAIR_STAGE_BYTES;
                    const uint64_t a_desc = ptx::smem_desc_sw128(sa, a_lbo, 1024);
                    const uint64_t b_desc = ptx::smem_desc_sw128(sa + A_BYTES, b_lbo, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        ptx::mma_f16_ss_pair(d_tmem, a_desc + a_step * k, b_desc + b_step * k, idesc, (kb | k) != 0);
                    }
                    ptx::mma_commit_pair(&empty[s]);
                }
                if (ok) {
                    ptx::mma_commit_pair(&tmem_full[acc]);
                }
            }
        }
        __syncwarp();
    }
    else {
        const int epi_warp = warp - 2;
        const int quarter  = warp & 3;
        epi.open(epi_warp);
        uint32_t tcount = 0;
        bool     ok     = true;
        for (int t = pair; t < total_tiles && ok; t += npairs, ++tcount) {
            const uint32_t acc = tcount & 1u;
            if (!ptx::mbar_wait(&tmem_full[acc], (tcount >> 1) & 1u)) {
                flag_error(core, ERR_EPI_WAIT);
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            int mt2, nt;
            pair_tile_coords(core, tiles_m2, t, mt2, nt);
            epi.tile(tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16), mt2 * 2 + static_cast<int>(half), nt,
                     quarter, lane);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive_cluster(ptx::cluster_addr(&tmem_empty[acc], 0));
            }
        }
        epi.close(threadIdx.x - 64);
    }

    // Neither CTA may free its tensor memory, or leave, while the other can still signal it or
    // read its shared memory.
    ptx::tc_fence_before();
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tmem_dealloc_pair<TMEM_COLS>(tmem_base);
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void epi_barrier()
{
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

}  // namespace gemm
}  // namespace fu
