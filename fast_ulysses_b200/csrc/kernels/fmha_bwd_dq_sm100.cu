// Flash attention backward, dQ pass (head_dim 128, non-causal) on the tcgen05 tensor cores.
//
// The backward is split in two passes so that neither needs atomics: this one keeps dQ stationary
// (one CTA owns 256 query rows as two 128-row tiles and sweeps the kv axis in steps of 64 rows),
// the other (fmha_bwd_sm100.cu) keeps dK/dV stationary. Per step and query tile:
//   S  = Q K^T , dP = dO V^T        (operands in shared memory, 128 x 64 accumulators in TMEM)
//   dS = exp2(S c - lse) o (dP - delta) * scale   one thread per query row; lse and delta of the
//                                                 row live in registers; dS goes back into TMEM
//                                                 as packed bf16 over S
//   dQ += dS K                      (dS read from TMEM as the A operand, K as an MN-major operand)
// TMEM per tile: S | dP | dQ = 64 + 64 + 128 columns; two tiles fill the 512 columns. The tiles are
// staggered exactly like the forward pass, so the element-wise work of one hides under the MMAs of
// the other. dQ leaves the kernel as bf16; there is no fp32 accumulator in global memory.
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D          = 128;
constexpr int BM         = 128;
constexpr int QT         = 2;
constexpr int BN         = 64;              // kv rows per step
constexpr int STAGES     = 2;
constexpr int TILE_BYTES = BM * D * 2;      // 32 KiB (Q or dO tile, two 64-column halves)
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_BYTES   = BN * D * 2;      // 16 KiB (K or V step tile, two 64-column halves of 8 KiB)
constexpr int KV_HALF    = KV_BYTES / 2;
constexpr int STAGE_BYTES = 2 * KV_BYTES;   // K | V
constexpr int SMEM_BYTES = 2 * QT * TILE_BYTES + STAGES * STAGE_BYTES + 1024;
constexpr int THREADS    = 32 * 18;         // TMA warp, MMA warp, 2 tiles x 8 element-wise warps

enum : uint32_t { ERR_LOAD = 31, ERR_MMA = 32, ERR_COMPUTE = 33 };

struct Params {
    CUtensorMap    map_q, map_do, map_k, map_v;   // q/dO boxes of 128 rows, k/v boxes of 64 rows
    const float*   lse2;    // (B, H, Sq_pad)
    const float*   delta;   // (B, H, Sq_pad)
    __nv_bfloat16* dq;
    int64_t        dq_row, dq_head, dq_batch;
    int            B, H, Sq, Skv, Sq_pad;
    int            q_blocks, total_work, n_kv;
    float          scale, scale_log2;
    uint32_t*      err;
};

__device__ __forceinline__ void flag(const Params& p, uint32_t code)
{
    if (p.err) {
        atomicCAS(p.err, 0u, code);
    }
}

struct Barriers {
    uint64_t q_full, q_empty;
    uint64_t kv_full[STAGES], kv_empty[STAGES];
    uint64_t sd_full[QT], ds_ready[QT], dq_final[QT], dq_free[QT];
};

__global__ void __launch_bounds__(THREADS, 1) fmha_bwd_dq_kernel(const __grid_constant__ Params p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ Barriers       bar;
    __shared__ uint32_t       tmem_holder;

    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t*       sm   = smem_raw + (base - ptx::smem_addr(smem_raw));
    // layout: Q0 | Q1 | dO0 | dO1 | stage0 (K|V) | stage1 (K|V)
    const uint32_t sq_addr  = base;
    const uint32_t sdo_addr = base + QT * TILE_BYTES;
    const uint32_t skv_addr = sdo_addr + QT * TILE_BYTES;
    uint8_t*       sq       = sm;
    uint8_t*       sdo      = sm + QT * TILE_BYTES;
    uint8_t*       skv      = sdo + QT * TILE_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar.q_full, 1);
        ptx::mbar_init(&bar.q_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&bar.kv_full[s], 1);
            ptx::mbar_init(&bar.kv_empty[s], 1);
        }
        for (int t = 0; t < QT; ++t) {
            ptx::mbar_init(&bar.sd_full[t], 1);
            ptx::mbar_init(&bar.ds_ready[t], 8);
            ptx::mbar_init(&bar.dq_final[t], 1);
            ptx::mbar_init(&bar.dq_free[t], 8);
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&p.map_q);
        ptx::tma_prefetch_desc(&p.map_do);
        ptx::tma_prefetch_desc(&p.map_k);
        ptx::tma_prefetch_desc(&p.map_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc<512>(&tmem_holder);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = tmem_holder;
    const int      n_kv = p.n_kv;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            uint32_t it = 0, wc = 0;
            bool     ok = true;
            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                const int qb = w % p.q_blocks;
                const int h  = (w / p.q_blocks) % p.H;
                const int b  = w / (p.q_blocks * p.H);
                if (!ptx::mbar_wait(&bar.q_empty, (wc & 1u) ^ 1u)) {
                    flag(p, ERR_LOAD);
                    break;
                }
                ptx::mbar_expect_tx(&bar.q_full, 2 * QT * TILE_BYTES);
                for (int t = 0; t < QT; ++t) {
                    for (int half = 0; half < 2; ++half) {
                        const int row = qb * (QT * BM) + t * BM;
                        ptx::tma_load_4d(sq + t * TILE_BYTES + half * HALF_BYTES, &p.map_q, half * 64, row, h, b,
                                         &bar.q_full);
                        ptx::tma_load_4d(sdo + t * TILE_BYTES + half * HALF_BYTES, &p.map_do, half * 64, row, h, b,
                                         &bar.q_full);
                    }
                }
                for (int j = 0; j < n_kv; ++j, ++it) {
                    const int s = it % STAGES;
                    if (!ptx::mbar_wait(&bar.kv_empty[s], ((it / STAGES) & 1u) ^ 1u)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    uint8_t* st = skv + s * STAGE_BYTES;
                    ptx::mbar_expect_tx(&bar.kv_full[s], STAGE_BYTES);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(st + half * KV_HALF, &p.map_k, half * 64, j * BN, h, b, &bar.kv_full[s]);
                        ptx::tma_load_4d(st + KV_BYTES + half * KV_HALF, &p.map_v, half * 64, j * BN, h, b,
                                         &bar.kv_full[s]);
                    }
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_sd = ptx::make_idesc(1, 1, BM, BN, 0, 0);  // 128 x 64, A and B K-major
            constexpr uint32_t idesc_dq = ptx::make_idesc(1, 1, BM, D, 0, 1);   // A from TMEM, K MN-major
            uint32_t           it = 0, wc = 0;
            uint32_t           rcount[QT] = {0, 0};
            bool               ok = true;

            auto issue_sd = [&](int t, int stage) {
                const uint32_t qa = sq_addr + t * TILE_BYTES, oa = sdo_addr + t * TILE_BYTES;
                const uint32_t ka = skv_addr + stage * STAGE_BYTES, va = ka + KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {  // S = Q K^T
                    const uint32_t a_off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    const uint32_t b_off = (kk >> 2) * KV_HALF + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem + t * 256, ptx::desc_advance(ptx::smem_desc_sw128(qa, 16, 1024), a_off),
                                    ptx::desc_advance(ptx::smem_desc_sw128(ka, 16, 1024), b_off), idesc_sd, kk != 0);
                }
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {  // dP = dO V^T
                    const uint32_t a_off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    const uint32_t b_off = (kk >> 2) * KV_HALF + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem + t * 256 + 64, ptx::desc_advance(ptx::smem_desc_sw128(oa, 16, 1024), a_off),
                                    ptx::desc_advance(ptx::smem_desc_sw128(va, 16, 1024), b_off), idesc_sd, kk != 0);
                }
                ptx::mma_commit(&bar.sd_full[t]);
            };
            auto issue_dq = [&](int t, int stage, bool accumulate) {
                const uint32_t ka = skv_addr + stage * STAGE_BYTES;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    // K step tile as an MN-major operand: 16 kv rows = 2048 bytes further down, the two
                    // 64-wide halves of d are KV_HALF apart, 8-row groups 1024 bytes apart
                    ptx::mma_f16_ts(tmem + t * 256 + 128, tmem + t * 256 + (kk >> 1) * 32 + (kk & 1) * 8,
                                    ptx::desc_advance(ptx::smem_desc_sw128(ka, KV_HALF, 1024), kk * 2048), idesc_dq, accumulate || kk != 0);
                }
            };

            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                if (!ptx::mbar_wait(&bar.q_full, wc & 1u)) {
                    flag(p, ERR_MMA);
                    break;
                }
                {
                    const int s = it % STAGES;
                    if (!ptx::mbar_wait(&bar.kv_full[s], (it / STAGES) & 1u)) {
                        flag(p, ERR_MMA);
                        break;
                    }
                    ptx::tc_fence_after();
                    issue_sd(0, s);
                    issue_sd(1, s);
                }
                for (int j = 0; j < n_kv && ok; ++j, ++it) {
                    const int  s    = it % STAGES;
                    const int  sn   = (it + 1) % STAGES;
                    const bool more = j + 1 < n_kv;
                    if (more && !ptx::mbar_wait(&bar.kv_full[sn], ((it + 1) / STAGES) & 1u)) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    for (int t = 0; t < QT; ++t) {
                        if (!ptx::mbar_wait(&bar.ds_ready[t], rcount[t] & 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        ++rcount[t];
                        if (j == 0 && !ptx::mbar_wait(&bar.dq_free[t], (wc & 1u) ^ 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        issue_dq(t, s, j != 0);
                        if (!more) {
                            ptx::mma_commit(&bar.dq_final[t]);
                        }
                        else {
                            issue_sd(t, sn);
                        }
                    }
                    if (!ok) {
                        break;
                    }
                    ptx::mma_commit(&bar.kv_empty[s]);  // K_j and V_j are no longer read
                }
                ptx::mma_commit(&bar.q_empty);
            }
        }
        __syncwarp();
    }
    else {
        // ---------------------------------------------------------------- dS and the dQ epilogue
        // two threads per query row: each takes 32 of the 64 kv columns of a step (the element-wise
        // work is latency-bound, so every scheduler gets two warps per tile)
        const int      t        = (warp - 2) >> 3;
        const int      colhalf  = ((warp - 2) >> 2) & 1;
        const int      quarter  = warp & 3;
        const int      row_in   = quarter * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t ts  = tmem + t * 256 + lane_off;        // S, then dS (bf16) over it
        const uint32_t tdp = ts + 64;
        const uint32_t tdq = ts + 128;
        const float    c   = p.scale_log2;
        uint32_t       scount = 0, wc = 0;
        bool           ok = true;

        for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
            const int     qb   = w % p.q_blocks;
            const int     h    = (w / p.q_blocks) % p.H;
            const int     b    = w / (p.q_blocks * p.H);
            const int     row  = qb * (QT * BM) + t * BM + row_in;   // < Sq_pad by construction
            const int64_t stat = (static_cast<int64_t>(b) * p.H + h) * p.Sq_pad + row;
            const float   lse2 = p.lse2[stat];   // +inf in the padding: its probabilities vanish
            const float   dl   = p.delta[stat];

            for (int j = 0; j < n_kv; ++j, ++scount) {
                if (!ptx::mbar_wait(&bar.sd_full[t], scount & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const int valid = min(BN, p.Skv - j * BN);
                uint32_t  rs[32], rd[32];
                ptx::tmem_ld_32x32(ts + colhalf * 32, rs);
                ptx::tmem_ld_32x32(tdp + colhalf * 32, rd);
                ptx::tmem_ld_wait();
                {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int k0 = colhalf * 32 + 2 * i;
                        float     p0 = ptx::ex2(fmaf(__uint_as_float(rs[2 * i]), c, -lse2));
                        float     p1 = ptx::ex2(fmaf(__uint_as_float(rs[2 * i + 1]), c, -lse2));
                        if (k0 >= valid) {
                            p0 = 0.0f;
                        }
                        if (k0 + 1 >= valid) {
                            p1 = 0.0f;
                        }
                        const float d0 = p0 * (__uint_as_float(rd[2 * i]) - dl) * p.scale;
                        const float d1 = p1 * (__uint_as_float(rd[2 * i + 1]) - dl) * p.scale;
                        pk[i]          = ptx::pack_bf16x2(d0, d1);
                    }
                    // dS over the start of the columns THIS warp read: kv 0..31 at columns 0..15,
                    // kv 32..63 at columns 32..47 (the MMA addresses its K-steps accordingly)
                    ptx::tmem_st_32x16(ts + colhalf * 32, pk);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.ds_ready[t]);
            }
            if (!ok) {
                break;
            }
            if (!ptx::mbar_wait(&bar.dq_final[t], wc & 1u)) {
                flag(p, ERR_COMPUTE);
                break;
            }
            ptx::tc_fence_after();
            const bool     row_ok = row < p.Sq;
            __nv_bfloat16* dst    = p.dq + b * p.dq_batch + static_cast<int64_t>(row) * p.dq_row + h * p.dq_head;
#pragma unroll 1
            for (int c2 = colhalf; c2 < colhalf + 1; ++c2) {
                uint32_t r[64];
                ptx::tmem_ld_32x32(tdq + c2 * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                ptx::tmem_ld_32x32(tdq + c2 * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                ptx::tmem_ld_wait();
                if (row_ok) {
                    uint4* out = reinterpret_cast<uint4*>(dst + c2 * 64);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        out[q4] = make_uint4(
                            ptx::pack_bf16x2(__uint_as_float(r[8 * q4]), __uint_as_float(r[8 * q4 + 1])),
                            ptx::pack_bf16x2(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3])),
                            ptx::pack_bf16x2(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5])),
                            ptx::pack_bf16x2(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7])));
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive_warp(&bar.dq_free[t]);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tmem_dealloc<512>(tmem);
    }
}

}  // namespace

// Launched by fu_fmha_bwd (fmha_bwd_sm100.cu) after its pre-pass has filled lse2 / delta.
int fu_fmha_bwd_dq_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream)
{
    Params p{};
    int    rc = make_map_bshd(&p.map_q, a->q, a->batch, a->seq_q, a->heads, a->q_row, a->q_head, a->q_batch, BM);
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_do, a->d_o, a->batch, a->seq_q, a->heads, a->o_row, a->o_head, a->o_batch, BM);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_k, a->k, a->batch, a->seq_kv, a->heads, a->k_row, a->k_head, a->k_batch, BN);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_v, a->v, a->batch, a->seq_kv, a->heads, a->v_row, a->v_head, a->v_batch, BN);
    }
    if (rc != FU_OK) {
        return rc;
    }
    p.lse2       = lse2;
    p.delta      = delta;
    p.dq         = static_cast<__nv_bfloat16*>(a->dq);
    p.dq_row     = a->q_row;
    p.dq_head    = a->q_head;
    p.dq_batch   = a->q_batch;
    p.B          = a->batch;
    p.H          = a->heads;
    p.Sq         = a->seq_q;
    p.Skv        = a->seq_kv;
    p.Sq_pad     = sq_pad;
    p.q_blocks   = (a->seq_q + QT * BM - 1) / (QT * BM);
    p.total_work = p.q_blocks * p.H * p.B;
    p.n_kv       = (a->seq_kv + BN - 1) / BN;
    p.scale      = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.err        = a->err;
    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static bool configured[64] = {};
    if (dev < 64 && !configured[dev]) {
        FU_CUDA_OK(cudaFuncSetAttribute(fmha_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev] = true;
    }
    int grid = a->ctas > 0 ? std::min(a->ctas, sms) : sms;
    grid     = std::max(1, std::min(grid, p.total_work));
    fmha_bwd_dq_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
