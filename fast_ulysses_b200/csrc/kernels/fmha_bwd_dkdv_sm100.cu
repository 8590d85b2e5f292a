// Flash attention backward, dK/dV pass (head_dim 128, non-causal) on the tcgen05 tensor cores.
//
// One persistent CTA per SM keeps a 128-row K/V block of one (batch, head) in shared memory and its
// dK and dV accumulators in tensor memory, and sweeps the query axis in steps of 64 rows:
//   S^T  = K Q^T , dP^T = V dO^T     128 x 64 accumulators, DOUBLE-buffered in TMEM, so the MMAs
//                                    of step h+1 run while the threads work on step h
//   P^T  = exp2(S^T c - lse[q])      two threads per kv row (32 query columns each: the element-wise
//                                    work is latency-bound, so it gets two warps per scheduler); lse and
//                                    delta of the 64 query rows come
//   dS^T = P^T o (dP^T - delta[q]) * scale   from shared memory (broadcast reads); both results go
//                                    back into TMEM as packed bf16 over S^T and dP^T
//   dV  += P^T dO ,  dK += dS^T Q    A operand from TMEM, dO / Q as MN-major shared-memory operands
// TMEM: buf0 (S^T|dP^T) | buf1 (S^T|dP^T) | dV | dK = 128 + 128 + 128 + 128 columns.
// dQ is produced by the dQ pass (fmha_bwd_dq_sm100.cu); nothing here is atomic.
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D          = 128;
constexpr int BKV        = 128;             // kv rows owned by the CTA
constexpr int BQ         = 64;              // query rows per step
constexpr int STAGES     = 3;
constexpr int TILE_BYTES = BKV * D * 2;     // 32 KiB: K or V block, two 64-column halves
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int Q_BYTES    = BQ * D * 2;      // 16 KiB: Q or dO step tile, two 64-column halves of 8 KiB
constexpr int Q_HALF     = Q_BYTES / 2;
constexpr int STAGE_BYTES = 2 * Q_BYTES + 1024;   // Q | dO | lse2[64] delta[64] (+ pad to keep 1 KiB alignment)
constexpr int SMEM_BYTES = 2 * TILE_BYTES + STAGES * STAGE_BYTES + 1024;
constexpr int THREADS    = 320;             // TMA warp, MMA warp, 8 element-wise warps

enum : uint32_t { ERR_LOAD = 41, ERR_MMA = 42, ERR_COMPUTE = 43 };

struct Params {
    CUtensorMap    map_q, map_do, map_k, map_v;   // q/dO boxes of 64 rows, k/v boxes of 128 rows
    const float*   lse2;
    const float*   delta;
    __nv_bfloat16* dk;
    __nv_bfloat16* dv;
    int64_t        dk_row, dk_head, dk_batch, dv_row, dv_head, dv_batch;
    int            B, H, Sq, Skv, Sq_pad;
    int            n_q, kv_blocks, total_work;   // n_q = Sq_pad / 64
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
    uint64_t kv_full, kv_empty;
    uint64_t full[STAGES], empty[STAGES];
    uint64_t sd_full[2], p_ready[2], acc_full, acc_free;
};

__global__ void __launch_bounds__(THREADS, 1) fmha_bwd_dkdv_kernel(const __grid_constant__ Params p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ Barriers       bar;
    __shared__ uint32_t       tmem_holder;

    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t*       sm   = smem_raw + (base - ptx::smem_addr(smem_raw));
    const uint32_t sk_addr = base, sv_addr = base + TILE_BYTES, st_addr = base + 2 * TILE_BYTES;
    uint8_t*       sk = sm;
    uint8_t*       sv = sm + TILE_BYTES;
    uint8_t*       sst = sm + 2 * TILE_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar.kv_full, 1);
        ptx::mbar_init(&bar.kv_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&bar.full[s], 1);
            ptx::mbar_init(&bar.empty[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            ptx::mbar_init(&bar.sd_full[g], 1);
            ptx::mbar_init(&bar.p_ready[g], 8);
        }
        ptx::mbar_init(&bar.acc_full, 1);
        ptx::mbar_init(&bar.acc_free, 8);
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
    const int      n_q  = p.n_q;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            uint32_t it = 0, wc = 0;
            bool     ok = true;
            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                const int jb = w % p.kv_blocks;
                const int h  = (w / p.kv_blocks) % p.H;
                const int b  = w / (p.kv_blocks * p.H);
                if (!ptx::mbar_wait(&bar.kv_empty, (wc & 1u) ^ 1u)) {
                    flag(p, ERR_LOAD);
                    break;
                }
                ptx::mbar_expect_tx(&bar.kv_full, 2 * TILE_BYTES);
                for (int half = 0; half < 2; ++half) {
                    ptx::tma_load_4d(sk + half * HALF_BYTES, &p.map_k, half * 64, jb * BKV, h, b, &bar.kv_full);
                    ptx::tma_load_4d(sv + half * HALF_BYTES, &p.map_v, half * 64, jb * BKV, h, b, &bar.kv_full);
                }
                const float* lse2  = p.lse2 + (static_cast<int64_t>(b) * p.H + h) * p.Sq_pad;
                const float* delta = p.delta + (static_cast<int64_t>(b) * p.H + h) * p.Sq_pad;
                for (int i = 0; i < n_q; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!ptx::mbar_wait(&bar.empty[s], ((it / STAGES) & 1u) ^ 1u)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    uint8_t* st = sst + s * STAGE_BYTES;
                    ptx::mbar_expect_tx(&bar.full[s], 2 * Q_BYTES + 512);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(st + half * Q_HALF, &p.map_q, half * 64, i * BQ, h, b, &bar.full[s]);
                        ptx::tma_load_4d(st + Q_BYTES + half * Q_HALF, &p.map_do, half * 64, i * BQ, h, b, &bar.full[s]);
                    }
                    ptx::bulk_g2s(st + 2 * Q_BYTES, lse2 + i * BQ, 256, &bar.full[s]);
                    ptx::bulk_g2s(st + 2 * Q_BYTES + 256, delta + i * BQ, 256, &bar.full[s]);
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_sd = ptx::make_idesc(1, 1, BKV, BQ, 0, 0);  // 128 x 64, A and B K-major
            constexpr uint32_t idesc_ac = ptx::make_idesc(1, 1, BKV, D, 0, 1);   // A from TMEM, B MN-major
            uint32_t           it = 0, wc = 0;
            bool               ok = true;

            auto issue_sd = [&](uint32_t step, int stage) {
                const uint32_t g  = step & 1u;
                const uint32_t qa = st_addr + stage * STAGE_BYTES, oa = qa + Q_BYTES;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {  // S^T = K Q^T
                    const uint32_t a_off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    const uint32_t b_off = (kk >> 2) * Q_HALF + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem + g * 128, ptx::desc_advance(ptx::smem_desc_sw128(sk_addr, 16, 1024), a_off),
                                    ptx::desc_advance(ptx::smem_desc_sw128(qa, 16, 1024), b_off), idesc_sd, kk != 0);
                }
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {  // dP^T = V dO^T
                    const uint32_t a_off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    const uint32_t b_off = (kk >> 2) * Q_HALF + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem + g * 128 + 64, ptx::desc_advance(ptx::smem_desc_sw128(sv_addr, 16, 1024), a_off),
                                    ptx::desc_advance(ptx::smem_desc_sw128(oa, 16, 1024), b_off), idesc_sd, kk != 0);
                }
                ptx::mma_commit(&bar.sd_full[g]);
            };
            auto issue_acc = [&](uint32_t step, int stage, bool accumulate) {
                const uint32_t g  = step & 1u;
                const uint32_t qa = st_addr + stage * STAGE_BYTES, oa = qa + Q_BYTES;
#pragma unroll
                for (int kk = 0; kk < BQ / 16; ++kk) {  // dV += P^T dO   (contraction over the 64 query rows)
                    ptx::mma_f16_ts(tmem + 256, tmem + g * 128 + (kk >> 1) * 32 + (kk & 1) * 8,
                                    ptx::desc_advance(ptx::smem_desc_sw128(oa, Q_HALF, 1024), kk * 2048), idesc_ac, accumulate || kk != 0);
                }
#pragma unroll
                for (int kk = 0; kk < BQ / 16; ++kk) {  // dK += dS^T Q
                    ptx::mma_f16_ts(tmem + 384, tmem + g * 128 + 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                                    ptx::desc_advance(ptx::smem_desc_sw128(qa, Q_HALF, 1024), kk * 2048), idesc_ac, accumulate || kk != 0);
                }
            };

            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                if (!ptx::mbar_wait(&bar.kv_full, wc & 1u)
                    || !ptx::mbar_wait(&bar.full[it % STAGES], (it / STAGES) & 1u)) {
                    flag(p, ERR_MMA);
                    break;
                }
                ptx::tc_fence_after();
                issue_sd(it, it % STAGES);
                for (int i = 0; i < n_q && ok; ++i, ++it) {
                    const int s = it % STAGES;
                    if (i + 1 < n_q) {
                        const int sn = (it + 1) % STAGES;
                        if (!ptx::mbar_wait(&bar.full[sn], ((it + 1) / STAGES) & 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        // buffer (it+1)&1 was last read by the accumulation MMAs of step it-1, which
                        // were issued before this and execute in order
                        issue_sd(it + 1, sn);
                    }
                    if (!ptx::mbar_wait(&bar.p_ready[it & 1u], (it >> 1) & 1u)
                        || (i == 0 && !ptx::mbar_wait(&bar.acc_free, (wc & 1u) ^ 1u))) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    issue_acc(it, s, i != 0);
                    ptx::mma_commit(&bar.empty[s]);
                }
                if (ok) {
                    ptx::mma_commit(&bar.acc_full);
                    ptx::mma_commit(&bar.kv_empty);
                }
            }
        }
        __syncwarp();
    }
    else {
        // ---------------------------------------------------------------- two threads per kv row
        const int      quarter  = warp & 3;
        const int      colhalf  = (warp - 2) >> 2;   // which 32 of the 64 query columns (and which half of d)
        const int      row_in   = quarter * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t t_dv = tmem + 256 + lane_off, t_dk = tmem + 384 + lane_off;
        const float    c = p.scale_log2;
        uint32_t       it = 0, wc = 0;
        bool           ok = true;
        for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
            const int  jb    = w % p.kv_blocks;
            const int  h     = (w / p.kv_blocks) % p.H;
            const int  b     = w / (p.kv_blocks * p.H);
            const int  kvr   = jb * BKV + row_in;
            const bool kv_ok = kvr < p.Skv;
            for (int i = 0; i < n_q; ++i, ++it) {
                const uint32_t g     = it & 1u;
                const float*   lse2  = reinterpret_cast<const float*>(sst + (it % STAGES) * STAGE_BYTES + 2 * Q_BYTES);
                const float*   delta = lse2 + 64;
                const uint32_t t_s   = tmem + g * 128 + lane_off;
                const uint32_t t_dp  = t_s + 64;
                if (!ptx::mbar_wait(&bar.sd_full[g], (it >> 1) & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                uint32_t rs[32], rd[32];
                ptx::tmem_ld_32x32(t_s + colhalf * 32, rs);
                ptx::tmem_ld_32x32(t_dp + colhalf * 32, rd);
                ptx::tmem_ld_wait();
                {
                    uint32_t pp[16], dd[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const int q0 = colhalf * 32 + 2 * k;
                        // lse2 is +inf for padding rows of q, so their probabilities are exactly 0
                        float p0 = ptx::ex2(fmaf(__uint_as_float(rs[2 * k]), c, -lse2[q0]));
                        float p1 = ptx::ex2(fmaf(__uint_as_float(rs[2 * k + 1]), c, -lse2[q0 + 1]));
                        if (!kv_ok) {
                            p0 = 0.0f;
                            p1 = 0.0f;
                        }
                        const float d0 = p0 * (__uint_as_float(rd[2 * k]) - delta[q0]) * p.scale;
                        const float d1 = p1 * (__uint_as_float(rd[2 * k + 1]) - delta[q0 + 1]) * p.scale;
                        pp[k]          = ptx::pack_bf16x2(p0, p1);
                        dd[k]          = ptx::pack_bf16x2(d0, d1);
                    }
                    // each warp writes its packed results over the start of the columns IT read (never
                    // over its partner's): P^T / dS^T for query rows 0..31 sit at columns 0..15, for
                    // rows 32..63 at columns 32..47; the MMA addresses its K-steps accordingly
                    ptx::tmem_st_32x16(t_s + colhalf * 32, pp);
                    ptx::tmem_st_32x16(t_dp + colhalf * 32, dd);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.p_ready[g]);
            }
            if (!ok) {
                break;
            }
            if (!ptx::mbar_wait(&bar.acc_full, wc & 1u)) {
                flag(p, ERR_COMPUTE);
                break;
            }
            ptx::tc_fence_after();
            __nv_bfloat16* dv = p.dv + b * p.dv_batch + static_cast<int64_t>(kvr) * p.dv_row + h * p.dv_head;
            __nv_bfloat16* dk = p.dk + b * p.dk_batch + static_cast<int64_t>(kvr) * p.dk_row + h * p.dk_head;
#pragma unroll 1
            for (int ch = colhalf * 2; ch < colhalf * 2 + 2; ++ch) {
                uint32_t rv[32], rk[32];
                ptx::tmem_ld_32x32(t_dv + ch * 32, rv);
                ptx::tmem_ld_32x32(t_dk + ch * 32, rk);
                ptx::tmem_ld_wait();
                if (kv_ok) {
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        uint4 a, bq;
                        a.x  = ptx::pack_bf16x2(__uint_as_float(rv[8 * k4]), __uint_as_float(rv[8 * k4 + 1]));
                        a.y  = ptx::pack_bf16x2(__uint_as_float(rv[8 * k4 + 2]), __uint_as_float(rv[8 * k4 + 3]));
                        a.z  = ptx::pack_bf16x2(__uint_as_float(rv[8 * k4 + 4]), __uint_as_float(rv[8 * k4 + 5]));
                        a.w  = ptx::pack_bf16x2(__uint_as_float(rv[8 * k4 + 6]), __uint_as_float(rv[8 * k4 + 7]));
                        bq.x = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4]), __uint_as_float(rk[8 * k4 + 1]));
                        bq.y = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 2]), __uint_as_float(rk[8 * k4 + 3]));
                        bq.z = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 4]), __uint_as_float(rk[8 * k4 + 5]));
                        bq.w = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 6]), __uint_as_float(rk[8 * k4 + 7]));
                        *reinterpret_cast<uint4*>(dv + ch * 32 + 8 * k4) = a;
                        *reinterpret_cast<uint4*>(dk + ch * 32 + 8 * k4) = bq;
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive_warp(&bar.acc_free);
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
int fu_fmha_bwd_dkdv_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream)
{
    Params p{};
    int    rc = make_map_bshd(&p.map_q, a->q, a->batch, a->seq_q, a->heads, a->q_row, a->q_head, a->q_batch, BQ);
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_do, a->d_o, a->batch, a->seq_q, a->heads, a->o_row, a->o_head, a->o_batch, BQ);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_k, a->k, a->batch, a->seq_kv, a->heads, a->k_row, a->k_head, a->k_batch, BKV);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_v, a->v, a->batch, a->seq_kv, a->heads, a->v_row, a->v_head, a->v_batch, BKV);
    }
    if (rc != FU_OK) {
        return rc;
    }
    p.lse2       = lse2;
    p.delta      = delta;
    p.dk         = static_cast<__nv_bfloat16*>(a->dk);
    p.dv         = static_cast<__nv_bfloat16*>(a->dv);
    p.dk_row     = a->k_row;
    p.dk_head    = a->k_head;
    p.dk_batch   = a->k_batch;
    p.dv_row     = a->v_row;
    p.dv_head    = a->v_head;
    p.dv_batch   = a->v_batch;
    p.B          = a->batch;
    p.H          = a->heads;
    p.Sq         = a->seq_q;
    p.Skv        = a->seq_kv;
    p.Sq_pad     = sq_pad;
    p.n_q        = sq_pad / BQ;
    p.kv_blocks  = (a->seq_kv + BKV - 1) / BKV;
    p.total_work = p.kv_blocks * p.H * p.B;
    p.scale      = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.err        = a->err;
    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static bool configured[64] = {};
    if (dev < 64 && !configured[dev]) {
        FU_CUDA_OK(cudaFuncSetAttribute(fmha_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev] = true;
    }
    int grid = a->ctas > 0 ? std::min(a->ctas, sms) : sms;
    grid     = std::max(1, std::min(grid, p.total_work));
    fmha_bwd_dkdv_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
