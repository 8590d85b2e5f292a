// Non-causal flash attention backward for head_dim 128: one software-pipelined pass on tcgen05.
//
// One persistent CTA per SM owns a 128-row K/V block of one (batch, head) at a time and sweeps all
// 128-row query blocks i. Five products per block pair, everything transposed so that the kv row
// sits on the TMEM lane axis and the probabilities can be fed back as the A operand:
//   S^T(i)  = K Q_i^T            (SS)      C1: P^T = exp2(S^T c - lse)               -> TMEM (bf16)
//   dP^T(i) = V dO_i^T           (SS)      C2: dS^T = P^T o (dP^T - delta)           -> TMEM + smem
//   dV     += P^T dO_i           (A from TMEM)
//   dK     += dS^T Q_i           (A from TMEM)
//   dQ_i^T  = K^T dS^T           (SS, both operands MN-major); drained by eight extra warps with
//                                coalesced fp32 reductions into a global accumulator
// Tensor memory: S^T/P^T | dP^T/dS^T/dQ^T | dV | dK, 128 fp32 columns each (all 512).
//
// Issue order per block: dP(i), dV(i), S(i+1), dK(i), dQ(i). C1(i+1) runs under dK(i) and dQ(i),
// C2(i) under dV(i) and S(i+1). dP(i+1) is the first product that needs the columns of dQ_i^T back:
// the drain warps copy them to registers, release the columns at once and only then issue their
// reductions, which overlap the next block. The softmax scale is applied to dK in the epilogue and
// to dQ when the accumulator is rounded, not to every element of dS.
//
// Measured limits (S = 32768, 5 heads, SM clock counter): a 128x128x16 MMA takes 64 clocks when its
// descriptors are ready (8 per product: 512), a tensor-memory load-and-wait about 200, and the fp32
// reductions of all SMs together move about 3.5 TB/s into L2, which bounds this algorithm near
// 1.1 PFLOP/s (64 KiB of reductions per 21 MFLOP). The dependent chain
// dP -> C2 -> dK, dQ -> drain -> dP is what sets the period, not the tensor pipe.
// Warps: 0 = TMA producer, 1 = MMA issuer, 2..9 = two threads per kv row, 10..17 = dQ drain.
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D           = 128;
constexpr int BLK         = 128;
constexpr int TILE_BYTES  = BLK * D * 2;  // 32 KiB
constexpr int HALF_BYTES  = TILE_BYTES / 2;
constexpr int STAGES      = 2;
constexpr int OFF_K       = 0;
constexpr int OFF_V       = OFF_K + TILE_BYTES;
constexpr int OFF_Q       = OFF_V + TILE_BYTES;            // STAGES tiles
constexpr int OFF_DO      = OFF_Q + STAGES * TILE_BYTES;   // STAGES tiles
constexpr int OFF_DS      = OFF_DO + STAGES * TILE_BYTES;  // dS^T, [kv x q], 128B-swizzled halves
constexpr int OFF_STATS   = OFF_DS + TILE_BYTES;           // per stage: lse2[128] | delta[128]
constexpr int OFF_BARS    = OFF_STATS + STAGES * 1024;
constexpr int SMEM_BYTES  = OFF_BARS + 256;
constexpr int THREADS     = 576;

static_assert(SMEM_BYTES <= 232448, "shared memory budget");

enum : uint32_t { ERR_ALIGN = 30, ERR_LOAD = 31, ERR_MMA = 32, ERR_COMPUTE = 33, ERR_DRAIN = 34 };

struct Params {
    CUtensorMap    map_q, map_k, map_v, map_do;
    const float*   lse2;    // (B, H, Sq_pad) log-sum-exp in base 2, +inf in the padding
    const float*   delta;   // (B, H, Sq_pad)
    float*         dq_acc;  // (B, Sq, H, 128) fp32, zeroed by the launcher
    __nv_bfloat16* dk;
    __nv_bfloat16* dv;
    int64_t        dk_row, dk_head, dk_batch, dv_row, dv_head, dv_batch;
    int            B, H, Sq, Skv, Sq_pad;
    int            n_q, kv_blocks, total_work;
    float          scale, scale_log2;
    uint32_t*      err;
    uint64_t*      trace;
};

struct Bars {
    uint64_t kv_full, kv_empty;
    uint64_t q_full[STAGES], do_full[STAGES], empty[STAGES];
    uint64_t s_full, dp_full, p_ready, ds_ready, dq_full, dq_free, acc_full, acc_free;
    uint32_t tmem_holder;
};
static_assert(sizeof(Bars) <= 256, "barrier block");

__device__ __forceinline__ void flag(const Params& p, uint32_t code)
{
    if (p.err) {
        atomicCAS(p.err, 0u, code);
    }
}

__device__ __forceinline__ void stamp(const Params& p, uint32_t it, int ev)
{
    if (p.trace && blockIdx.x == 0 && it >= 64u && it < 72u) {
        p.trace[(it - 64u) * 16 + ev] = clock64();
    }
}

// CTAs that run at the same time own neighbouring K/V blocks of one head. Each starts its sweep
// over the query blocks at a different block, so that their dQ reductions do not all land on the
// same addresses at the same moment.
__device__ __forceinline__ int first_block(const Params& p, int jb)
{
    return static_cast<int>(static_cast<int64_t>(jb) * p.n_q / p.kv_blocks);
}

__device__ __forceinline__ void red_add(float* addr, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// 16 query columns of S^T -> 8 packed probability pairs
template <int C>
__device__ __forceinline__ void c1_chunk(const uint32_t (&r)[16], uint32_t (&pk)[32], const float* lse2, float c,
                                         bool kv_ok)
{
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float p0 = ptx::ex2(fmaf(__uint_as_float(r[2 * k]), c, -lse2[C * 16 + 2 * k]));
        const float p1 = ptx::ex2(fmaf(__uint_as_float(r[2 * k + 1]), c, -lse2[C * 16 + 2 * k + 1]));
        pk[C * 8 + k]  = kv_ok ? ptx::pack_bf16x2(p0, p1) : 0u;
    }
}

// 16 query columns of dP^T -> 8 packed dS pairs (without the softmax scale), stored over the first
// columns this thread has already read and into the swizzled shared-memory row
template <int C>
__device__ __forceinline__ void c2_chunk(const uint32_t (&r)[16], const uint32_t (&pk)[32], const float* delta,
                                         uint32_t t_dp, uint8_t* ds_row, int row_in)
{
    // the difference in fp32 (it cancels), the product with the bf16 probabilities as a packed pair
    uint32_t dd[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float d0 = __uint_as_float(r[2 * k]) - delta[C * 16 + 2 * k];
        const float d1 = __uint_as_float(r[2 * k + 1]) - delta[C * 16 + 2 * k + 1];
        dd[k]          = ptx::mul_bf16x2(pk[C * 8 + k], ptx::pack_bf16x2(d0, d1));
    }
    ptx::tmem_st_32x8(t_dp + C * 8, dd);
    *reinterpret_cast<uint4*>(ds_row + (((2 * C) ^ (row_in & 7)) << 4))     = make_uint4(dd[0], dd[1], dd[2], dd[3]);
    *reinterpret_cast<uint4*>(ds_row + (((2 * C + 1) ^ (row_in & 7)) << 4)) = make_uint4(dd[4], dd[5], dd[6], dd[7]);
}

__global__ void __launch_bounds__(THREADS, 1) fmha_bwd_fused_kernel(const __grid_constant__ Params p)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    const uint32_t base = ptx::smem_addr(sm);
    Bars&          bar  = *reinterpret_cast<Bars*>(sm + OFF_BARS);
    const int      warp = threadIdx.x >> 5;
    const int      lane = threadIdx.x & 31;
    if (base & 1023u) {
        if (threadIdx.x == 0) {
            flag(p, ERR_ALIGN);
        }
        return;
    }

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar.kv_full, 1);
        ptx::mbar_init(&bar.kv_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&bar.q_full[s], 1);
            ptx::mbar_init(&bar.do_full[s], 1);
            ptx::mbar_init(&bar.empty[s], 1);
        }
        ptx::mbar_init(&bar.s_full, 1);
        ptx::mbar_init(&bar.dp_full, 1);
        ptx::mbar_init(&bar.p_ready, 8);  // one arrival per warp
        ptx::mbar_init(&bar.ds_ready, 8);  // one arrival per warp
        ptx::mbar_init(&bar.dq_full, 1);
        ptx::mbar_init(&bar.dq_free, 8);  // one arrival per warp
        ptx::mbar_init(&bar.acc_full, 1);
        ptx::mbar_init(&bar.acc_free, 8);  // one arrival per warp
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&p.map_q);
        ptx::tma_prefetch_desc(&p.map_k);
        ptx::tma_prefetch_desc(&p.map_v);
        ptx::tma_prefetch_desc(&p.map_do);
    }
    if (warp == 1) {
        ptx::tmem_alloc<512>(&bar.tmem_holder);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = bar.tmem_holder;
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
                    ptx::tma_load_4d(sm + OFF_K + half * HALF_BYTES, &p.map_k, half * 64, jb * BLK, h, b, &bar.kv_full);
                    ptx::tma_load_4d(sm + OFF_V + half * HALF_BYTES, &p.map_v, half * 64, jb * BLK, h, b, &bar.kv_full);
                }
                const float* lse2  = p.lse2 + (static_cast<int64_t>(b) * p.H + h) * p.Sq_pad;
                const float* delta = p.delta + (static_cast<int64_t>(b) * p.H + h) * p.Sq_pad;
                const int    first = first_block(p, jb);
                for (int i0 = 0; i0 < n_q; ++i0, ++it) {
                    const int      i  = i0 + first < n_q ? i0 + first : i0 + first - n_q;
                    const int      s  = it % STAGES;
                    const uint32_t ph = ((it / STAGES) & 1u) ^ 1u;
                    uint8_t*       ss = sm + OFF_STATS + s * 1024;
                    // one release per stage (after dK of the block that used it): the statistics of
                    // a stage are read by the element-wise warps until then
                    if (!ptx::mbar_wait(&bar.empty[s], ph)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    ptx::mbar_expect_tx(&bar.q_full[s], TILE_BYTES + 512);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(sm + OFF_Q + s * TILE_BYTES + half * HALF_BYTES, &p.map_q, half * 64, i * BLK, h,
                                         b, &bar.q_full[s]);
                    }
                    ptx::bulk_g2s(ss, lse2 + i * BLK, 512, &bar.q_full[s]);
                    ptx::mbar_expect_tx(&bar.do_full[s], TILE_BYTES + 512);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(sm + OFF_DO + s * TILE_BYTES + half * HALF_BYTES, &p.map_do, half * 64, i * BLK,
                                         h, b, &bar.do_full[s]);
                    }
                    ptx::bulk_g2s(ss + 512, delta + i * BLK, 512, &bar.do_full[s]);
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_kk = ptx::make_idesc(1, 1, BLK, BLK, 0, 0);  // A, B K-major
            constexpr uint32_t idesc_tn = ptx::make_idesc(1, 1, BLK, D, 0, 1);    // A from TMEM, B MN-major
            constexpr uint32_t idesc_nn = ptx::make_idesc(1, 1, D, BLK, 1, 1);    // A, B MN-major
            // one descriptor per operand and role, built once; every MMA below only steps it
            const uint64_t k_kmaj  = ptx::smem_desc_sw128(base + OFF_K, 16, 1024);
            const uint64_t v_kmaj  = ptx::smem_desc_sw128(base + OFF_V, 16, 1024);
            const uint64_t q_kmaj  = ptx::smem_desc_sw128(base + OFF_Q, 16, 1024);
            const uint64_t do_kmaj = ptx::smem_desc_sw128(base + OFF_DO, 16, 1024);
            const uint64_t k_mn    = ptx::smem_desc_sw128(base + OFF_K, HALF_BYTES, 1024);
            const uint64_t q_mn    = ptx::smem_desc_sw128(base + OFF_Q, HALF_BYTES, 1024);
            const uint64_t do_mn   = ptx::smem_desc_sw128(base + OFF_DO, HALF_BYTES, 1024);
            const uint64_t ds_mn   = ptx::smem_desc_sw128(base + OFF_DS, HALF_BYTES, 1024);
            uint32_t           it = 0, wc = 0;
            bool               ok = true;
            auto issue_s = [&](int stage) {  // S^T = K Q^T
                const uint64_t qd = ptx::desc_advance(q_kmaj, stage * TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem, ptx::desc_advance(k_kmaj, off), ptx::desc_advance(qd, off), idesc_kk, kk != 0);
                }
                ptx::mma_commit(&bar.s_full);
            };
            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                if (!ptx::mbar_wait(&bar.kv_full, wc & 1u) || !ptx::mbar_wait(&bar.q_full[it % STAGES], (it / STAGES) & 1u)) {
                    flag(p, ERR_MMA);
                    break;
                }
                ptx::tc_fence_after();
                issue_s(it % STAGES);
                for (int i = 0; i < n_q; ++i, ++it) {
                    const int      s  = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    const uint64_t o_k = ptx::desc_advance(do_kmaj, s * TILE_BYTES);
                    const uint64_t o_m = ptx::desc_advance(do_mn, s * TILE_BYTES);
                    const uint64_t q_m = ptx::desc_advance(q_mn, s * TILE_BYTES);
                    // the previous block's dQ^T must have left the columns dP^T is written to
                    if (!ptx::mbar_wait(&bar.do_full[s], ph) || !ptx::mbar_wait(&bar.dq_free, (it & 1u) ^ 1u)) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    stamp(p, it, 1);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {  // dP^T = V dO^T
                        const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                        ptx::mma_f16_ss(tmem + 128, ptx::desc_advance(v_kmaj, off), ptx::desc_advance(o_k, off), idesc_kk,
                                        kk != 0);
                    }
                    ptx::mma_commit(&bar.dp_full);
                    if (!ptx::mbar_wait(&bar.p_ready, it & 1u)
                        || (i == 0 && !ptx::mbar_wait(&bar.acc_free, (wc & 1u) ^ 1u))) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    stamp(p, it, 0);
#pragma unroll
                    for (int kk = 0; kk < BLK / 16; ++kk) {  // dV += P^T dO   (contraction over q)
                        ptx::mma_f16_ts(tmem + 256, tmem + (kk >> 2) * 64 + (kk & 3) * 8, ptx::desc_advance(o_m, kk * 2048),
                                        idesc_tn, i != 0 || kk != 0);
                    }
                    if (i + 1 < n_q) {
                        const uint32_t n = it + 1;
                        if (!ptx::mbar_wait(&bar.q_full[n % STAGES], (n / STAGES) & 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        issue_s(n % STAGES);
                    }
                    stamp(p, it, 2);
                    if (!ptx::mbar_wait(&bar.ds_ready, it & 1u)) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    stamp(p, it, 3);
#pragma unroll
                    for (int kk = 0; kk < BLK / 16; ++kk) {  // dK += dS^T Q
                        ptx::mma_f16_ts(tmem + 384, tmem + 128 + (kk >> 2) * 64 + (kk & 3) * 8,
                                        ptx::desc_advance(q_m, kk * 2048), idesc_tn, i != 0 || kk != 0);
                    }
                    ptx::mma_commit(&bar.empty[s]);
#pragma unroll
                    for (int kk = 0; kk < BLK / 16; ++kk) {  // dQ^T = K^T dS^T   (contraction over kv)
                        ptx::mma_f16_ss(tmem + 128, ptx::desc_advance(k_mn, kk * 2048), ptx::desc_advance(ds_mn, kk * 2048),
                                        idesc_nn, kk != 0);
                    }
                    ptx::mma_commit(&bar.dq_full);
                    stamp(p, it, 4);
                }
                if (ok) {
                    ptx::mma_commit(&bar.acc_full);
                    ptx::mma_commit(&bar.kv_empty);
                }
            }
        }
        __syncwarp();
    }
    else if (warp < 10) {
        // ---------------------------------------------------------------- element-wise warps
        // two threads per kv row: warps 2..5 take query columns 0..63 of a block, warps 6..9 columns
        // 64..127; each writes its packed bf16 results over the start of the columns it read itself
        const int      quarter  = warp & 3;
        const int      c2       = (warp - 2) >> 2;
        const int      row_in   = quarter * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_off + c2 * 64, t_dp = tmem + 128 + lane_off + c2 * 64;
        const uint32_t t_dv = tmem + 256 + lane_off, t_dk = tmem + 384 + lane_off;
        uint8_t*       ds_row = sm + OFF_DS + c2 * HALF_BYTES + row_in * 128;
        const float    c = p.scale_log2;
        uint32_t       it = 0, wc = 0;
        bool           ok = true;
        for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
            const int  jb    = w % p.kv_blocks;
            const int  h     = (w / p.kv_blocks) % p.H;
            const int  b     = w / (p.kv_blocks * p.H);
            const int  kvr   = jb * BLK + row_in;
            const bool kv_ok = kvr < p.Skv;
            for (int i = 0; i < n_q; ++i, ++it) {
                const int    s     = it % STAGES;
                const float* lse2  = reinterpret_cast<const float*>(sm + OFF_STATS + s * 1024) + c2 * 64;
                const float* delta = lse2 + 128;
                uint32_t     pk[32];  // this thread's 64 probabilities, bf16 pairs
                if (!ptx::mbar_wait(&bar.s_full, it & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (threadIdx.x == 64) {
                    stamp(p, it, 5);
                }
                {
                    // loads run one 16-column chunk ahead of the arithmetic
                    uint32_t ra[16], rb[16];
                    ptx::tmem_ld_32x16(t_s, ra);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_s + 16, rb);
                    c1_chunk<0>(ra, pk, lse2, c, kv_ok);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_s + 32, ra);
                    c1_chunk<1>(rb, pk, lse2, c, kv_ok);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_s + 48, rb);
                    c1_chunk<2>(ra, pk, lse2, c, kv_ok);
                    ptx::tmem_ld_wait();
                    c1_chunk<3>(rb, pk, lse2, c, kv_ok);
                    ptx::tmem_st_32x32(t_s, pk);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.p_ready);
                if (threadIdx.x == 64) {
                    stamp(p, it, 6);
                }

                if (!ptx::mbar_wait(&bar.dp_full, it & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (threadIdx.x == 64) {
                    stamp(p, it, 7);
                }
                {
                    uint32_t ra[16], rb[16];
                    ptx::tmem_ld_32x16(t_dp, ra);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_dp + 16, rb);
                    c2_chunk<0>(ra, pk, delta, t_dp, ds_row, row_in);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_dp + 32, ra);
                    c2_chunk<1>(rb, pk, delta, t_dp, ds_row, row_in);
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x16(t_dp + 48, rb);
                    c2_chunk<2>(ra, pk, delta, t_dp, ds_row, row_in);
                    ptx::tmem_ld_wait();
                    c2_chunk<3>(rb, pk, delta, t_dp, ds_row, row_in);
                }
                ptx::tmem_st_wait();
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.ds_ready);
                if (threadIdx.x == 64) {
                    stamp(p, it, 8);
                }
            }
            if (!ok) {
                break;
            }
            // dK, dV of this block
            if (!ptx::mbar_wait(&bar.acc_full, wc & 1u)) {
                flag(p, ERR_COMPUTE);
                break;
            }
            ptx::tc_fence_after();
            __nv_bfloat16* dv = p.dv + b * p.dv_batch + static_cast<int64_t>(kvr) * p.dv_row + h * p.dv_head;
            __nv_bfloat16* dk = p.dk + b * p.dk_batch + static_cast<int64_t>(kvr) * p.dk_row + h * p.dk_head;
#pragma unroll 1
            for (int ch = 2 * c2; ch < 2 * c2 + 2; ++ch) {
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
                        bq.x = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4]) * p.scale, __uint_as_float(rk[8 * k4 + 1]) * p.scale);
                        bq.y = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 2]) * p.scale, __uint_as_float(rk[8 * k4 + 3]) * p.scale);
                        bq.z = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 4]) * p.scale, __uint_as_float(rk[8 * k4 + 5]) * p.scale);
                        bq.w = ptx::pack_bf16x2(__uint_as_float(rk[8 * k4 + 6]) * p.scale, __uint_as_float(rk[8 * k4 + 7]) * p.scale);
                        *reinterpret_cast<uint4*>(dv + ch * 32 + 8 * k4) = a;
                        *reinterpret_cast<uint4*>(dk + ch * 32 + 8 * k4) = bq;
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive_warp(&bar.acc_free);
        }
    }
    else {
        // ---------------------------------------------------------------- dQ drain
        // dQ_i^T sits in tensor memory with the head dimension on the lanes: lane d of a warp adds
        // its query columns into dq_acc[q][d], so that every warp-wide reduction covers 128
        // contiguous bytes of one query row. Warps 10..13 take query columns 0..63, warps 14..17
        // columns 64..127. The columns are released as soon as they are in registers.
        const int      quarter  = warp & 3;
        const int      qh       = (warp - 10) >> 2;
        const int      dcol     = quarter * 32 + lane;
        const uint32_t t_dq     = tmem + 128 + qh * 64 + (static_cast<uint32_t>(quarter * 32) << 16);
        const int64_t  q_stride = static_cast<int64_t>(p.H) * D;
        uint32_t       it       = 0;
        bool           ok       = true;
        for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
            const int h  = (w / p.kv_blocks) % p.H;
            const int b  = w / (p.kv_blocks * p.H);
            float*    dq = p.dq_acc + (static_cast<int64_t>(b) * p.Sq * p.H + h) * D + dcol;
            const int first = first_block(p, w % p.kv_blocks);
            for (int i0 = 0; i0 < n_q; ++i0, ++it) {
                const int i = i0 + first < n_q ? i0 + first : i0 + first - n_q;
                if (!ptx::mbar_wait(&bar.dq_full, it & 1u)) {
                    flag(p, ERR_DRAIN);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (threadIdx.x == 320) {
                    stamp(p, it, 9);
                }
                uint32_t r0[32], r1[32];
                ptx::tmem_ld_32x32(t_dq, r0);
                ptx::tmem_ld_32x32(t_dq + 32, r1);
                ptx::tmem_ld_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.dq_free);
                if (threadIdx.x == 320) {
                    stamp(p, it, 10);
                }
                const int q0    = i * BLK + qh * 64;
                const int valid = p.Sq - q0;  // query rows of this half that exist
                float*    row   = dq + static_cast<int64_t>(q0) * q_stride;
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    if (k < valid) {
                        red_add(row + k * q_stride, __uint_as_float(r0[k]));
                    }
                }
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    if (32 + k < valid) {
                        red_add(row + (32 + k) * q_stride, __uint_as_float(r1[k]));
                    }
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tmem_dealloc<512>(tmem);
    }
}

}  // namespace

// Launched by fu_fmha_bwd (fmha_bwd_sm100.cu) after its pre-pass has filled lse2 / delta and the
// fp32 dQ accumulator has been zeroed; the caller rounds the accumulator to bf16 afterwards.
int fu_fmha_bwd_fused_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream)
{
    Params p{};
    int    rc = make_map_bshd(&p.map_q, a->q, a->batch, a->seq_q, a->heads, a->q_row, a->q_head, a->q_batch, BLK);
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_do, a->d_o, a->batch, a->seq_q, a->heads, a->o_row, a->o_head, a->o_batch, BLK);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_k, a->k, a->batch, a->seq_kv, a->heads, a->k_row, a->k_head, a->k_batch, BLK);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_v, a->v, a->batch, a->seq_kv, a->heads, a->v_row, a->v_head, a->v_batch, BLK);
    }
    if (rc != FU_OK) {
        return rc;
    }
    p.lse2       = lse2;
    p.delta      = delta;
    p.dq_acc     = a->dq_acc;
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
    p.n_q        = sq_pad / BLK;
    p.kv_blocks  = (a->seq_kv + BLK - 1) / BLK;
    p.total_work = p.kv_blocks * p.H * p.B;
    p.scale      = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.err        = a->err;
    p.trace      = a->trace;
    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static bool configured[64] = {};
    if (dev < 64 && !configured[dev]) {
        FU_CUDA_OK(cudaFuncSetAttribute(fmha_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev] = true;
    }
    int grid = a->ctas > 0 ? std::min(a->ctas, sms) : sms;
    grid     = std::max(1, std::min(grid, p.total_work));
    fmha_bwd_fused_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
