// Non-causal flash attention forward for head_dim 128 on the tcgen05 tensor cores.
//
// One persistent CTA per SM works on (batch, head, 256 query rows) items: two 128-row query tiles
// that share every K/V tile. Warp roles:
//   warp 0       TMA producer: Q (once per item), then K and V tiles through two-stage rings
//   warp 1       MMA issuer: S_t = Q_t K^T (operands in shared memory), O_t += P_t V (P read
//                from tensor memory, V as an MN-major shared-memory operand)
//   warps 2, 3   idle (they fill warpgroup 0 so that register counts can be set per warpgroup:
//                warpgroup 0 gives registers away, the softmax warpgroups take them)
//   warps 4..7   softmax for query tile 0, warps 8..11 for query tile 1: one thread per row;
//                exp2 with a lazily updated reference maximum, P written back over S in tensor
//                memory as packed bf16, O rescaled in tensor memory only when the maximum grew by
//                more than 2^8; final normalisation, bf16 store and log-sum-exp
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t aliases S_t.
// The two query tiles are staggered (QK of tile 0 for step j+1 is issued between the two PV of
// step j), so each softmax has two MMA slots of cover.
//
// q, k, v, o use the (batch, seq, heads, 128) layout of the all-to-all windows, so attention reads
// what the fused QKV kernel scattered and writes what the output projection pulls, with no copy.
// The reference has no attention kernel (examples/dit_attention.py:57 calls torch SDPA).
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D         = 128;
constexpr int BM        = 128;  // rows per query tile
constexpr int QT        = 2;    // query tiles per CTA
constexpr int BN        = 128;  // kv rows per step
constexpr int KV_STAGES = 2;
constexpr int TILE_BYTES = 128 * D * 2;       // 32 KiB: a 128 x 128 bf16 tile as two 64-column halves
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int SMEM_BYTES = (QT + 2 * KV_STAGES) * TILE_BYTES + 1024;
constexpr int THREADS    = 32 * 12;            // three warpgroups: {producer, MMA, 2 idle}, softmax 0, softmax 1
constexpr int REGS_SMALL = 104;                 // warpgroup 0 after it has given registers away
constexpr int REGS_SOFTMAX = 200;              // per scheduler: 32 x (104 + 2 x 200) = 16128 of 16384 registers
constexpr float RESCALE_THRESHOLD = 8.0f;     // in log2 units
constexpr int   kPolyPairs = 0;               // of every 16 exponential pairs, on the FMA pipe by default

enum : uint32_t { ERR_LOAD = 11, ERR_MMA = 12, ERR_SOFTMAX = 13 };

struct Params {
    CUtensorMap    map_q, map_k, map_v;
    __nv_bfloat16* o;
    float*         lse;         // (B, H, Sq)
    int64_t        o_row, o_head, o_batch;  // element strides of o
    int            B, H, Sq, Skv;
    int            q_blocks, total_work, n_kv;
    float          scale, scale_log2;
    uint32_t*      err;
    uint64_t*      trace;
};

__device__ __forceinline__ void flag(const Params& p, uint32_t code)
{
    if (p.err) {
        atomicCAS(p.err, 0u, code);
    }
}

struct Barriers {
    uint64_t q_full, q_empty;
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[QT], p_lo[QT], p_hi[QT], o_final[QT], o_free[QT];
};

// exp2 of a pair on the FMA pipe instead of the special-function unit: floor by a round-down add of
// 1.5 * 2^23 (the integer part lands in the low mantissa bits), a cubic for 2^fraction (relative
// error 7.5e-5, far below the bf16 rounding of P that follows), and the integer part added to the
// exponent field. Arguments below -126 are clamped: their exponent field would wrap.
__device__ __forceinline__ void ex2_poly2(float& e0, float& e1, float x0, float x1)
{
    constexpr float MAGIC = 12582912.0f;
    constexpr float C0 = 0.9999251961708069f, C1 = 0.695833683013916f, C2 = 0.22606723010540009f,
                    C3 = 0.07802422344684601f;
    x0 = fmaxf(x0, -126.0f);
    x1 = fmaxf(x1, -126.0f);
    float t0, t1, i0, i1, f0, f1, p0, p1;
    ptx::add2_rm(t0, t1, x0, x1, MAGIC, MAGIC);
    ptx::add2(i0, i1, t0, t1, -MAGIC, -MAGIC);
    ptx::fma2(f0, f1, i0, i1, -1.0f, -1.0f, x0, x1);
    ptx::fma2(p0, p1, f0, f1, C3, C3, C2, C2);
    ptx::fma2(p0, p1, p0, p1, f0, f1, C1, C1);
    ptx::fma2(p0, p1, p0, p1, f0, f1, C0, C0);
    e0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
    e1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// 32 columns of one row: P = exp2(S * c - m * c) as packed bf16, row sum into l4. NP of every 16
// pairs take the FMA-pipe path (spread evenly so both pipes stay fed), the rest the special-function unit.
template <int NP>
__device__ __forceinline__ void exp_chunk(const uint32_t* r, float c, float nmc, float (&l4)[4], uint32_t (&pk)[16])
{
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float x0, x1, e0, e1;
        ptx::fma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), c, c, nmc, nmc);
        if (NP > 0 && (i * NP) % 16 < NP) {
            ex2_poly2(e0, e1, x0, x1);
        }
        else {
            e0 = ptx::ex2(x0);
            e1 = ptx::ex2(x1);
        }
        ptx::add2(l4[(2 * i) & 3], l4[(2 * i + 1) & 3], l4[(2 * i) & 3], l4[(2 * i + 1) & 3], e0, e1);
        pk[i] = ptx::pack_bf16x2(e0, e1);
    }
}

// Optional timeline (TRACE builds only): CTA 0 stores the SM clock of pipeline events of kv steps
// 64..71 of its first work item, 32 slots per step: 0..9 softmax tile 0, 10..19 softmax tile 1,
// 20..31 the MMA issuer.
template <bool TRACE>
__device__ __forceinline__ void stamp(const Params& p, uint32_t step, int ev)
{
    if (TRACE && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && step >= 64u && step < 72u) {
        p.trace[(step - 64u) * 32 + ev] = clock64();
    }
}

template <int NP, bool TRACE>
__global__ void __launch_bounds__(THREADS, 1) fmha_fwd_kernel(const __grid_constant__ Params p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ Barriers       bar;
    __shared__ uint32_t       tmem_holder;

    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t*       sm   = smem_raw + (base - ptx::smem_addr(smem_raw));
    // layout: Q0 | Q1 | K[0] | K[1] | V[0] | V[1]
    const uint32_t sq_addr = base;
    const uint32_t sk_addr = base + QT * TILE_BYTES;
    const uint32_t sv_addr = sk_addr + KV_STAGES * TILE_BYTES;
    uint8_t*       sq      = sm;
    uint8_t*       sk      = sm + QT * TILE_BYTES;
    uint8_t*       sv      = sk + KV_STAGES * TILE_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar.q_full, 1);
        ptx::mbar_init(&bar.q_empty, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            ptx::mbar_init(&bar.k_full[s], 1);
            ptx::mbar_init(&bar.k_empty[s], 1);
            ptx::mbar_init(&bar.v_full[s], 1);
            ptx::mbar_init(&bar.v_empty[s], 1);
        }
        for (int t = 0; t < QT; ++t) {
            ptx::mbar_init(&bar.s_full[t], 1);
            ptx::mbar_init(&bar.p_lo[t], 4);  // one arrival per warp
            ptx::mbar_init(&bar.p_hi[t], 4);
            ptx::mbar_init(&bar.o_final[t], 1);
            ptx::mbar_init(&bar.o_free[t], 4);
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&p.map_q);
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

    if (warp < 4) {
    ptx::setmaxnreg_dec<REGS_SMALL>();
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
                ptx::mbar_expect_tx(&bar.q_full, QT * TILE_BYTES);
                for (int t = 0; t < QT; ++t) {
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(sq + t * TILE_BYTES + half * HALF_BYTES, &p.map_q, half * 64,
                                         qb * (QT * BM) + t * BM, h, b, &bar.q_full);
                    }
                }
                for (int j = 0; j < n_kv; ++j, ++it) {
                    const int      s      = it % KV_STAGES;
                    const uint32_t parity = ((it / KV_STAGES) & 1u) ^ 1u;
                    if (!ptx::mbar_wait(&bar.k_empty[s], parity)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    ptx::mbar_expect_tx(&bar.k_full[s], TILE_BYTES);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(sk + s * TILE_BYTES + half * HALF_BYTES, &p.map_k, half * 64, j * BN, h, b,
                                         &bar.k_full[s]);
                    }
                    if (!ptx::mbar_wait(&bar.v_empty[s], parity)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    ptx::mbar_expect_tx(&bar.v_full[s], TILE_BYTES);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(sv + s * TILE_BYTES + half * HALF_BYTES, &p.map_v, half * 64, j * BN, h, b,
                                         &bar.v_full[s]);
                    }
                }
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ptx::make_idesc(1, 1, BM, BN, 0, 0);  // both K-major
            constexpr uint32_t idesc_pv = ptx::make_idesc(1, 1, BM, D, 0, 1);   // V is MN-major
            uint32_t           it = 0, wc = 0;
            uint32_t           pcount[QT] = {0, 0};
            bool               ok = true;

            // one descriptor per operand, built once; every MMA below only steps it
            const uint64_t desc_q = ptx::smem_desc_sw128(sq_addr, 16, 1024);
            const uint64_t desc_k = ptx::smem_desc_sw128(sk_addr, 16, 1024);
            const uint64_t desc_v = ptx::smem_desc_sw128(sv_addr, HALF_BYTES, 1024);

            auto issue_qk = [&](int t, int stage) {
                const uint64_t qa = ptx::desc_advance(desc_q, t * TILE_BYTES);
                const uint64_t ka = ptx::desc_advance(desc_k, stage * TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    ptx::mma_f16_ss(tmem + t * 128, ptx::desc_advance(qa, off), ptx::desc_advance(ka, off), idesc_qk,
                                    kk != 0);
                }
                ptx::mma_commit(&bar.s_full[t]);
            };
            // One half (64 kv rows) of P_t V: the softmax hands P over in two halves so that the
            // first half's products run under the second half's exponentials.
            auto issue_pv = [&](int t, int stage, int half, bool accumulate) {
                // 16 kv rows = 2048 bytes further down; the two 64-wide halves of d are HALF_BYTES
                // apart (leading byte offset), 8-row groups 1024 bytes apart
                const uint64_t va = ptx::desc_advance(desc_v, stage * TILE_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < BN / 32; ++k4) {
                    const int kk = half * (BN / 32) + k4;
                    ptx::mma_f16_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, ptx::desc_advance(va, kk * 2048),
                                    idesc_pv, accumulate || kk != 0);
                }
            };

            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                if (!ptx::mbar_wait(&bar.q_full, wc & 1u)) {
                    flag(p, ERR_MMA);
                    break;
                }
                // prologue: S for both query tiles of kv step 0
                {
                    const int s = it % KV_STAGES;
                    if (!ptx::mbar_wait(&bar.k_full[s], (it / KV_STAGES) & 1u)) {
                        flag(p, ERR_MMA);
                        break;
                    }
                    ptx::tc_fence_after();
                    issue_qk(0, s);
                    issue_qk(1, s);
                    ptx::mma_commit(&bar.k_empty[s]);
                }
                for (int j = 0; j < n_kv && ok; ++j, ++it) {
                    const int  s    = it % KV_STAGES;
                    const int  sn   = (it + 1) % KV_STAGES;
                    const bool more = j + 1 < n_kv;
                    if (!ptx::mbar_wait(&bar.v_full[s], (it / KV_STAGES) & 1u)) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    if (more && !ptx::mbar_wait(&bar.k_full[sn], ((it + 1) / KV_STAGES) & 1u)) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    for (int t = 0; t < QT; ++t) {
                        stamp<TRACE>(p, it, 20 + t * 6 + 0);
                        if (!ptx::mbar_wait(&bar.p_lo[t], pcount[t] & 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        stamp<TRACE>(p, it, 20 + t * 6 + 1);
                        if (j == 0 && !ptx::mbar_wait(&bar.o_free[t], (wc & 1u) ^ 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        issue_pv(t, s, 0, j != 0);
                        stamp<TRACE>(p, it, 20 + t * 6 + 2);
                        if (!ptx::mbar_wait(&bar.p_hi[t], pcount[t] & 1u)) {
                            flag(p, ERR_MMA);
                            ok = false;
                            break;
                        }
                        stamp<TRACE>(p, it, 20 + t * 6 + 3);
                        ++pcount[t];
                        ptx::tc_fence_after();
                        issue_pv(t, s, 1, true);
                        if (!more) {
                            ptx::mma_commit(&bar.o_final[t]);
                        }
                        else {
                            issue_qk(t, sn);  // S_t is free again: PV_t above is ordered before it
                        }
                        stamp<TRACE>(p, it, 20 + t * 6 + 4);
                    }
                    if (!ok) {
                        break;
                    }
                    ptx::mma_commit(&bar.v_empty[s]);
                    if (more) {
                        ptx::mma_commit(&bar.k_empty[sn]);
                    }
                }
                ptx::mma_commit(&bar.q_empty);
            }
        }
        __syncwarp();
    }
    }
    else {
        ptx::setmaxnreg_inc<REGS_SOFTMAX>();
        // ---------------------------------------------------------------- softmax + epilogue
        const int      t       = (warp - 4) >> 2;          // query tile
        const int      quarter = warp & 3;                 // TMEM lane quarter of this warp
        const int      row_in  = quarter * 32 + lane;      // row inside the query tile
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t ts      = tmem + t * 128 + lane_off;        // S_t / P_t
        const uint32_t to      = tmem + 256 + t * 128 + lane_off;  // O_t
        const float    c       = p.scale_log2;
        uint32_t       scount = 0, wc = 0;
        bool           ok = true;

        for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
            const int qb  = w % p.q_blocks;
            const int h   = (w / p.q_blocks) % p.H;
            const int b   = w / (p.q_blocks * p.H);
            const int row = qb * (QT * BM) + t * BM + row_in;
            float     m_ref = -INFINITY, l = 0.0f;

            for (int j = 0; j < n_kv; ++j, ++scount) {
                if (!ptx::mbar_wait(&bar.s_full[t], scount & 1u)) {
                    flag(p, ERR_SOFTMAX);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                stamp<TRACE>(p, scount, t * 10 + 0);
                const int valid = min(BN, p.Skv - j * BN);  // columns of this step that exist
                // The whole row of S in registers with a single wait: the softmax sits on the
                // critical path between two MMAs, so its latency matters more than its register use.
                uint32_t r[BN];
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    ptx::tmem_ld_32x32(ts + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[ch * 32]));
                }
                ptx::tmem_ld_wait();
                stamp<TRACE>(p, scount, t * 10 + 1);
                if (valid < BN) {
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        if (i >= valid) {
                            r[i] = 0xff800000u;  // -inf: exp2 gives exactly 0
                        }
                    }
                }
                // row maximum with three-input max: 64 instructions in four independent chains
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < BN; i += 8) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        mx4[u] = ptx::max3(mx4[u], __uint_as_float(r[i + 2 * u]), __uint_as_float(r[i + 2 * u + 1]));
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // lazy reference maximum: rescale only when it grew by more than the threshold
                const bool grow = (j == 0) || ((mx - m_ref) * c > RESCALE_THRESHOLD);
                if (__any_sync(0xffffffffu, grow && j != 0)) {
                    const float alpha = (grow && j != 0) ? ptx::ex2((m_ref - mx) * c) : 1.0f;
                    l *= alpha;
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        uint32_t ro[32];
                        ptx::tmem_ld_32x32(to + ch * 32, ro);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
                        }
                        ptx::tmem_st_32x32(to + ch * 32, ro);
                    }
                    ptx::tmem_st_wait();
                }
                if (grow) {
                    m_ref = mx;
                }
                stamp<TRACE>(p, scount, t * 10 + 2);
                const float mc = m_ref * c;
                // P = exp2(S * c - m_ref * c), written over S as packed bf16
                const float nmc = -mc;
                float       l4[4] = {0.f, 0.f, 0.f, 0.f};
                // The last block of a ragged sequence holds -inf columns: those take the
                // special-function unit only (the FMA-pipe form clamps instead of returning 0).
                uint32_t pk[16];
                if (valid == BN) {
                    exp_chunk<NP>(&r[0], c, nmc, l4, pk);
                    ptx::tmem_st_32x16(ts, pk);
                    exp_chunk<NP>(&r[32], c, nmc, l4, pk);
                    ptx::tmem_st_32x16(ts + 16, pk);
                    // third quarter's exponentials are issued before waiting for the first half's
                    // stores, so the store latency hides under them
                    exp_chunk<NP>(&r[64], c, nmc, l4, pk);
                }
                else {
                    exp_chunk<0>(&r[0], c, nmc, l4, pk);
                    ptx::tmem_st_32x16(ts, pk);
                    exp_chunk<0>(&r[32], c, nmc, l4, pk);
                    ptx::tmem_st_32x16(ts + 16, pk);
                    exp_chunk<0>(&r[64], c, nmc, l4, pk);
                }
                stamp<TRACE>(p, scount, t * 10 + 3);
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.p_lo[t]);
                stamp<TRACE>(p, scount, t * 10 + 4);
                ptx::tmem_st_32x16(ts + 32, pk);
                if (valid == BN) {
                    exp_chunk<NP>(&r[96], c, nmc, l4, pk);
                }
                else {
                    exp_chunk<0>(&r[96], c, nmc, l4, pk);
                }
                ptx::tmem_st_32x16(ts + 48, pk);
                l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                stamp<TRACE>(p, scount, t * 10 + 5);
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive_warp(&bar.p_hi[t]);
                stamp<TRACE>(p, scount, t * 10 + 6);
            }
            if (!ok) {
                break;
            }
            // epilogue: O / l -> bf16, log-sum-exp
            if (!ptx::mbar_wait(&bar.o_final[t], wc & 1u)) {
                flag(p, ERR_SOFTMAX);
                break;
            }
            ptx::tc_fence_after();
            const float    inv    = 1.0f / l;
            const bool     row_ok = row < p.Sq;
            __nv_bfloat16* dst    = p.o + b * p.o_batch + static_cast<int64_t>(row) * p.o_row + h * p.o_head;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(to + ch * 32, r);
                ptx::tmem_ld_wait();
                if (row_ok) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        pk[i] = ptx::pack_bf16x2(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                    }
                    uint4* out = reinterpret_cast<uint4*>(dst + ch * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        out[q4] = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                    }
                }
            }
            if (row_ok && p.lse) {
                p.lse[(static_cast<int64_t>(b) * p.H + h) * p.Sq + row] = (m_ref * c + ptx::lg2(l)) * 0.6931471805599453f;
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive_warp(&bar.o_free[t]);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tmem_dealloc<512>(tmem);
    }
}

}  // namespace

extern "C" int fu_fmha_fwd(const FuFmhaArgs* a, void* stream)
{
    if (!a || !a->q || !a->k || !a->v || !a->o) {
        return fu::fail(FU_E_ARG, "fu_fmha_fwd: null operand");
    }
    if (a->head_dim != D) {
        return fu::fail(FU_E_UNSUPPORTED, "fu_fmha_fwd: head_dim %d (only 128 is built)", a->head_dim);
    }
    if (a->batch < 1 || a->heads < 1 || a->seq_q < 1 || a->seq_kv < 1) {
        return fu::fail(FU_E_ARG, "fu_fmha_fwd: empty problem");
    }
    if ((reinterpret_cast<uintptr_t>(a->o) & 15u) || (a->o_row % 8) || (a->o_head % 8) || (a->o_batch % 8)) {
        return fu::fail(FU_E_ARG, "fu_fmha_fwd: o needs 16-byte aligned rows");
    }
    Params p{};
    int    rc = make_map_bshd(&p.map_q, a->q, a->batch, a->seq_q, a->heads, a->q_row, a->q_head, a->q_batch, BM);
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_k, a->k, a->batch, a->seq_kv, a->heads, a->k_row, a->k_head, a->k_batch, BN);
    }
    if (rc == FU_OK) {
        rc = make_map_bshd(&p.map_v, a->v, a->batch, a->seq_kv, a->heads, a->v_row, a->v_head, a->v_batch, BN);
    }
    if (rc != FU_OK) {
        return rc;
    }
    p.o          = static_cast<__nv_bfloat16*>(a->o);
    p.lse        = a->lse;
    p.o_row      = a->o_row;
    p.o_head     = a->o_head;
    p.o_batch    = a->o_batch;
    p.B          = a->batch;
    p.H          = a->heads;
    p.Sq         = a->seq_q;
    p.Skv        = a->seq_kv;
    p.q_blocks   = (a->seq_q + QT * BM - 1) / (QT * BM);
    p.total_work = p.q_blocks * p.H * p.B;
    p.n_kv       = (a->seq_kv + BN - 1) / BN;
    p.scale      = a->scale;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.err        = a->err;

    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int grid = a->ctas > 0 ? std::min(a->ctas, sms) : sms;
    grid     = std::max(1, std::min(grid, p.total_work));
    // how many of every 16 exponential pairs go to the FMA pipe: FU_FMHA_POLY(n) in flags, default kPolyPairs
    const int np = (a->flags & FU_FMHA_POLY_SET) ? ((a->flags >> 8) & 15) : kPolyPairs;
    if (np < 0 || np > 6 || (np & 1)) {
        return fu::fail(FU_E_ARG, "fu_fmha_fwd: %d of 16 exponential pairs on the FMA pipe is not built (0, 2, 4, 6)", np);
    }
    static bool configured[64][8] = {};
    auto launch = [&](auto kernel) -> int {
        if (dev >= 64 || a->trace || !configured[dev][np]) {
            FU_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            if (dev < 64) {
                configured[dev][np] = true;
            }
        }
        kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
        FU_CUDA_OK(cudaGetLastError());
        return FU_OK;
    };
    p.trace = a->trace;
    if (a->trace) {
        if (np != 0) {
            return fu::fail(FU_E_ARG, "fu_fmha_fwd: the timeline build exists for the default exponential split only");
        }
        return launch(fmha_fwd_kernel<0, true>);
    }
    switch (np) {
    case 0: return launch(fmha_fwd_kernel<0, false>);
    case 2: return launch(fmha_fwd_kernel<2, false>);
    case 4: return launch(fmha_fwd_kernel<4, false>);
    case 6: return launch(fmha_fwd_kernel<6, false>);
    default: return fu::fail(FU_E_ARG, "fu_fmha_fwd: %d of 16 exponential pairs on the FMA pipe is not built (0, 2, 4, 6)", np);
    }
}
