// Non-causal flash attention backward for head_dim 128 on the tcgen05 tensor cores.
//
// One persistent CTA per SM owns a 128-row K/V block of one (batch, head) at a time and sweeps all
// 128-row query blocks. Everything is computed transposed, so that the probabilities land in
// tensor memory with the kv row on the lane axis and can be fed back as the A operand:
//   S^T  = K Q^T           (SS)                 P^T  = exp2(S^T c - lse)          -> TMEM, bf16
//   dP^T = V dO^T          (SS)                 dS^T = P^T o (dP^T - delta) scale -> TMEM + smem
//   dV  += P^T dO          (A from TMEM, dO as an MN-major smem operand)
//   dK  += dS^T Q          (A from TMEM, Q as an MN-major smem operand)
//   dQ_i = dS K            (dS^T in smem read as an MN-major A, K as an MN-major B); added into an
//                          fp32 accumulator in global memory with vector reductions
// Tensor memory: S^T/P^T/dQ | dP^T/dS^T | dV | dK, 128 fp32 columns each.
// Warps: 0 = TMA producer, 1 = MMA issuer, 2..9 = two threads per kv row (and per q row for dQ).
//
// A small pre-pass computes delta = rowsum(O o dO) and rescales the log-sum-exp to base 2, both
// padded to whole query blocks; a post-pass rounds the fp32 dQ accumulator to bf16.
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D          = 128;
constexpr int BLK        = 128;
constexpr int TILE_BYTES = BLK * D * 2;  // 32 KiB
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int STAGES     = 2;
// dynamic shared memory layout (no static shared memory in this kernel, every byte is budgeted)
constexpr int OFF_K      = 0;
constexpr int OFF_V      = OFF_K + TILE_BYTES;
constexpr int OFF_STAGE  = OFF_V + TILE_BYTES;            // per stage: Q | dO
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int OFF_DS     = OFF_STAGE + STAGES * STAGE_BYTES;
constexpr int OFF_STATS  = OFF_DS + TILE_BYTES;           // per stage: lse2[128] | delta[128]
constexpr int OFF_BARS   = OFF_STATS + STAGES * 1024;
constexpr int SMEM_BYTES = OFF_BARS + 256;
constexpr int THREADS    = 320;   // TMA warp, MMA warp, 8 element-wise warps (two threads per row)

static_assert(SMEM_BYTES <= 232448, "shared memory budget");

enum : uint32_t { ERR_ALIGN = 20, ERR_LOAD = 21, ERR_MMA = 22, ERR_COMPUTE = 23 };

struct Params {
    CUtensorMap    map_q, map_k, map_v, map_do;
    const float*   lse2;    // (B, H, Sq_pad) log-sum-exp in base 2, +inf in the padding
    const float*   delta;   // (B, H, Sq_pad)
    float*         dq_acc;  // (B, Sq, H, 128) fp32
    __nv_bfloat16* dk;
    __nv_bfloat16* dv;
    int64_t        dk_row, dk_head, dk_batch, dv_row, dv_head, dv_batch;
    int            B, H, Sq, Skv, Sq_pad;
    int            n_q, kv_blocks, total_work;
    float          scale, scale_log2;
    uint32_t*      err;
};

struct Bars {
    uint64_t kv_full, kv_empty, full[STAGES], empty[STAGES];
    uint64_t s_full, p_ready, dq_full, st_free, acc_full, acc_free;
    uint32_t tmem_holder;
};

__device__ __forceinline__ void flag(const Params& p, uint32_t code)
{
    if (p.err) {
        atomicCAS(p.err, 0u, code);
    }
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// kDq = true: the single-pass variant that also produces dQ (atomic reductions into dq_acc).
// kDq = false (default path): dK and dV only; dQ comes from the dQ pass in fmha_bwd_dq_sm100.cu.
template <bool kDq>
__global__ void __launch_bounds__(THREADS, 1) fmha_bwd_kernel(const __grid_constant__ Params p)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    const uint32_t base = ptx::smem_addr(sm);
    Bars&          bar  = *reinterpret_cast<Bars*>(sm + OFF_BARS);
    const int      warp = threadIdx.x >> 5;
    const int      lane = threadIdx.x & 31;
    if (base & 1023u) {
        // The swizzled tiles need 1024-byte alignment and there is no room for slack: refuse.
        if (threadIdx.x == 0) {
            flag(p, ERR_ALIGN);
        }
        return;
    }

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar.kv_full, 1);
        ptx::mbar_init(&bar.kv_empty, 1);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&bar.full[s], 1);
            ptx::mbar_init(&bar.empty[s], 1);
        }
        ptx::mbar_init(&bar.s_full, 1);
        ptx::mbar_init(&bar.p_ready, 256);
        ptx::mbar_init(&bar.dq_full, 1);
        ptx::mbar_init(&bar.st_free, 256);
        ptx::mbar_init(&bar.acc_full, 1);
        ptx::mbar_init(&bar.acc_free, 256);
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
                for (int i = 0; i < n_q; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!ptx::mbar_wait(&bar.empty[s], ((it / STAGES) & 1u) ^ 1u)) {
                        flag(p, ERR_LOAD);
                        ok = false;
                        break;
                    }
                    uint8_t* st = sm + OFF_STAGE + s * STAGE_BYTES;
                    uint8_t* ss = sm + OFF_STATS + s * 1024;
                    ptx::mbar_expect_tx(&bar.full[s], STAGE_BYTES + 1024);
                    for (int half = 0; half < 2; ++half) {
                        ptx::tma_load_4d(st + half * HALF_BYTES, &p.map_q, half * 64, i * BLK, h, b, &bar.full[s]);
                        ptx::tma_load_4d(st + TILE_BYTES + half * HALF_BYTES, &p.map_do, half * 64, i * BLK, h, b,
                                         &bar.full[s]);
                    }
                    ptx::bulk_g2s(ss, lse2 + i * BLK, 512, &bar.full[s]);
                    ptx::bulk_g2s(ss + 512, delta + i * BLK, 512, &bar.full[s]);
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
            constexpr uint32_t idesc_nn = ptx::make_idesc(1, 1, BLK, D, 1, 1);    // A, B MN-major
            const uint32_t     ka = base + OFF_K, va = base + OFF_V, dsa = base + OFF_DS;
            uint32_t           it = 0, wc = 0;
            bool               ok = true;
            for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++wc) {
                if (!ptx::mbar_wait(&bar.kv_full, wc & 1u)) {
                    flag(p, ERR_MMA);
                    break;
                }
                for (int i = 0; i < n_q; ++i, ++it) {
                    const int      s  = it % STAGES;
                    const uint32_t qa = base + OFF_STAGE + s * STAGE_BYTES;
                    const uint32_t oa = qa + TILE_BYTES;
                    if (!ptx::mbar_wait(&bar.full[s], (it / STAGES) & 1u)
                        || (kDq && !ptx::mbar_wait(&bar.st_free, (it & 1u) ^ 1u))) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {  // S^T = K Q^T
                        const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                        ptx::mma_f16_ss(tmem, ptx::smem_desc_sw128(ka + off, 16, 1024),
                                        ptx::smem_desc_sw128(qa + off, 16, 1024), idesc_kk, kk != 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {  // dP^T = V dO^T
                        const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                        ptx::mma_f16_ss(tmem + 128, ptx::smem_desc_sw128(va + off, 16, 1024),
                                        ptx::smem_desc_sw128(oa + off, 16, 1024), idesc_kk, kk != 0);
                    }
                    ptx::mma_commit(&bar.s_full);
                    if (!ptx::mbar_wait(&bar.p_ready, it & 1u)
                        || (i == 0 && !ptx::mbar_wait(&bar.acc_free, (wc & 1u) ^ 1u))) {
                        flag(p, ERR_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < BLK / 16; ++kk) {  // dV += P^T dO   (contraction over q)
                        ptx::mma_f16_ts(tmem + 256, tmem + (kk >> 2) * 64 + (kk & 3) * 8,
                                        ptx::smem_desc_sw128(oa + kk * 2048, HALF_BYTES, 1024), idesc_tn,
                                        i != 0 || kk != 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < BLK / 16; ++kk) {  // dK += dS^T Q
                        ptx::mma_f16_ts(tmem + 384, tmem + 128 + (kk >> 2) * 64 + (kk & 3) * 8,
                                        ptx::smem_desc_sw128(qa + kk * 2048, HALF_BYTES, 1024), idesc_tn,
                                        i != 0 || kk != 0);
                    }
                    if (kDq) {
#pragma unroll
                        for (int kk = 0; kk < BLK / 16; ++kk) {  // dQ_i = dS K      (contraction over kv)
                            ptx::mma_f16_ss(tmem, ptx::smem_desc_sw128(dsa + kk * 2048, HALF_BYTES, 1024),
                                            ptx::smem_desc_sw128(ka + kk * 2048, HALF_BYTES, 1024), idesc_nn, kk != 0);
                        }
                    }
                    ptx::mma_commit(&bar.empty[s]);
                    if (kDq) {
                        ptx::mma_commit(&bar.dq_full);
                    }
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
        // ---------------------------------------------------------------- compute: one thread per row
        // two threads per row: warps 2..5 take columns 0..63 of a tile, warps 6..9 columns 64..127;
        // each writes its packed bf16 results over the start of the columns it read itself
        const int      quarter  = warp & 3;
        const int      c2       = (warp - 2) >> 2;
        const int      row_in   = quarter * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_off, t_dp = tmem + 128 + lane_off;
        const uint32_t t_dv = tmem + 256 + lane_off, t_dk = tmem + 384 + lane_off;
        uint8_t*       ds_row = sm + OFF_DS + row_in * 128;  // this kv row inside each 64-column half
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
                const float* lse2  = reinterpret_cast<const float*>(sm + OFF_STATS + s * 1024);
                const float* delta = lse2 + 128;
                if (!ptx::mbar_wait(&bar.s_full, it & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
#pragma unroll 1
                for (int ch = 2 * c2; ch < 2 * c2 + 2; ++ch) {
                    uint32_t rs[32], rd[32];
                    ptx::tmem_ld_32x32(t_s + ch * 32, rs);
                    ptx::tmem_ld_32x32(t_dp + ch * 32, rd);
                    ptx::tmem_ld_wait();
                    uint32_t pp[16], dd[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const int   q0 = ch * 32 + 2 * k;
                        float       p0 = ptx::ex2(fmaf(__uint_as_float(rs[2 * k]), c, -lse2[q0]));
                        float       p1 = ptx::ex2(fmaf(__uint_as_float(rs[2 * k + 1]), c, -lse2[q0 + 1]));
                        if (!kv_ok) {
                            p0 = 0.0f;
                            p1 = 0.0f;
                        }
                        const float d0 = p0 * (__uint_as_float(rd[2 * k]) - delta[q0]) * p.scale;
                        const float d1 = p1 * (__uint_as_float(rd[2 * k + 1]) - delta[q0 + 1]) * p.scale;
                        pp[k]          = ptx::pack_bf16x2(p0, p1);
                        dd[k]          = ptx::pack_bf16x2(d0, d1);
                    }
                    ptx::tmem_st_32x16(t_s + c2 * 64 + (ch & 1) * 16, pp);
                    ptx::tmem_st_32x16(t_dp + c2 * 64 + (ch & 1) * 16, dd);
                    // dS^T row into the 128B-swizzled [kv x q] tile the dQ MMA reads from shared memory
                    uint8_t* half_base = ds_row + (ch >> 1) * HALF_BYTES;
#pragma unroll
                    for (int k4 = 0; kDq && k4 < 4; ++k4) {
                        const int chunk = (ch & 1) * 4 + k4;
                        *reinterpret_cast<uint4*>(half_base + ((chunk ^ (row_in & 7)) << 4)) =
                            make_uint4(dd[4 * k4], dd[4 * k4 + 1], dd[4 * k4 + 2], dd[4 * k4 + 3]);
                    }
                }
                ptx::tmem_st_wait();
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before();
                ptx::mbar_arrive(&bar.p_ready);
                if (!kDq) {
                    continue;
                }

                // dQ_i: this thread now owns query row i * 128 + row_in
                if (!ptx::mbar_wait(&bar.dq_full, it & 1u)) {
                    flag(p, ERR_COMPUTE);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const int qrow = i * BLK + row_in;
                float*    dq   = p.dq_acc + ((static_cast<int64_t>(b) * p.Sq + qrow) * p.H + h) * D;
#pragma unroll 1
                for (int ch = 2 * c2; ch < 2 * c2 + 2; ++ch) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(t_s + ch * 32, r);
                    ptx::tmem_ld_wait();
                    if (qrow < p.Sq) {
#pragma unroll
                        for (int k4 = 0; k4 < 8; ++k4) {
                            red_add_v4(dq + ch * 32 + 4 * k4, __uint_as_float(r[4 * k4]), __uint_as_float(r[4 * k4 + 1]),
                                       __uint_as_float(r[4 * k4 + 2]), __uint_as_float(r[4 * k4 + 3]));
                        }
                    }
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(&bar.st_free);
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
            ptx::mbar_arrive(&bar.acc_free);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tmem_dealloc<512>(tmem);
    }
}

// delta[b,h,s] = sum_x O[b,s,h,x] * dO[b,s,h,x]; lse2 = lse * log2(e); padding rows get lse2 = +inf
// (so that their probabilities vanish) and delta = 0. One warp per (b, h, s).
struct PreParams {
    const __nv_bfloat16 *o, *d_o;
    const float*         lse;
    float *              lse2, *delta;
    int64_t              o_row, o_head, o_batch, do_row, do_head, do_batch;
    int                  B, H, Sq, Sq_pad;
};

__global__ void fmha_bwd_pre_kernel(const PreParams p)
{
    const int64_t gw    = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int     lane  = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.B) * p.H * p.Sq_pad;
    if (gw >= total) {
        return;
    }
    const int s = static_cast<int>(gw % p.Sq_pad);
    const int h = static_cast<int>((gw / p.Sq_pad) % p.H);
    const int b = static_cast<int>(gw / (static_cast<int64_t>(p.Sq_pad) * p.H));
    if (s >= p.Sq) {
        if (lane == 0) {
            p.lse2[gw]  = INFINITY;
            p.delta[gw] = 0.0f;
        }
        return;
    }
    const uint2 ov = *reinterpret_cast<const uint2*>(p.o + b * p.o_batch + static_cast<int64_t>(s) * p.o_row
                                                     + h * p.o_head + lane * 4);
    const uint2 dv = *reinterpret_cast<const uint2*>(p.d_o + b * p.do_batch + static_cast<int64_t>(s) * p.do_row
                                                     + h * p.do_head + lane * 4);
    const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.x));
    const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.y));
    const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.x));
    const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.y));
    float        acc = o0.x * d0.x + o0.y * d0.y + o1.x * d1.x + o1.y * d1.y;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
    }
    if (lane == 0) {
        p.delta[gw] = acc;
        p.lse2[gw]  = p.lse[(static_cast<int64_t>(b) * p.H + h) * p.Sq + s] * 1.4426950408889634f;
    }
}

// dq[b,s,h,:] = bf16(dq_acc[b,s,h,:] * scale)
__global__ void fmha_bwd_post_kernel(const float* acc, __nv_bfloat16* dq, int64_t dq_row, int64_t dq_head,
                                     int64_t dq_batch, int B, int H, int Sq, float scale)
{
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // one per 8 elements
    const int64_t total = static_cast<int64_t>(B) * Sq * H * 16;
    if (idx >= total) {
        return;
    }
    const int     x8 = static_cast<int>(idx & 15);
    const int64_t r  = idx >> 4;
    const int     h  = static_cast<int>(r % H);
    const int64_t bs = r / H;
    const int     s  = static_cast<int>(bs % Sq);
    const int     b  = static_cast<int>(bs / Sq);
    const float4  a0 = *reinterpret_cast<const float4*>(acc + r * 128 + x8 * 8);
    const float4  a1 = *reinterpret_cast<const float4*>(acc + r * 128 + x8 * 8 + 4);
    uint4         o;
    o.x = ptx::pack_bf16x2(a0.x * scale, a0.y * scale);
    o.y = ptx::pack_bf16x2(a0.z * scale, a0.w * scale);
    o.z = ptx::pack_bf16x2(a1.x * scale, a1.y * scale);
    o.w = ptx::pack_bf16x2(a1.z * scale, a1.w * scale);
    *reinterpret_cast<uint4*>(dq + b * dq_batch + static_cast<int64_t>(s) * dq_row + h * dq_head + x8 * 8) = o;
}

}  // namespace

int fu_fmha_bwd_dq_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream);
int fu_fmha_bwd_dkdv_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream);
int fu_fmha_bwd_fused_launch(const FuFmhaArgs* a, const float* lse2, const float* delta, int sq_pad, void* stream);

extern "C" int fu_fmha_bwd(const FuFmhaArgs* a, void* stream_v)
{
    if (!a || !a->q || !a->k || !a->v || !a->o || !a->lse || !a->d_o || !a->dq || !a->dk || !a->dv || !a->delta
        || ((a->pad_ & 5) && !a->dq_acc)) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd: null operand");
    }
    if (a->head_dim != D) {
        return fu::fail(FU_E_UNSUPPORTED, "fu_fmha_bwd: head_dim %d (only 128 is built)", a->head_dim);
    }
    if (a->batch < 1 || a->heads < 1 || a->seq_q < 1 || a->seq_kv < 1) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd: empty problem");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int    sq_pad = (a->seq_q + BLK - 1) / BLK * BLK;
    const int64_t stats = static_cast<int64_t>(a->batch) * a->heads * sq_pad;

    PreParams pre{};
    pre.o = static_cast<const __nv_bfloat16*>(a->o);
    pre.d_o = static_cast<const __nv_bfloat16*>(a->d_o);
    pre.lse = a->lse;
    pre.lse2 = a->delta;
    pre.delta = a->delta + stats;
    pre.o_row = pre.do_row = a->o_row;
    pre.o_head = pre.do_head = a->o_head;
    pre.o_batch = pre.do_batch = a->o_batch;
    pre.B = a->batch;
    pre.H = a->heads;
    pre.Sq = a->seq_q;
    pre.Sq_pad = sq_pad;
    {
        const int64_t threads = stats * 32;
        fmha_bwd_pre_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(pre);
        FU_CUDA_OK(cudaGetLastError());
    }
    const bool single_pass = (a->pad_ & 1) != 0;
    const bool fused       = (a->pad_ & 4) != 0;
    if (single_pass || fused) {
        FU_CUDA_OK(cudaMemsetAsync(a->dq_acc, 0,
                                   sizeof(float) * a->batch * static_cast<int64_t>(a->seq_q) * a->heads * D, stream));
    }

    auto round_dq = [&](float scale) -> int {
        const int64_t n = static_cast<int64_t>(a->batch) * a->seq_q * a->heads * 16;
        fmha_bwd_post_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
            a->dq_acc, static_cast<__nv_bfloat16*>(a->dq), a->q_row, a->q_head, a->q_batch, a->batch, a->heads, a->seq_q, scale);
        FU_CUDA_OK(cudaGetLastError());
        return FU_OK;
    };
    if (fused) {
        // one software-pipelined pass (fmha_bwd_fused_sm100.cu); dQ is reduced in fp32
        const int rc_f = fu_fmha_bwd_fused_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
        return rc_f != FU_OK ? rc_f : round_dq(a->scale);
    }

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
    p.lse2       = pre.lse2;
    p.delta      = pre.delta;
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

    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static bool configured[64] = {};
    if (dev < 64 && !configured[dev]) {
        FU_CUDA_OK(cudaFuncSetAttribute(fmha_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        FU_CUDA_OK(cudaFuncSetAttribute(fmha_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[dev] = true;
    }
    int grid = a->ctas > 0 ? std::min(a->ctas, sms) : sms;
    grid     = std::max(1, std::min(grid, p.total_work));
    if (!single_pass) {
        // Two passes, no atomics: dK/dV with the K/V block stationary, then dQ with the query rows
        // stationary (fmha_bwd_dq_sm100.cu). Both read the statistics prepared above.
        if (a->pad_ & 2) {
            // the earlier dK/dV pass without double buffering, kept for comparison
            fmha_bwd_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(p);
            FU_CUDA_OK(cudaGetLastError());
        }
        else {
            rc = fu_fmha_bwd_dkdv_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
            if (rc != FU_OK) {
                return rc;
            }
        }
        return fu_fmha_bwd_dq_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
    }
    fmha_bwd_kernel<true><<<grid, THREADS, SMEM_BYTES, stream>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return round_dq(1.0f);
}

// ---- attention backward for callers that cannot allocate ------------------------------------------
// Some callers of this library are not allowed to obtain device memory at the point where they
// need the backward pass: code running while a CUDA graph is being recorded, plugins living inside
// a host application that owns the only allocator, or a real-time loop in which cudaMalloc's
// implicit device synchronisation is unacceptable. For them the two scratch buffers of
// fu_fmha_bwd (the padded softmax statistics and the fp32 dQ accumulator) live in the array below,
// which is part of the library image: every GPU that loads the library holds these bytes until the
// process exits. The price is a fixed upper bound on the problem size and no concurrency: every
// call uses the same bytes.
constexpr size_t kNoAllocStatsBytes = 512u << 10;   // 2 * batch * heads * roundup(seq_q, 128) floats
constexpr size_t kNoAllocAccBytes   = 8u << 20;     // batch * seq_q * heads * 128 floats
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocStatsBytes + kNoAllocAccBytes];

extern "C" int fu_fmha_bwd_noalloc(const FuFmhaArgs* a, void* stream)
{
    if (!a) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd_noalloc: null args");
    }
    if (a->batch < 1 || a->heads < 1 || a->seq_q < 1) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd_noalloc: empty problem");
    }
    const size_t sq_pad = (static_cast<size_t>(a->seq_q) + BLK - 1) / BLK * BLK;
    const size_t stats  = 2 * sizeof(float) * a->batch * a->heads * sq_pad;
    const size_t acc    = sizeof(float) * a->batch * static_cast<size_t>(a->seq_q) * a->heads * D;
    if (stats > kNoAllocStatsBytes || acc > kNoAllocAccBytes) {
        return fu::fail(FU_E_ARG,
                        "fu_fmha_bwd_noalloc: batch %d x heads %d x seq_q %d needs %zu + %zu scratch bytes, the built-in "
                        "scratch holds %zu + %zu (batch*heads*seq_q <= 16384); use fu_fmha_bwd with your own buffers",
                        a->batch, a->heads, a->seq_q, stats, acc, kNoAllocStatsBytes, kNoAllocAccBytes);
    }
    // The array's name is only a host-side handle; the device address has to be asked for, once
    // per device, with that device current. This happens on the first call on each device.
    static void* base[64] = {};
    int          dev      = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        return fu::fail(FU_E_UNSUPPORTED, "fu_fmha_bwd_noalloc: device index %d", dev);
    }
    if (!base[dev]) {
        void* ptr = nullptr;
        FU_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        base[dev] = ptr;
    }
    FuFmhaArgs local = *a;
    local.delta      = reinterpret_cast<float*>(base[dev]);
    local.dq_acc     = reinterpret_cast<float*>(static_cast<unsigned char*>(base[dev]) + kNoAllocStatsBytes);
    // fu_fmha_bwd zeroes the accumulator and rewrites every statistic it reads, so nothing of an
    // earlier call survives into this one.
    return fu_fmha_bwd(&local, stream);
}
