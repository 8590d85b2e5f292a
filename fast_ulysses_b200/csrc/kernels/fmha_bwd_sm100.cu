// Non-causal flash attention backward for head_dim 128 on the tcgen05 tensor cores: the entry
// points, the small pre- and post-passes, and the choice between the two implementations.
//
//   default        one software-pipelined pass (fmha_bwd_fused_sm100.cu). dK and dV stay in tensor
//                  memory for a whole K/V block; dQ is summed over the K/V blocks with fp32
//                  reductions into a scratch accumulator, so its last bits depend on their order.
//   deterministic  two passes without atomics: dK/dV with the K/V block stationary
//                  (fmha_bwd_dkdv_sm100.cu), then dQ with the query rows stationary
//                  (fmha_bwd_dq_sm100.cu). Seven products instead of five.
//
// The pre-pass computes delta = rowsum(O o dO) and rescales the log-sum-exp to base 2, both padded
// to whole query blocks; the post-pass of the default path scales and rounds the fp32 dQ
// accumulator to bf16.
#include "fu_kernels.h"
#include "host_util.h"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <algorithm>

namespace {

using namespace fu;

constexpr int D   = 128;
constexpr int BLK = 128;

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
    const bool deterministic = a && (a->flags & FU_FMHA_DETERMINISTIC) != 0;
    if (!a || !a->q || !a->k || !a->v || !a->o || !a->lse || !a->d_o || !a->dq || !a->dk || !a->dv || !a->delta
        || (!deterministic && !a->dq_acc)) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd: null operand");
    }
    if (a->head_dim != D) {
        return fu::fail(FU_E_UNSUPPORTED, "fu_fmha_bwd: head_dim %d (only 128 is built)", a->head_dim);
    }
    if (a->batch < 1 || a->heads < 1 || a->seq_q < 1 || a->seq_kv < 1) {
        return fu::fail(FU_E_ARG, "fu_fmha_bwd: empty problem");
    }
    cudaStream_t  stream = static_cast<cudaStream_t>(stream_v);
    const int     sq_pad = (a->seq_q + BLK - 1) / BLK * BLK;
    const int64_t stats  = static_cast<int64_t>(a->batch) * a->heads * sq_pad;

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
    if (deterministic) {
        const int rc = fu_fmha_bwd_dkdv_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
        return rc != FU_OK ? rc : fu_fmha_bwd_dq_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
    }
    FU_CUDA_OK(cudaMemsetAsync(a->dq_acc, 0, sizeof(float) * a->batch * static_cast<int64_t>(a->seq_q) * a->heads * D,
                               stream));
    const int rc = fu_fmha_bwd_fused_launch(a, pre.lse2, pre.delta, sq_pad, stream_v);
    if (rc != FU_OK) {
        return rc;
    }
    const int64_t n = static_cast<int64_t>(a->batch) * a->seq_q * a->heads * 16;
    fmha_bwd_post_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
        a->dq_acc, static_cast<__nv_bfloat16*>(a->dq), a->q_row, a->q_head, a->q_batch, a->batch, a->heads, a->seq_q,
        a->scale);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
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
    // Two limits, each named in its own message: the dQ accumulator bounds the number of query rows,
    // the statistics bound the number of rows AFTER seq_q has been rounded up to 128 per (batch,
    // head), which is the one that bites for many heads with short sequences.
    if (acc > kNoAllocAccBytes) {
        return fu::fail(FU_E_ARG,
                        "fu_fmha_bwd_noalloc: batch %d x heads %d x seq_q %d is %zu query rows; the built-in dQ "
                        "accumulator holds batch*heads*seq_q <= 16384 rows (%zu bytes). Use fu_fmha_bwd with your own "
                        "buffers",
                        a->batch, a->heads, a->seq_q, static_cast<size_t>(a->batch) * a->heads * a->seq_q,
                        kNoAllocAccBytes);
    }
    if (stats > kNoAllocStatsBytes) {
        return fu::fail(FU_E_ARG,
                        "fu_fmha_bwd_noalloc: batch %d x heads %d x seq_q %d needs statistics for %zu padded rows; the "
                        "built-in scratch holds batch*heads*roundup(seq_q, 128) <= 65536 rows (%zu bytes). Use "
                        "fu_fmha_bwd with your own buffers",
                        a->batch, a->heads, a->seq_q, static_cast<size_t>(a->batch) * a->heads * sq_pad,
                        kNoAllocStatsBytes);
    }
    // The array's name is only a host-side handle; the device address has to be asked for, once
    // per device, with that device current. This happens on the first call on each device. The
    // address is remembered for the life of the process: after cudaDeviceReset() it is stale, and
    // this entry point must not be used again in that process.
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
