// Block-scaled fp8 (e4m3) payloads for the exchange: every run of 128 values (one head of one
// token) is scaled by amax / 448 and rounded to e4m3; the fp32 scale travels with its payload in
// the same row of the packed tensor, so one all_to_all_4d moves both and a tile never arrives
// without its scale. Packed layout per (token, head): 128 bytes of e4m3 followed by 16 bytes whose
// first four hold the fp32 scale (the rest keeps rows 16-byte granular): last dimension 144.
//
//
// fu_a2a4d_fp8 is the exchange itself in that format, in ONE launch and with no pass of its own over
// HBM for the quantisation: every rank reads its bf16 input once, quantises each (token, head) row in
// registers and stores payload and scale straight into the owning peer's window (0.52 of the bf16
// bytes cross NVLink; inside the windows payloads and scales lie in two planes, see below); after
// the closing handshake each rank expands its window into the bf16 result. The stand-alone kernels remain for callers that want the packed tensor itself.
//
// The reference moves fp8/int8 tensors as opaque bytes (src/group.cc:54-62) and has no scaling.
#include "fu_kernels.h"
#include "handshake.cuh"
#include "host_util.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>

namespace {

constexpr int kBlock  = 128;
constexpr int kPacked = 144;

// one warp per block of 128 values: lane holds 4 consecutive values
__global__ void __launch_bounds__(256) quant_e4m3_kernel(const __nv_bfloat16* x, uint8_t* packed, int64_t blocks)
{
    const int     lane   = threadIdx.x & 31;
    const int64_t warp0  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t blk = warp0; blk < blocks; blk += nwarps) {
        const uint2  raw = *reinterpret_cast<const uint2*>(x + blk * kBlock + lane * 4);
        const float2 a   = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b   = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        float        amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        }
        const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
        const float inv   = 1.0f / scale;
        uint32_t    q     = 0;
        q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3));
        q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3)) << 8;
        q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3)) << 16;
        q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3)) << 24;
        uint8_t* row = packed + blk * kPacked;
        *reinterpret_cast<uint32_t*>(row + lane * 4) = q;
        if (lane < 4) {
            *reinterpret_cast<float*>(row + kBlock + lane * 4) = lane == 0 ? scale : 0.0f;
        }
    }
}

__global__ void __launch_bounds__(256) dequant_e4m3_kernel(const uint8_t* packed, __nv_bfloat16* x, int64_t blocks)
{
    const int     lane   = threadIdx.x & 31;
    const int64_t warp0  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t blk = warp0; blk < blocks; blk += nwarps) {
        const uint8_t* row   = packed + blk * kPacked;
        const float    scale = *reinterpret_cast<const float*>(row + kBlock);
        const uint32_t q     = *reinterpret_cast<const uint32_t*>(row + lane * 4);
        float          v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((q >> (8 * k)) & 0xff), __NV_E4M3);
            v[k]               = __half2float(*reinterpret_cast<const __half*>(&h)) * scale;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2                out;
        out.x = *reinterpret_cast<const uint32_t*>(&lo);
        out.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(x + blk * kBlock + lane * 4) = out;
    }
}

// ---- the exchange with quantisation in the store path ---------------------------------------------------
// Inside the windows of this kernel the payloads and the scales lie in two planes: row i of a window
// (rows in the order of the result: batch, token, local head) has its 128 e4m3 bytes at i * 128 and
// its fp32 scale at win_rows * 128 + i * 4, with win_rows = win_bytes / 144 on every rank. A warp
// quantises four neighbouring heads of a token at a time, so what it stores into a peer's window
// is 512 contiguous, aligned payload bytes and 16 contiguous scale bytes: NVLink carries whole
// 128-byte lines at its full rate and odd-sized pieces (a 144-byte row) at a fraction of it.
struct Fp8Route {
    const uint8_t* src;  // bf16 rows of 256 bytes
    uint8_t*       dst;  // the peer's window
    int64_t        src_pitch, src_batch;              // bytes
    int64_t        dst_row0, dst_pitch, dst_batch;    // window rows
    int64_t        rows, batches, heads_per_row, groups, count;  // groups of 4 heads; count = batches * rows * groups
};

struct Fp8Args {
    Fp8Route       r[FU_MAX_WORLD];
    int            n;
    fu::Peers      peers;
    const uint8_t* window;  // own window
    __nv_bfloat16* out;
    int64_t        out_rows;  // (token, head) rows of the result
    int64_t        scale_off; // byte offset of the scale plane in every window
    int            handshake;
};

constexpr int kFp8Unroll = 2;  // groups of four rows whose loads are in flight per warp

__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float inv)
{
    uint32_t q = 0;
    q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(a * inv, __NV_SATFINITE, __NV_E4M3));
    q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(b * inv, __NV_SATFINITE, __NV_E4M3)) << 8;
    q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(c * inv, __NV_SATFINITE, __NV_E4M3)) << 16;
    q |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(d * inv, __NV_SATFINITE, __NV_E4M3)) << 24;
    return q;
}

__device__ __forceinline__ void dequant4(uint32_t q, float scale, uint32_t& lo, uint32_t& hi)
{
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((q >> (8 * k)) & 0xff), __NV_E4M3);
        v[k]               = __half2float(*reinterpret_cast<const __half*>(&h)) * scale;
    }
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    const __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
    lo = *reinterpret_cast<const uint32_t*>(&a);
    hi = *reinterpret_cast<const uint32_t*>(&b);
}

__global__ void __launch_bounds__(256) a2a4d_fp8_kernel(const __grid_constant__ Fp8Args a)
{
    __shared__ uint32_t ticket;
    const int      lane   = threadIdx.x & 31;
    const int      warp   = threadIdx.x >> 5;
    const int      sub    = lane >> 3;  // which of the warp's four rows this lane works on
    const int      part   = lane & 7;   // which 16 values of that row
    const int64_t  warp0  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t  nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    FuCtrl*        own    = a.peers.own;
    const uint64_t base   = *reinterpret_cast<volatile uint64_t*>(&own->epoch);
    // Opening: nobody overwrites a window before its owner has finished reading it.
    if (a.handshake && warp == 0) {
        if (blockIdx.x == 0) {
            fu::hs_announce(a.peers, base + 1);
        }
        fu::hs_await(a.peers, base + 1, FU_ST_OPEN_TIMEOUT);
    }
    __syncthreads();
    // Push: every (token, head) row is read once, quantised in registers and stored into the
    // window of the rank that owns the head (mode 0) or the token (mode 1).
    for (int ri = 0; ri < a.n; ++ri) {
        const Fp8Route& r = a.r[ri];
        for (int64_t i0 = warp0 * kFp8Unroll; i0 < r.count; i0 += nwarps * kFp8Unroll) {
            uint4   raw[kFp8Unroll][2];
            int64_t to[kFp8Unroll];  // window row this lane's values belong to, or -1
#pragma unroll
            for (int u = 0; u < kFp8Unroll; ++u) {
                const int64_t i = i0 + u;
                to[u]           = -1;
                if (i < r.count) {
                    const int64_t g     = i % r.groups;
                    const int64_t row   = (i / r.groups) % r.rows;
                    const int64_t batch = i / (r.groups * r.rows);
                    const int64_t h     = g * 4 + sub;
                    if (h < r.heads_per_row) {
                        const uint4* from = reinterpret_cast<const uint4*>(r.src + batch * r.src_batch + row * r.src_pitch
                                                                           + h * 256 + part * 32);
                        raw[u][0] = from[0];
                        raw[u][1] = from[1];
                        to[u]     = r.dst_row0 + batch * r.dst_batch + row * r.dst_pitch + h;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kFp8Unroll; ++u) {
                float v[16];
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const uint32_t w[4] = {raw[u][k].x, raw[u][k].y, raw[u][k].z, raw[u][k].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f   = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                        v[k * 8 + 2 * j]     = to[u] >= 0 ? f.x : 0.0f;
                        v[k * 8 + 2 * j + 1] = to[u] >= 0 ? f.y : 0.0f;
                    }
                }
                float amax = 0.0f;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    amax = fmaxf(amax, fabsf(v[k]));
                }
#pragma unroll
                for (int off = 4; off > 0; off >>= 1) {  // the eight lanes of one row
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                }
                const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
                const float inv   = 1.0f / scale;
                if (to[u] >= 0) {
                    const uint4 q = make_uint4(quant4(v[0], v[1], v[2], v[3], inv), quant4(v[4], v[5], v[6], v[7], inv),
                                               quant4(v[8], v[9], v[10], v[11], inv), quant4(v[12], v[13], v[14], v[15], inv));
                    *reinterpret_cast<uint4*>(r.dst + to[u] * kBlock + part * 16) = q;
                    if (part == 0) {
                        *reinterpret_cast<float*>(r.dst + a.scale_off + to[u] * 4) = scale;
                    }
                }
            }
        }
    }
    // Closing: "all my writes have landed"; every CTA waits for everyone's, because every CTA reads
    // the window next.
    fu::ptx::fence_sys();
    __syncthreads();
    if (threadIdx.x == 0) {
        ticket = atomicAdd(&own->arrive[0], 1u);
    }
    __syncthreads();
    if (a.handshake && warp == 0) {
        if (ticket == gridDim.x - 1) {
            fu::ptx::fence_sys();
            fu::hs_announce(a.peers, base + 2);
        }
        fu::hs_await(a.peers, base + 2, FU_ST_CLOSE_TIMEOUT);
    }
    __syncthreads();
    // Expand the own window (what the peers and this rank itself have written) into the result:
    // four rows per warp, 512 bytes of payload in, 1 KiB of bf16 out.
    const int64_t out_groups = (a.out_rows + 3) / 4;
    for (int64_t i0 = warp0 * kFp8Unroll; i0 < out_groups; i0 += nwarps * kFp8Unroll) {
        uint4 q[kFp8Unroll];
        float sc[kFp8Unroll];
#pragma unroll
        for (int u = 0; u < kFp8Unroll; ++u) {
            const int64_t row = (i0 + u) * 4 + sub;
            if (row < a.out_rows) {
                const uint8_t* from = a.window + row * kBlock + part * 16;
                asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(q[u].x), "=r"(q[u].y), "=r"(q[u].z), "=r"(q[u].w)
                             : "l"(from));
                asm volatile("ld.global.f32 %0, [%1];" : "=f"(sc[u]) : "l"(a.window + a.scale_off + row * 4));
            }
        }
#pragma unroll
        for (int u = 0; u < kFp8Unroll; ++u) {
            const int64_t row = (i0 + u) * 4 + sub;
            if (row < a.out_rows) {
                uint4 lo, hi;
                dequant4(q[u].x, sc[u], lo.x, lo.y);
                dequant4(q[u].y, sc[u], lo.z, lo.w);
                dequant4(q[u].z, sc[u], hi.x, hi.y);
                dequant4(q[u].w, sc[u], hi.z, hi.w);
                uint4* to = reinterpret_cast<uint4*>(a.out + row * kBlock + part * 16);
                to[0]     = lo;
                to[1]     = hi;
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        ticket = atomicAdd(&own->arrive[1], 1u);
    }
    __syncthreads();
    if (ticket == gridDim.x - 1 && threadIdx.x == 0) {
        own->arrive[0] = 0;
        own->arrive[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint64_t*>(&own->epoch) = base + 2;
    }
}

int grid_for(int64_t blocks)
{
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = (blocks + 7) / 8;
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sms) * 16)));
}

}  // namespace

extern "C" int fu_quant_e4m3_block128(const void* x_bf16, void* packed, int64_t blocks, void* stream)
{
    if (!x_bf16 || !packed || blocks < 0) {
        return fu::fail(FU_E_ARG, "fu_quant_e4m3_block128: bad argument");
    }
    if (blocks == 0) {
        return FU_OK;
    }
    quant_e4m3_kernel<<<grid_for(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(packed), blocks);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_dequant_e4m3_block128(const void* packed, void* x_bf16, int64_t blocks, void* stream)
{
    if (!x_bf16 || !packed || blocks < 0) {
        return fu::fail(FU_E_ARG, "fu_dequant_e4m3_block128: bad argument");
    }
    if (blocks == 0) {
        return FU_OK;
    }
    dequant_e4m3_kernel<<<grid_for(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), static_cast<__nv_bfloat16*>(x_bf16), blocks);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

// Routes are the bf16 plan's (offsets, pitches and row lengths in bytes of (b, s, n, 128) bf16
// tensors, all multiples of 256); the destination side is rescaled to packed rows here.
extern "C" int fu_a2a4d_fp8_check(const FuA2AFp8Args* a)
{
    if (!a || !a->src || !a->out) {
        return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: null operand");
    }
    if (a->world < 1 || a->world > FU_MAX_WORLD || a->rank < 0 || a->rank >= a->world || a->n_routes < 0
        || a->n_routes > FU_MAX_WORLD) {
        return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: rank %d / world %d / %d routes", a->rank, a->world, a->n_routes);
    }
    if ((reinterpret_cast<uintptr_t>(a->src) & 15u) || (reinterpret_cast<uintptr_t>(a->out) & 15u) || a->out_rows < 0
        || a->out_rows * kPacked > a->win_bytes) {
        return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: unaligned operand, or %lld result rows in a window of %lld bytes",
                        (long long)a->out_rows, (long long)a->win_bytes);
    }
    for (int p = 0; p < a->world; ++p) {
        if (!a->peer_win[p] || !a->peer_ctrl[p] || (reinterpret_cast<uintptr_t>(a->peer_win[p]) & 15u)) {
            return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: no (aligned) window or control block for rank %d", p);
        }
    }
    for (int i = 0; i < a->n_routes; ++i) {
        const FuRoute& r = a->routes[i];
        if (r.peer < 0 || r.peer >= a->world) {
            return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: route %d names rank %d", i, r.peer);
        }
        if (((r.row_bytes | r.src_off | r.dst_off | r.src_pitch | r.dst_pitch | r.src_batch | r.dst_batch) & 255)
            || (r.src_off | r.dst_off | r.src_pitch | r.dst_pitch | r.src_batch | r.dst_batch | r.row_bytes) < 0) {
            return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: route %d is not made of whole 128-value rows", i);
        }
        if (r.rows <= 0 || r.batches <= 0 || r.row_bytes <= 0) {
            continue;
        }
        const int64_t src_end = r.src_off + (r.batches - 1) * r.src_batch + (r.rows - 1) * r.src_pitch + r.row_bytes;
        const int64_t dst_end = (r.dst_off + (r.batches - 1) * r.dst_batch + (r.rows - 1) * r.dst_pitch + r.row_bytes) / 256 * kPacked;
        if (src_end > a->src_bytes) {
            return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: route %d reads up to byte %lld of an input of %lld bytes", i,
                            (long long)src_end, (long long)a->src_bytes);
        }
        if (dst_end > a->win_bytes) {
            return fu::fail(FU_E_ARG, "fu_a2a4d_fp8: route %d writes up to byte %lld of rank %d's window of %lld bytes", i,
                            (long long)dst_end, r.peer, (long long)a->win_bytes);
        }
    }
    return FU_OK;
}

extern "C" int fu_a2a4d_fp8(const FuA2AFp8Args* a, void* stream)
{
    const int rc = fu_a2a4d_fp8_check(a);
    if (rc != FU_OK) {
        return rc;
    }
    Fp8Args k{};
    for (int i = 0; i < a->n_routes; ++i) {
        const FuRoute& r = a->routes[i];
        if (r.rows <= 0 || r.batches <= 0 || r.row_bytes <= 0) {
            continue;
        }
        Fp8Route& o     = k.r[k.n++];
        o.src           = static_cast<const uint8_t*>(a->src) + r.src_off;
        o.dst           = static_cast<uint8_t*>(a->peer_win[r.peer]);
        o.src_pitch     = r.src_pitch;
        o.src_batch     = r.src_batch;
        o.dst_row0      = r.dst_off / 256;
        o.dst_pitch     = r.dst_pitch / 256;
        o.dst_batch     = r.dst_batch / 256;
        o.rows          = r.rows;
        o.batches       = r.batches;
        o.heads_per_row = r.row_bytes / 256;
        o.groups        = (o.heads_per_row + 3) / 4;
        o.count         = o.batches * o.rows * o.groups;
    }
    k.scale_off = a->win_bytes / kPacked * kBlock;  // the same on every rank: windows have one size
    for (int p = 0; p < a->world; ++p) {
        k.peers.ctrl[p] = a->peer_ctrl[p];
    }
    k.peers.own        = a->peer_ctrl[a->rank];
    k.peers.rank       = a->rank;
    k.peers.world      = a->world;
    k.peers.mute       = (a->flags & FU_A2A_MUTE) ? 1 : 0;
    k.peers.timeout_ns = static_cast<uint64_t>(a->timeout_ms ? a->timeout_ms : 10000) * 1000000ull;
    k.handshake        = (a->flags & FU_A2A_NO_HANDSHAKE) ? 0 : 1;
    k.window           = static_cast<const uint8_t*>(a->peer_win[a->rank]);
    k.out              = static_cast<__nv_bfloat16*>(a->out);
    k.out_rows         = a->out_rows;
    int dev = 0, sms = 0, per_sm = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    FU_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a2a4d_fp8_kernel, 256, 0));
    // Every CTA waits for the peers between its two phases, so the grid must be resident at once;
    // with peers it takes two thirds of what fits, like the bf16 exchange, so that an asynchronous
    // exchange of the same rank always finds room beside it.
    int grid = sms * std::max(1, std::min(per_sm, 4));
    if (a->world > 1) {
        grid = grid * 2 / 3;
    }
    grid = std::max(1, a->ctas > 0 ? std::min(a->ctas, grid) : grid);
    a2a4d_fp8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(k);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
