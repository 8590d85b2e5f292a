// Memory-bound companions of the fused GEMMs.
//
//   fu_qk_norm_rope_bwd   backward of "per-head RMSNorm -> RoPE" for q and k in one pass: takes the
//                         gradients that came back from the head owners, the pre-norm projections
//                         saved by the forward kernel, and writes the gradient of the projection
//                         output (ready to be the A operand of the dgrad/wgrad GEMMs) plus the
//                         gradients of the two norm weights.
//   fu_pull_qkv_grads     the same pass fused with the exchange that brings dq, dk and dv home
//                         (mode 1 of the all-to-all): every head-row is loaded straight from the
//                         rank that owns the head, over NVLink, transformed on the way (q, k) or
//                         passed through (v), and stored where the dgrad/wgrad GEMMs read it. One
//                         launch replaces the stand-alone exchange, this kernel's local form and a
//                         slice copy; the handshakes are those of every kernel that touches peers.
#include "fu_kernels.h"
#include "handshake.cuh"
#include "host_util.h"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace {

struct NormRopeBwd {
    const __nv_bfloat16* g[2];      // dq, dk: (m, heads, 128) dense
    const __nv_bfloat16* y;         // (m, 2 * heads * 128) pre-norm projections, leading dim ld_y
    __nv_bfloat16*       dy;        // (m, ...) output, leading dim ld_dy; q at column 0, k at heads * 128
    const float2*        rope;      // (s_local, 64)
    const float*         gamma[2];
    float*               dgamma[2];
    int64_t              ld_y, ld_dy;
    int64_t              m, s_local;
    int                  heads;
    float                eps;
};

__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const NormRopeBwd p)
{
    const int     lane   = threadIdx.x & 31;
    const int64_t warp0  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int64_t items  = p.m * p.heads;  // per projection
    for (int t = 0; t < 2; ++t) {
        const float4 gm = *reinterpret_cast<const float4*>(p.gamma[t] + lane * 4);
        float        dg[4] = {0.f, 0.f, 0.f, 0.f};
        for (int64_t it = warp0; it < items; it += nwarps) {
            const int64_t row  = it / p.heads;
            const int     head = static_cast<int>(it - row * p.heads);
            const int64_t s    = row % p.s_local;
            const uint2   gv   = *reinterpret_cast<const uint2*>(p.g[t] + (row * p.heads + head) * 128 + lane * 4);
            const uint2   yv   = *reinterpret_cast<const uint2*>(p.y + row * p.ld_y + (t * p.heads + head) * 128 + lane * 4);
            const float2  g01  = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.x));
            const float2  g23  = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.y));
            const float2  y01  = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.x));
            const float2  y23  = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.y));
            const float4  cs   = *reinterpret_cast<const float4*>(p.rope + s * 64 + lane * 2);  // (c0, s0, c1, s1)
            // undo the rotation: the transpose of a rotation is the opposite rotation
            const float dx[4] = {g01.x * cs.x + g01.y * cs.y, -g01.x * cs.y + g01.y * cs.x,
                                 g23.x * cs.z + g23.y * cs.w, -g23.x * cs.w + g23.y * cs.z};
            const float yy[4] = {y01.x, y01.y, y23.x, y23.y};
            float       ss    = yy[0] * yy[0] + yy[1] * yy[1] + yy[2] * yy[2] + yy[3] * yy[3];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, off);
            }
            const float rstd  = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
            const float gmv[4] = {gm.x, gm.y, gm.z, gm.w};
            float       n[4], dn[4], dot = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                n[k]  = yy[k] * rstd;
                dn[k] = dx[k] * gmv[k];
                dg[k] += dx[k] * n[k];
                dot += dn[k] * n[k];
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, off);
            }
            dot *= (1.0f / 128.0f);
            uint2 out;
            out.x = fu::ptx::pack_bf16x2(rstd * (dn[0] - n[0] * dot), rstd * (dn[1] - n[1] * dot));
            out.y = fu::ptx::pack_bf16x2(rstd * (dn[2] - n[2] * dot), rstd * (dn[3] - n[3] * dot));
            *reinterpret_cast<uint2*>(p.dy + row * p.ld_dy + (t * p.heads + head) * 128 + lane * 4) = out;
        }
        if (p.dgamma[t]) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                atomicAdd(p.dgamma[t] + lane * 4 + k, dg[k]);
            }
        }
    }
}

// ---- LayerNorm without affine parameters ----------------------------------------------------------------
// One warp per row, two passes over the row (the second is an L1/L2 hit): statistics in fp32.
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, float* stats,
                                                            int64_t rows, int64_t cols, int64_t ldx, int64_t ldy, float eps)
{
    const int     lane = threadIdx.x & 31;
    const int64_t row  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) {
        return;
    }
    const __nv_bfloat16* xr = x + row * ldx;
    float                s = 0.f, ss = 0.f;
    for (int64_t c = lane * 8; c < cols; c += 256) {
        const uint4           v = *reinterpret_cast<const uint4*>(xr + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            s += f.x + f.y;
            ss += f.x * f.x + f.y * f.y;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, off);
        ss += __shfl_xor_sync(0xffffffffu, ss, off);
    }
    const float mean = s / static_cast<float>(cols);
    const float rstd = rsqrtf(fmaxf(ss / static_cast<float>(cols) - mean * mean, 0.f) + eps);
    if (lane == 0 && stats) {
        stats[2 * row]     = mean;
        stats[2 * row + 1] = rstd;
    }
    __nv_bfloat16* yr = y + row * ldy;
    for (int64_t c = lane * 8; c < cols; c += 256) {
        const uint4           v = *reinterpret_cast<const uint4*>(xr + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint32_t              o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            o[j]           = fu::ptx::pack_bf16x2((f.x - mean) * rstd, (f.y - mean) * rstd);
        }
        *reinterpret_cast<uint4*>(yr + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const __nv_bfloat16* dy, const __nv_bfloat16* x,
                                                            const float* stats, __nv_bfloat16* dx, int64_t rows,
                                                            int64_t cols, int64_t ld)
{
    const int     lane = threadIdx.x & 31;
    const int64_t row  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) {
        return;
    }
    const float          mean = stats[2 * row], rstd = stats[2 * row + 1];
    const __nv_bfloat16* xr = x + row * ld;
    const __nv_bfloat16* gr = dy + row * ld;
    float                sg = 0.f, sgx = 0.f;
    for (int64_t c = lane * 8; c < cols; c += 256) {
        const uint4           xv = *reinterpret_cast<const uint4*>(xr + c);
        const uint4           gv = *reinterpret_cast<const uint4*>(gr + c);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 xf = __bfloat1622float2(xh[j]), gf = __bfloat1622float2(gh[j]);
            sg += gf.x + gf.y;
            sgx += gf.x * (xf.x - mean) * rstd + gf.y * (xf.y - mean) * rstd;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        sg += __shfl_xor_sync(0xffffffffu, sg, off);
        sgx += __shfl_xor_sync(0xffffffffu, sgx, off);
    }
    const float mg = sg / static_cast<float>(cols), mgx = sgx / static_cast<float>(cols);
    __nv_bfloat16* dr = dx + row * ld;
    for (int64_t c = lane * 8; c < cols; c += 256) {
        const uint4           xv = *reinterpret_cast<const uint4*>(xr + c);
        const uint4           gv = *reinterpret_cast<const uint4*>(gr + c);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
        uint32_t              o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 xf = __bfloat1622float2(xh[j]), gf = __bfloat1622float2(gh[j]);
            o[j] = fu::ptx::pack_bf16x2(rstd * (gf.x - mg - (xf.x - mean) * rstd * mgx),
                                        rstd * (gf.y - mg - (xf.y - mean) * rstd * mgx));
        }
        *reinterpret_cast<uint4*>(dr + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- the same backward, fed by the head owners' memory ----------------------------------------------
constexpr int MAX_HEADS = 128;

struct PullGrads {
    const uint8_t*       src[3][FU_MAX_WORLD];  // dq, dk, dv of every rank: (b, s_total, heads_of[p], 128) bf16
    fu::Peers            peers;
    const __nv_bfloat16* y;                     // (m, 2 * heads * 128) pre-norm q | k, leading dim ld_y
    __nv_bfloat16*       dy;                    // (m, 3 * heads * 128): d(projection) for q | k | v
    const float2*        rope;                  // (s_local, 64)
    const float*         gamma[2];
    float*               dgamma[2];
    int64_t              ld_y, ld_dy;
    int64_t              m, s_local, seq_off, s_total;
    int                  heads, handshake;
    float                eps;
    uint8_t              owner[MAX_HEADS], local[MAX_HEADS], heads_of[FU_MAX_WORLD];
};

__global__ void __launch_bounds__(256) pull_qkv_grads_kernel(const __grid_constant__ PullGrads p)
{
    __shared__ uint32_t ticket;
    const int      lane = threadIdx.x & 31;
    const int      warp = threadIdx.x >> 5;
    const uint64_t base = *reinterpret_cast<volatile uint64_t*>(&p.peers.own->epoch);
    // Opening: every rank says "my dq, dk, dv are complete" (stream order put this kernel after its
    // attention backward); nobody reads a peer before that. Every CTA polls the local flags itself.
    if (p.handshake && warp == 0) {
        if (blockIdx.x == 0) {
            fu::hs_announce(p.peers, base + 1);
        }
        fu::hs_await(p.peers, base + 1, FU_ST_OPEN_TIMEOUT);
    }
    __syncthreads();

    const int64_t warp0  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int64_t items  = p.m * p.heads;  // per projection
    for (int t = 0; t < 3; ++t) {
        float4 gm    = make_float4(0.f, 0.f, 0.f, 0.f);
        float  dg[4] = {0.f, 0.f, 0.f, 0.f};
        if (t < 2) {
            gm = *reinterpret_cast<const float4*>(p.gamma[t] + lane * 4);
        }
        // Four rows per warp in flight: a load from a peer takes microseconds, and with one per
        // warp the kernel would wait on latency instead of on the link.
        constexpr int kInFlight = 4;
        for (int64_t it0 = warp0; it0 < items; it0 += nwarps * kInFlight) {
            uint2   gvs[kInFlight], yvs[kInFlight];
            int64_t rows[kInFlight];
            int     hds[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int64_t it = it0 + u * nwarps;
                rows[u]          = -1;
                if (it < items) {
                    const int64_t  row   = it / p.heads;
                    const int      head  = static_cast<int>(it - row * p.heads);
                    const int64_t  batch = row / p.s_local;
                    const int64_t  s     = row - batch * p.s_local;
                    const int      peer  = p.owner[head];
                    const int64_t  hp    = p.heads_of[peer];
                    const uint8_t* from  = p.src[t][peer]
                                          + (((batch * p.s_total + p.seq_off + s) * hp + p.local[head]) * 128 + lane * 4) * 2;
                    asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(gvs[u].x), "=r"(gvs[u].y) : "l"(from));
                    if (t < 2) {
                        yvs[u] = *reinterpret_cast<const uint2*>(p.y + row * p.ld_y + (t * p.heads + head) * 128 + lane * 4);
                    }
                    rows[u] = row;
                    hds[u]  = head;
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (rows[u] < 0) {
                    continue;
                }
                const int64_t row  = rows[u];
                const int     head = hds[u];
                const int64_t s    = row % p.s_local;
                const uint2   gv   = gvs[u];
                __nv_bfloat16* to = p.dy + row * p.ld_dy + (static_cast<int64_t>(t) * p.heads + head) * 128 + lane * 4;
                if (t == 2) {
                    *reinterpret_cast<uint2*>(to) = gv;  // dv needs no transformation
                    continue;
                }
                const uint2  yv  = yvs[u];
                const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.x));
                const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.y));
                const float2 y01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.x));
                const float2 y23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.y));
                const float4 cs  = *reinterpret_cast<const float4*>(p.rope + s * 64 + lane * 2);  // (c0, s0, c1, s1)
                // undo the rotation: the transpose of a rotation is the opposite rotation
                const float dx[4] = {g01.x * cs.x + g01.y * cs.y, -g01.x * cs.y + g01.y * cs.x,
                                     g23.x * cs.z + g23.y * cs.w, -g23.x * cs.w + g23.y * cs.z};
                const float yy[4] = {y01.x, y01.y, y23.x, y23.y};
                float       ss    = yy[0] * yy[0] + yy[1] * yy[1] + yy[2] * yy[2] + yy[3] * yy[3];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    ss += __shfl_xor_sync(0xffffffffu, ss, off);
                }
                const float rstd   = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
                const float gmv[4] = {gm.x, gm.y, gm.z, gm.w};
                float       n[4], dn[4], dot = 0.0f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    n[k]  = yy[k] * rstd;
                    dn[k] = dx[k] * gmv[k];
                    dg[k] += dx[k] * n[k];
                    dot += dn[k] * n[k];
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    dot += __shfl_xor_sync(0xffffffffu, dot, off);
                }
                dot *= (1.0f / 128.0f);
                uint2 out;
                out.x = fu::ptx::pack_bf16x2(rstd * (dn[0] - n[0] * dot), rstd * (dn[1] - n[1] * dot));
                out.y = fu::ptx::pack_bf16x2(rstd * (dn[2] - n[2] * dot), rstd * (dn[3] - n[3] * dot));
                *reinterpret_cast<uint2*>(to) = out;
            }
        }
        if (t < 2 && p.dgamma[t]) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                atomicAdd(p.dgamma[t] + lane * 4 + k, dg[k]);
            }
        }
    }
    // Closing: "I have finished reading everybody's gradients", so that their owners may overwrite
    // them; the CTA that finishes last says it and waits for the same word from every peer.
    __syncthreads();
    if (threadIdx.x == 0) {
        ticket = atomicAdd(&p.peers.own->arrive[0], 1u);
    }
    __syncthreads();
    if (ticket == gridDim.x - 1 && warp == 0) {
        if (p.handshake) {
            fu::ptx::fence_sys();
            fu::hs_announce(p.peers, base + 2);
            fu::hs_await(p.peers, base + 2, FU_ST_CLOSE_TIMEOUT);
        }
        if (lane == 0) {
            p.peers.own->arrive[0] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint64_t*>(&p.peers.own->epoch) = base + 2;
        }
    }
}

}  // namespace

extern "C" int fu_qk_norm_rope_bwd(const FuNormRopeBwdArgs* a, void* stream)
{
    if (!a || !a->dq || !a->dk || !a->y || !a->dy || !a->rope || !a->gamma_q || !a->gamma_k) {
        return fu::fail(FU_E_ARG, "fu_qk_norm_rope_bwd: null operand");
    }
    if (a->m <= 0 || a->heads <= 0 || a->s_local <= 0 || (a->ld_y % 4) || (a->ld_dy % 4)) {
        return fu::fail(FU_E_ARG, "fu_qk_norm_rope_bwd: bad shape");
    }
    NormRopeBwd p{};
    p.g[0]      = static_cast<const __nv_bfloat16*>(a->dq);
    p.g[1]      = static_cast<const __nv_bfloat16*>(a->dk);
    p.y         = static_cast<const __nv_bfloat16*>(a->y);
    p.dy        = static_cast<__nv_bfloat16*>(a->dy);
    p.rope      = reinterpret_cast<const float2*>(a->rope);
    p.gamma[0]  = a->gamma_q;
    p.gamma[1]  = a->gamma_k;
    p.dgamma[0] = a->dgamma_q;
    p.dgamma[1] = a->dgamma_k;
    p.ld_y      = a->ld_y;
    p.ld_dy     = a->ld_dy;
    p.m         = a->m;
    p.s_local   = a->s_local;
    p.heads     = a->heads;
    p.eps       = a->eps;
    int dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    qk_norm_rope_bwd_kernel<<<sms * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_pull_qkv_grads_check(const FuPullGradsArgs* a)
{
    if (!a || !a->y || !a->dy || !a->rope || !a->gamma_q || !a->gamma_k) {
        return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: null operand");
    }
    if (a->world < 1 || a->world > FU_MAX_WORLD || a->rank < 0 || a->rank >= a->world) {
        return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: rank %d / world %d", a->rank, a->world);
    }
    if (a->m <= 0 || a->heads <= 0 || a->heads > MAX_HEADS || a->s_local <= 0 || a->m % a->s_local || (a->ld_y % 4)
        || (a->ld_dy % 4)) {
        return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: bad shape (m=%lld heads=%d s_local=%lld)", (long long)a->m, a->heads,
                        (long long)a->s_local);
    }
    if (a->seq_off < 0 || a->s_total <= 0 || a->seq_off + a->s_local > a->s_total) {
        return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: rows %lld..%lld do not lie inside a sequence of %lld",
                        (long long)a->seq_off, (long long)(a->seq_off + a->s_local), (long long)a->s_total);
    }
    int heads_seen = 0;
    const int64_t batches = a->m / a->s_local;
    for (int p = 0; p < a->world; ++p) {
        if (a->head_splits[p] < 0 || a->head_splits[p] > 255 || !a->peer_dq[p] || !a->peer_dk[p] || !a->peer_dv[p]
            || !a->peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: bad shard or missing buffer for rank %d", p);
        }
        heads_seen += a->head_splits[p];
        // row (batch, seq_off + s) of rank p's buffers starts at ((batch * s_total + seq_off + s) * head_splits[p]) * 256
        const int64_t last = ((batches - 1) * a->s_total + a->seq_off + a->s_local) * a->head_splits[p] * 256;
        if (last > a->src_bytes) {
            return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: the loads from rank %d reach byte %lld of buffers of %lld bytes", p,
                            (long long)last, (long long)a->src_bytes);
        }
    }
    if (heads_seen != a->heads) {
        return fu::fail(FU_E_ARG, "fu_pull_qkv_grads: head_splits sum to %d, expected %d", heads_seen, a->heads);
    }
    return FU_OK;
}

extern "C" int fu_pull_qkv_grads(const FuPullGradsArgs* a, void* stream)
{
    const int rc = fu_pull_qkv_grads_check(a);
    if (rc != FU_OK) {
        return rc;
    }
    PullGrads p{};
    int       h = 0;
    for (int r = 0; r < a->world; ++r) {
        p.src[0][r]     = static_cast<const uint8_t*>(a->peer_dq[r]);
        p.src[1][r]     = static_cast<const uint8_t*>(a->peer_dk[r]);
        p.src[2][r]     = static_cast<const uint8_t*>(a->peer_dv[r]);
        p.peers.ctrl[r] = a->peer_ctrl[r];
        p.heads_of[r]   = static_cast<uint8_t>(a->head_splits[r]);
        for (int i = 0; i < a->head_splits[r]; ++i, ++h) {
            p.owner[h] = static_cast<uint8_t>(r);
            p.local[h] = static_cast<uint8_t>(i);
        }
    }
    p.peers.own        = a->peer_ctrl[a->rank];
    p.peers.rank       = a->rank;
    p.peers.world      = a->world;
    p.peers.mute       = (a->flags & FU_A2A_MUTE) ? 1 : 0;
    p.peers.timeout_ns = static_cast<uint64_t>(a->timeout_ms ? a->timeout_ms : 10000) * 1000000ull;
    p.handshake        = (a->flags & FU_A2A_NO_HANDSHAKE) ? 0 : 1;
    p.y                = static_cast<const __nv_bfloat16*>(a->y);
    p.dy               = static_cast<__nv_bfloat16*>(a->dy);
    p.rope             = reinterpret_cast<const float2*>(a->rope);
    p.gamma[0]         = a->gamma_q;
    p.gamma[1]         = a->gamma_k;
    p.dgamma[0]        = a->dgamma_q;
    p.dgamma[1]        = a->dgamma_k;
    p.ld_y             = a->ld_y;
    p.ld_dy            = a->ld_dy;
    p.m                = a->m;
    p.s_local          = a->s_local;
    p.seq_off          = a->seq_off;
    p.s_total          = a->s_total;
    p.heads            = a->heads;
    p.eps              = a->eps;
    int dev = 0, sms = 0, per_sm = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // One wave: the CTA that finishes last waits for the peers, and CTAs that have not started yet
    // must not be what a peer is waiting for. Every CTA of the first wave gets to run whatever
    // else is on the device, and a resident grid keeps the closing handshake prompt.
    FU_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pull_qkv_grads_kernel, 256, 0));
    const int grid = sms * (per_sm > 0 ? per_sm : 1);
    pull_qkv_grads_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_layernorm_fwd(const void* x, void* y, float* stats, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                                float eps, void* stream)
{
    if (!x || !y || rows <= 0 || cols <= 0 || (cols % 8) || (ldx % 8) || (ldy % 8)
        || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u)) {
        return fu::fail(FU_E_ARG, "fu_layernorm_fwd: needs 16-byte aligned rows of a multiple of 8 columns");
    }
    const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);  // eight warps, one row each
    layernorm_fwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), stats, rows, cols, ldx, ldy, eps);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_layernorm_bwd(const void* dy, const void* x, const float* stats, void* dx, int64_t rows, int64_t cols,
                                int64_t ld, void* stream)
{
    if (!dy || !x || !stats || !dx || rows <= 0 || cols <= 0 || (cols % 8) || (ld % 8)
        || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15u)) {
        return fu::fail(FU_E_ARG, "fu_layernorm_bwd: needs 16-byte aligned rows of a multiple of 8 columns");
    }
    const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
    layernorm_bwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stats,
        static_cast<__nv_bfloat16*>(dx), rows, cols, ld);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
