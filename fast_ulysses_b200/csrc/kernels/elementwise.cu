// Memory-bound companions of the fused GEMMs.
//
//   fu_qk_norm_rope_bwd   backward of "per-head RMSNorm -> RoPE" for q and k in one pass: takes the
//                         gradients that came back from the head owners, the pre-norm projections
//                         saved by the forward kernel, and writes the gradient of the projection
//                         output (ready to be the A operand of the dgrad/wgrad GEMMs) plus the
//                         gradients of the two norm weights.
#include "fu_kernels.h"
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
