// Block-scaled fp8 (e4m3) payloads for the exchange: every run of 128 values (one head of one
// token) is scaled by amax / 448 and rounded to e4m3; the fp32 scale travels with its payload in
// the same row of the packed tensor, so one all_to_all_4d moves both and a tile never arrives
// without its scale. Packed layout per (token, head): 128 bytes of e4m3 followed by 16 bytes whose
// first four hold the fp32 scale (the rest keeps rows 16-byte granular): last dimension 144.
//
// The reference moves fp8/int8 tensors as opaque bytes (src/group.cc:54-62) and has no scaling.
#include "fu_kernels.h"
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
