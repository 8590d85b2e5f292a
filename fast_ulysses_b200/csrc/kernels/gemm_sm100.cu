// tcgen05 GEMM kernels built on gemm_sm100.cuh:
//
//   fu_gemm_bf16          C = act(A * B^T + bias) + residual, bf16 in/out, fp32 accumulate.
//   fu_qkv_rope_scatter   the fused mode-0 path: QKV projection whose epilogue applies per-head
//                         RMSNorm and 3D RoPE to q and k in registers and stores every head-row
//                         straight into the owning rank's q/k/v window at its permuted
//                         (sequence-gathered, head-scattered) position over NVLink. The all-to-all
//                         is the address of the store; there is no separate exchange or permute.
//
// The reference has no GEMM: its example wraps nn.Linear + separate norm/RoPE around two
// all_to_all_4d calls (examples/dit_attention.py:45-63). These kernels replace that composition.
#include "fu_kernels.h"
#include "gemm_sm100.cuh"
#include "host_util.h"
#include "tma_host.h"

#include <algorithm>
#include <cstdlib>

namespace {

using namespace fu;
using namespace fu::gemm;

// ---- plain epilogue --------------------------------------------------------------------------------
struct PlainEpi {
    __nv_bfloat16*       c;
    const __nv_bfloat16* residual;
    const float*         bias;
    int64_t              ldc;
    int                  M, N, act;
    const __nv_bfloat16* aux;    // act 3: where the tanh-form GELU's derivative is evaluated
    __nv_bfloat16*       c_pre;  // optional second output: the value before the activation

    __device__ void open(int) {}
    __device__ void close(int) {}

    __device__ __forceinline__ static float gelu_tanh(float x)
    {
        const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    __device__ __forceinline__ static float gelu_erf(float x)
    {
        return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    }
    __device__ __forceinline__ static float gelu_tanh_grad(float x)
    {
        const float x2 = x * x;
        const float th = tanhf(0.7978845608028654f * (x + 0.044715f * x * x2));
        return 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * 0.7978845608028654f * (1.0f + 0.134145f * x2);
    }

    __device__ void tile(uint32_t tmem_acc, int mt, int nt, int quarter, int lane)
    {
        const int  row    = mt * BM + quarter * 32 + lane;
        const bool row_ok = row < M;
#pragma unroll 1
        for (int chunk = 0; chunk < BN / 32; ++chunk) {
            const int col0 = nt * BN + chunk * 32;
            if (col0 >= N) {
                break;  // warp-uniform
            }
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem_acc + chunk * 32, r);
            ptx::tmem_ld_wait();
            if (!row_ok) {
                continue;
            }
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                v[j] = __uint_as_float(r[j]);
            }
            if (bias) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (col0 + j < N) {
                        v[j] += bias[col0 + j];
                    }
                }
            }
            if (c_pre) {  // the pre-activation, for the backward (whole 8-column groups only: N % 8 == 0 is checked)
                uint4* pre = reinterpret_cast<uint4*>(c_pre + static_cast<int64_t>(row) * ldc + col0);
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    if (col0 + g8 * 8 + 8 <= N) {
                        pre[g8] = make_uint4(pack_bf16(v[g8 * 8 + 0], v[g8 * 8 + 1]), pack_bf16(v[g8 * 8 + 2], v[g8 * 8 + 3]),
                                             pack_bf16(v[g8 * 8 + 4], v[g8 * 8 + 5]), pack_bf16(v[g8 * 8 + 6], v[g8 * 8 + 7]));
                    }
                }
            }
            if (act == 3) {
                const __nv_bfloat16* at = aux + static_cast<int64_t>(row) * ldc + col0;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    if (col0 + g8 * 8 + 8 <= N) {
                        const uint4           av = *reinterpret_cast<const uint4*>(at + g8 * 8);
                        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(ap[j]);
                            v[g8 * 8 + 2 * j] *= gelu_tanh_grad(f.x);
                            v[g8 * 8 + 2 * j + 1] *= gelu_tanh_grad(f.y);
                        }
                    }
                }
            }
            if (act == 1) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    v[j] = gelu_tanh(v[j]);
                }
            }
            else if (act == 2) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    v[j] = gelu_erf(v[j]);
                }
            }
            __nv_bfloat16*       dst = c + static_cast<int64_t>(row) * ldc + col0;
            const __nv_bfloat16* res = residual ? residual + static_cast<int64_t>(row) * ldc + col0 : nullptr;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
                if (col0 + g8 * 8 + 8 <= N) {
                    if (res) {
                        const uint4 rv = *reinterpret_cast<const uint4*>(res + g8 * 8);
                        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(rp[j]);
                            v[g8 * 8 + 2 * j] += f.x;
                            v[g8 * 8 + 2 * j + 1] += f.y;
                        }
                    }
                    uint4 o;
                    o.x = pack_bf16(v[g8 * 8 + 0], v[g8 * 8 + 1]);
                    o.y = pack_bf16(v[g8 * 8 + 2], v[g8 * 8 + 3]);
                    o.z = pack_bf16(v[g8 * 8 + 4], v[g8 * 8 + 5]);
                    o.w = pack_bf16(v[g8 * 8 + 6], v[g8 * 8 + 7]);
                    *reinterpret_cast<uint4*>(dst + g8 * 8) = o;
                }
                else {
                    for (int j = 0; j < 8; ++j) {
                        if (col0 + g8 * 8 + j < N) {
                            float x = v[g8 * 8 + j];
                            if (res) {
                                x += __bfloat162float(res[g8 * 8 + j]);
                            }
                            dst[g8 * 8 + j] = __float2bfloat16(x);
                        }
                    }
                }
            }
        }
    }
};

struct PlainArgs {
    Core     core;
    PlainEpi epi;
};

__global__ void __launch_bounds__(THREADS, 1) gemm_plain_kernel(const __grid_constant__ PlainArgs a)
{
    PlainEpi epi = a.epi;
    run(a.core, epi);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1) gemm_pair_kernel(const __grid_constant__ PlainArgs a)
{
    PlainEpi epi = a.epi;
    run_pair(a.core, epi);
}

// ---- fused QKV epilogue: RMSNorm + 3D RoPE + scatter ---------------------------------------------------
constexpr int HEAD_DIM = 128;
constexpr int MAX_HEADS = 128;

struct QkvParams {
    uint8_t*      win[3][FU_MAX_WORLD];  // q, k, v window base on every rank
    Peers         peers;
    const float2* rope;     // [s_local][64] (cos, sin) per rotated pair
    const float*  gamma_q;  // [128]
    const float*  gamma_k;
    float         eps;
    int           M, heads;          // rows = b * s_local; heads per projection
    int64_t       s_local, seq_off, s_total;
    uint8_t       owner[MAX_HEADS];  // head -> rank that owns it
    uint8_t       local[MAX_HEADS];  // head -> index inside its owner's shard
    uint8_t       heads_of[FU_MAX_WORLD];
    int           handshake;
    int           n_types, n_normed;
    __nv_bfloat16* y_save;
    int64_t       ld_y;
};

// The functor keeps a reference to the parameters (they stay in the kernel's constant bank) and
// only its own mutable state in registers.
struct QkvEpi {
    const QkvParams& p;
    uint64_t         base_epoch;

    __device__ explicit QkvEpi(const QkvParams& params) : p(params), base_epoch(0) {}

    __device__ void open(int epi_warp)
    {
        const Peers& peers     = p.peers;
        const int    handshake = p.handshake;
        base_epoch = *reinterpret_cast<volatile uint64_t*>(&peers.own->epoch);
        if (handshake && epi_warp == 0) {
            if (blockIdx.x == 0) {
                hs_announce(peers, base_epoch + 1);
            }
            hs_await(peers, base_epoch + 1, FU_ST_OPEN_TIMEOUT);
        }
        epi_barrier();  // no epilogue thread stores to a peer before the owners said "go"
    }

    __device__ void close(int epi_tid)
    {
        __shared__ uint32_t ticket;
        const Peers& peers     = p.peers;
        const int    handshake = p.handshake;
        ptx::fence_sys();
        epi_barrier();
        if (epi_tid == 0) {
            ticket = atomicAdd(&peers.own->arrive[0], 1u);
        }
        epi_barrier();
        if (ticket == gridDim.x - 1 && epi_tid < 32) {
            if (handshake) {
                ptx::fence_sys();
                hs_announce(peers, base_epoch + 2);
                hs_await(peers, base_epoch + 2, FU_ST_CLOSE_TIMEOUT);
            }
            if (epi_tid == 0) {
                peers.own->arrive[0] = 0;
                __threadfence();
                *reinterpret_cast<volatile uint64_t*>(&peers.own->epoch) = base_epoch + 2;
            }
        }
    }

    __device__ void tile(uint32_t tmem_acc, int mt, int nt, int quarter, int lane)
    {
        const int     M = p.M, heads = p.heads;
        const int64_t s_local = p.s_local, s_total = p.s_total, seq_off = p.seq_off;
        const float   eps = p.eps;
        const int     row    = mt * BM + quarter * 32 + lane;
        const bool    row_ok = row < M;
        const int64_t batch  = row / s_local;
        const int64_t s      = row - batch * s_local;
#pragma unroll 1
        for (int hh = 0; hh < BN / HEAD_DIM; ++hh) {
            const int head_global = nt * (BN / HEAD_DIM) + hh;
            const int type        = head_global / heads;  // 0 q, 1 k, 2 v
            if (type >= p.n_types) {
                break;
            }
            const bool normed = type < p.n_normed;
            const int      head  = head_global - type * heads;
            const int      peer  = p.owner[head];
            const int64_t  hp    = p.heads_of[peer];
            uint8_t*       dst   = p.win[type][peer]
                           + (((batch * s_total + seq_off + s) * hp + p.local[head]) * HEAD_DIM) * 2;
            const uint32_t tcol  = tmem_acc + hh * HEAD_DIM;
            float          scale = 1.0f;
            if (normed) {
                float ss = 0.0f;
#pragma unroll 1
                for (int chunk = 0; chunk < 4; ++chunk) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tcol + chunk * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float x = __uint_as_float(r[j]);
                        ss += x * x;
                    }
                }
                scale = rsqrtf(ss * (1.0f / HEAD_DIM) + eps);
            }
            const float*  gamma = type == 0 ? p.gamma_q : p.gamma_k;
            const float2* cs    = p.rope + (row_ok ? s : 0) * (HEAD_DIM / 2);
            // The finished head rows (256 bytes each) go through a per-warp staging buffer so that
            // every store instruction to the owner's window writes whole rows: lanes 0-15 one row,
            // lanes 16-31 the next. Written straight from the accumulator layout (a lane is a row)
            // each instruction would scatter 32 separate 16-byte pieces, which NVLink carries at a
            // fraction of its rate. 16-byte units are XOR-swizzled by the row so that neither the
            // row-wise writes nor the row-wide reads conflict on shared-memory banks.
            uint8_t* stage = stage_of(quarter);
#pragma unroll 1
            for (int chunk = 0; chunk < 4; ++chunk) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tcol + chunk * 32, r);
                ptx::tmem_ld_wait();
                uint32_t o[16];
                if (normed) {
                    if (p.y_save && row_ok) {
                        uint4* ys = reinterpret_cast<uint4*>(p.y_save + static_cast<int64_t>(row) * p.ld_y
                                                             + head_global * HEAD_DIM + chunk * 32);
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            ys[q4] = make_uint4(pack_bf16(__uint_as_float(r[8 * q4]), __uint_as_float(r[8 * q4 + 1])),
                                                pack_bf16(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3])),
                                                pack_bf16(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5])),
                                                pack_bf16(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7])));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int    c0 = chunk * 32 + 2 * i;
                        const float  x0 = __uint_as_float(r[2 * i]) * scale * gamma[c0];
                        const float  x1 = __uint_as_float(r[2 * i + 1]) * scale * gamma[c0 + 1];
                        const float2 t  = cs[chunk * 16 + i];
                        o[i]            = pack_bf16(x0 * t.x - x1 * t.y, x0 * t.y + x1 * t.x);
                    }
                }
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        o[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    }
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int unit = (chunk * 4 + q4) ^ (lane & 15);
                    *reinterpret_cast<uint4*>(stage + lane * 256 + unit * 16) =
                        make_uint4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]);
                }
            }
            __syncwarp();
            const unsigned long long my_dst = row_ok ? reinterpret_cast<unsigned long long>(dst) : 0ull;
            const int                unit   = lane & 15;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
                const int                r_src = 2 * i + (lane >> 4);
                const unsigned long long to    = __shfl_sync(0xffffffffu, my_dst, r_src);
                const uint4 v = *reinterpret_cast<const uint4*>(stage + r_src * 256 + ((unit ^ (r_src & 15)) * 16));
                if (to) {
                    ptx::st_v4(reinterpret_cast<uint4*>(to) + unit, v);
                }
            }
            __syncwarp();  // the buffer is refilled by the next head
        }
    }

    // 8 KiB of staging per epilogue warp, behind the operand ring in dynamic shared memory.
    static constexpr int kStageBytesPerWarp = 32 * HEAD_DIM * 2;
    static constexpr int kExtraSmem         = 4 * kStageBytesPerWarp;
    __device__ static uint8_t* stage_of(int quarter)
    {
        extern __shared__ uint8_t smem_raw[];
        const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
        return smem_raw + (base - ptx::smem_addr(smem_raw)) + STAGES * STAGE_BYTES + quarter * kStageBytesPerWarp;
    }
};

struct QkvArgs {
    Core      core;
    QkvParams epi;
};

__global__ void __launch_bounds__(THREADS, 1) qkv_rope_scatter_kernel(const __grid_constant__ QkvArgs a)
{
    QkvEpi epi(a.epi);
    run(a.core, epi);
}

// ---- fused mode-1 path: pull attention output from peers, feed the output projection -----------------
// A[m, head*128 + x] = O_owner(head)[batch, seq_off + s, local head, x]. Four extra warps per CTA
// copy (M-tile, peer) blocks from the peers' O buffers into a local gather buffer with plain
// loads over NVLink and publish a flag per block; the TMA producer of whichever CTA needs that
// part of A waits for the flag (bounded) and then loads it from local memory, so every remote byte
// crosses NVLink once and the transfer overlaps the GEMM tile by tile. No multicast anywhere.
struct PullParams {
    const uint8_t* peer_o[FU_MAX_WORLD];
    Peers          peers;
    uint8_t*       gather;   // (M, heads_total * 128) bf16, local
    uint32_t*      ready;    // [tiles_m * world], zero before launch
    int            M, tiles_m, heads_total;
    int64_t        s_local, seq_off, s_total;
    uint8_t        heads_of[FU_MAX_WORLD];
    uint16_t       head_start[FU_MAX_WORLD];
    uint8_t        owner[MAX_HEADS];
    int            handshake;
    uint32_t*      err;
};

struct PullSrc {
    const PullParams& p;
    int               seen_mt, seen_peer;
    __device__ explicit PullSrc(const PullParams& params) : p(params), seen_mt(-1), seen_peer(-1) {}

    __device__ bool ready(int mt, int kb)
    {
        const int peer = p.owner[kb >> 1];  // BK = 64: two K-blocks per head
        if (mt == seen_mt && peer == seen_peer) {
            return true;
        }
        const uint32_t* f  = p.ready + mt * p.peers.world + peer;
        const uint64_t  t0 = ptx::globaltimer_ns();
        uint32_t        spins = 0;
        while (ptx::ld_acquire_gpu_u32(f) == 0u) {
            if ((++spins & 255u) == 0u && ptx::globaltimer_ns() - t0 > p.peers.timeout_ns) {
                return false;
            }
        }
        ptx::fence_proxy_async();  // generic-proxy writes by the pullers -> TMA reads below
        seen_mt   = mt;
        seen_peer = peer;
        return true;
    }
};

struct PullAux {
    static constexpr int kWarps = 4;
    const PullParams&    p;
    __device__ explicit PullAux(const PullParams& params) : p(params) {}

    __device__ static void aux_barrier() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

    __device__ void run(int aux_warp, int lane) const
    {
        __shared__ uint32_t ticket;
        const Peers&   peers = p.peers;
        const int      tid   = aux_warp * 32 + lane;
        const uint64_t base  = *reinterpret_cast<volatile uint64_t*>(&peers.own->epoch);
        // Opening: every rank says "my attention output is complete" (stream order put this kernel
        // after its attention kernel) and nobody reads a peer before that.
        if (p.handshake && aux_warp == 0) {
            if (blockIdx.x == 0) {
                hs_announce(peers, base + 1);
            }
            hs_await(peers, base + 1, FU_ST_OPEN_TIMEOUT);
        }
        aux_barrier();
        const int units = p.tiles_m * peers.world;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int mt   = u / peers.world;
            const int peer = (peers.rank + (u - mt * peers.world)) % peers.world;
            const int rows = min(BM, p.M - mt * BM);
            const uint32_t vpr  = static_cast<uint32_t>(p.heads_of[peer]) * 16u;  // 16-byte vectors per row
            const uint32_t nvec = vpr * rows;
            const uint8_t* src  = p.peer_o[peer];
            const int64_t  src_pitch = static_cast<int64_t>(p.heads_of[peer]) * 256;
            const int64_t  dst_pitch = static_cast<int64_t>(p.heads_total) * 256;
            uint8_t*       dst  = p.gather + static_cast<int64_t>(p.head_start[peer]) * 256;
            for (uint32_t v0 = tid; v0 < nvec; v0 += 8 * 128) {
                uint4    val[8];
                uint8_t* to[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t v = v0 + k * 128;
                    if (v < nvec) {
                        const uint32_t r     = v / vpr;
                        const uint32_t c     = v - r * vpr;
                        const int64_t  row   = static_cast<int64_t>(mt) * BM + r;
                        const int64_t  batch = row / p.s_local;
                        const int64_t  s     = row - batch * p.s_local;
                        val[k] = ptx::ld_v4(src + (batch * p.s_total + p.seq_off + s) * src_pitch + (c << 4));
                        to[k]  = dst + row * dst_pitch + (c << 4);
                    }
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (v0 + k * 128 < nvec) {
                        ptx::st_v4(to[k], val[k]);
                    }
                }
            }
            __threadfence();
            aux_barrier();
            if (tid == 0) {
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ready + mt * peers.world + peer), "r"(1u)
                             : "memory");
            }
        }
        // Closing: "I have finished reading everybody's output", so that the owners may overwrite
        // it; the last CTA also waits for the same word from all peers before the kernel ends.
        aux_barrier();
        if (tid == 0) {
            ticket = atomicAdd(&peers.own->arrive[0], 1u);
        }
        aux_barrier();
        if (ticket == gridDim.x - 1 && aux_warp == 0) {
            if (p.handshake) {
                ptx::fence_sys();
                hs_announce(peers, base + 2);
                hs_await(peers, base + 2, FU_ST_CLOSE_TIMEOUT);
            }
            if (lane == 0) {
                peers.own->arrive[0] = 0;
                __threadfence();
                *reinterpret_cast<volatile uint64_t*>(&peers.own->epoch) = base + 2;
            }
        }
    }
};

struct PullArgs {
    Core       core;
    PlainEpi   epi;
    PullParams pull;
};

__global__ void __launch_bounds__(THREADS + 128, 1) pull_outproj_kernel(const __grid_constant__ PullArgs a)
{
    PlainEpi epi = a.epi;
    run(a.core, epi, PullSrc(a.pull), PullAux(a.pull));
}

int launch_grid(int ctas, int tiles)
{
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int g = ctas > 0 ? std::min(ctas, sms) : sms;
    return std::max(1, std::min(g, tiles));
}

// Raises a kernel's dynamic shared-memory limit once per (device, kernel). Keyed by the kernel's
// address: two kernels with the same signature share one instantiation of this template.
template <class K>
int set_smem(K kernel, int bytes = SMEM_BYTES)
{
    struct Done {
        int         dev;
        const void* fn;
    };
    static Done done[256];
    static int  n_done = 0;
    int         dev    = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    const void* fn = reinterpret_cast<const void*>(kernel);
    for (int i = 0; i < n_done; ++i) {
        if (done[i].dev == dev && done[i].fn == fn) {
            return FU_OK;
        }
    }
    FU_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (n_done < 256) {
        done[n_done++] = Done{dev, fn};
    }
    return FU_OK;
}

// How many CTA pairs of the pair kernel the device holds at once (GPCs with an odd number of SMs
// leave one SM without a partner). Asked once per device.
int pair_capacity()
{
    static int cached[64] = {};
    int        dev        = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) {
        return 0;
    }
    if (cached[dev] == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim          = dim3(2, 1, 1);
        cfg.blockDim         = dim3(THREADS, 1, 1);
        cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
        cudaLaunchAttribute attr{};
        attr.id               = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs             = &attr;
        cfg.numAttrs          = 1;
        int n                 = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess || n < 1) {
            (void)cudaGetLastError();
            // the kernel carries its cluster shape itself; ask again without naming it
            cfg.attrs    = nullptr;
            cfg.numAttrs = 0;
            n            = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess || n < 1) {
                (void)cudaGetLastError();
                // Pairs do not wait for one another, so a grid larger than what is resident at once
                // is merely scheduled in turns: assume every SM finds a partner.
                int sms = 0;
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
                n = sms / 2;
            }
        }
        cached[dev] = n > 0 ? n : -1;
    }
    return cached[dev] > 0 ? cached[dev] : 0;
}

int fill_core(Core& core, const void* a, const void* b, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
              uint32_t* err, int flags = 0)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return fu::fail(FU_E_ARG, "gemm: empty problem (m=%lld n=%lld k=%lld)", (long long)m, (long long)n, (long long)k);
    }
    // K itself may be anything (TMA zero-fills the part of a box that lies past it); what TMA needs
    // is a 16-byte row pitch, which make_map_2d checks on lda and ldb.
    core.a_mn = (flags & FU_GEMM_A_KM) ? 1 : 0;
    core.b_mn = (flags & FU_GEMM_B_KN) ? 1 : 0;
    int rc = core.a_mn ? make_map_2d(&core.map_a, a, 2, k, m, lda, 64, 64) : make_map_2d(&core.map_a, a, 2, m, k, lda, BM, BK);
    if (rc != FU_OK) {
        return rc;
    }
    // a CTA pair splits B's rows of a tile between its two CTAs
    const int b_rows = (flags & FU_GEMM_PAIR) ? BN / 2 : BN;
    rc = core.b_mn ? make_map_2d(&core.map_b, b, 2, k, n, ldb, 64, 64) : make_map_2d(&core.map_b, b, 2, n, k, ldb, b_rows, BK);
    if (rc != FU_OK) {
        return rc;
    }
    core.M       = static_cast<int>(m);
    core.N       = static_cast<int>(n);
    core.K       = static_cast<int>(k);
    core.tiles_m = static_cast<int>((m + BM - 1) / BM);
    core.tiles_n = static_cast<int>((n + BN - 1) / BN);
    core.err     = err;
    return FU_OK;
}

}  // namespace

extern "C" int fu_gemm_bf16(const FuGemmArgs* g, void* stream)
{
    if (!g || !g->a || !g->b || !g->c) {
        return fu::fail(FU_E_ARG, "fu_gemm_bf16: null operand");
    }
    if ((g->ldc % 8) || (reinterpret_cast<uintptr_t>(g->c) & 15u)
        || (g->residual && (reinterpret_cast<uintptr_t>(g->residual) & 15u))) {
        return fu::fail(FU_E_ARG, "fu_gemm_bf16: C (and the residual) need 16-byte aligned rows");
    }
    // CTA pairs are chosen per call (FU_GEMM_PAIR / FU_GEMM_SINGLE) or, for calls that say nothing,
    // by the environment variable FU_GEMM_PAIR (read once).
    static const bool pair_default = [] {
        const char* e = std::getenv("FU_GEMM_PAIR");
        return e && e[0] == '1';
    }();
    const bool pair  = (g->flags & FU_GEMM_PAIR) || (pair_default && !(g->flags & FU_GEMM_SINGLE));
    const int  flags = pair ? (g->flags | FU_GEMM_PAIR) : (g->flags & ~FU_GEMM_PAIR);
    PlainArgs a{};
    int       rc = fill_core(a.core, g->a, g->b, g->m, g->n, g->k, g->lda, g->ldb, g->err, flags);
    if (rc != FU_OK) {
        return rc;
    }
    a.epi.c        = static_cast<__nv_bfloat16*>(g->c);
    a.epi.residual = static_cast<const __nv_bfloat16*>(g->residual);
    a.epi.bias     = g->bias;
    a.epi.ldc      = g->ldc;
    a.epi.M        = a.core.M;
    a.epi.N        = a.core.N;
    a.epi.act      = g->act;
    a.epi.aux      = static_cast<const __nv_bfloat16*>(g->aux);
    a.epi.c_pre    = static_cast<__nv_bfloat16*>(g->c_pre);
    if (g->act < 0 || g->act > 3 || (g->act == 3 && !g->aux)) {
        return fu::fail(FU_E_ARG, "fu_gemm_bf16: act=%d (0..3; 3 needs aux)", g->act);
    }
    if ((g->aux || g->c_pre) && ((g->n % 8) || (reinterpret_cast<uintptr_t>(g->aux) & 15u)
                                 || (reinterpret_cast<uintptr_t>(g->c_pre) & 15u))) {
        return fu::fail(FU_E_ARG, "fu_gemm_bf16: aux / c_pre need n %% 8 == 0 and 16-byte aligned rows");
    }
    if (pair) {
        rc = set_smem(gemm_pair_kernel, PAIR_SMEM_BYTES);
        if (rc != FU_OK) {
            return rc;
        }
        const int pairs = pair_capacity();
        if (pairs < 1) {
            return fu::fail(FU_E_CUDA, "fu_gemm_bf16: this device cannot hold a cluster of two CTAs of the pair kernel");
        }
        const int tiles = ((a.core.tiles_m + 1) / 2) * a.core.tiles_n;
        int       want  = g->ctas > 0 ? std::max(1, g->ctas / 2) : pairs;
        want            = std::max(1, std::min(std::min(want, pairs), tiles));
        gemm_pair_kernel<<<2 * want, THREADS, PAIR_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(a);
        FU_CUDA_OK(cudaGetLastError());
        return FU_OK;
    }
    rc             = set_smem(gemm_plain_kernel);
    if (rc != FU_OK) {
        return rc;
    }
    const int grid = launch_grid(g->ctas, a.core.tiles_m * a.core.tiles_n);
    gemm_plain_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(a);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_qkv_rope_scatter_check(const FuQkvArgs* q)
{
    if (!q || !q->x || !q->w) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: null operand");
    }
    const int n_types  = q->n_types > 0 ? q->n_types : 3;
    const int n_normed = q->n_types > 0 ? q->n_normed : 2;
    if (n_types > 3 || n_normed > 2 || n_normed > n_types) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: %d projections, %d normed", n_types, n_normed);
    }
    if (n_normed > 0 && (!q->rope || !q->gamma_q || (n_normed > 1 && !q->gamma_k))) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: RMSNorm + RoPE need rope and gamma tables");
    }
    if (q->world < 1 || q->world > FU_MAX_WORLD || q->rank < 0 || q->rank >= q->world) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: rank %d / world %d", q->rank, q->world);
    }
    if (q->heads < 1 || q->heads > MAX_HEADS) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: heads=%d (need 1..%d)", q->heads, MAX_HEADS);
    }
    if (q->s_local <= 0 || q->m % q->s_local) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: m=%lld is not a multiple of s_local=%lld", (long long)q->m,
                        (long long)q->s_local);
    }
    int heads_seen = 0;
    for (int p = 0; p < q->world; ++p) {
        if (q->head_splits[p] < 0 || q->head_splits[p] > 255) {
            return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: head_splits[%d]=%d", p, q->head_splits[p]);
        }
        heads_seen += q->head_splits[p];
        if (!q->win_q[p] || (n_types > 1 && !q->win_k[p]) || (n_types > 2 && !q->win_v[p]) || !q->peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: no window for rank %d", p);
        }
    }
    if (heads_seen != q->heads) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: head_splits sum to %d, expected %d", heads_seen, q->heads);
    }
    // The epilogue stores row (batch, seq_off + s) of head `local` of rank p at
    // ((batch * s_total + seq_off + s) * head_splits[p] + local) * 256 bytes behind that rank's base.
    if (q->seq_off < 0 || q->s_total <= 0 || q->seq_off + q->s_local > q->s_total) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: rows %lld..%lld do not lie inside a sequence of %lld",
                        (long long)q->seq_off, (long long)(q->seq_off + q->s_local), (long long)q->s_total);
    }
    const int64_t batches = q->m / q->s_local;
    for (int p = 0; p < q->world; ++p) {
        const int64_t last = ((batches - 1) * q->s_total + q->seq_off + q->s_local) * q->head_splits[p] * 256;
        if (q->head_splits[p] > 0 && last > q->win_bytes) {
            return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: the stores to rank %d reach byte %lld of windows of %lld bytes",
                            p, (long long)last, (long long)q->win_bytes);
        }
    }
    return FU_OK;
}

extern "C" int fu_qkv_rope_scatter(const FuQkvArgs* q, void* stream)
{
    int rc = fu_qkv_rope_scatter_check(q);
    if (rc != FU_OK) {
        return rc;
    }
    const int n_types  = q->n_types > 0 ? q->n_types : 3;
    const int n_normed = q->n_types > 0 ? q->n_normed : 2;
    QkvArgs a{};
    rc = fill_core(a.core, q->x, q->w, q->m, static_cast<int64_t>(n_types) * q->heads * HEAD_DIM, q->k, q->ldx, q->ldw,
                   q->err, (q->flags & FU_QKV_W_KN) ? FU_GEMM_B_KN : 0);
    if (rc != FU_OK) {
        return rc;
    }
    QkvParams& e = a.epi;
    int     h = 0;
    for (int p = 0; p < q->world; ++p) {
        if (q->head_splits[p] < 0 || q->head_splits[p] > 255) {
            return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: head_splits[%d]=%d", p, q->head_splits[p]);
        }
        e.heads_of[p] = static_cast<uint8_t>(q->head_splits[p]);
        for (int i = 0; i < q->head_splits[p]; ++i, ++h) {
            if (h >= MAX_HEADS) {
                return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: too many heads");
            }
            e.owner[h] = static_cast<uint8_t>(p);
            e.local[h] = static_cast<uint8_t>(i);
        }
        if (!q->win_q[p] || (n_types > 1 && !q->win_k[p]) || (n_types > 2 && !q->win_v[p]) || !q->peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: no window for rank %d", p);
        }
        e.win[0][p]     = static_cast<uint8_t*>(q->win_q[p]);
        e.win[1][p]     = static_cast<uint8_t*>(q->win_k[p]);
        e.win[2][p]     = static_cast<uint8_t*>(q->win_v[p]);
        e.peers.ctrl[p] = q->peer_ctrl[p];
    }
    if (h != q->heads) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: head_splits sum to %d, expected %d", h, q->heads);
    }
    e.peers.own        = q->peer_ctrl[q->rank];
    e.peers.rank       = q->rank;
    e.peers.world      = q->world;
    e.peers.mute       = (q->flags & FU_A2A_MUTE) ? 1 : 0;
    e.peers.timeout_ns = static_cast<uint64_t>(q->timeout_ms ? q->timeout_ms : 10000) * 1000000ull;
    e.handshake        = (q->flags & FU_A2A_NO_HANDSHAKE) ? 0 : 1;
    e.rope             = reinterpret_cast<const float2*>(q->rope);
    e.gamma_q          = q->gamma_q;
    e.gamma_k          = q->gamma_k;
    e.eps              = q->eps;
    e.M                = a.core.M;
    e.heads            = q->heads;
    e.s_local          = q->s_local;
    e.seq_off          = q->seq_off;
    e.s_total          = q->s_total;
    e.n_types          = n_types;
    e.n_normed         = n_normed;
    e.y_save           = static_cast<__nv_bfloat16*>(q->y_save);
    e.ld_y             = q->ld_y;
    if (q->y_save && ((q->ld_y % 8) || (reinterpret_cast<uintptr_t>(q->y_save) & 15u))) {
        return fu::fail(FU_E_ARG, "fu_qkv_rope_scatter: y_save needs 16-byte aligned rows");
    }
    rc                 = set_smem(qkv_rope_scatter_kernel, SMEM_BYTES + QkvEpi::kExtraSmem);
    if (rc != FU_OK) {
        return rc;
    }
    const int grid = launch_grid(q->ctas, a.core.tiles_m * a.core.tiles_n);
    qkv_rope_scatter_kernel<<<grid, THREADS, SMEM_BYTES + QkvEpi::kExtraSmem, static_cast<cudaStream_t>(stream)>>>(a);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_pull_outproj_check(const FuPullArgs* q)
{
    if (!q || !q->w || !q->c || !q->gather || !q->ready) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: null operand");
    }
    if (q->world < 1 || q->world > FU_MAX_WORLD || q->rank < 0 || q->rank >= q->world) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: rank %d / world %d", q->rank, q->world);
    }
    if (q->s_local <= 0 || q->m % q->s_local) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: m=%lld is not a multiple of s_local=%lld", (long long)q->m,
                        (long long)q->s_local);
    }
    if ((q->ldc % 8) || (reinterpret_cast<uintptr_t>(q->c) & 15u)) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: C needs 16-byte aligned rows");
    }
    int heads_seen = 0;
    for (int p = 0; p < q->world; ++p) {
        if (q->head_splits[p] < 0 || q->head_splits[p] > 255 || !q->peer_o[p] || !q->peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_pull_outproj: bad shard or missing buffer for rank %d", p);
        }
        heads_seen += q->head_splits[p];
    }
    if (heads_seen < 1 || heads_seen > MAX_HEADS) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: %d heads (need 1..%d)", heads_seen, MAX_HEADS);
    }
    // The puller warps read row (batch, seq_off + s) of rank p's buffer at
    // ((batch * s_total + seq_off + s) * head_splits[p]) * 256 bytes, head_splits[p] * 256 bytes long.
    if (q->seq_off < 0 || q->s_total <= 0 || q->seq_off + q->s_local > q->s_total) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: rows %lld..%lld do not lie inside a sequence of %lld",
                        (long long)q->seq_off, (long long)(q->seq_off + q->s_local), (long long)q->s_total);
    }
    const int64_t batches = q->m / q->s_local;
    for (int p = 0; p < q->world; ++p) {
        const int64_t last = ((batches - 1) * q->s_total + q->seq_off + q->s_local) * q->head_splits[p] * 256;
        if (last > q->o_bytes) {
            return fu::fail(FU_E_ARG, "fu_pull_outproj: the loads from rank %d reach byte %lld of buffers of %lld bytes", p,
                            (long long)last, (long long)q->o_bytes);
        }
    }
    if (q->m * heads_seen * 256 > q->gather_bytes) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: the gathered operand needs %lld bytes, `gather` holds %lld",
                        (long long)(q->m * heads_seen * 256), (long long)q->gather_bytes);
    }
    if (((q->m + BM - 1) / BM) * q->world > q->ready_words) {
        return fu::fail(FU_E_ARG, "fu_pull_outproj: %lld flags needed, `ready` holds %lld",
                        (long long)(((q->m + BM - 1) / BM) * q->world), (long long)q->ready_words);
    }
    return FU_OK;
}

extern "C" int fu_pull_outproj(const FuPullArgs* q, void* stream_v)
{
    int rc = fu_pull_outproj_check(q);
    if (rc != FU_OK) {
        return rc;
    }
    PullArgs a{};
    PullParams& e = a.pull;
    int heads = 0;
    for (int p = 0; p < q->world; ++p) {
        if (q->head_splits[p] < 0 || q->head_splits[p] > 255 || !q->peer_o[p] || !q->peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_pull_outproj: bad shard or missing buffer for rank %d", p);
        }
        e.heads_of[p]   = static_cast<uint8_t>(q->head_splits[p]);
        e.head_start[p] = static_cast<uint16_t>(heads);
        for (int i = 0; i < q->head_splits[p]; ++i, ++heads) {
            if (heads >= MAX_HEADS) {
                return fu::fail(FU_E_ARG, "fu_pull_outproj: too many heads");
            }
            e.owner[heads] = static_cast<uint8_t>(p);
        }
        e.peer_o[p]     = static_cast<const uint8_t*>(q->peer_o[p]);
        e.peers.ctrl[p] = q->peer_ctrl[p];
    }
    const int64_t k = static_cast<int64_t>(heads) * HEAD_DIM;
    rc = fill_core(a.core, q->gather, q->w, q->m, q->n, k, k, q->ldw, q->err);
    if (rc != FU_OK) {
        return rc;
    }
    e.peers.own        = q->peer_ctrl[q->rank];
    e.peers.rank       = q->rank;
    e.peers.world      = q->world;
    e.peers.mute       = (q->flags & FU_A2A_MUTE) ? 1 : 0;
    e.peers.timeout_ns = static_cast<uint64_t>(q->timeout_ms ? q->timeout_ms : 10000) * 1000000ull;
    e.handshake        = (q->flags & FU_A2A_NO_HANDSHAKE) ? 0 : 1;
    e.gather           = static_cast<uint8_t*>(q->gather);
    e.ready            = q->ready;
    e.M                = a.core.M;
    e.tiles_m          = a.core.tiles_m;
    e.heads_total      = heads;
    e.s_local          = q->s_local;
    e.seq_off          = q->seq_off;
    e.s_total          = q->s_total;
    e.err              = q->err;
    a.epi.c            = static_cast<__nv_bfloat16*>(q->c);
    a.epi.residual     = static_cast<const __nv_bfloat16*>(q->residual);
    a.epi.bias         = q->bias;
    a.epi.ldc          = q->ldc;
    a.epi.M            = a.core.M;
    a.epi.N            = a.core.N;
    a.epi.act          = 0;
    rc                 = set_smem(pull_outproj_kernel);
    if (rc != FU_OK) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    FU_CUDA_OK(cudaMemsetAsync(q->ready, 0, sizeof(uint32_t) * a.core.tiles_m * q->world, stream));
    // One CTA per SM and never more than the SM count: CTAs wait on flags other CTAs publish.
    const int grid = launch_grid(q->ctas, 1 << 30);
    pull_outproj_kernel<<<grid, THREADS + 128, SMEM_BYTES, stream>>>(a);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
