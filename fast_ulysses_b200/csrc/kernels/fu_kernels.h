#pragma once
// C interface of the sm_100a kernel library. Everything here takes raw device pointers and a CUDA
// stream: the kernels never learn where a peer address came from (symmetric memory, IPC, or a fake
// peer on the same device in a single-GPU test), and nothing in this library includes torch.
//
// Every launcher returns 0 on success or a negative FU_E_* code; fu_last_error() gives the text.
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FU_API __attribute__((visibility("default")))
#define FU_MAX_WORLD 8

enum {
    FU_OK            = 0,
    FU_E_ARG         = -1,  // an argument the launcher refuses before launching anything
    FU_E_CUDA        = -2,  // a CUDA runtime/driver call failed
    FU_E_UNSUPPORTED = -3,
};

// ---- control block ------------------------------------------------------------------------------
// One per window, inside the same symmetric allocation, so that two collectives on two windows can
// never disturb each other's handshake. `flags[p]` is written by rank p (remotely); everything else
// is local to the owning rank.
typedef struct FuCtrl {
    uint64_t flags[FU_MAX_WORLD];  // last phase number rank p has announced to this rank
    uint64_t epoch;                // phases this rank has completed on this window (+2 per call)
    uint32_t arrive[2];            // CTA arrival counters used inside one launch
    uint32_t status[6];            // [0] code, [1] peer, [2,3] expected, [4,5] seen (FU_ST_*)
    uint64_t stamps[8];            // globaltimer ns: start, opened, pushed, closed, done
    uint8_t  slot_of[FU_MAX_WORLD];  // written by rank p with its opening announcement: where rank p
                                   // wants this call's payload (0 = its window, k = its pool buffer k)
    uint64_t pad_[10];
} FuCtrl;  // 256 bytes

#define FU_CTRL_BYTES 256

enum {
    FU_ST_OK            = 0,
    FU_ST_OPEN_TIMEOUT  = 1,  // a peer never announced that it had finished reading the window
    FU_ST_CLOSE_TIMEOUT = 2,  // a peer never announced that its writes had landed
    FU_ST_COPY_TIMEOUT  = 3,  // a bulk copy inside the kernel did not complete
};

// ---- all-to-all -----------------------------------------------------------------------------------
typedef struct FuRoute {
    int32_t peer;
    int32_t pad_;
    int64_t src_off, dst_off;
    int64_t src_pitch, dst_pitch;
    int64_t row_bytes, rows;
    int64_t batches, src_batch, dst_batch;
} FuRoute;

enum {
    FU_A2A_NO_HANDSHAKE  = 1,   // skip both handshakes: single-device emulation of several ranks
    FU_A2A_STAMPS        = 2,   // record per-phase globaltimer stamps into ctrl->stamps
    FU_A2A_EARLY_PUBLISH = 4,   // TEST ONLY negative control: announce completion before the payload
    FU_A2A_LDST          = 8,   // move data with 16-byte ld/st instead of bulk (TMA) copies
    FU_A2A_MUTE          = 16,  // TEST ONLY: never announce anything, so that peers' waits run out
    FU_A2A_MINOR_SHARE   = 32,  // this launch may run beside another collective of the same rank on
                                // an unordered stream: take a third of the device, not two thirds
    FU_A2A_COPY_ENGINE   = 128, // move the payload with the copy engines (one cudaMemcpy2DAsync per
                                // route and batch) between two one-warp handshake kernels: no SM is
                                // held while the payload moves, so GEMMs beside the call keep the
                                // whole device. Same handshake protocol as the kernel transport, so
                                // ranks may mix the two. Not available to a call that may use the
                                // output pool (the host cannot know which buffer a peer chose).
    FU_A2A_KEEP_EPOCH    = 256, // leave the window's phase counter alone (a helper launch inside a
                                // call whose handshakes are run by other launches)
    FU_A2A_CE_LOCAL_COPIES = 512, // with FU_A2A_COPY_ENGINE: the copies that stay on this device (own
                                // share, copy-out) also go through cudaMemcpy2DAsync instead of a
                                // small launch of the exchange kernel
};

// Output pool. A rank may ask its peers, per call, to write into one of up to FU_POOL_SLOTS extra
// symmetric buffers instead of its window: the result is then already where the caller will read
// it and nothing is copied out. Each rank chooses for itself (whichever of its buffers is free, or
// none) and tells the others in the opening handshake, so ranks never have to agree.
#define FU_POOL_SLOTS 4

typedef struct FuA2AArgs {
    const void* src;                    // this rank's input
    void*       peer_win[FU_MAX_WORLD]; // window base on every rank (own entry included)
    FuCtrl*     peer_ctrl[FU_MAX_WORLD];
    void*       out;                    // if non-null: after the closing handshake copy the dense
    int64_t     out_bytes;              //   prefix of the own window here (fused copy-out)
    int32_t     rank, world;
    int32_t     n_routes;
    int32_t     flags;
    int32_t     ctas;                   // 0 = library default
    uint32_t    timeout_ms;             // bound on every cross-rank wait; 0 = library default
    FuRoute     routes[FU_MAX_WORLD];
    // Copy-out refinement (append-only fields). When `own_direct` is set and `out` is given, the
    // route whose peer is this rank writes straight into `out` instead of the window, and only
    // the `n_out_routes` regions below (offsets relative to the window base and to `out` alike)
    // are copied out after the closing handshake. With n_out_routes == 0 the whole dense prefix
    // of `out_bytes` is copied.
    int32_t     own_direct;
    int32_t     n_out_routes;
    FuRoute     out_routes[2];
    // Output pool (append-only fields): buffer k of every rank, how many there are, and this rank's
    // choice for this call (0 = window; then `out`, if given, is filled by the fused copy-out as
    // before; k > 0 = pool buffer k - 1, and `out` must be that buffer's local address).
    // `peer_slot` replaces the exchanged choices when FU_A2A_NO_HANDSHAKE is set.
    void*       peer_pool[FU_MAX_WORLD][FU_POOL_SLOTS];
    int32_t     n_pool;
    int32_t     my_slot;
    int8_t      peer_slot[FU_MAX_WORLD];
    // Capacities (append-only fields), in bytes: of every rank's window, of every pool buffer and of
    // the readable extent behind `src`. The launcher computes the last byte every route reads and
    // writes and refuses the launch when one lies beyond its buffer: a route is an address formula
    // applied to another GPU's memory, and nothing on the device would catch a wrong one.
    int64_t     win_bytes;
    int64_t     pool_bytes;
    int64_t     src_bytes;
} FuA2AArgs;

FU_API int fu_a2a4d(const FuA2AArgs* args, void* stream);
// The argument checks of fu_a2a4d alone (everything it would refuse), without launching anything:
// no CUDA call is made, so it runs on a machine without a GPU.
FU_API int fu_a2a4d_check(const FuA2AArgs* args);

// Standalone cross-rank barrier on a window's control block (epoch += 1).
FU_API int fu_barrier(FuCtrl* const* peer_ctrl, int rank, int world, uint32_t timeout_ms, int flags, void* stream);

// ---- tcgen05 GEMMs ------------------------------------------------------------------------------
// C[m,n] = act(A[m,k] * B[n,k]^T + bias[n]) + residual[m,n]; bf16 operands, fp32 accumulation.
// act: 0 none, 1 GELU (tanh form), 2 GELU (erf form), 3 = multiply by the derivative of the tanh-form
// GELU at aux[m, n] (the backward of act 1 fused into the dgrad GEMM that produces its incoming
// gradient). `c_pre` (nullable, leading dimension ldc) additionally receives the value before the
// activation, which that backward needs. `err` (nullable) is a device word that receives a
// non-zero code if a wait inside the kernel ran out.
// flags: an operand may be given with the contraction along its rows instead of its columns
// (A stored k x m with pitch lda, B stored k x n with pitch ldb). The weight gradient of a linear
// layer, dW = dY^T X, is then a GEMM over dY and X as they lie in memory.
enum {
    FU_GEMM_A_KM = 1,
    FU_GEMM_B_KN = 2,
    FU_GEMM_PAIR = 4,    // run on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2) whatever the default is
    FU_GEMM_SINGLE = 8,  // run on single CTAs (128 x 256 tiles) whatever the default is
};
typedef struct FuGemmArgs {
    const void*  a;
    const void*  b;
    void*        c;
    int64_t      m, n, k, lda, ldb, ldc;
    const float* bias;
    const void*  residual;
    int32_t      act;
    int32_t      ctas;
    uint32_t*    err;
    int32_t      flags;
    const void*  aux;    // act 3: bf16 (m, n) with leading dimension ldc
    void*        c_pre;  // bf16 (m, n) with leading dimension ldc, or null
} FuGemmArgs;
FU_API int fu_gemm_bf16(const FuGemmArgs* args, void* stream);

// Fused mode-0 path: [q|k|v] = x * W^T (W rows ordered q heads, k heads, v heads; head_dim 128),
// per-head RMSNorm and RoPE on q and k, each head-row stored into the owning rank's window at
// (batch, seq_off + s, local head). Windows have layout (b, s_total, head_splits[p], 128) bf16.
// FuQkvArgs::flags: the weight is given with the contraction along its rows, (k, n) with pitch ldw,
// and read as it lies in memory (the scatter of d(attention output) = dY W_o uses W_o as stored).
#define FU_QKV_W_KN 64
typedef struct FuQkvArgs {
    const void*  x;
    const void*  w;
    int64_t      m, k, ldx, ldw;
    int32_t      heads;
    int32_t      pad_;
    int64_t      s_local, seq_off, s_total;
    const float* rope;     // (s_local, 64, 2): cos, sin per rotated pair
    const float* gamma_q;  // (128)
    const float* gamma_k;
    float        eps;
    int32_t      rank, world;
    int32_t      head_splits[FU_MAX_WORLD];
    void*        win_q[FU_MAX_WORLD];
    void*        win_k[FU_MAX_WORLD];
    void*        win_v[FU_MAX_WORLD];
    FuCtrl*      peer_ctrl[FU_MAX_WORLD];
    int32_t      flags;    // FU_A2A_NO_HANDSHAKE, FU_A2A_MUTE, FU_QKV_W_KN
    uint32_t     timeout_ms;
    int32_t      ctas;
    uint32_t*    err;
    // Generalisation (append-only). `n_types` projections share the head layout (3 = q, k, v;
    // 1 = a single tensor, e.g. the gradient of the attention output on its way back to the head
    // owners); the first `n_normed` of them get RMSNorm + RoPE. 0 / 0 means the default 3 / 2.
    // `y_save` (nullable) receives the pre-norm values of the normed projections, row-major
    // (m, n_normed * heads * 128) bf16 with leading dimension `ld_y`, for the backward pass.
    int32_t      n_types, n_normed;
    void*        y_save;
    int64_t      ld_y;
    // Bytes available behind every win_q / win_k / win_v base (append-only). The largest offset the
    // epilogue can store to, ((batches * s_total - (s_total - seq_off - s_local)) * head_splits[p]) * 256,
    // is checked against it before the launch.
    int64_t      win_bytes;
} FuQkvArgs;
FU_API int fu_qkv_rope_scatter(const FuQkvArgs* args, void* stream);
FU_API int fu_qkv_rope_scatter_check(const FuQkvArgs* args);  // the argument checks alone; no CUDA call

// Backward of per-head RMSNorm -> RoPE for q and k. dq, dk: (m, heads, 128) bf16 dense; y: the
// pre-norm projections saved by fu_qkv_rope_scatter; dy receives d(projection) for q at column 0
// and for k at column heads*128; dgamma_* (nullable, fp32[128]) are accumulated into.
typedef struct FuNormRopeBwdArgs {
    const void*  dq;
    const void*  dk;
    const void*  y;
    void*        dy;
    const float* rope;
    const float* gamma_q;
    const float* gamma_k;
    float*       dgamma_q;
    float*       dgamma_k;
    int64_t      m, s_local, ld_y, ld_dy;
    int32_t      heads;
    float        eps;
} FuNormRopeBwdArgs;
FU_API int fu_qk_norm_rope_bwd(const FuNormRopeBwdArgs* args, void* stream);

// The backward of the fused mode-0 path before its GEMMs: dq, dk and dv are loaded from the ranks
// that own the heads (each rank's buffers have layout (b, s_total, head_splits[p], 128) bf16 with
// `src_bytes` bytes behind every base), RoPE and RMSNorm are undone for q and k, and the result is
// written as d(projection) for q | k | v into `dy` (m, 3 * heads * 128), the A operand of the
// dgrad and wgrad GEMMs. Replaces a stand-alone mode-1 exchange, fu_qk_norm_rope_bwd and a copy.
typedef struct FuPullGradsArgs {
    const void*  peer_dq[FU_MAX_WORLD];
    const void*  peer_dk[FU_MAX_WORLD];
    const void*  peer_dv[FU_MAX_WORLD];
    FuCtrl*      peer_ctrl[FU_MAX_WORLD];
    int64_t      src_bytes;
    const void*  y;        // pre-norm q | k saved by fu_qkv_rope_scatter, (m, 2 * heads * 128), leading dim ld_y
    void*        dy;
    const float* rope;
    const float* gamma_q;
    const float* gamma_k;
    float*       dgamma_q; // nullable; accumulated into
    float*       dgamma_k;
    int64_t      m, s_local, seq_off, s_total, ld_y, ld_dy;
    int32_t      heads, rank, world;
    int32_t      head_splits[FU_MAX_WORLD];
    int32_t      flags;    // FU_A2A_NO_HANDSHAKE, FU_A2A_MUTE
    uint32_t     timeout_ms;
    float        eps;
} FuPullGradsArgs;
FU_API int fu_pull_qkv_grads(const FuPullGradsArgs* args, void* stream);
FU_API int fu_pull_qkv_grads_check(const FuPullGradsArgs* args);  // the argument checks alone; no CUDA call

// Fused mode-1 path: C[m, n] = A[m, :] * W[n, :]^T + bias + residual where A is the attention output
// gathered from its owners: A[m, head*128 + x] = O_owner(head)[batch, seq_off + s, local head, x].
// Every rank's O buffer has layout (b, s_total, head_splits[p], 128) bf16. `gather` is local scratch
// of m x (heads*128) bf16 and `ready` of ceil(m/128)*world uint32 (zeroed by the launcher).
typedef struct FuPullArgs {
    const void*  w;
    void*        c;
    int64_t      m, n, ldw, ldc;
    const float* bias;
    const void*  residual;
    int64_t      s_local, seq_off, s_total;
    int32_t      rank, world;
    int32_t      head_splits[FU_MAX_WORLD];
    const void*  peer_o[FU_MAX_WORLD];
    FuCtrl*      peer_ctrl[FU_MAX_WORLD];
    void*        gather;
    uint32_t*    ready;
    int32_t      flags;
    uint32_t     timeout_ms;
    int32_t      ctas;
    int32_t      pad_;
    uint32_t*    err;
    // Capacities (append-only): bytes readable behind every peer_o base, bytes of `gather`, words of `ready`.
    int64_t      o_bytes;
    int64_t      gather_bytes;
    int64_t      ready_words;
} FuPullArgs;
FU_API int fu_pull_outproj(const FuPullArgs* args, void* stream);
FU_API int fu_pull_outproj_check(const FuPullArgs* args);  // the argument checks alone; no CUDA call

// ---- flash attention (head_dim 128, non-causal, bf16) -----------------------------------------------
// q, k, v, o are addressed as (batch, seq, head, 128) with explicit element strides for the seq, head
// and batch axes, so both the window layout (b, s, h, d) and (b, h, s, d) work without a copy.
// lse (nullable) is (batch, heads, seq_q) fp32, natural log. do/dq/dk/dv follow the layout of
// o/q/k/v respectively; delta and dq_acc are scratch the caller provides for the backward.
// Backward: two passes without atomics (bit-reproducible dQ, about 1.5x the time of the default
// single pass, which sums dQ over the K/V blocks with fp32 reductions).
enum { FU_FMHA_DETERMINISTIC = 1 };
// Forward tuning knob: FU_FMHA_POLY(n) computes n of every 16 exponential pairs on the FMA pipe
// (a cubic) instead of the special-function unit; n in {0, 2, 4, 6}. Without it the library default applies.
#define FU_FMHA_POLY_SET 0x1000
#define FU_FMHA_POLY(n) (FU_FMHA_POLY_SET | (((n) & 15) << 8))
typedef struct FuFmhaArgs {
    const void* q;
    const void* k;
    const void* v;
    void*       o;
    float*      lse;
    int32_t     batch, heads, seq_q, seq_kv, head_dim;
    float       scale;
    int64_t     q_row, q_head, q_batch;
    int64_t     k_row, k_head, k_batch;
    int64_t     v_row, v_head, v_batch;
    int64_t     o_row, o_head, o_batch;
    int32_t     ctas;
    int32_t     flags;   // backward: FU_FMHA_* bits
    uint32_t*   err;
    // backward only
    const void* d_o;
    void*       dq;
    void*       dk;
    void*       dv;
    float*      delta;   // fp32 scratch of 2 * batch * heads * roundup(seq_q, 128) floats
    float*      dq_acc;  // (batch, seq_q, heads, 128) fp32 scratch, zeroed by the launcher; not needed
                         // (may be null) with FU_FMHA_DETERMINISTIC
    // optional timeline of the fused backward: CTA 0 stores the SM clock of 16 pipeline events for
    // each of its blocks 64..71 (128 words); null = no trace
    uint64_t*   trace;
} FuFmhaArgs;
FU_API int fu_fmha_fwd(const FuFmhaArgs* args, void* stream);
// d_o is addressed with o's strides, dq / dk / dv with q's / k's / v's strides.
FU_API int fu_fmha_bwd(const FuFmhaArgs* args, void* stream);

// The same backward pass for callers that may not allocate device memory where they call it (while
// a graph is being recorded, inside a host application that owns the allocator, in a loop that
// cannot afford cudaMalloc's synchronisation). This entry point has no counterpart in the
// reference. `delta` and `dq_acc` in `args` are ignored: the scratch is a fixed array inside the
// library (8.5 MiB of every GPU that loads it, held until the process exits). Limits and rules:
//   * two size limits, both checked, a problem beyond either is refused with an error that names it:
//     batch * heads * seq_q <= 16384 query rows (the dQ accumulator), and
//     batch * heads * roundup(seq_q, 128) <= 65536 (the softmax statistics are padded to whole
//     128-row blocks per (batch, head), so many heads with short sequences meet this one first:
//     1024 (batch, head) pairs of one row each are refused although they are only 1024 rows);
//   * the first call on each device looks up the array's device address, so make that first call
//     outside any stream capture; the address is kept for the life of the process and is stale
//     after cudaDeviceReset();
//   * all calls share the one array: two calls that overlap on the GPU (different streams, or
//     different threads) corrupt each other. Calls ordered on one stream are safe, each clears
//     what it needs to start from zero;
//   * nothing is allocated or freed: no cudaMalloc/cudaFree, no torch, no library allocator.
FU_API int fu_fmha_bwd_noalloc(const FuFmhaArgs* args, void* stream);

// ---- LayerNorm without affine parameters (bf16 in and out, fp32 statistics) -------------------------
// y = (x - mean) * rstd per row; `stats` (rows, 2) fp32 receives (mean, rstd) for the backward.
FU_API int fu_layernorm_fwd(const void* x, void* y, float* stats, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                            float eps, void* stream);
// dx = rstd * (dy - mean(dy) - xhat * mean(dy * xhat)), xhat recomputed from x and the saved statistics.
FU_API int fu_layernorm_bwd(const void* dy, const void* x, const float* stats, void* dx, int64_t rows, int64_t cols,
                            int64_t ld, void* stream);

// ---- block-scaled fp8 payloads ----------------------------------------------------------------------
// `blocks` runs of 128 bf16 values <-> `blocks` packed rows of 144 bytes (128 e4m3 + fp32 scale + pad).
FU_API int fu_quant_e4m3_block128(const void* x_bf16, void* packed, int64_t blocks, void* stream);
FU_API int fu_dequant_e4m3_block128(const void* packed, void* x_bf16, int64_t blocks, void* stream);

// The all-to-all of a (b, s, n, 128) bf16 tensor with the payload carried as block-scaled e4m3, in
// one launch: quantised in the store path into the peers' windows, expanded into the bf16 result
// `out` after the closing handshake. `routes` are the routes of the bf16 plan (byte quantities of
// 256-byte rows); the launcher rescales the destination side. `win_bytes` is the size of every
// window, THE SAME ON EVERY RANK, at 144 bytes per (token, head) row it must hold (inside, 128-byte
// payloads and 4-byte scales lie in two planes whose split follows from `win_bytes`); `out_rows`
// the (token, head) rows of the result, `src_bytes` the extent of the input. 16-byte aligned operands.
typedef struct FuA2AFp8Args {
    const void* src;
    void*       out;
    void*       peer_win[FU_MAX_WORLD];
    FuCtrl*     peer_ctrl[FU_MAX_WORLD];
    int64_t     win_bytes, src_bytes, out_rows;
    int32_t     rank, world, n_routes, flags, ctas;
    uint32_t    timeout_ms;
    FuRoute     routes[FU_MAX_WORLD];
} FuA2AFp8Args;
FU_API int fu_a2a4d_fp8(const FuA2AFp8Args* args, void* stream);
FU_API int fu_a2a4d_fp8_check(const FuA2AFp8Args* args);  // the argument checks alone; no CUDA call

FU_API const char* fu_last_error(void);
FU_API const char* fu_build_info(void);  // "sm_100a;<nvcc version>;<library version>"

#ifdef __cplusplus
}
#endif
