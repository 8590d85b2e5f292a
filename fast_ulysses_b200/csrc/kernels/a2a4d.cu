// The Ulysses 4D all-to-all as ONE persistent sm_100a kernel: opening handshake, payload pushed to
// every peer's window at its permuted offset, closing handshake, and (optionally) the copy-out of
// the own window into a caller-owned tensor. The relayout is expressed in the addresses of the
// copies, so there is no permute pass.
//
// Parity with the reference: replaces src/barrier.cu:31-49 (two one-block barrier launches),
// src/transfer.cu:68-126 (one cudaMemcpy2D/3DAsync per peer on the copy engines) and
// src/bindings.cc:216-223 (the flat copy-out) with a single launch whose data plane is SM-issued
// bulk (TMA) copies: local global -> shared -> the peer's window over NVLink, all peers in flight
// at once. Ordering rests on the PTX memory model only: payload copies complete, fence.acq_rel.sys,
// CTA arrival counter, then red.release.sys on the peer's flag; the reader spins with
// ld.acquire.sys. Every spin is bounded and reports through the control block's status words.
//
// Where a rank's payload lands is that rank's choice per call: its window, or one of its pooled
// output buffers (then nothing is copied out afterwards). The choice travels with the opening
// announcement (FuCtrl::slot_of) and every sender shifts its routes to that rank accordingly, so
// ranks with different numbers of live results need not agree on anything.
//
// A second transport, chosen per launch (FU_A2A_COPY_ENGINE), moves the same routes with the copy
// engines between two one-warp handshake kernels (the reference's data plane, src/transfer.cu:26-52):
// slower to start, but it holds no SM while the payload moves, which is what a call that runs beside
// GEMMs wants. Both transports speak the same handshake, so ranks may mix them.
#include "fu_kernels.h"
#include "handshake.cuh"
#include "host_util.h"
#include "ptx.cuh"

#include <algorithm>

static_assert(sizeof(FuCtrl) == FU_CTRL_BYTES, "control block layout");

namespace {

using namespace fu::ptx;

constexpr int      kStages      = 4;
constexpr int      kStageBytes  = 48 * 1024;
constexpr int      kAhead       = kStages - 2;  // loads issued this many chunks ahead of the stores
constexpr int      kLdstThreads = 512;
constexpr int      kLdstUnroll  = 8;           // 16-byte loads in flight per thread
constexpr int      kLdstChunkBytes = 64 * 1024;  // = threads x unroll x 16 B: one pass per chunk
constexpr int      kLdstCtasPerSm  = 1;           // 128 registers per thread: eight 16-byte vectors in flight without spilling
constexpr uint32_t kDefaultTimeoutMs = 10000;

// A route plus its decomposition into chunks of at most one stage.
struct RouteX {
    const uint8_t* src;
    uint8_t*       dst;
    int64_t        src_pitch, dst_pitch, src_batch, dst_batch;
    int64_t        rows, batches;
    int64_t        row_bytes;
    int64_t        piece_bytes;     // bytes of a row moved by one chunk when a row exceeds a stage
    int32_t        pieces_per_row;  // > 1 only when rows_per_chunk == 1
    int32_t        rows_per_chunk;
    int64_t        row_groups;      // ceil(rows / rows_per_chunk)
    int64_t        count;           // chunks in this route
    int32_t        peer;            // rank whose choice of buffer shifts `dst` (-1: dst is final)
};

struct RouteSet {
    int     n;
    int64_t max_count;
    RouteX  r[FU_MAX_WORLD];
    // When `pinned`, CTAs [first[g], first[g + 1]) serve route g and nothing else; the host sizes the
    // ranges by what each route costs (bytes, and a local copy is several times cheaper per byte
    // than one that crosses NVLink), so all routes end at about the same time.
    int32_t pinned;
    int16_t first[FU_MAX_WORLD + 1];
};

struct KArgs {
    RouteSet push;
    RouteSet copy_out;  // n == 0 when there is no fused copy-out
    fu::Peers peers;  // control blocks, rank, world size, time limit of every cross-rank wait
    int       flags;
    // Output pool: `dst` of a route to rank p is built for p's window; if p announces pool buffer
    // k for this call, the route is shifted by pool_delta[p][k - 1] = buffer - window.
    int64_t  pool_delta[FU_MAX_WORLD][FU_POOL_SLOTS];
    int32_t  n_pool, my_slot;
    int8_t   peer_slot[FU_MAX_WORLD];
};

struct Chunk {
    const uint8_t* src;
    uint8_t*       dst;
    int64_t        src_pitch, dst_pitch;
    uint32_t       nrows, row_bytes;
};

// Round-robin over routes: virtual index v names (route v % n, chunk v / n); a route that has run
// out of chunks yields nothing for that v. With gridDim a multiple of n each CTA streams to one peer.
// The route a CTA is pinned to, or -1 when the set deals its chunks round-robin.
__device__ __forceinline__ int pinned_route(const RouteSet& s, int cta)
{
    if (!s.pinned) {
        return -1;
    }
    int g = 0;
    while (g + 1 < s.n && cta >= s.first[g + 1]) {
        ++g;
    }
    return g;
}

struct ChunkCursor {
    int64_t        v, stride, end;
    int            route;  // >= 0: this CTA walks that route only (v is then a chunk index)
    const int64_t* shift;  // per-rank destination shift (shared memory), or null
    __device__ ChunkCursor(const RouteSet& s, int cta, int ctas, const int64_t* shift_ = nullptr)
        : v(cta), stride(ctas), end(s.max_count * s.n), route(pinned_route(s, cta)), shift(shift_)
    {
        if (route >= 0) {
            v      = cta - s.first[route];
            stride = s.first[route + 1] - s.first[route];
            end    = s.r[route].count;
        }
    }
    __device__ bool next(const RouteSet& s, Chunk& c)
    {
        while (v < end) {
            const int     ri  = route >= 0 ? route : static_cast<int>(v % s.n);
            const int64_t idx = route >= 0 ? v : v / s.n;
            v += stride;
            const RouteX& r = s.r[ri];
            if (idx >= r.count) {
                continue;
            }
            const int64_t per_batch = r.row_groups * r.pieces_per_row;
            const int64_t batch     = idx / per_batch;
            const int64_t rem       = idx - batch * per_batch;
            const int64_t group     = rem / r.pieces_per_row;
            const int64_t piece     = rem - group * r.pieces_per_row;
            const int64_t row0      = group * r.rows_per_chunk;
            const int64_t col0      = piece * r.piece_bytes;
            c.nrows     = static_cast<uint32_t>(min(static_cast<int64_t>(r.rows_per_chunk), r.rows - row0));
            c.row_bytes = static_cast<uint32_t>(min(r.piece_bytes, r.row_bytes - col0));
            c.src       = r.src + batch * r.src_batch + row0 * r.src_pitch + col0;
            c.dst       = r.dst + batch * r.dst_batch + row0 * r.dst_pitch + col0;
            if (shift && r.peer >= 0) {
                c.dst += shift[r.peer];
            }
            c.src_pitch = r.src_pitch;
            c.dst_pitch = r.dst_pitch;
            return true;
        }
        return false;
    }
};

// ---- data movers ------------------------------------------------------------------------------------
struct BulkPipe {
    uint8_t*  base;  // kStages buffers of kStageBytes each (an address computed, not an array indexed
                     // at run time: that would live in local memory)
    uint64_t* full;  // kStages mbarriers
    __device__ __forceinline__ uint8_t* stage(int s) const { return base + s * kStageBytes; }
};

__device__ __forceinline__ void bulk_issue_loads(const BulkPipe& p, int s, const Chunk& c, int lane)
{
    const uint32_t total = c.nrows * c.row_bytes;
    if (lane == 0) {
        mbar_expect_tx(&p.full[s], total);
    }
    __syncwarp();
    if (c.src_pitch == c.row_bytes) {
        if (lane == 0) {
            bulk_g2s(p.stage(s), c.src, total, &p.full[s]);
        }
    }
    else {
        for (uint32_t r = lane; r < c.nrows; r += 32) {
            bulk_g2s(p.stage(s) + r * c.row_bytes, c.src + r * c.src_pitch, c.row_bytes, &p.full[s]);
        }
    }
}

__device__ __forceinline__ void bulk_issue_stores(const BulkPipe& p, int s, const Chunk& c, int lane)
{
    if (c.dst_pitch == c.row_bytes) {
        if (lane == 0) {
            bulk_s2g(c.dst, p.stage(s), c.nrows * c.row_bytes);
        }
    }
    else {
        for (uint32_t r = lane; r < c.nrows; r += 32) {
            bulk_s2g(c.dst + r * c.dst_pitch, p.stage(s) + r * c.row_bytes, c.row_bytes);
        }
    }
    bulk_commit();  // every lane commits one (possibly empty) group per chunk
}

// Moves this CTA's share of a route set with one warp. `jbase` continues the stage/parity sequence
// across successive calls in one kernel. Returns false if a load never completed.
__device__ bool bulk_move(const RouteSet& set, const BulkPipe& p, int64_t& jbase, FuCtrl* own,
                          const int64_t* shift = nullptr)
{
    const int   lane = threadIdx.x & 31;
    ChunkCursor load_cur(set, blockIdx.x, gridDim.x, shift);
    ChunkCursor store_cur(set, blockIdx.x, gridDim.x, shift);
    Chunk       c;
    int64_t     jl = jbase;  // next chunk number to load
    int64_t     js = jbase;  // next chunk number to store
    bool        ok = true;
    for (int q = 0; q < kAhead; ++q) {
        if (!load_cur.next(set, c)) {
            break;
        }
        // stage reuse across calls: the previous call drained every group before returning
        bulk_issue_loads(p, static_cast<int>(jl % kStages), c, lane);
        ++jl;
    }
    while (store_cur.next(set, c)) {
        Chunk ahead;
        if (load_cur.next(set, ahead)) {
            // the stage about to be refilled was last read by the store issued two chunks ago
            bulk_wait_read<1>();
            __syncwarp();
            bulk_issue_loads(p, static_cast<int>(jl % kStages), ahead, lane);
            ++jl;
        }
        const int      s      = static_cast<int>(js % kStages);
        const uint32_t parity = static_cast<uint32_t>((js / kStages) & 1);
        if (!mbar_wait(&p.full[s], parity)) {
            fu::hs_report(own, FU_ST_COPY_TIMEOUT, 0, static_cast<uint64_t>(js), 0);
            ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            break;
        }
        fence_proxy_async_smem();
        bulk_issue_stores(p, s, c, lane);
        ++js;
    }
    bulk_wait<0>();  // writes performed, not merely read out of shared memory
    __syncwarp();
    jbase = ok ? js : jl;
    return ok;
}

// `kCoherent` selects plain loads: required when the source was written during this launch (the own
// window, filled by peers), where the read-only path must not be used.
template <bool kCoherent>
__device__ void ldst_move(const RouteSet& set, const int64_t* shift = nullptr)
{
    ChunkCursor cur(set, blockIdx.x, gridDim.x, shift);
    Chunk       c;
    while (cur.next(set, c)) {
        const uint32_t vpr  = c.row_bytes >> 4;
        const uint32_t nvec = vpr * c.nrows;
        for (uint32_t v0 = threadIdx.x; v0 < nvec; v0 += kLdstUnroll * kLdstThreads) {
            // only the data stays in registers between the loads and the stores: the destination of
            // each vector is recomputed (two integer divisions are cheaper than 16 spilled registers)
            uint4 val[kLdstUnroll];
#pragma unroll
            for (int u = 0; u < kLdstUnroll; ++u) {
                const uint32_t v = v0 + u * kLdstThreads;
                if (v < nvec) {
                    const uint32_t row = v / vpr;
                    const uint32_t col = v - row * vpr;
                    const uint8_t* from = c.src + row * c.src_pitch + (static_cast<int64_t>(col) << 4);
                    val[u]             = kCoherent ? ld_v4(from) : ld_nc_v4(from);
                }
            }
#pragma unroll
            for (int u = 0; u < kLdstUnroll; ++u) {
                const uint32_t v = v0 + u * kLdstThreads;
                if (v < nvec) {
                    const uint32_t row = v / vpr;
                    const uint32_t col = v - row * vpr;
                    st_v4(c.dst + row * c.dst_pitch + (static_cast<int64_t>(col) << 4), val[u]);
                }
            }
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------------------------
template <bool kBulk>
__global__ void __launch_bounds__(kBulk ? 32 : kLdstThreads, kBulk ? 1 : kLdstCtasPerSm) a2a4d_kernel(const __grid_constant__ KArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t                       full_bar[kStages];
    __shared__ uint32_t                       ticket_s;
    __shared__ int64_t                        shift_s[FU_MAX_WORLD];  // destination shift per rank (output pool)
    __shared__ int                            alive_s;                // did the opening handshake complete

    const int  warp      = threadIdx.x >> 5;
    const bool handshake = !(a.flags & FU_A2A_NO_HANDSHAKE);
    const bool stamps    = (a.flags & FU_A2A_STAMPS) && blockIdx.x == 0 && threadIdx.x == 0;
    FuCtrl*    own       = a.peers.own;

    BulkPipe pipe;
    if (kBulk) {
        pipe.base = smem;
        pipe.full = full_bar;
        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(&full_bar[s], 1);
            }
            mbar_fence_init();
        }
        __syncthreads();
    }

    // Stable for the whole launch: only the last CTA to finish advances it.
    const uint64_t base = *reinterpret_cast<volatile uint64_t*>(&own->epoch);
    if (stamps) {
        own->stamps[0] = globaltimer_ns();
    }

    // Opening: "writers wait for readers". Each rank announces that everything it had queued before
    // this launch, its reads of its own window included, is finished; nobody overwrites a window
    // before its owner said so. Every CTA polls the (local) flags itself, so there is no grid-wide
    // dependency here.
    // A CTA pinned to one route writes one rank's memory only, so it waits for that rank alone and
    // starts pushing the moment that rank has announced, however late the others are. A route
    // whose destination is final (the own share going straight to the caller's tensor) touches
    // no window and waits for nobody.
    uint32_t  who = 0xffffffffu;
    const int pin = pinned_route(a.push, blockIdx.x);
    if (pin >= 0) {
        who = a.push.r[pin].peer >= 0 ? (1u << a.push.r[pin].peer) : 0u;
    }
    bool alive = true;
    if (handshake && warp == 0) {
        if (blockIdx.x == 0) {
            fu::hs_announce(a.peers, base + 1, a.my_slot);
            if (a.flags & FU_A2A_EARLY_PUBLISH) {
                fu::hs_announce(a.peers, base + 2);
            }
        }
        alive = fu::hs_await(a.peers, base + 1, FU_ST_OPEN_TIMEOUT, who);
    }
    if (warp == 0) {
        // Which buffer each rank wants this call's payload in: announced with the opening flag
        // (the acquire in await() orders this read, so only the ranks waited for are read), or
        // given by the host when there is no handshake.
        const int lane = threadIdx.x & 31;
        if (lane < a.peers.world && ((who >> lane) & 1u)) {
            int slot = handshake ? static_cast<int>(*reinterpret_cast<volatile uint8_t*>(&own->slot_of[lane]))
                                 : static_cast<int>(a.peer_slot[lane]);
            if (slot < 0 || slot > a.n_pool) {
                slot = 0;  // a rank that announced nothing usable is reported by the handshake itself
            }
            shift_s[lane] = slot > 0 ? a.pool_delta[lane][slot - 1] : 0;
        }
        if (lane == 0) {
            alive_s = alive ? 1 : 0;
        }
        __syncwarp();
    }
    if (stamps) {
        own->stamps[1] = globaltimer_ns();
    }

    int64_t chunk_no = 0;
    if (kBulk) {
        if (alive) {
            alive = bulk_move(a.push, pipe, chunk_no, own, shift_s);
        }
    }
    else {
        __syncthreads();
        // Nothing is pushed after an opening handshake that ran out of time: a rank that never
        // announced has not said where it wants its payload either.
        if (alive_s) {
            ldst_move<false>(a.push, shift_s);
        }
    }
    // Make this CTA's payload visible system-wide before its arrival can be observed.
    fence_sys();
    __syncthreads();
    if (stamps) {
        own->stamps[2] = globaltimer_ns();
    }

    if (threadIdx.x == 0) {
        ticket_s = atomicAdd(&own->arrive[0], 1u);
    }
    __syncthreads();
    const bool last_in = (ticket_s == gridDim.x - 1);
    const bool copying = a.copy_out.n > 0;

    // Closing: "all my writes have landed". The CTA that arrives last has, through the arrival
    // counter and the fences around it, every other CTA's payload ordered before its announcement.
    if (handshake && warp == 0) {
        if (last_in) {
            fence_sys();
            fu::hs_announce(a.peers, base + 2);
        }
        if (last_in || copying) {
            fu::hs_await(a.peers, base + 2, FU_ST_CLOSE_TIMEOUT);
        }
    }
    if (stamps) {
        own->stamps[3] = globaltimer_ns();
    }

    if (copying) {
        __syncthreads();
        if (kBulk) {
            fence_proxy_async();  // the bulk loads below read what peers wrote through the generic proxy
            bulk_move(a.copy_out, pipe, chunk_no, own);
        }
        else {
            ldst_move<true>(a.copy_out);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            ticket_s = atomicAdd(&own->arrive[1], 1u);
        }
        __syncthreads();
    }
    const bool last_out = copying ? (ticket_s == gridDim.x - 1) : last_in;
    if (last_out && threadIdx.x == 0) {
        own->arrive[0] = 0;
        own->arrive[1] = 0;
        if (a.flags & FU_A2A_STAMPS) {
            own->stamps[4] = globaltimer_ns();
        }
        __threadfence();
        if (!(a.flags & FU_A2A_KEEP_EPOCH)) {
            *reinterpret_cast<volatile uint64_t*>(&own->epoch) = base + 2;
        }
    }
}

__global__ void __launch_bounds__(32, 1)
    barrier_kernel(FuCtrl* own, const __grid_constant__ KArgs a)
{
    const uint64_t base = *reinterpret_cast<volatile uint64_t*>(&own->epoch);
    fu::hs_announce(a.peers, base + 1);
    fu::hs_await(a.peers, base + 1, FU_ST_OPEN_TIMEOUT);
    __syncwarp();
    if (threadIdx.x == 0) {
        *reinterpret_cast<volatile uint64_t*>(&own->epoch) = base + 1;
    }
}

// The two handshakes of the copy-engine transport, one warp each. Phase 1 opens (announce "my reads
// of my window are finished", wait for every rank's); phase 2 runs after the copies in stream order
// and closes (announce "my writes have landed", wait for every rank's, advance the phase counter).
// A copy that precedes this kernel in its stream has completed, destination writes included, before
// the kernel starts; the system-scope fence and the release on the flags order it for the peers.
__global__ void __launch_bounds__(32, 1) ce_phase_kernel(const __grid_constant__ fu::Peers p, int phase, int flags)
{
    FuCtrl*        own    = p.own;
    const uint64_t base   = *reinterpret_cast<volatile uint64_t*>(&own->epoch);
    const bool     stamps = (flags & FU_A2A_STAMPS) && threadIdx.x == 0;
    if (phase == 1) {
        if (stamps) {
            own->stamps[0] = globaltimer_ns();
        }
        fu::hs_announce(p, base + 1, 0);  // buffer 0: this call's payload goes to the window
        if (flags & FU_A2A_EARLY_PUBLISH) {
            fu::hs_announce(p, base + 2);
        }
        fu::hs_await(p, base + 1, FU_ST_OPEN_TIMEOUT);
        if (stamps) {
            own->stamps[1] = globaltimer_ns();
        }
        return;
    }
    if (stamps) {
        own->stamps[2] = globaltimer_ns();
    }
    fence_sys();
    fu::hs_announce(p, base + 2);
    fu::hs_await(p, base + 2, FU_ST_CLOSE_TIMEOUT);
    __syncwarp();
    if (threadIdx.x == 0) {
        if (flags & FU_A2A_STAMPS) {
            own->stamps[3] = own->stamps[4] = globaltimer_ns();
        }
        __threadfence();
        *reinterpret_cast<volatile uint64_t*>(&own->epoch) = base + 2;
    }
}

// ---- host side ----------------------------------------------------------------------------------------
// Cuts a route into chunks of at most `chunk` bytes. A route that is dense on both sides is first
// folded into one long row, so that its chunks are large whatever the row length was.
void decompose(RouteX& x, int64_t chunk)
{
    if (x.row_bytes <= 0 || x.rows <= 0 || x.batches <= 0) {
        x.count = 0;
        return;
    }
    if (x.src_pitch == x.row_bytes && x.dst_pitch == x.row_bytes && x.rows > 1) {
        x.row_bytes *= x.rows;
        x.rows      = 1;
        x.src_pitch = x.dst_pitch = x.row_bytes;
    }
    if (x.row_bytes <= chunk) {
        x.piece_bytes    = x.row_bytes;
        x.pieces_per_row = 1;
        x.rows_per_chunk = static_cast<int32_t>(std::min<int64_t>(chunk / x.row_bytes, x.rows));
    }
    else {
        x.piece_bytes    = chunk;
        x.pieces_per_row = static_cast<int32_t>((x.row_bytes + chunk - 1) / chunk);
        x.rows_per_chunk = 1;
    }
    x.row_groups = (x.rows + x.rows_per_chunk - 1) / x.rows_per_chunk;
    x.count      = x.batches * x.row_groups * x.pieces_per_row;
}

// Deals `ctas` CTAs to the routes of a set in proportion to what each route costs: its bytes, with
// a route that stays on this device (the own share) counted at kLocalCost of a route that crosses
// NVLink. Every route gets at least one CTA; with fewer CTAs than routes the set stays unpinned and
// its chunks are dealt round-robin.
constexpr double kLocalCost = 0.3;
void pin_ctas(RouteSet& set, int ctas, int rank)
{
    set.pinned = 0;
    if (set.n < 1 || ctas < set.n) {
        return;
    }
    double cost[FU_MAX_WORLD], total = 0.0;
    for (int g = 0; g < set.n; ++g) {
        const RouteX& r     = set.r[g];
        const bool    local = r.peer < 0 || r.peer == rank;
        cost[g] = static_cast<double>(r.row_bytes) * static_cast<double>(r.rows) * static_cast<double>(r.batches)
                  * (local ? kLocalCost : 1.0);
        total += cost[g];
    }
    int given[FU_MAX_WORLD], sum = 0;
    for (int g = 0; g < set.n; ++g) {
        given[g] = std::max(1, static_cast<int>(ctas * cost[g] / total));
        sum += given[g];
    }
    // hand the remainder (or take the excess) one CTA at a time where it changes the load per CTA most
    while (sum != ctas) {
        int best = -1;
        for (int g = 0; g < set.n; ++g) {
            if (sum > ctas && given[g] <= 1) {
                continue;
            }
            const double load = cost[g] / given[g];
            if (best < 0 || (sum < ctas ? load > cost[best] / given[best] : load < cost[best] / given[best])) {
                best = g;
            }
        }
        if (best < 0) {
            return;  // cannot happen with ctas >= n; stay unpinned rather than guess
        }
        given[best] += sum < ctas ? 1 : -1;
        sum += sum < ctas ? 1 : -1;
    }
    set.first[0] = 0;
    for (int g = 0; g < set.n; ++g) {
        set.first[g + 1] = static_cast<int16_t>(set.first[g] + given[g]);
    }
    set.pinned = 1;
}

bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace

namespace {

// One past the last byte a route touches on one side, relative to that side's base.
int64_t route_extent(int64_t off, int64_t pitch, int64_t batch_stride, const FuRoute& r)
{
    if (r.rows <= 0 || r.batches <= 0 || r.row_bytes <= 0) {
        return 0;
    }
    return off + (r.batches - 1) * batch_stride + (r.rows - 1) * pitch + r.row_bytes;
}

// Everything fu_a2a4d refuses, and the kernel arguments when it refuses nothing. Host arithmetic only.
int build_args(const FuA2AArgs* args, KArgs& k)
{
    if (!args) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: null args");
    }
    const FuA2AArgs& in = *args;
    if (in.world < 1 || in.world > FU_MAX_WORLD || in.rank < 0 || in.rank >= in.world) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: rank %d / world %d out of range", in.rank, in.world);
    }
    if (in.n_routes < 0 || in.n_routes > FU_MAX_WORLD) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: %d routes", in.n_routes);
    }
    k.peers.rank       = in.rank;
    k.peers.world      = in.world;
    k.peers.mute       = (in.flags & FU_A2A_MUTE) ? 1 : 0;
    k.peers.timeout_ns = static_cast<uint64_t>(in.timeout_ms ? in.timeout_ms : kDefaultTimeoutMs) * 1000000ull;
    k.flags            = in.flags;
    for (int p = 0; p < in.world; ++p) {
        if (!in.peer_win[p] || !in.peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: no window or control block for rank %d", p);
        }
        k.peers.ctrl[p] = in.peer_ctrl[p];
    }
    k.peers.own = in.peer_ctrl[in.rank];
    if (in.n_routes > 0 && !aligned16(in.src)) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: the input is not 16-byte aligned");
    }
    if (in.n_pool < 0 || in.n_pool > FU_POOL_SLOTS || in.my_slot < 0 || in.my_slot > in.n_pool) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: pool buffer %d of %d", in.my_slot, in.n_pool);
    }
    if ((in.flags & FU_A2A_COPY_ENGINE) && in.n_pool > 0) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: the copy-engine transport cannot serve a call that may use the output "
                                  "pool (which buffer a peer chose is known on the device only)");
    }
    k.n_pool  = in.n_pool;
    k.my_slot = in.my_slot;
    for (int p = 0; p < in.world; ++p) {
        k.peer_slot[p] = in.peer_slot[p];
        if ((in.flags & FU_A2A_NO_HANDSHAKE) && (in.peer_slot[p] < 0 || in.peer_slot[p] > in.n_pool)) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: rank %d is given pool buffer %d of %d", p, in.peer_slot[p], in.n_pool);
        }
        for (int s = 0; s < in.n_pool; ++s) {
            if (!in.peer_pool[p][s] || !aligned16(in.peer_pool[p][s])) {
                return fu::fail(FU_E_ARG, "fu_a2a4d: pool buffer %d of rank %d is missing or not 16-byte aligned", s, p);
            }
            k.pool_delta[p][s] = static_cast<const uint8_t*>(in.peer_pool[p][s]) - static_cast<const uint8_t*>(in.peer_win[p]);
        }
    }
    if (in.my_slot > 0 && in.out != in.peer_pool[in.rank][in.my_slot - 1]) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: with pool buffer %d chosen, `out` must be that buffer", in.my_slot);
    }
    const bool    ldst  = (in.flags & FU_A2A_LDST) != 0;
    const int64_t chunk = ldst ? kLdstChunkBytes : kStageBytes;
    const bool    copy_out = in.out && in.out_bytes > 0;
    if (copy_out && (!aligned16(in.out) || (in.out_bytes & 15))) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: the copy-out destination is not 16-byte granular");
    }
    if (in.n_out_routes < 0 || in.n_out_routes > 2) {
        return fu::fail(FU_E_ARG, "fu_a2a4d: %d copy-out routes", in.n_out_routes);
    }
    auto granular = [](const FuRoute& r) {
        return ((r.row_bytes | r.src_off | r.dst_off | r.src_pitch | r.dst_pitch | r.src_batch | r.dst_batch) & 15) == 0;
    };
    auto expand = [&](const FuRoute& r, const uint8_t* src_base, uint8_t* dst_base, int shift_peer = -1) {
        RouteX x{};
        x.peer      = shift_peer;
        x.src       = src_base + r.src_off;
        x.dst       = dst_base + r.dst_off;
        x.src_pitch = r.src_pitch;
        x.dst_pitch = r.dst_pitch;
        x.src_batch = r.src_batch;
        x.dst_batch = r.dst_batch;
        x.rows      = r.rows;
        x.batches   = r.batches;
        x.row_bytes = r.row_bytes;
        decompose(x, chunk);
        return x;
    };
    k.push.n = 0;
    for (int i = 0; i < in.n_routes; ++i) {
        const FuRoute& r = in.routes[i];
        if (r.peer < 0 || r.peer >= in.world) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: route %d names rank %d", i, r.peer);
        }
        if (!granular(r)) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: route %d is not 16-byte granular", i);
        }
        if (!aligned16(in.peer_win[r.peer])) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: rank %d's window is not 16-byte aligned", r.peer);
        }
        if ((r.src_off | r.dst_off | r.src_pitch | r.dst_pitch | r.src_batch | r.dst_batch) < 0) {
            return fu::fail(FU_E_ARG, "fu_a2a4d: route %d has a negative offset or stride", i);
        }
        // The own share never needs the window when the caller wants the result elsewhere.
        const bool direct = copy_out && in.own_direct && r.peer == in.rank;
        {
            const int64_t src_end = route_extent(r.src_off, r.src_pitch, r.src_batch, r);
            const int64_t dst_end = route_extent(r.dst_off, r.dst_pitch, r.dst_batch, r);
            if (src_end > in.src_bytes) {
                return fu::fail(FU_E_ARG, "fu_a2a4d: route %d reads up to byte %lld of an input of %lld bytes", i,
                                (long long)src_end, (long long)in.src_bytes);
            }
            if (direct) {
                if (dst_end > in.out_bytes) {
                    return fu::fail(FU_E_ARG, "fu_a2a4d: route %d writes up to byte %lld of an output of %lld bytes", i,
                                    (long long)dst_end, (long long)in.out_bytes);
                }
            }
            else {
                if (dst_end > in.win_bytes) {
                    return fu::fail(FU_E_ARG, "fu_a2a4d: route %d writes up to byte %lld of rank %d's window of %lld bytes",
                                    i, (long long)dst_end, r.peer, (long long)in.win_bytes);
                }
                // rank r.peer may ask for this call's payload in any of its pool buffers instead
                if (in.n_pool > 0 && dst_end > in.pool_bytes) {
                    return fu::fail(FU_E_ARG, "fu_a2a4d: route %d writes up to byte %lld but the pool buffers hold %lld bytes",
                                    i, (long long)dst_end, (long long)in.pool_bytes);
                }
            }
        }
        uint8_t*   dst    = direct ? static_cast<uint8_t*>(in.out) : static_cast<uint8_t*>(in.peer_win[r.peer]);
        // a route into another rank's memory follows that rank's choice of buffer for this call
        RouteX     x      = expand(r, static_cast<const uint8_t*>(in.src), dst, direct ? -1 : r.peer);
        if (x.count > 0) {
            k.push.r[k.push.n++] = x;
            k.push.max_count     = std::max(k.push.max_count, x.count);
        }
    }
    k.copy_out.n = 0;
    if (copy_out) {
        const uint8_t* win = static_cast<const uint8_t*>(in.peer_win[in.rank]);
        if (in.n_out_routes > 0 || in.own_direct) {
            for (int i = 0; i < in.n_out_routes; ++i) {
                if (!granular(in.out_routes[i])) {
                    return fu::fail(FU_E_ARG, "fu_a2a4d: copy-out route %d is not 16-byte granular", i);
                }
                {
                    const FuRoute& r = in.out_routes[i];
                    if ((r.src_off | r.dst_off | r.src_pitch | r.dst_pitch | r.src_batch | r.dst_batch) < 0
                        || route_extent(r.src_off, r.src_pitch, r.src_batch, r) > in.win_bytes
                        || route_extent(r.dst_off, r.dst_pitch, r.dst_batch, r) > in.out_bytes) {
                        return fu::fail(FU_E_ARG, "fu_a2a4d: copy-out route %d leaves the window (%lld bytes) or the "
                                        "output (%lld bytes)", i, (long long)in.win_bytes, (long long)in.out_bytes);
                    }
                }
                RouteX x = expand(in.out_routes[i], win, static_cast<uint8_t*>(in.out));
                if (x.count > 0) {
                    k.copy_out.r[k.copy_out.n++] = x;
                    k.copy_out.max_count         = std::max(k.copy_out.max_count, x.count);
                }
            }
        }
        else {
            if (in.out_bytes > in.win_bytes) {
                return fu::fail(FU_E_ARG, "fu_a2a4d: copy-out of %lld bytes from a window of %lld bytes",
                                (long long)in.out_bytes, (long long)in.win_bytes);
            }
            FuRoute flat{};
            flat.row_bytes = in.out_bytes;
            flat.rows = flat.batches = 1;
            flat.src_pitch = flat.dst_pitch = in.out_bytes;
            RouteX x = expand(flat, win, static_cast<uint8_t*>(in.out));
            k.copy_out.r[k.copy_out.n++] = x;
            k.copy_out.max_count         = x.count;
        }
    }
    // `copy_out.n` doubles as "every CTA must see the closing handshake"; with nothing left to copy
    // (a single rank whose own share went straight to `out`) the plain closing path is taken.

    return FU_OK;
}

}  // namespace

extern "C" int fu_a2a4d(const FuA2AArgs* args, void* stream_v);

namespace {

// One route on the copy engines: a pitched copy per batch (a flat one where both sides are dense).
int copy_route(const FuRoute& r, const uint8_t* src_base, uint8_t* dst_base, cudaStream_t stream)
{
    if (r.rows <= 0 || r.batches <= 0 || r.row_bytes <= 0) {
        return FU_OK;
    }
    for (int64_t b = 0; b < r.batches; ++b) {
        const uint8_t* s = src_base + r.src_off + b * r.src_batch;
        uint8_t*       d = dst_base + r.dst_off + b * r.dst_batch;
        if (r.rows == 1 || (r.src_pitch == r.row_bytes && r.dst_pitch == r.row_bytes)) {
            FU_CUDA_OK(cudaMemcpyAsync(d, s, static_cast<size_t>(r.row_bytes * r.rows), cudaMemcpyDeviceToDevice, stream));
        }
        else {
            FU_CUDA_OK(cudaMemcpy2DAsync(d, static_cast<size_t>(r.dst_pitch), s, static_cast<size_t>(r.src_pitch),
                                         static_cast<size_t>(r.row_bytes), static_cast<size_t>(r.rows),
                                         cudaMemcpyDeviceToDevice, stream));
        }
    }
    return FU_OK;
}

// The whole call with the copy engines as the data plane. `in` has passed build_args(), so every
// route lies inside the buffers it names. The routes to peers run one after another on the
// caller's stream: one copy-engine flow fills a GPU's NVLink egress, so nothing is gained by
// spreading them over streams, and the order in which `in.routes` lists the peers (next rank up
// first) keeps every rank's ingress fed by one sender at a time.
// What stays on this device (the own share, and the copy-out of a copying call) is moved by a
// small launch of the exchange kernel itself, with handshakes off: the driver serves a pitched
// copy within one device with a kernel of its own choosing, not with a copy engine, so nothing
// is saved by asking it. FU_A2A_CE_LOCAL_COPIES asks it all the same (for measurements).
constexpr int kCeLocalCtas = 16;

int launch_copy_engine(const FuA2AArgs& in, const KArgs& k, cudaStream_t stream)
{
    const bool handshake    = !(in.flags & FU_A2A_NO_HANDSHAKE);
    const bool copy_out     = in.out && in.out_bytes > 0;
    const bool local_kernel = !(in.flags & FU_A2A_CE_LOCAL_COPIES);
    // A launch of the exchange kernel that moves only local data and leaves the handshakes and the
    // phase counter to the one-warp kernels around the copies.
    auto helper = [&](bool own_share) -> int {
        FuA2AArgs h = in;
        h.flags     = (in.flags & (FU_A2A_LDST | FU_A2A_MINOR_SHARE)) | FU_A2A_NO_HANDSHAKE | FU_A2A_KEEP_EPOCH;
        h.ctas      = in.ctas > 0 ? std::min(in.ctas, kCeLocalCtas) : kCeLocalCtas;
        for (int p = 0; p < FU_MAX_WORLD; ++p) {
            h.peer_slot[p] = 0;
        }
        if (own_share) {
            h.n_routes = 0;
            for (int i = 0; i < in.n_routes; ++i) {
                if (in.routes[i].peer == in.rank) {
                    h.routes[h.n_routes++] = in.routes[i];
                }
            }
            h.n_out_routes = 0;
            if (!(copy_out && in.own_direct)) {  // the own share goes to the own window: nothing else is written
                h.out       = nullptr;
                h.out_bytes = 0;
            }
            if (h.n_routes == 0) {
                return FU_OK;
            }
        }
        else {
            h.n_routes = 0;  // only the copy-out runs
        }
        return fu_a2a4d(&h, stream);
    };
    if (local_kernel) {
        // Touches the caller's tensor or the own window only, which no peer reads: it need not
        // wait for anybody, so it goes first.
        const int rc = helper(true);
        if (rc != FU_OK) {
            return rc;
        }
    }
    if (handshake) {
        ce_phase_kernel<<<1, 32, 0, stream>>>(k.peers, 1, in.flags);
        FU_CUDA_OK(cudaGetLastError());
    }
    for (int i = 0; i < in.n_routes; ++i) {
        const FuRoute& r = in.routes[i];
        if (local_kernel && r.peer == in.rank) {
            continue;
        }
        const bool direct = copy_out && in.own_direct && r.peer == in.rank;
        uint8_t*   dst    = direct ? static_cast<uint8_t*>(in.out) : static_cast<uint8_t*>(in.peer_win[r.peer]);
        const int  rc     = copy_route(r, static_cast<const uint8_t*>(in.src), dst, stream);
        if (rc != FU_OK) {
            return rc;
        }
    }
    if (handshake) {
        ce_phase_kernel<<<1, 32, 0, stream>>>(k.peers, 2, in.flags);
        FU_CUDA_OK(cudaGetLastError());
    }
    if (copy_out) {
        const bool routed = in.n_out_routes > 0 || in.own_direct;
        if (local_kernel && (!routed || in.n_out_routes > 0)) {
            return helper(false);
        }
        const uint8_t* win = static_cast<const uint8_t*>(in.peer_win[in.rank]);
        if (routed) {
            for (int i = 0; i < in.n_out_routes; ++i) {
                const int rc = copy_route(in.out_routes[i], win, static_cast<uint8_t*>(in.out), stream);
                if (rc != FU_OK) {
                    return rc;
                }
            }
        }
        else {
            FU_CUDA_OK(cudaMemcpyAsync(in.out, win, static_cast<size_t>(in.out_bytes), cudaMemcpyDeviceToDevice, stream));
        }
    }
    return FU_OK;
}

}  // namespace

extern "C" int fu_a2a4d_check(const FuA2AArgs* args)
{
    KArgs k{};
    return build_args(args, k);
}

extern "C" int fu_a2a4d(const FuA2AArgs* args, void* stream_v)
{
    KArgs     k{};
    const int rc = build_args(args, k);
    if (rc != FU_OK) {
        return rc;
    }
    const FuA2AArgs& in   = *args;
    const bool       ldst = (in.flags & FU_A2A_LDST) != 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (in.flags & FU_A2A_COPY_ENGINE) {
        return launch_copy_engine(in, k, stream);
    }
    int          dev = 0, sms = 0;
    FU_CUDA_OK(cudaGetDevice(&dev));
    FU_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // Every CTA must be resident at once (the CTAs that finish first wait for peers while the rest
    // still have payload to push), so the grid never exceeds what the device can hold. Two
    // collectives of one rank may run side by side on unordered streams (the sync and the async
    // call); if each could fill the device, rank A might hold every SM with the one while rank B
    // holds every SM with the other, each waiting for the peer's other kernel to start. So with
    // peers a launch takes two thirds of the device, or one third when flagged as the minor
    // partner, and both always fit together. A single rank waits for nobody and takes it all.
    const int capacity = ldst ? sms * kLdstCtasPerSm : sms;
    int       share    = capacity;
    if (in.world > 1) {
        share = (in.flags & FU_A2A_MINOR_SHARE) ? capacity / 3 : (2 * capacity) / 3;
    }
    int ctas = in.ctas > 0 ? std::min(in.ctas, share) : share;
    ctas     = std::max(1, ctas);
    pin_ctas(k.push, ctas, in.rank);
    if (ldst) {
        a2a4d_kernel<false><<<ctas, kLdstThreads, 0, stream>>>(k);
    }
    else {
        static bool configured[64] = {};
        const int   smem_bytes     = kStages * kStageBytes;
        if (dev < 64 && !configured[dev]) {
            FU_CUDA_OK(cudaFuncSetAttribute(a2a4d_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            smem_bytes));
            configured[dev] = true;
        }
        a2a4d_kernel<true><<<ctas, 32, smem_bytes, stream>>>(k);
    }
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}

extern "C" int fu_barrier(FuCtrl* const* peer_ctrl, int rank, int world, uint32_t timeout_ms, int flags,
                          void* stream_v)
{
    if (world < 1 || world > FU_MAX_WORLD || rank < 0 || rank >= world || !peer_ctrl) {
        return fu::fail(FU_E_ARG, "fu_barrier: rank %d / world %d out of range", rank, world);
    }
    KArgs k{};
    k.peers.rank       = rank;
    k.peers.world      = world;
    k.peers.mute       = (flags & FU_A2A_MUTE) ? 1 : 0;
    k.peers.timeout_ns = static_cast<uint64_t>(timeout_ms ? timeout_ms : kDefaultTimeoutMs) * 1000000ull;
    k.flags            = flags;
    for (int p = 0; p < world; ++p) {
        if (!peer_ctrl[p]) {
            return fu::fail(FU_E_ARG, "fu_barrier: no control block for rank %d", p);
        }
        k.peers.ctrl[p] = peer_ctrl[p];
    }
    k.peers.own = peer_ctrl[rank];
    barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(k.peers.own, k);
    FU_CUDA_OK(cudaGetLastError());
    return FU_OK;
}
