#pragma once
// The cross-rank handshake shared by every kernel that writes peers' windows: announce a phase
// number into every peer's flag slot (red.release.sys), wait until every peer has announced it
// (ld.acquire.sys on the own, local slots). Waits are bounded by the global timer and report
// through the control block's status words instead of spinning for ever.
#include "fu_kernels.h"
#include "ptx.cuh"

namespace fu {

struct Peers {
    FuCtrl*  own;
    FuCtrl*  ctrl[FU_MAX_WORLD];
    int      rank, world, mute;
    uint64_t timeout_ns;
};

__device__ inline void hs_report(FuCtrl* own, uint32_t code, uint32_t peer, uint64_t expected, uint64_t seen)
{
    if (atomicCAS(&own->status[0], 0u, code) == 0u) {
        own->status[1] = peer;
        own->status[2] = static_cast<uint32_t>(expected);
        own->status[3] = static_cast<uint32_t>(expected >> 32);
        own->status[4] = static_cast<uint32_t>(seen);
        own->status[5] = static_cast<uint32_t>(seen >> 32);
    }
}

// One full warp: lane p < world announces `value` to rank p. With `slot >= 0` the announcement
// carries a byte for rank p's FuCtrl::slot_of (where this rank wants the payload of this call):
// written first by the same thread to the same rank, so the release below orders it.
__device__ inline void hs_announce(const Peers& p, uint64_t value, int slot = -1)
{
    const int lane = threadIdx.x & 31;
    if (lane < p.world && !p.mute) {
        if (slot >= 0) {
            *reinterpret_cast<volatile uint8_t*>(&p.ctrl[lane]->slot_of[p.rank]) = static_cast<uint8_t>(slot);
        }
        ptx::red_release_sys_max(&p.ctrl[lane]->flags[p.rank], value);
    }
}

// One full warp: lane p < world waits until rank p has announced at least `target`, for the ranks
// named in `who` (bit p). False on every lane after the time limit, with the missing rank recorded.
__device__ inline bool hs_await(const Peers& p, uint64_t target, uint32_t code, uint32_t who = 0xffffffffu)
{
    const int lane = threadIdx.x & 31;
    bool      ok   = true;
    if (lane < p.world && ((who >> lane) & 1u)) {
        const uint64_t t0    = ptx::globaltimer_ns();
        uint32_t       spins = 0;
        uint64_t       seen;
        while ((seen = ptx::ld_acquire_sys(&p.own->flags[lane])) < target) {
            ++spins;
            if ((spins & 63u) == 0u) {
                if (ptx::globaltimer_ns() - t0 > p.timeout_ns || spins > 0x7fffff00u) {
                    hs_report(p.own, code, static_cast<uint32_t>(lane), target, seen);
                    ok = false;
                    break;
                }
                __nanosleep(64);
            }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

}  // namespace fu
