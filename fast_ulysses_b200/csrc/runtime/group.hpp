#pragma once
// The per-group runtime: everything that outlives one call. Symmetric windows (with their
// handshake control blocks inside the same allocation), the plan cache, the lend pool, the
// buffers handed out by empty_output(), and the launch of the all-to-all kernel. A group whose
// device index is negative runs on CPU tensors over the process group's own all-to-all (gloo),
// which is what lets every host-side rule be tested without a GPU.
//
// Parity: include/fast_ulysses/group.hpp:24-200 and src/group.cc of the reference. Differences
// that follow from the SM-driven design: windows are byte buffers keyed by role only (the kernel
// moves bytes, so a dtype change never reallocates); there is no transfer stream and no staging
// pool (the kernel reads the caller's tensor directly); the handshake state is a FuCtrl block at
// the tail of each window rather than a slice of torch's signal pad.
#include <ATen/ATen.h>
#include <torch/custom_class.h>

#include <array>
#include <atomic>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "../kernels/fu_kernels.h"
#include "../plan/a2a_plan.hpp"

namespace fu {

using Splits = std::optional<std::vector<int64_t>>;

enum class Role : int64_t {
    kSync  = 0,  // all_to_all_4d on the caller's stream
    kAsync = 1,  // all_to_all_4d_async on the comm stream; unordered against kSync, hence separate
};

struct Window {
    at::Tensor            bytes;  // uint8, payload capacity followed by the control block
    int64_t               capacity = 0;  // payload bytes
    std::vector<uint8_t*> base;   // payload base on every rank (peer-mapped)
    std::vector<FuCtrl*>  ctrl;   // control block on every rank (peer-mapped)
    bool                  valid() const { return bytes.defined(); }
};

constexpr int     kLentSlots     = 4;
constexpr int     kPoolSlots     = 3;  // <= FU_POOL_SLOTS

// One buffer of the output pool: a symmetric allocation (shared with the tensors handed out of it,
// so it outlives the pool if it must) and whether a tensor handed out of it is still alive.
struct PoolSlot {
    std::shared_ptr<Window>           w;
    std::shared_ptr<std::atomic<int>> busy;
    // The stream of the call that last filled this buffer. A tensor is dropped on the host while
    // its readers may still be queued on that stream; a later call on the same stream is ordered
    // after them, a call on another stream first waits for that stream (see take_pool_slot).
    void* last_stream = nullptr;
    bool  used        = false;
};
constexpr size_t  kPlanCacheCap  = 512;

class Group : public torch::CustomClassHolder {
public:
    Group(std::string group_name, int64_t rank, int64_t world, int64_t device_index);
    ~Group() override;

    bool    on_cuda() const { return device_index_ >= 0; }
    int64_t device_index() const { return device_index_; }
    int     rank() const { return rank_; }
    int     world() const { return world_; }
    void    check_alive() const;

    // Validation on rank-uniform quantities only, then the cached plan. Throws before anything
    // collective has happened, so a rejected argument is rejected on every rank together.
    const Plan& plan(at::IntArrayRef sizes, at::IntArrayRef strides, at::ScalarType dtype, int64_t mode,
                     const Splits& seq, const Splits& heads);

    Window&       window(Role role, int64_t bytes);
    Window&       lend_window(int64_t bytes);
    // Output pool of the copying call. `take_pool_slot` is COLLECTIVE when the pool has to be
    // created or grown (every rank calls it with the same `bytes` at the same point) and otherwise
    // a local decision: the index + 1 of a buffer no live tensor refers to, or 0 when there is
    // none (the call then goes through the window and is copied out, on this rank only).
    int           take_pool_slot(int64_t bytes, void* stream);
    at::Tensor    pool_output(int slot, at::IntArrayRef shape, at::ScalarType dtype);
    // Gives back a buffer taken with take_pool_slot for which no tensor came to exist.
    void          release_pool_slot(int slot);
    bool          output_pool() const { return pool_enabled_; }
    void          set_output_pool(bool on) { pool_enabled_ = on; }
    int64_t       pool_hits() const { return pool_hits_; }
    // Whether the asynchronous call moves its payload with the copy engines (FU_A2A_COPY_ENGINE)
    // instead of the kernel. A local choice: both transports speak the same handshake.
    bool          async_copy_engine() const { return async_copy_engine_; }
    void          set_async_copy_engine(bool on) { async_copy_engine_ = on; }
    at::Tensor    make_output(at::IntArrayRef shape, at::ScalarType dtype, int64_t window_bytes);
    const Window* window_of(const at::Tensor& t) const;
    // A caller-owned symmetric byte buffer for the fused operators (q/k/v windows, attention
    // output): COLLECTIVE. `symm_ptrs` gives its base address on every rank followed by its control
    // block address on every rank.
    at::Tensor           symm_alloc(int64_t bytes);
    std::vector<int64_t> symm_ptrs(const at::Tensor& t) const;
    void          prune_owned();

    // Typed view of a window's dense prefix.
    static at::Tensor view_of(const Window& w, at::IntArrayRef shape, at::ScalarType dtype);

    // Launch on `stream`. `out` may be null (result stays in the window). `src_bytes` is the extent
    // of the input behind `src`; with the capacities of the window and the pool it lets the launcher
    // refuse a route that would leave its buffer.
    // `pool_possible`: some rank may have chosen a pool buffer for this call (the same on every rank).
    void launch(const Plan& plan, const void* src, int64_t src_bytes, const Window& w, void* out, int64_t out_bytes,
                void* stream, int extra_flags, int pool_slot = 0, bool pool_possible = false);
    void barrier(Role role, void* stream);

    // CPU/gloo execution of the same plan.
    void run_cpu(const Plan& plan, const at::Tensor& x, at::Tensor& out);

    // Reads (synchronising) the first non-zero status word among this group's windows and throws
    // a description of it; returns silently when every window is clean.
    void    check();
    int64_t epoch(int64_t role_or_ptr, const at::Tensor& probe);
    std::vector<int64_t> stamps(int64_t role);

    void set_timeout_ms(int64_t ms) { timeout_ms_ = static_cast<uint32_t>(ms); }
    void set_test_flags(int64_t flags) { test_flags_ = static_cast<int>(flags); }
    void set_ctas(int64_t ctas) { ctas_ = static_cast<int>(ctas); }
    int64_t windows_allocated() const { return allocations_; }

    void destroy();

private:
    Window allocate(int64_t bytes);

    std::string group_name_;
    int         rank_;
    int         world_;
    int64_t     device_index_;
    bool        alive_      = true;
    uint32_t    timeout_ms_ = 0;
    int         test_flags_ = 0;
    bool        async_copy_engine_ = false;
    int         ctas_       = 0;
    int64_t     allocations_ = 0;

    std::map<std::vector<int64_t>, Plan> plans_;
    std::map<int64_t, Window>            windows_;  // by role
    std::array<Window, kLentSlots>       lent_;
    uint64_t                             lend_calls_ = 0;
    std::map<void*, Window>              owned_;    // empty_output() buffers by data pointer
    std::vector<PoolSlot>                pool_;
    int64_t                              pool_capacity_ = 0;
    bool                                 pool_enabled_  = true;
    int64_t                              pool_hits_     = 0;
};

}  // namespace fu
