#include "group.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/csrc/distributed/c10d/symm_mem/SymmetricMemory.hpp>

#include <cstring>
#include <sstream>

namespace fu {

namespace symm = c10d::symmetric_memory;

namespace {

constexpr int64_t kAlign = 256;

int64_t round_up(int64_t v, int64_t to)
{
    return (v + to - 1) / to * to;
}

void cuda_ok(cudaError_t e, const char* what)
{
    TORCH_CHECK(e == cudaSuccess, "fast_ulysses_b200: ", what, " failed: ", cudaGetErrorString(e));
}

bool supported_dtype(at::ScalarType t)
{
    return t == at::kHalf || t == at::kBFloat16 || t == at::kFloat || t == at::kFloat8_e4m3fn
           || t == at::kFloat8_e5m2 || t == at::kChar || t == at::kByte;
}

Geometry geometry_for(at::IntArrayRef sizes, at::ScalarType dtype, int64_t mode, int world, int rank,
                      const Splits& seq, const Splits& heads)
{
    TORCH_CHECK(sizes.size() == 4, "input must be 4D (b, s, n, d), got ", sizes.size(), " dims");
    TORCH_CHECK(supported_dtype(dtype),
                "dtype must be float16, bfloat16, float32, float8_e4m3fn, float8_e5m2, int8 or uint8, got ", dtype);
    const int64_t s = sizes[1], n = sizes[2], d = sizes[3];
    const int64_t elem = static_cast<int64_t>(c10::elementSize(dtype));
    // Every offset, pitch and row length in the plan is a multiple of d * elem, and the kernel moves
    // 16-byte granules, so this one rule makes the whole exchange granular.
    TORCH_CHECK((d * elem) % 16 == 0, "the head dim must be 16-byte aligned: d=", d, " x ", elem, " B is ", d * elem,
                " B");
    TORCH_CHECK(mode == 0 || mode == 1, "mode must be 0 or 1, got ", mode);

    Geometry g;
    g.b     = sizes[0];
    g.d     = d;
    g.rank  = rank;
    g.world = world;
    if (seq.has_value() || heads.has_value()) {
        TORCH_CHECK(seq.has_value() && heads.has_value(),
                    "pass both seq_splits and head_splits, or neither: each describes the whole group and "
                    "neither can be inferred from a shape that is already sharded");
        g.seq   = *seq;
        g.heads = *heads;
        try {
            g.validate();
        }
        catch (const std::invalid_argument& e) {
            TORCH_CHECK(false, e.what());
        }
        const int64_t want_s = mode == 0 ? g.seq[rank] : g.seq_total();
        const int64_t want_n = mode == 0 ? g.head_total() : g.heads[rank];
        TORCH_CHECK(s == want_s && n == want_n, "input is [", g.b, ", ", s, ", ", n, ", ", d,
                    "] but the splits imply [", g.b, ", ", want_s, ", ", want_n, ", ", d, "] on rank ", rank);
        return g;
    }
    if (mode == 0) {
        TORCH_CHECK(n % world == 0, "mode 0 scatters the head axis, so n_global (", n, ") must divide world_size (",
                    world, ") -- or pass seq_splits and head_splits");
        g.seq.assign(world, s);
        g.heads.assign(world, n / world);
    }
    else {
        TORCH_CHECK(s % world == 0, "mode 1 scatters the sequence axis, so s_global (", s,
                    ") must divide world_size (", world, ") -- or pass seq_splits and head_splits");
        g.seq.assign(world, s / world);
        g.heads.assign(world, n);
    }
    return g;
}

const char* status_name(uint32_t code)
{
    switch (code) {
        case FU_ST_OPEN_TIMEOUT: return "opening handshake timed out (a peer never said it had finished reading)";
        case FU_ST_CLOSE_TIMEOUT: return "closing handshake timed out (a peer never said its writes had landed)";
        case FU_ST_COPY_TIMEOUT: return "a bulk copy inside the kernel never completed";
        default: return "unknown status";
    }
}

}  // namespace

Group::Group(std::string group_name, int64_t rank, int64_t world, int64_t device_index)
    : group_name_(std::move(group_name)), rank_(static_cast<int>(rank)), world_(static_cast<int>(world)),
      device_index_(device_index)
{
    TORCH_CHECK(world >= 1 && world <= FU_MAX_WORLD, "world_size must be in [1, ", FU_MAX_WORLD,
                "]: the exchange runs inside one NVLink domain, got ", world);
    TORCH_CHECK(rank >= 0 && rank < world, "rank ", rank, " is outside a group of ", world);
}

Group::~Group()
{
    // Windows may still be the target of a kernel in flight on some stream; wait for the device
    // before the allocations go back. No collective here: a destructor is no place for one.
    if (alive_ && on_cuda() && (!windows_.empty() || lend_calls_ > 0)) {
        int prev = 0;
        if (cudaGetDevice(&prev) == cudaSuccess) {
            cudaSetDevice(static_cast<int>(device_index_));
            cudaDeviceSynchronize();
            cudaSetDevice(prev);
        }
    }
}

void Group::check_alive() const
{
    TORCH_CHECK(alive_, "this UlyssesGroup has been destroyed; build a new one");
}

const Plan& Group::plan(at::IntArrayRef sizes, at::IntArrayRef strides, at::ScalarType dtype, int64_t mode,
                        const Splits& seq, const Splits& heads)
{
    std::vector<int64_t> key;
    key.reserve(16 + 2 * world_);
    key.push_back(mode);
    key.push_back(static_cast<int64_t>(c10::elementSize(dtype)));
    key.push_back(static_cast<int64_t>(dtype));
    key.insert(key.end(), sizes.begin(), sizes.end());
    key.push_back(-1);
    key.insert(key.end(), strides.begin(), strides.end());
    key.push_back(seq.has_value() ? static_cast<int64_t>(seq->size()) : -2);
    if (seq.has_value()) {
        key.insert(key.end(), seq->begin(), seq->end());
    }
    key.push_back(heads.has_value() ? static_cast<int64_t>(heads->size()) : -2);
    if (heads.has_value()) {
        key.insert(key.end(), heads->begin(), heads->end());
    }
    auto it = plans_.find(key);
    if (it != plans_.end()) {
        return it->second;
    }
    const Geometry       g    = geometry_for(sizes, dtype, mode, world_, rank_, seq, heads);
    const int64_t        elem = static_cast<int64_t>(c10::elementSize(dtype));
    std::vector<int64_t> in_strides;
    if (!strides.empty()) {
        in_strides.assign(strides.begin(), strides.begin() + 3);
    }
    Plan p;
    try {
        p = make_plan(g, static_cast<int>(mode), elem, in_strides);
    }
    catch (const std::invalid_argument& e) {
        TORCH_CHECK(false, e.what());
    }
    // Identical on every rank (it is a max over all ranks), so this raises on all of them together.
    TORCH_CHECK(p.window_numel > 0,
                "this call moves no data: every rank's shard is empty. Check the shape and the splits -- a "
                "sequence or head axis of 0 on ALL ranks has nothing to exchange");
    if (plans_.size() >= kPlanCacheCap) {
        plans_.clear();
    }
    return plans_.emplace(std::move(key), std::move(p)).first->second;
}

Window Group::allocate(int64_t bytes)
{
    TORCH_CHECK(on_cuda(), "symmetric windows exist only on the CUDA backend");
    TORCH_CHECK(bytes > 0, "this call moves no data: every rank's shard is empty");
    const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
    const int64_t              payload = round_up(bytes, kAlign);
    const int64_t              total   = payload + FU_CTRL_BYTES;
    const c10::Device          dev(c10::DeviceType::CUDA, static_cast<c10::DeviceIndex>(device_index_));
    cudaStream_t               stream = at::cuda::getCurrentCUDAStream();

    Window w;
    w.capacity = payload;
    if (world_ == 1) {
        // One rank has no peers to map; an ordinary allocation keeps a single-GPU run independent
        // of the symmetric-memory bootstrap.
        w.bytes = at::empty({total}, at::TensorOptions().dtype(at::kByte).device(dev));
        w.base  = {static_cast<uint8_t*>(w.bytes.data_ptr())};
        w.ctrl  = {reinterpret_cast<FuCtrl*>(w.base[0] + payload)};
        cuda_ok(cudaMemsetAsync(w.ctrl[0], 0, FU_CTRL_BYTES, stream), "cudaMemsetAsync");
        cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        ++allocations_;
        return w;
    }
    // The allocator entry point itself, so that no unrelated allocation can slip between the ranks'
    // rendezvous calls and desynchronise them.
    w.bytes  = symm::empty_strided_p2p({total}, {1}, at::kByte, dev, group_name_, std::nullopt);
    auto sym = symm::rendezvous(w.bytes, group_name_);
    TORCH_CHECK(sym, "torch symmetric memory could not rendezvous a ", total, "-byte window on group '", group_name_,
                "'. Is the group registered for symmetric memory, and are all ranks on one NVLink domain?");
    const std::vector<void*> ptrs = sym->get_buffer_ptrs();
    TORCH_CHECK(static_cast<int>(ptrs.size()) == world_, "rendezvous returned ", ptrs.size(),
                " peers for a group of ", world_);
    for (void* p : ptrs) {
        w.base.push_back(static_cast<uint8_t*>(p));
        w.ctrl.push_back(reinterpret_cast<FuCtrl*>(static_cast<uint8_t*>(p) + payload));
    }
    // The memory may be recycled from an earlier window, and every counter must start at zero.
    // Clear the own block, then hold all ranks until everyone has: otherwise a fast rank's first
    // announcement could land in a block its owner has yet to clear, and be erased.
    cuda_ok(cudaMemsetAsync(w.ctrl[rank_], 0, FU_CTRL_BYTES, stream), "cudaMemsetAsync");
    sym->barrier(0, 0);
    cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    ++allocations_;
    return w;
}

Window& Group::window(Role role, int64_t bytes)
{
    check_alive();
    const int64_t key = static_cast<int64_t>(role);
    auto          it  = windows_.find(key);
    if (it != windows_.end() && it->second.capacity >= bytes) {
        return it->second;
    }
    if (it != windows_.end()) {
        // Growth is triggered by a rank-uniform size, so every rank reallocates at the same call.
        // The old window may still be read by work queued on this device.
        const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
        cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        windows_.erase(it);
    }
    return windows_.emplace(key, allocate(bytes)).first->second;
}

Window& Group::lend_window(int64_t bytes)
{
    check_alive();
    // The slot is chosen by the call count, a quantity every rank shares; a search for a free slot
    // would read local reference counts and let ranks pick different windows.
    const size_t idx  = static_cast<size_t>(lend_calls_++ % kLentSlots);
    Window&      slot = lent_[idx];
    if (!slot.valid()) {
        slot = allocate(bytes);
        return slot;
    }
    TORCH_CHECK(slot.bytes.storage().use_count() == 1,
                "all_to_all_4d_async(lend=True) has rotated back to a window that a live result still refers "
                "to: at most ",
                kLentSlots,
                " lent results may be alive at once. Drop the older ones before issuing more calls, or pass "
                "out= and own the buffer. Every rank must drop them at the same point in its program.");
    if (slot.capacity < bytes) {
        const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
        cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        slot = Window{};
        slot = allocate(bytes);
    }
    return slot;
}

int Group::take_pool_slot(int64_t bytes, void* stream)
{
    check_alive();
    if (pool_.empty() || pool_capacity_ < bytes) {
        // Collective: `bytes` is the window size of the plan, which every rank computes alike, so
        // all ranks arrive here in the same call. Buffers of the old pool that tensors still refer
        // to stay alive through those tensors.
        pool_.clear();
        for (int k = 0; k < kPoolSlots; ++k) {
            PoolSlot s;
            s.w    = std::make_shared<Window>(allocate(bytes));
            s.busy = std::make_shared<std::atomic<int>>(0);
            pool_.push_back(std::move(s));
        }
        pool_capacity_ = pool_[0].w->capacity;
    }
    for (size_t k = 0; k < pool_.size(); ++k) {
        int expected = 0;
        if (pool_[k].busy->compare_exchange_strong(expected, 1)) {
            PoolSlot& s = pool_[k];
            if (s.used && s.last_stream != stream) {
                // Readers of the previous result were queued on the stream that produced it (a
                // reader on a third stream is the caller's to order, as with any allocator).
                // Everything queued there so far must finish before the peers may write again.
                const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
                cudaEvent_t ev = nullptr;
                cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreateWithFlags");
                // `last_stream` is only a handle: the caller may have destroyed that stream since.
                // A stream that no longer exists has nothing queued, but CUDA refuses the handle; a
                // rank that threw here would leave its peers waiting in the collective, so fall
                // back to waiting for the whole device instead.
                if (cudaEventRecord(ev, static_cast<cudaStream_t>(s.last_stream)) == cudaSuccess) {
                    cuda_ok(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ev, 0), "cudaStreamWaitEvent");
                }
                else {
                    (void)cudaGetLastError();
                    cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
                }
                cuda_ok(cudaEventDestroy(ev), "cudaEventDestroy");
            }
            s.last_stream = stream;
            s.used        = true;
            ++pool_hits_;
            return static_cast<int>(k) + 1;
        }
    }
    return 0;
}

void Group::release_pool_slot(int slot)
{
    if (slot >= 1 && slot <= static_cast<int>(pool_.size())) {
        pool_[static_cast<size_t>(slot - 1)].busy->store(0);
    }
}

at::Tensor Group::pool_output(int slot, at::IntArrayRef shape, at::ScalarType dtype)
{
    TORCH_CHECK(slot >= 1 && slot <= static_cast<int>(pool_.size()), "pool buffer ", slot, " does not exist");
    const PoolSlot& s      = pool_[static_cast<size_t>(slot - 1)];
    const int64_t   nbytes = c10::multiply_integers(shape) * static_cast<int64_t>(c10::elementSize(dtype));
    TORCH_CHECK(nbytes <= s.w->capacity, "pool buffer of ", s.w->capacity, " bytes cannot hold ", nbytes);
    // The tensor owns the buffer's "in use" mark and a reference to the allocation: the buffer goes
    // back to the pool when the last reference to the tensor's storage is dropped, and the memory
    // stays mapped even if the pool itself has been replaced or the group destroyed by then.
    std::shared_ptr<Window>           keep = s.w;
    std::shared_ptr<std::atomic<int>> busy = s.busy;
    const c10::Device dev(c10::DeviceType::CUDA, static_cast<c10::DeviceIndex>(device_index_));
    return at::from_blob(
        s.w->base[static_cast<size_t>(rank_)], shape, [keep, busy](void*) { busy->store(0); },
        at::TensorOptions().dtype(dtype).device(dev));
}

at::Tensor Group::view_of(const Window& w, at::IntArrayRef shape, at::ScalarType dtype)
{
    const int64_t nbytes = c10::multiply_integers(shape) * static_cast<int64_t>(c10::elementSize(dtype));
    TORCH_INTERNAL_ASSERT(nbytes <= w.capacity);
    return w.bytes.narrow(0, 0, nbytes).view(dtype).view(shape);
}

at::Tensor Group::make_output(at::IntArrayRef shape, at::ScalarType dtype, int64_t window_bytes)
{
    check_alive();
    if (!on_cuda()) {
        return at::empty(shape, at::TensorOptions().dtype(dtype));
    }
    prune_owned();
    Window     w   = allocate(window_bytes);
    at::Tensor out = view_of(w, shape, dtype);
    owned_.emplace(w.bytes.data_ptr(), std::move(w));
    return out;
}

at::Tensor Group::symm_alloc(int64_t bytes)
{
    check_alive();
    TORCH_CHECK(on_cuda(), "symmetric buffers exist only on the CUDA backend");
    prune_owned();
    Window     w   = allocate(bytes);
    at::Tensor out = w.bytes.narrow(0, 0, bytes);
    owned_.emplace(w.bytes.data_ptr(), std::move(w));
    return out;
}

std::vector<int64_t> Group::symm_ptrs(const at::Tensor& t) const
{
    const Window* w = window_of(t);
    TORCH_CHECK(w, "this tensor is not the base of a symmetric buffer of this group");
    std::vector<int64_t> out;
    for (uint8_t* p : w->base) {
        out.push_back(reinterpret_cast<int64_t>(p));
    }
    for (FuCtrl* p : w->ctrl) {
        out.push_back(reinterpret_cast<int64_t>(p));
    }
    return out;
}

const Window* Group::window_of(const at::Tensor& t) const
{
    auto it = owned_.find(t.data_ptr());
    return it == owned_.end() ? nullptr : &it->second;
}

void Group::prune_owned()
{
    // The caller's tensor is a view over the window's storage: one holder left means it is ours only.
    for (auto it = owned_.begin(); it != owned_.end();) {
        it = it->second.bytes.storage().use_count() == 1 ? owned_.erase(it) : std::next(it);
    }
}

void Group::launch(const Plan& plan, const void* src, int64_t src_bytes, const Window& w, void* out,
                   int64_t out_bytes, void* stream, int extra_flags, int pool_slot, bool pool_possible)
{
    FuA2AArgs a{};
    a.src        = src;
    a.src_bytes  = src_bytes;
    a.win_bytes  = w.capacity;
    a.pool_bytes = pool_capacity_;
    // Every rank passes the whole pool, whatever it chose itself: a peer may have chosen any buffer.
    // A call that cannot use the pool on any rank (asynchronous, out=, captured, pool switched off)
    // passes none: the kernel then ignores whatever a control block still says from an earlier call.
    TORCH_INTERNAL_ASSERT(pool_possible || pool_slot == 0);
    const size_t n_pool = pool_possible ? pool_.size() : 0;
    a.n_pool  = static_cast<int32_t>(n_pool);
    a.my_slot = pool_slot;
    for (size_t k = 0; k < n_pool; ++k) {
        for (int p = 0; p < world_; ++p) {
            a.peer_pool[p][k] = pool_[k].w->base[static_cast<size_t>(p)];
        }
    }
    for (int p = 0; p < world_; ++p) {
        a.peer_win[p]  = w.base[p];
        a.peer_ctrl[p] = w.ctrl[p];
    }
    a.out        = out;
    a.out_bytes  = out_bytes;
    a.rank       = rank_;
    a.world      = world_;
    a.flags      = test_flags_ | extra_flags;
    a.ctas       = ctas_;
    a.timeout_ms = timeout_ms_;
    // Start with the next rank up and finish with the own share, so that at any moment every
    // rank's ingress is fed by a different sender.
    int n = 0;
    for (int i = 1; i <= world_; ++i) {
        const int peer = (rank_ + i) % world_;
        for (const Route& r : plan.sends) {
            if (r.peer != peer) {
                continue;
            }
            FuRoute& o  = a.routes[n++];
            o.peer      = r.peer;
            o.src_off   = r.src_off;
            o.dst_off   = r.dst_off;
            o.src_pitch = r.src_pitch;
            o.dst_pitch = r.dst_pitch;
            o.row_bytes = r.row_bytes;
            o.rows      = r.rows;
            o.batches   = r.batches;
            o.src_batch = r.src_batch;
            o.dst_batch = r.dst_batch;
        }
    }
    a.n_routes = n;
    if (out) {
        // Own share straight into the caller's tensor; only what peers wrote is copied out.
        a.own_direct   = 1;
        a.n_out_routes = 0;
        // With a pool buffer chosen the peers write `out` themselves: nothing is copied out.
        for (const Route& r : (pool_slot > 0 ? std::vector<Route>{} : plan.from_peers)) {
            FuRoute& o  = a.out_routes[a.n_out_routes++];
            o.peer      = rank_;
            o.src_off   = r.src_off;
            o.dst_off   = r.dst_off;
            o.src_pitch = r.src_pitch;
            o.dst_pitch = r.dst_pitch;
            o.row_bytes = r.row_bytes;
            o.rows      = r.rows;
            o.batches   = r.batches;
            o.src_batch = r.src_batch;
            o.dst_batch = r.dst_batch;
        }
    }
    const int rc = fu_a2a4d(&a, stream);
    TORCH_CHECK(rc == FU_OK, "fast_ulysses_b200: ", fu_last_error());
}

void Group::barrier(Role role, void* stream)
{
    check_alive();
    TORCH_CHECK(on_cuda(), "barrier() is the device-side barrier; use torch.distributed.barrier on CPU");
    Window& w = window(role, kAlign);
    const int rc = fu_barrier(w.ctrl.data(), rank_, world_, timeout_ms_, test_flags_, stream);
    TORCH_CHECK(rc == FU_OK, "fast_ulysses_b200: ", fu_last_error());
}

void Group::run_cpu(const Plan& plan, const at::Tensor& x, at::Tensor& out)
{
    // The same routes, executed as: pack each peer's share densely, one all_to_all over the
    // process group with per-peer byte counts, unpack each arrival at its permuted offset.
    std::vector<int64_t> send_counts(world_, 0), recv_counts(world_, 0);
    for (const Route& r : plan.sends) {
        send_counts[r.peer] = r.bytes();
    }
    for (const Route& r : plan.recvs) {
        recv_counts[r.peer] = r.bytes();
    }
    int64_t send_total = 0, recv_total = 0;
    for (int p = 0; p < world_; ++p) {
        send_total += send_counts[p];
        recv_total += recv_counts[p];
    }
    at::Tensor send = at::empty({send_total}, at::kByte);
    at::Tensor recv = at::empty({recv_total}, at::kByte);
    const auto* src = static_cast<const uint8_t*>(x.data_ptr());
    auto*       sb  = static_cast<uint8_t*>(send.data_ptr());
    {
        std::vector<int64_t> start(world_, 0);
        for (int p = 1; p < world_; ++p) {
            start[p] = start[p - 1] + send_counts[p - 1];
        }
        for (const Route& r : plan.sends) {
            uint8_t* dst = sb + start[r.peer];
            for (int64_t bi = 0; bi < r.batches; ++bi) {
                for (int64_t row = 0; row < r.rows; ++row) {
                    std::memcpy(dst, src + r.src_off + bi * r.src_batch + row * r.src_pitch,
                                static_cast<size_t>(r.row_bytes));
                    dst += r.row_bytes;
                }
            }
        }
    }
    if (world_ == 1) {
        std::memcpy(recv.data_ptr(), send.data_ptr(), static_cast<size_t>(send_total));
    }
    else {
        auto pg = c10d::resolve_process_group(group_name_);
        pg->alltoall_base(recv, send, recv_counts, send_counts)->wait();
    }
    auto*       dst_base = static_cast<uint8_t*>(out.data_ptr());
    const auto* rb       = static_cast<const uint8_t*>(recv.data_ptr());
    std::vector<int64_t> start(world_, 0);
    for (int p = 1; p < world_; ++p) {
        start[p] = start[p - 1] + recv_counts[p - 1];
    }
    for (const Route& r : plan.recvs) {
        const uint8_t* from = rb + start[r.peer];
        for (int64_t bi = 0; bi < r.batches; ++bi) {
            for (int64_t row = 0; row < r.rows; ++row) {
                std::memcpy(dst_base + r.dst_off + bi * r.dst_batch + row * r.dst_pitch, from,
                            static_cast<size_t>(r.row_bytes));
                from += r.row_bytes;
            }
        }
    }
}

void Group::check()
{
    if (!on_cuda()) {
        return;
    }
    const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
    cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    auto probe = [&](const Window& w, const char* what) {
        if (!w.valid()) {
            return;
        }
        uint32_t st[6] = {};
        cuda_ok(cudaMemcpy(st, w.ctrl[rank_]->status, sizeof(st), cudaMemcpyDeviceToHost), "cudaMemcpy");
        if (st[0] == FU_ST_OK) {
            return;
        }
        cuda_ok(cudaMemset(w.ctrl[rank_]->status, 0, sizeof(st)), "cudaMemset");
        const uint64_t expected = (static_cast<uint64_t>(st[3]) << 32) | st[2];
        const uint64_t seen     = (static_cast<uint64_t>(st[5]) << 32) | st[4];
        TORCH_CHECK(false, "fast_ulysses_b200: rank ", rank_, ", ", what, " window: ", status_name(st[0]),
                    "; waiting on rank ", st[1], " for phase ", expected, ", last saw ", seen,
                    ". The result of that call is not valid.");
    };
    for (auto& kv : windows_) {
        probe(kv.second, kv.first == 0 ? "sync" : "async");
    }
    for (auto& w : lent_) {
        probe(w, "lent");
    }
    for (auto& kv : owned_) {
        probe(kv.second, "caller-owned");
    }
}

int64_t Group::epoch(int64_t which, const at::Tensor& probe)
{
    if (!on_cuda()) {
        return -1;
    }
    const Window* w = nullptr;
    if (which == 0 || which == 1) {
        auto it = windows_.find(which);
        w       = it == windows_.end() ? nullptr : &it->second;
    }
    else if (which == 2) {
        w = window_of(probe);
    }
    else if (which >= 3 && which < 3 + kLentSlots) {
        w = lent_[which - 3].valid() ? &lent_[which - 3] : nullptr;
    }
    if (!w) {
        return -1;
    }
    const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
    cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    uint64_t e = 0;
    cuda_ok(cudaMemcpy(&e, &w->ctrl[rank_]->epoch, sizeof(e), cudaMemcpyDeviceToHost), "cudaMemcpy");
    return static_cast<int64_t>(e);
}

std::vector<int64_t> Group::stamps(int64_t role)
{
    std::vector<int64_t> out(8, 0);
    auto                 it = windows_.find(role);
    if (!on_cuda() || it == windows_.end()) {
        return out;
    }
    const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
    cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    uint64_t raw[8];
    cuda_ok(cudaMemcpy(raw, it->second.ctrl[rank_]->stamps, sizeof(raw), cudaMemcpyDeviceToHost), "cudaMemcpy");
    for (int i = 0; i < 8; ++i) {
        out[i] = static_cast<int64_t>(raw[i]);
    }
    return out;
}

void Group::destroy()
{
    if (!alive_) {
        return;
    }
    if (on_cuda()) {
        const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index_));
        cudaDeviceSynchronize();
    }
    plans_.clear();
    windows_.clear();
    pool_.clear();
    pool_capacity_ = 0;
    for (auto& w : lent_) {
        w = Window{};
    }
    prune_owned();
    alive_ = false;
}

}  // namespace fu
