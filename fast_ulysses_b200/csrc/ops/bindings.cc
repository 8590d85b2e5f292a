// The torch operator layer: schemas, dispatcher registrations, autograd (reverse and forward
// mode), shape propagation for FakeTensor, the refusal of vmap, and the small pybind module.
//
// Parity: src/bindings.cc:89-811 and src/plan_bindings.cc of the reference. The call path differs:
// one kernel launch per collective (handshakes, payload and copy-out fused), the input is read in
// place by that kernel (no staging copy, strided views accepted), and CPU tensors run the same
// plan over the process group's all-to-all.
#include <nvtx3/nvToolsExt.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/autograd.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "../runtime/group.hpp"
#include "../runtime/nvlink.hpp"
#include "../runtime/work.hpp"

namespace py = pybind11;

namespace fu {

using GroupPtr = c10::intrusive_ptr<Group>;

namespace {

void cuda_ok(cudaError_t e, const char* what)
{
    TORCH_CHECK(e == cudaSuccess, "fast_ulysses_b200: ", what, " failed: ", cudaGetErrorString(e));
}

bool overlaps(const void* a, int64_t a_bytes, const void* b, int64_t b_bytes)
{
    const auto a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a_bytes > 0 && b_bytes > 0 && a0 < b0 + static_cast<uintptr_t>(b_bytes)
           && b0 < a0 + static_cast<uintptr_t>(a_bytes);
}

int64_t nbytes_of(at::IntArrayRef shape, at::ScalarType dtype)
{
    return c10::multiply_integers(shape) * static_cast<int64_t>(c10::elementSize(dtype));
}

void require_backend(const Group& g, const at::Tensor& t, const char* name)
{
    if (g.on_cuda()) {
        TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor for this group (it was built for cuda:", g.device_index(),
                    "), got ", t.device());
        // static_cast: a DeviceIndex is an int8_t and would print as a character.
        TORCH_CHECK(t.device().index() == g.device_index(), name, " is on cuda:",
                    static_cast<int64_t>(t.device().index()), " but this UlyssesGroup was built for cuda:",
                    g.device_index(), "; one group serves exactly one device");
    }
    else {
        TORCH_CHECK(t.is_cpu(), name, " must be a CPU tensor: this UlyssesGroup runs the CPU/gloo backend");
    }
}

// What a call has decided before anything collective happens.
struct Prepared {
    const Plan* plan = nullptr;
    at::Tensor  x;              // the tensor the kernel reads (the input, or a densified copy)
    at::Tensor  output;
    Window*     window        = nullptr;
    bool        out_is_window = false;
    int         pool_slot     = 0;  // > 0: `output` is that buffer of the output pool
    // Every rank evaluates the same condition (role, no out=, pool switched on, no capture): when it
    // holds, any rank may ask for this call's payload in one of its pool buffers; when it does not,
    // no rank can, and the kernel is told that there is no pool at all.
    bool        pool_possible = false;
};

// The kernel reads a view in place when only the batch and sequence strides are irregular.
bool readable_in_place(const at::Tensor& t)
{
    if (t.dim() != 4 || t.numel() == 0) {
        return false;
    }
    const int64_t elem = static_cast<int64_t>(t.element_size());
    return t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(1) >= t.size(2) * t.size(3) && t.stride(0) >= 0
           && (t.stride(0) * elem) % 16 == 0 && (t.stride(1) * elem) % 16 == 0
           && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
}

Prepared prepare(Group& g, const at::Tensor& input, int64_t mode, const Splits& seq, const Splits& heads,
                 const std::optional<at::Tensor>& out, Role role, bool lend)
{
    g.check_alive();
    g.prune_owned();
    require_backend(g, input, "input");
    TORCH_CHECK(input.dim() == 4, "input must be 4D (b, s, n, d), got ", input.dim(), " dims");

    Prepared             p;
    std::vector<int64_t> strides;
    if (input.is_contiguous() && (!g.on_cuda() || reinterpret_cast<uintptr_t>(input.data_ptr()) % 16 == 0)) {
        p.x = input;
    }
    else if (g.on_cuda() && readable_in_place(input)) {
        p.x     = input;
        strides = input.strides().vec();
    }
    else {
        p.x = input.contiguous();
        if (g.on_cuda() && reinterpret_cast<uintptr_t>(p.x.data_ptr()) % 16 != 0) {
            p.x = p.x.clone();
        }
    }
    p.plan = &g.plan(p.x.sizes(), strides, p.x.scalar_type(), mode, seq, heads);
    const auto    dtype        = p.x.scalar_type();
    const int64_t elem         = static_cast<int64_t>(c10::elementSize(dtype));
    const int64_t window_bytes = p.plan->window_numel * elem;
    const int64_t out_bytes    = p.plan->out_numel * elem;

    if (out.has_value()) {
        const at::Tensor& o = *out;
        TORCH_CHECK(o.is_contiguous() && (g.on_cuda() ? o.is_cuda() : o.is_cpu()), "out must be a contiguous ",
                    g.on_cuda() ? "CUDA" : "CPU", " tensor");
        require_backend(g, o, "out");
        TORCH_CHECK(o.sizes().vec() == p.plan->out_shape, "out has shape ", o.sizes(), " but this call produces ",
                    at::IntArrayRef(p.plan->out_shape));
        TORCH_CHECK(o.scalar_type() == dtype, "out has dtype ", o.scalar_type(), " but the input is ", dtype);
        p.output = o;
    }
    if (!g.on_cuda()) {
        if (!p.output.defined()) {
            p.output = at::empty(p.plan->out_shape, input.options());
        }
        return p;
    }

    if (out.has_value()) {
        const Window* owned = g.window_of(*out);
        if (owned && owned->capacity >= window_bytes) {
            p.window        = const_cast<Window*>(owned);
            p.out_is_window = true;
        }
    }
    if (!p.window) {
        if (lend) {
            p.window        = &g.lend_window(window_bytes);
            p.output        = Group::view_of(*p.window, p.plan->out_shape, dtype);
            p.out_is_window = true;
        }
        else {
            p.window = &g.window(role, window_bytes);
            // Not while a CUDA graph is being captured: a replay keeps writing the buffer chosen at
            // capture time, whoever holds it by then, so a captured call takes the window and a
            // tensor from the graph's own memory pool instead.
            cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
            const cudaStream_t      cur = at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(g.device_index()));
            cudaStreamIsCapturing(cur, &capture);
            if (!p.output.defined() && role == Role::kSync && g.output_pool()
                && capture == cudaStreamCaptureStatusNone) {
                // The result is born in a pooled symmetric buffer that the peers write directly
                // (this rank tells them which one in the opening handshake). When every buffer is
                // still referenced by a live tensor, this rank alone falls back to window + copy-out.
                p.pool_possible = true;
                p.pool_slot     = g.take_pool_slot(window_bytes, cur);
                if (p.pool_slot > 0) {
                    // the buffer is marked busy from here; only the tensor's deleter clears the mark,
                    // so a failure before the tensor exists must clear it by hand
                    try {
                        p.output = g.pool_output(p.pool_slot, p.plan->out_shape, dtype);
                    }
                    catch (...) {
                        g.release_pool_slot(p.pool_slot);
                        throw;
                    }
                }
            }
            if (!p.output.defined()) {
                p.output = at::empty(p.plan->out_shape, p.x.options().memory_format(at::MemoryFormat::Contiguous));
            }
        }
    }
    // Peers write the window while this rank's kernel is still reading the input.
    const uint8_t* win_base = p.window->base[g.rank()];
    const int64_t span = p.x.numel() == 0 ? 0
                                          : ((p.x.size(0) - 1) * p.x.stride(0) + (p.x.size(1) - 1) * p.x.stride(1)
                                             + p.x.size(2) * p.x.size(3))
                                                * elem;
    TORCH_CHECK(!overlaps(p.x.data_ptr(), span, win_base, p.window->capacity),
                "input overlaps the window this call writes: the peers would overwrite it while it is being "
                "read. Pass a copy, or a different out=");
    if (!p.out_is_window) {
        TORCH_CHECK(!overlaps(p.output.data_ptr(), out_bytes, win_base, p.window->capacity),
                    "out partially overlaps a window of this group");
    }
    return p;
}

// An NVTX range around the host side of one collective (argument checks, plan lookup, launch):
// a timeline profiler shows which call of the library a kernel on the stream belongs to. The
// header-only NVTX costs a null check when no profiler is attached.
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&)            = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

void run_prepared(Group& g, Prepared& p, cudaStream_t stream, int extra_flags)
{
    if (!g.on_cuda()) {
        g.run_cpu(*p.plan, p.x, p.output);
        return;
    }
    const int64_t out_bytes = nbytes_of(p.plan->out_shape, p.x.scalar_type());
    const int64_t elem      = static_cast<int64_t>(p.x.element_size());
    // one past the last byte of the (possibly strided) input: what the routes may read
    const int64_t src_bytes = p.x.numel() == 0 ? 0
                                               : ((p.x.size(0) - 1) * p.x.stride(0) + (p.x.size(1) - 1) * p.x.stride(1)
                                                  + (p.x.size(2) - 1) * p.x.stride(2) + p.x.size(3))
                                                     * elem;
    g.launch(*p.plan, p.x.data_ptr(), src_bytes, *p.window, p.out_is_window ? nullptr : p.output.data_ptr(),
             p.out_is_window ? 0 : out_bytes, stream, extra_flags, p.pool_slot, p.pool_possible);
}

cudaStream_t current_stream(const Group& g)
{
    return at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(g.device_index()));
}

std::vector<int64_t> output_shape_for(const Group& g, const at::Tensor& input, int64_t mode, const Splits& seq,
                                      const Splits& heads)
{
    // Shape rule only; shares the validation with the real kernel through a throw-away plan.
    Group& mut = const_cast<Group&>(g);
    return mut.plan(input.sizes(), {}, input.scalar_type(), mode, seq, heads).out_shape;
}

}  // namespace

// ---- vmap -----------------------------------------------------------------------------------------
// vmap has no batching rule for a collective and would fall back to one call per batch element;
// ranks that disagree on the batch size would then issue different numbers of collectives.
void refuse_vmap(const c10::OperatorHandle& op, c10::Stack*)
{
    TORCH_CHECK(false, op.schema().operator_name().name,
                " does not support torch.vmap: it is a collective, and vmap would run it once per batch "
                "element, so ranks that disagree on the batch size would wait on each other for ever. Fold the "
                "batch into the leading axis and call it once. (torch.autograd.grad(is_grads_batched=True) "
                "arrives here too.)");
}

// ---- functional op ----------------------------------------------------------------------------------
at::Tensor all_to_all_4d(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                         const Splits& heads)
{
    const NvtxRange range(mode == 0 ? "fast_ulysses_b200::all_to_all_4d[mode 0]" : "fast_ulysses_b200::all_to_all_4d[mode 1]");
    Prepared p = prepare(*group, input, mode, seq, heads, std::nullopt, Role::kSync, false);
    if (group->on_cuda()) {
        const c10::cuda::CUDAGuard guard(input.device());
        run_prepared(*group, p, current_stream(*group), 0);
    }
    else {
        run_prepared(*group, p, nullptr, 0);
    }
    return p.output;
}

at::Tensor all_to_all_4d_meta(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                              const Splits& heads)
{
    return at::empty(output_shape_for(*group, input, mode, seq, heads), input.options());
}

void all_to_all_4d_out(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                       const Splits& heads, at::Tensor out)
{
    const NvtxRange range(mode == 0 ? "fast_ulysses_b200::all_to_all_4d_out[mode 0]"
                                    : "fast_ulysses_b200::all_to_all_4d_out[mode 1]");
    Prepared p = prepare(*group, input, mode, seq, heads, out, Role::kSync, false);
    if (group->on_cuda()) {
        const c10::cuda::CUDAGuard guard(input.device());
        run_prepared(*group, p, current_stream(*group), 0);
    }
    else {
        run_prepared(*group, p, nullptr, 0);
    }
}

void all_to_all_4d_out_meta(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                            const Splits& heads, at::Tensor out)
{
    const auto shape = output_shape_for(*group, input, mode, seq, heads);
    TORCH_CHECK(out.sizes().vec() == shape, "out has shape ", out.sizes(), " but this call produces ",
                at::IntArrayRef(shape));
}

// ---- async (comm-stream) op ---------------------------------------------------------------------------
// Runs with the comm stream current. The kernel reads the caller's tensor directly: the comm
// stream waits for the caller's stream to have produced it, and the caching allocator is told that
// the comm stream uses the block, so there is no staging copy.
namespace {

at::Tensor run_async(Group& g, const at::Tensor& input, int64_t mode, const Splits& seq, const Splits& heads,
                     const std::optional<at::Tensor>& out, int64_t caller_stream_id, int64_t caller_device_index,
                     bool lend)
{
    g.check_alive();
    require_backend(g, input, "input");
    const NvtxRange range("fast_ulysses_b200::all_to_all_4d_async");
    if (!g.on_cuda()) {
        Prepared p = prepare(g, input, mode, seq, heads, out, Role::kAsync, false);
        run_prepared(g, p, nullptr, 0);
        return p.output;
    }
    const c10::cuda::CUDAGuard guard(input.device());
    const auto                 comm = at::cuda::getCurrentCUDAStream(input.device().index());
    const c10::cuda::CUDAStream caller(c10::Stream(
        c10::Stream::UNSAFE, c10::Device(c10::DeviceType::CUDA, static_cast<c10::DeviceIndex>(caller_device_index)),
        caller_stream_id));
    TORCH_CHECK(caller.device_index() == input.device().index(),
                "the caller's stream is on another device than the input");

    Prepared p;
    {
        // Densifying a view the kernel cannot read in place belongs on the stream that produced it.
        const c10::cuda::CUDAStreamGuard on_caller(caller);
        p = prepare(g, input, mode, seq, heads, out, Role::kAsync, lend);
    }
    if (p.output.defined() && !out.has_value() && !p.out_is_window) {
        // Allocated while the caller's stream was current; the comm stream writes it.
        c10::cuda::CUDACachingAllocator::recordStream(p.output.storage().data_ptr(), comm);
    }
    cudaEvent_t ready = nullptr;
    cuda_ok(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming), "cudaEventCreateWithFlags");
    cuda_ok(cudaEventRecord(ready, caller.stream()), "cudaEventRecord");
    cuda_ok(cudaStreamWaitEvent(comm.stream(), ready, 0), "cudaStreamWaitEvent");
    cuda_ok(cudaEventDestroy(ready), "cudaEventDestroy");
    c10::cuda::CUDACachingAllocator::recordStream(p.x.storage().data_ptr(), comm);
    run_prepared(g, p, comm.stream(), FU_A2A_MINOR_SHARE | (g.async_copy_engine() ? FU_A2A_COPY_ENGINE : 0));
    return p.output;
}

}  // namespace

at::Tensor all_to_all_4d_staged(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                                const Splits& heads, int64_t caller_stream_id, int64_t caller_device_index, bool lend)
{
    return run_async(*group, input, mode, seq, heads, std::nullopt, caller_stream_id, caller_device_index, lend);
}

void all_to_all_4d_staged_out(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                              const Splits& heads, at::Tensor out, int64_t caller_stream_id,
                              int64_t caller_device_index)
{
    run_async(*group, input, mode, seq, heads, out, caller_stream_id, caller_device_index, false);
}

at::Tensor all_to_all_4d_staged_meta(const GroupPtr&, const at::Tensor&, int64_t, const Splits&, const Splits&, int64_t,
                                     int64_t, bool)
{
    TORCH_CHECK(false, "all_to_all_4d_async cannot be traced: it is bound to live CUDA streams and to windows that "
                       "exist only at run time. Trace all_to_all_4d instead.");
}

void all_to_all_4d_staged_out_meta(const GroupPtr&, const at::Tensor&, int64_t, const Splits&, const Splits&,
                                   at::Tensor, int64_t, int64_t)
{
    TORCH_CHECK(false, "all_to_all_4d_async(out=) cannot be traced: it is bound to live CUDA streams.");
}

// ---- empty_output ---------------------------------------------------------------------------------------
at::Tensor empty_output(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                        const Splits& heads)
{
    group->check_alive();
    require_backend(*group, input, "input");
    const Plan&   plan = group->plan(input.sizes(), {}, input.scalar_type(), mode, seq, heads);
    const int64_t elem = static_cast<int64_t>(input.element_size());
    return group->make_output(plan.out_shape, input.scalar_type(), plan.window_numel * elem);
}

at::Tensor empty_output_meta(const GroupPtr&, const at::Tensor&, int64_t, const Splits&, const Splits&)
{
    TORCH_CHECK(false, "empty_output() cannot be traced: it is a collective allocation of symmetric memory, "
                       "which has to happen once, outside the traced region. Allocate before tracing.");
}

// ---- timed -----------------------------------------------------------------------------------------------
// BENCHMARKS ONLY. The phases are fused into one launch, so they are timed by the kernel itself:
// globaltimer stamps taken by CTA 0 (opening, own share of the payload) and by the last CTA to
// finish (closing, copy-out). Synchronises.
std::tuple<at::Tensor, std::vector<double>> all_to_all_4d_timed(const GroupPtr& group, const at::Tensor& input,
                                                                int64_t mode, const Splits& seq, const Splits& heads)
{
    TORCH_CHECK(group->on_cuda(), "all_to_all_4d_timed needs the CUDA backend");
    Prepared                   p = prepare(*group, input, mode, seq, heads, std::nullopt, Role::kSync, false);
    const c10::cuda::CUDAGuard guard(input.device());
    run_prepared(*group, p, current_stream(*group), FU_A2A_STAMPS);
    const std::vector<int64_t> t = group->stamps(static_cast<int64_t>(Role::kSync));
    std::vector<double>        ms(4, 0.0);
    for (int i = 0; i < 4; ++i) {
        ms[i] = static_cast<double>(t[i + 1] - t[i]) * 1e-6;
    }
    return {p.output, ms};
}

std::tuple<at::Tensor, std::vector<double>> all_to_all_4d_timed_meta(const GroupPtr&, const at::Tensor&, int64_t,
                                                                     const Splits&, const Splits&)
{
    TORCH_CHECK(false, "all_to_all_4d_timed reads device timers and cannot be traced.");
}

// ---- autograd ----------------------------------------------------------------------------------------------
namespace {

using A2ASig = at::Tensor(const GroupPtr&, const at::Tensor&, int64_t, const Splits&, const Splits&);

// Back into the dispatcher with the autograd keys masked, so that Python modes, FakeTensor and the
// Meta kernel below are still consulted.
at::Tensor redispatch(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                      const Splits& heads)
{
    at::AutoDispatchBelowADInplaceOrView below;
    static auto op =
        c10::Dispatcher::singleton().findSchemaOrThrow("fast_ulysses_b200::all_to_all_4d", "").typed<A2ASig>();
    return op.call(group, input, mode, seq, heads);
}

// The exchange is a permutation of the global element set, so its vector-Jacobian product is the
// inverse permutation: the other mode with the SAME splits (they describe the group's geometry,
// not one call's send/receive counts, so they do not swap).
struct Exchange : public torch::autograd::Function<Exchange> {
    static at::Tensor forward(torch::autograd::AutogradContext* ctx, const GroupPtr& group, const at::Tensor& input,
                              int64_t mode, const Splits& seq, const Splits& heads)
    {
        ctx->saved_data["group"] = group;  // the graph keeps the group alive
        ctx->saved_data["mode"]  = mode;
        ctx->saved_data["seq"]   = seq.has_value() ? c10::IValue(*seq) : c10::IValue();
        ctx->saved_data["heads"] = heads.has_value() ? c10::IValue(*heads) : c10::IValue();
        return redispatch(group, input, mode, seq, heads);
    }

    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list    grads)
    {
        torch::autograd::variable_list out(5);
        if (!grads[0].defined()) {
            return out;
        }
        auto          group = ctx->saved_data["group"].toCustomClass<Group>();
        const int64_t mode  = ctx->saved_data["mode"].toInt();
        Splits        seq, heads;
        if (!ctx->saved_data["seq"].isNone()) {
            seq = ctx->saved_data["seq"].toIntVector();
        }
        if (!ctx->saved_data["heads"].isNone()) {
            heads = ctx->saved_data["heads"].toIntVector();
        }
        // The copying call: an allocation inside backward would put a collective rendezvous at the
        // mercy of the engine's node order. apply() so that double backward comes back here.
        out[1] = Exchange::apply(group, grads[0], 1 - mode, seq, heads);
        return out;
    }
};

at::Tensor reverse_mode(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                        const Splits& heads)
{
    if (at::GradMode::is_enabled() && input.requires_grad()) {
        return Exchange::apply(group, input, mode, seq, heads);
    }
    return redispatch(group, input, mode, seq, heads);
}

}  // namespace

at::Tensor all_to_all_4d_autograd(const GroupPtr& group, const at::Tensor& input, int64_t mode, const Splits& seq,
                                  const Splits& heads)
{
    // Forward-mode AD: a C++ autograd::Function has no jvp hook, so a dual input is split here. The
    // Jacobian-vector product of a permutation is the permutation, so the tangent takes the same
    // trip: a second collective, issued by every rank because every rank runs the same program.
    constexpr uint64_t level   = 0;
    const at::Tensor   tangent = input._fw_grad(level);
    if (!tangent.defined()) {
        return reverse_mode(group, input, mode, seq, heads);
    }
    at::Tensor primal_out = reverse_mode(group, input._fw_primal(level), mode, seq, heads);
    primal_out._set_fw_grad(reverse_mode(group, tangent, mode, seq, heads), level, /*is_inplace_op=*/false);
    return primal_out;
}

// ---- plan debug ----------------------------------------------------------------------------------------------
// The plan as tensors, so that a CPU test can replay it over plain byte arrays for any rank.
std::tuple<std::vector<int64_t>, int64_t, at::Tensor, at::Tensor, at::Tensor> a2a_plan_debug(
    int64_t b, int64_t d, int64_t rank, int64_t world, std::vector<int64_t> seq, std::vector<int64_t> heads,
    int64_t mode, int64_t elem_size)
{
    Geometry g;
    g.b     = b;
    g.d     = d;
    g.rank  = static_cast<int>(rank);
    g.world = static_cast<int>(world);
    g.seq   = std::move(seq);
    g.heads = std::move(heads);
    Plan plan;
    try {
        plan = make_plan(g, static_cast<int>(mode), elem_size);
    }
    catch (const std::invalid_argument& e) {
        TORCH_CHECK(false, e.what());
    }
    auto pack = [](const std::vector<Route>& routes) {
        at::Tensor t = at::zeros({static_cast<int64_t>(routes.size()), 10}, at::kLong);
        auto       a = t.accessor<int64_t, 2>();
        for (size_t i = 0; i < routes.size(); ++i) {
            const Route& r = routes[i];
            const int64_t row[10] = {r.peer,      r.src_off, r.dst_off,   r.src_pitch, r.dst_pitch,
                                     r.row_bytes, r.rows,    r.batches,   r.src_batch, r.dst_batch};
            for (int j = 0; j < 10; ++j) {
                a[i][j] = row[j];
            }
        }
        return t;
    };
    return {plan.out_shape, plan.window_numel, pack(plan.sends), pack(plan.recvs), pack(plan.from_peers)};
}

}  // namespace fu

#define FU_GROUP_T "__torch__.torch.classes.fast_ulysses_b200.UlyssesGroup"

TORCH_LIBRARY(fast_ulysses_b200, m)
{
    m.class_<fu::Group>("UlyssesGroup")
        .def(torch::init<std::string, int64_t, int64_t, int64_t>())
        .def("destroy", &fu::Group::destroy)
        .def("check", &fu::Group::check)
        .def("set_timeout_ms", &fu::Group::set_timeout_ms)
        .def("set_ctas", &fu::Group::set_ctas)
        .def("windows_allocated", &fu::Group::windows_allocated)
        .def("set_output_pool", [](const c10::intrusive_ptr<fu::Group>& g, bool on) { g->set_output_pool(on); })
        .def("output_pool", [](const c10::intrusive_ptr<fu::Group>& g) { return g->output_pool(); })
        .def("pool_hits", [](const c10::intrusive_ptr<fu::Group>& g) { return g->pool_hits(); })
        .def("set_async_copy_engine",
             [](const c10::intrusive_ptr<fu::Group>& g, bool on) { g->set_async_copy_engine(on); })
        .def("async_copy_engine", [](const c10::intrusive_ptr<fu::Group>& g) { return g->async_copy_engine(); })
        .def("symm_alloc", &fu::Group::symm_alloc)
        .def("symm_ptrs", &fu::Group::symm_ptrs)
        .def("barrier",
             [](const c10::intrusive_ptr<fu::Group>& self, int64_t role) {
                 const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(self->device_index()));
                 self->barrier(static_cast<fu::Role>(role), fu::current_stream(*self));
             })
        // TESTS ONLY: completed handshake phases on a window (0 sync, 1 async, 2 the window behind
        // `probe`, 3.. lent slots); -1 when there is no such window. Synchronises.
        .def("epoch_debug", [](const c10::intrusive_ptr<fu::Group>& self, const at::Tensor& probe,
                               int64_t which) { return self->epoch(which, probe); })
        // TESTS ONLY: FU_A2A_* bits OR-ed into every launch (negative controls, ld/st data path).
        .def("set_test_flags", &fu::Group::set_test_flags);

    auto refuse_batching = [&m](const char* name) {
        for (const c10::DispatchKey key : {c10::DispatchKey::FuncTorchBatched, c10::DispatchKey::Batched}) {
            m.impl(name, key, torch::CppFunction::makeFromBoxedFunction<&fu::refuse_vmap>());
        }
    };

    m.def("all_to_all_4d(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits=None, "
          "int[]? head_splits=None) -> Tensor");
    m.impl("all_to_all_4d", c10::DispatchKey::CompositeExplicitAutograd, &fu::all_to_all_4d);
    m.impl("all_to_all_4d", c10::DispatchKey::Autograd, &fu::all_to_all_4d_autograd);
    m.impl("all_to_all_4d", c10::DispatchKey::Meta, &fu::all_to_all_4d_meta);
    refuse_batching("all_to_all_4d");

    m.def("all_to_all_4d_out(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits, "
          "int[]? head_splits, Tensor(a!) out) -> ()");
    m.impl("all_to_all_4d_out", c10::DispatchKey::CompositeExplicitAutograd, &fu::all_to_all_4d_out);
    m.impl("all_to_all_4d_out", c10::DispatchKey::Meta, &fu::all_to_all_4d_out_meta);
    refuse_batching("all_to_all_4d_out");

    m.def("all_to_all_4d_staged(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits, "
          "int[]? head_splits, int caller_stream_id, int caller_device_index, bool lend=False) -> Tensor");
    m.impl("all_to_all_4d_staged", c10::DispatchKey::CompositeExplicitAutograd, &fu::all_to_all_4d_staged);
    m.impl("all_to_all_4d_staged", c10::DispatchKey::Meta, &fu::all_to_all_4d_staged_meta);
    refuse_batching("all_to_all_4d_staged");

    m.def("all_to_all_4d_staged_out(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits, "
          "int[]? head_splits, Tensor(a!) out, int caller_stream_id, int caller_device_index) -> ()");
    m.impl("all_to_all_4d_staged_out", c10::DispatchKey::CompositeExplicitAutograd, &fu::all_to_all_4d_staged_out);
    m.impl("all_to_all_4d_staged_out", c10::DispatchKey::Meta, &fu::all_to_all_4d_staged_out_meta);
    refuse_batching("all_to_all_4d_staged_out");

    m.def("empty_output(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits=None, "
          "int[]? head_splits=None) -> Tensor");
    m.impl("empty_output", c10::DispatchKey::CompositeExplicitAutograd, &fu::empty_output);
    m.impl("empty_output", c10::DispatchKey::Meta, &fu::empty_output_meta);
    // A fresh buffer does not depend on the tensor its shape was taken from.
    m.impl("empty_output", c10::DispatchKey::Autograd, torch::CppFunction::makeFallthrough());
    refuse_batching("empty_output");

    m.def("all_to_all_4d_timed(" FU_GROUP_T " group, Tensor input, int mode, int[]? seq_splits=None, "
          "int[]? head_splits=None) -> (Tensor, float[])");
    m.impl("all_to_all_4d_timed", c10::DispatchKey::CompositeExplicitAutograd, &fu::all_to_all_4d_timed);
    m.impl("all_to_all_4d_timed", c10::DispatchKey::Meta, &fu::all_to_all_4d_timed_meta);
    m.impl("all_to_all_4d_timed", c10::DispatchKey::Autograd, torch::CppFunction::makeFallthrough());
    refuse_batching("all_to_all_4d_timed");

    m.def("a2a_plan_debug(int b, int d, int rank, int world_size, int[] seq_splits, int[] head_splits, "
          "int mode, int elem_size) -> (int[], int, Tensor, Tensor, Tensor)",
          &fu::a2a_plan_debug);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("register_stream_completion", &fu::register_stream_completion);
    m.def("nvlink_matrix", [](const std::vector<int64_t>& devices) -> py::object {
        const auto matrix = fu::nvlink_matrix(devices);
        if (!matrix.has_value()) {
            return py::none();
        }
        py::dict out;
        for (const auto& e : *matrix) {
            out[py::make_tuple(e.first.first, e.first.second)] = py::bool_(e.second);
        }
        return out;
    });
    m.def("_nvlink_matrix_by_bus_id",
          [](const std::vector<std::string>& bus_ids, const std::vector<int64_t>& labels) -> py::object {
              const auto matrix = fu::nvlink_matrix_by_bus_id(bus_ids, labels);
              if (!matrix.has_value()) {
                  return py::none();
              }
              py::dict out;
              for (const auto& e : *matrix) {
                  out[py::make_tuple(e.first.first, e.first.second)] = py::bool_(e.second);
              }
              return out;
          });
    m.def("check_nvlink", &fu::check_nvlink);
    m.def("_set_nvml_library", &fu::set_nvml_library);
    m.def("build_info", []() {
        std::map<std::string, std::string> out;
        out["version"]        = "0.1.0";
        out["cuda_arch_list"] = "100a";
        out["kernels"]        = fu_build_info();
        return out;
    });
}
