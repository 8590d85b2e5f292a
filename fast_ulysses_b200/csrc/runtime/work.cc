#include "work.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

namespace fu {
namespace {

void ok(cudaError_t e, const char* what)
{
    TORCH_CHECK(e == cudaSuccess, "fast_ulysses_b200: ", what, " failed: ", cudaGetErrorString(e));
}

// Completion is an event on the comm stream; waiting means "whatever stream is current now must
// not run past that event".
class EventWork : public c10d::Work {
public:
    explicit EventWork(cudaEvent_t ev) : ev_(ev) {}
    ~EventWork() override { cudaEventDestroy(ev_); }

    bool wait(std::chrono::milliseconds) override
    {
        ok(cudaStreamWaitEvent(at::cuda::getCurrentCUDAStream(), ev_, 0), "cudaStreamWaitEvent");
        return true;
    }
    void synchronize() override { ok(cudaEventSynchronize(ev_), "cudaEventSynchronize"); }
    bool isCompleted() override { return cudaEventQuery(ev_) == cudaSuccess; }
    bool isSuccess() const override { return true; }

private:
    cudaEvent_t ev_;
};

}  // namespace

bool register_stream_completion(const at::Tensor& tensor, int64_t comm_stream)
{
    const c10::cuda::CUDAGuard guard(tensor.device());
    cudaEvent_t                ev = nullptr;
    ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreateWithFlags");
    ok(cudaEventRecord(ev, reinterpret_cast<cudaStream_t>(comm_stream)), "cudaEventRecord");
#if FU_HAS_WORK_REGISTRY
    c10d::register_work(tensor, c10::make_intrusive<EventWork>(ev));
    return true;
#else
    ok(cudaStreamWaitEvent(at::cuda::getCurrentCUDAStream(), ev, 0), "cudaStreamWaitEvent");
    ok(cudaEventDestroy(ev), "cudaEventDestroy");
    return false;
#endif
}

}  // namespace fu
