#pragma once
// Binds the completion of work queued on a communication stream to torch's work registry, so that
// an AsyncCollectiveTensor's wait() becomes a GPU-side stream dependency and the host never blocks.
// Parity: include/fast_ulysses/work.hpp and src/work.cc:22-80 of the reference.
#include <ATen/ATen.h>

namespace fu {
// Records an event on `comm_stream` and registers it for `tensor`. Returns false (after making the
// current stream wait directly) when this libtorch exposes no registry.
bool register_stream_completion(const at::Tensor& tensor, int64_t comm_stream);
}  // namespace fu
