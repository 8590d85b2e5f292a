#pragma once
// NVLink topology probe. For a list of CUDA devices: which ordered pairs are joined by NVLink,
// either by a direct GPU-to-GPU link or by both sitting on one NVSwitch fabric. NVML is loaded at
// run time; when it is missing, or any device cannot be probed, the answer is "cannot say"
// (nullopt) and callers fail open.
//
// Parity: include/fast_ulysses/nvlink.hpp:25-29 and src/nvlink.cc:114-220 of the reference.
#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace fu {

using LinkMatrix = std::map<std::pair<int64_t, int64_t>, bool>;

// Probe by PCI bus id ("0000:1b:00.0"); index i of `bus_ids` is reported as device `labels[i]`.
std::optional<LinkMatrix> nvlink_matrix_by_bus_id(const std::vector<std::string>& bus_ids,
                                                  const std::vector<int64_t>&     labels);
std::optional<LinkMatrix> nvlink_matrix(const std::vector<int64_t>& devices);
// Empty when every pair is joined or when NVML cannot say; otherwise a refusal message.
std::string check_nvlink(const std::vector<int64_t>& devices);
// TESTS: load this shared object instead of libnvidia-ml.so.1 (a fake NVML built by the test).
void set_nvml_library(const std::string& path);

}  // namespace fu
