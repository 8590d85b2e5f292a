#include "nvlink.hpp"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cctype>
#include <cstring>
#include <mutex>
#include <set>
#include <sstream>

namespace fu {
namespace {

// The slice of NVML's ABI this probe needs, declared here so that no NVML header is required.
struct PciInfo {
    char         bus_id_legacy[16];
    unsigned int domain, bus, device, pci_device_id, pci_subsystem_id;
    char         bus_id[32];
};
using Device = void*;
constexpr int kSuccess        = 0;
constexpr int kMaxLinks       = 32;
constexpr int kRemoteGpu      = 0;  // NVML_NVLINK_DEVICE_TYPE_GPU
constexpr int kRemoteSwitch   = 2;  // NVML_NVLINK_DEVICE_TYPE_SWITCH

struct Nvml {
    void* lib = nullptr;
    int (*init)()                                              = nullptr;
    int (*by_bus_id)(const char*, Device*)                     = nullptr;
    int (*link_state)(Device, unsigned, unsigned*)             = nullptr;
    int (*remote_pci)(Device, unsigned, PciInfo*)              = nullptr;
    int (*remote_type)(Device, unsigned, int*)                 = nullptr;
    bool ok = false;
};

std::mutex  g_mu;
std::string g_path = "libnvidia-ml.so.1";
Nvml        g_nvml;
bool        g_loaded = false;

Nvml& nvml()
{
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_loaded) {
        return g_nvml;
    }
    g_loaded = true;
    Nvml& n  = g_nvml;
    n        = Nvml{};
    n.lib    = dlopen(g_path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!n.lib) {
        return n;
    }
    auto sym = [&](const char* name) { return dlsym(n.lib, name); };
    n.init        = reinterpret_cast<int (*)()>(sym("nvmlInit_v2"));
    n.by_bus_id   = reinterpret_cast<int (*)(const char*, Device*)>(sym("nvmlDeviceGetHandleByPciBusId_v2"));
    n.link_state  = reinterpret_cast<int (*)(Device, unsigned, unsigned*)>(sym("nvmlDeviceGetNvLinkState"));
    n.remote_pci  = reinterpret_cast<int (*)(Device, unsigned, PciInfo*)>(sym("nvmlDeviceGetNvLinkRemotePciInfo_v2"));
    n.remote_type = reinterpret_cast<int (*)(Device, unsigned, int*)>(sym("nvmlDeviceGetNvLinkRemoteDeviceType"));
    n.ok = n.init && n.by_bus_id && n.link_state && n.remote_pci && n.remote_type && n.init() == kSuccess;
    return n;
}

std::string canonical(const std::string& bus_id)
{
    // NVML prints an 8-digit domain, CUDA a 4-digit one; compare on the last 12 characters, lower case.
    std::string s = bus_id;
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
    return s.size() > 12 ? s.substr(s.size() - 12) : s;
}

}  // namespace

void set_nvml_library(const std::string& path)
{
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_nvml.lib) {
        dlclose(g_nvml.lib);
    }
    g_nvml   = Nvml{};
    g_loaded = false;
    g_path   = path.empty() ? "libnvidia-ml.so.1" : path;
}

std::optional<LinkMatrix> nvlink_matrix_by_bus_id(const std::vector<std::string>& bus_ids,
                                                  const std::vector<int64_t>&     labels)
{
    Nvml& n = nvml();
    if (!n.ok || bus_ids.size() != labels.size()) {
        return std::nullopt;
    }
    const size_t                       count = bus_ids.size();
    std::vector<std::set<std::string>> direct(count);
    std::vector<bool>                  on_switch(count, false);
    for (size_t i = 0; i < count; ++i) {
        Device dev = nullptr;
        if (n.by_bus_id(bus_ids[i].c_str(), &dev) != kSuccess) {
            return std::nullopt;  // one device we cannot see makes the whole answer unknowable
        }
        for (unsigned link = 0; link < kMaxLinks; ++link) {
            unsigned active = 0;
            if (n.link_state(dev, link, &active) != kSuccess || !active) {
                continue;
            }
            int kind = -1;
            if (n.remote_type(dev, link, &kind) != kSuccess) {
                continue;
            }
            if (kind == kRemoteSwitch) {
                on_switch[i] = true;
            }
            else if (kind == kRemoteGpu) {
                PciInfo info;
                std::memset(&info, 0, sizeof(info));
                if (n.remote_pci(dev, link, &info) == kSuccess) {
                    direct[i].insert(canonical(info.bus_id));
                }
            }
        }
    }
    LinkMatrix out;
    for (size_t i = 0; i < count; ++i) {
        for (size_t j = 0; j < count; ++j) {
            if (i == j) {
                continue;
            }
            // Every GPU with a link into the switch fabric reaches every other such GPU.
            const bool joined = (on_switch[i] && on_switch[j]) || direct[i].count(canonical(bus_ids[j])) > 0;
            out[{labels[i], labels[j]}] = joined;
        }
    }
    return out;
}

std::optional<LinkMatrix> nvlink_matrix(const std::vector<int64_t>& devices)
{
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess) {
        return std::nullopt;
    }
    std::vector<std::string> bus_ids;
    for (int64_t d : devices) {
        if (d < 0 || d >= visible) {
            return std::nullopt;
        }
        char buf[64] = {0};
        if (cudaDeviceGetPCIBusId(buf, sizeof(buf), static_cast<int>(d)) != cudaSuccess) {
            return std::nullopt;
        }
        bus_ids.emplace_back(buf);
    }
    return nvlink_matrix_by_bus_id(bus_ids, devices);
}

std::string check_nvlink(const std::vector<int64_t>& devices)
{
    const auto matrix = nvlink_matrix(devices);
    if (!matrix.has_value()) {
        return "";
    }
    std::ostringstream missing;
    int                n = 0;
    for (const auto& e : *matrix) {
        if (!e.second && e.first.first < e.first.second) {
            missing << (n++ ? ", " : "") << "cuda:" << e.first.first << "<->cuda:" << e.first.second;
        }
    }
    if (n == 0) {
        return "";
    }
    return "these GPUs are not joined by NVLink: " + missing.str()
           + ". The exchange writes peers' memory directly and over PCIe it is slower than "
             "torch.distributed; pass require_nvlink=False only to measure that case.";
}

}  // namespace fu
