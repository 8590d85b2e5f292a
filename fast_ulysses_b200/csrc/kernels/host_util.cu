#include "fu_kernels.h"
#include "host_util.h"

namespace fu {
char* error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}
}  // namespace fu

#define FU_STR2(x) #x
#define FU_STR(x) FU_STR2(x)

extern "C" const char* fu_last_error(void)
{
    return fu::error_buffer();
}

extern "C" const char* fu_build_info(void)
{
    return "sm_100a;nvcc " FU_STR(__CUDACC_VER_MAJOR__) "." FU_STR(__CUDACC_VER_MINOR__) "." FU_STR(
        __CUDACC_VER_BUILD__) ";fast_ulysses_b200 0.1.0";
}
