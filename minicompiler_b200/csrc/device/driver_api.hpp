#pragma once
// Driver-API entry points used by the device layer, resolved at run time with
// cudaGetDriverEntryPoint so that the library has no link-time dependency on
// libcuda and still loads on a machine without a driver.

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <string>
#include <vector>

namespace mcd {

struct DriverApi {
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                             void**, void**) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};

// nullptr when no driver is present.
const DriverApi* driver_api();

int fail(const std::string& message);              // records the message, returns 1
int check_rt(cudaError_t err, const char* what);   // 0, or records "<what>: <text>"
int check_drv(CUresult err, const char* what);

int compile_to_cubin(const char* source, const char* options, std::vector<char>* cubin, std::string* log);

}  // namespace mcd
