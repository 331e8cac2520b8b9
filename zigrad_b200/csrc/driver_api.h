// Driver-API access without linking libcuda: entry points are resolved at
// run time through cudaGetDriverEntryPoint (see driver_symbol in runtime.cu).
#pragma once

#include <cuda.h>

namespace zg {

void* driver_symbol(const char* name);
bool check_cu(CUresult r, const char* what, const char* file, int line);

}  // namespace zg

// ZG_DRV(cuMemCreate) -> typed function pointer (nullptr + sticky error if missing)
#define ZG_DRV(fn) reinterpret_cast<decltype(&fn)>(::zg::driver_symbol(#fn))
#define ZG_CU(expr) ::zg::check_cu((expr), #expr, __FILE__, __LINE__)
