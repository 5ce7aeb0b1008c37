// CUDA driver entry points used by the library (virtual-memory management and TMA descriptor encoding),
// resolved through the runtime at first use so that the shared library carries no link-time dependency on the
// driver library and can be loaded (symbols inspected, host-only helpers called) on a machine without a GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

namespace gh {

struct DriverApi
{
  CUresult ( *MemAddressReserve )( CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long ) = nullptr;
  CUresult ( *MemAddressFree )( CUdeviceptr, size_t ) = nullptr;
  CUresult ( *MemCreate )( CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long )
    = nullptr;
  CUresult ( *MemRelease )( CUmemGenericAllocationHandle ) = nullptr;
  CUresult ( *MemMap )( CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long ) = nullptr;
  CUresult ( *MemUnmap )( CUdeviceptr, size_t ) = nullptr;
  CUresult ( *MemSetAccess )( CUdeviceptr, size_t, const CUmemAccessDesc*, size_t ) = nullptr;
  CUresult ( *MemGetAllocationGranularity )( size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags )
    = nullptr;
  CUresult ( *TensorMapEncodeTiled )( CUtensorMap*,
                                      CUtensorMapDataType,
                                      cuuint32_t,
                                      void*,
                                      const cuuint64_t*,
                                      const cuuint64_t*,
                                      const cuuint32_t*,
                                      const cuuint32_t*,
                                      CUtensorMapInterleave,
                                      CUtensorMapSwizzle,
                                      CUtensorMapL2promotion,
                                      CUtensorMapFloatOOBfill )
    = nullptr;
  CUresult ( *GetErrorString )( CUresult, const char** ) = nullptr;
};

// Returns the process-wide table, resolving it on the first call; nullptr (and a message) if the driver is
// not reachable.
const DriverApi* driver_api( std::string& err );
std::string driver_error( const DriverApi* api, CUresult r );

} // namespace gh
