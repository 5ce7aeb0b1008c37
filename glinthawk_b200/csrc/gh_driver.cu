#include "gh_driver.hh"

#include <mutex>

namespace gh {

namespace {

DriverApi g_api;
bool g_ok = false;
std::string g_err;
std::once_flag g_once;

template<typename F>
bool resolve( F& slot, const char* name )
{
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  const cudaError_t e = cudaGetDriverEntryPoint( name, &fn, cudaEnableDefault, &q );
  if ( e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr ) {
    g_err = std::string( "cannot resolve driver entry point " ) + name + ": "
            + ( e != cudaSuccess ? cudaGetErrorString( e ) : "not available" );
    (void)cudaGetLastError();
    return false;
  }
  slot = reinterpret_cast<F>( fn );
  return true;
}

void resolve_all()
{
  g_ok = resolve( g_api.MemAddressReserve, "cuMemAddressReserve" ) && resolve( g_api.MemAddressFree, "cuMemAddressFree" )
         && resolve( g_api.MemCreate, "cuMemCreate" ) && resolve( g_api.MemRelease, "cuMemRelease" )
         && resolve( g_api.MemMap, "cuMemMap" ) && resolve( g_api.MemUnmap, "cuMemUnmap" )
         && resolve( g_api.MemSetAccess, "cuMemSetAccess" )
         && resolve( g_api.MemGetAllocationGranularity, "cuMemGetAllocationGranularity" )
         && resolve( g_api.TensorMapEncodeTiled, "cuTensorMapEncodeTiled" )
         && resolve( g_api.GetErrorString, "cuGetErrorString" );
}

} // namespace

const DriverApi* driver_api( std::string& err )
{
  std::call_once( g_once, resolve_all );
  if ( !g_ok ) {
    err = g_err;
    return nullptr;
  }
  return &g_api;
}

std::string driver_error( const DriverApi* api, CUresult r )
{
  const char* s = nullptr;
  if ( api != nullptr && api->GetErrorString != nullptr && api->GetErrorString( r, &s ) == CUDA_SUCCESS && s != nullptr )
    return s;
  return "CUresult " + std::to_string( static_cast<int>( r ) );
}

} // namespace gh
