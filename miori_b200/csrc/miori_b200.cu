// Single translation unit of libmiori_b200.so: the device-side error record and the
// kernels' templates are shared by inclusion, so the library has no relocatable device
// code and every kernel is compiled once for sm_100a.
#include "backend.cu"
#include "ops_api.cu"
#include "gemm_tcgen05.cu"
#include "neighbors.cu"
#include "peers.cu"
