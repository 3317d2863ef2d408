// Single translation unit of the kernel library: the pieces share one device status word
// and are compiled together so no relocatable device code is needed.
#include <mutex>
#include "host_common.cu"
#include "gemm_tcgen05.cu"
#include "rownorm.cu"
#include "pointwise.cu"
#include "mla_decode.cu"
#include "allreduce.cu"
#include "allgather.cu"
