// DSD / DDS kernels (mma.sync / FFMA path) instantiated for float.
#include "dsd_impl.cuh"
namespace bsp {
template int dsd_mma_t<float>(const void*, const void*, void*, int, int, int, int64_t, int,
                           int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                           const Meta&, cudaStream_t);
}
