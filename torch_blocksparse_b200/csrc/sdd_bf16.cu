// SDD kernels (mma.sync / FFMA path) instantiated for __nv_bfloat16.
#include "sdd_impl.cuh"
namespace bsp {
template int sdd_mma_t<__nv_bfloat16>(const void*, const void*, void*, int, int, int,
                            int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                            int64_t, const Meta&, cudaStream_t);
}
