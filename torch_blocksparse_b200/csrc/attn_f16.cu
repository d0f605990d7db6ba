// Fused attention kernels (mma.sync path) instantiated for __half.
#include "attn_impl.cuh"
namespace bsp {
template int attn_fwd_t<__half>(const AttnArgs&, int, int, int, cudaStream_t);
template int attn_bwd_t<__half>(const AttnArgs&, int, int, int, int, cudaStream_t);
}
