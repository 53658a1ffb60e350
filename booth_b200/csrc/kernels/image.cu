// image.cu -- the single translation unit behind the sm_100a kernel image.
// nvcc turns it into one cubin that the C shim embeds (image.S) and loads with
// cuModuleLoadData; the same file is what bc_load_kernel is given as a path.
#include "stream.cu"
#include "reduce.cu"
#include "asian.cu"
#include "tile.cu"
#include "canonical.cu"
#include "pipe_probe.cu"
#if __has_include("gemm_tf32x3.cu")
#include "gemm_tf32x3.cu"
#endif
