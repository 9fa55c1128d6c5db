// Host helper: kernel launches that let the NEXT kernel of the stream begin its prologue before this one has drained
// (programmatic dependent launch).  Every kernel launched through launch_pdl calls pdl_trigger() on entry and
// pdl_wait() before its first access to global memory another kernel may have written or may still read, so the only
// work that overlaps is barrier initialisation, tensor-memory allocation and descriptor prefetch, plus the launch
// latency itself.  ITTAI_PDL=0 in the environment turns the attribute off (plain stream order).
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace ittai {

inline bool pdl_enabled() {
    static const bool on = [] { const char* e = std::getenv("ITTAI_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ittai
