// Kernel launch helper: every decode-path kernel is launched with programmatic dependent launch (PDL) enabled, so its
// prologue (barrier init, TMEM allocation, descriptor prefetch, block scheduling) overlaps the tail of the kernel before
// it.  Kernels call pdl_launch_dependents() at entry and pdl_wait() before their first global-memory access; without the
// launch attribute both are no-ops.  FB_PDL=0 in the environment turns the attribute off.
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>

namespace fb {

// Kernel function attributes (dynamic shared-memory limit) belong to a device's context: set them once per device.
struct DeviceOnce {
  bool done[64] = {};
  bool need() {
    int d = 0;
    cudaGetDevice(&d);
    d &= 63;
    if (done[d]) return false;
    done[d] = true;
    return true;
  }
};

// Kernel classes for the FB_PDL bit mask: which launches carry the PDL attribute.  Default: the tensor-core GEMM kernels
// only.  Measured on Llama-3-8B decode (64 x 1024): GEMM-only 5.67 ms/step vs 5.95 without PDL; adding the attention kernel
// (+0.19 ms), its combine (+0.12 ms) or the row kernels (+0.04 ms) each made the step slower -- CTAs of a multi-CTA-per-SM
// grid that become resident while the previous kernel still holds some SMs end up unevenly spread.
enum PdlClass { PDL_GEMM = 1, PDL_ATTN = 2, PDL_COMBINE = 4, PDL_ROW = 8 };
inline bool pdl_enabled(int cls) {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("FB_PDL");
    v = e != nullptr ? std::atoi(e) : PDL_GEMM;
  }
  return (v & cls) != 0;
}

// appends the PDL attribute to attr[n] when enabled; returns the new attribute count
inline int add_pdl_attr(cudaLaunchAttribute* attr, int n) {
  if (!pdl_enabled(PDL_GEMM)) return n;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  return n + 1;
}

// cluster_x = 0: no cluster attribute
template <int CLS = PDL_ROW, typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 0) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled(CLS)) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace fb
