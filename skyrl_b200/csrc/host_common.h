// Host-side helpers shared by the kernel translation units: error codes, the
// driver entry point for tensor-map encoding and a small tensor-map cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_OK 0
#define SB_ERR_ARG 1        // unsupported shape / alignment
#define SB_ERR_CUDA 2       // a CUDA runtime call failed
#define SB_ERR_TMAP 3       // tensor-map encode failed
#define SB_ERR_TOO_LARGE 4  // size beyond a stated maximum

namespace sb {

// 2-D bf16 row-major tensor [rows, cols] with row stride `ld` elements; box is
// [box_rows, 64] elements with the 128-byte swizzle. Returns nullptr on failure.
const CUtensorMap* get_tmap_bf16_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                    uint32_t box_cols = 64);
// 3-D bf16 tensor [d2, d1, d0] (d0 innermost) with byte strides for d1 and d2.
const CUtensorMap* get_tmap_bf16_3d(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                    uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2);

int* device_status_ptr();  // per-device status word (device address); nullptr when it cannot be resolved
int device_index();        // current CUDA device clamped to [0, 63]: index of per-device "configured once" tables
int sm_count();
bool pdl_enabled();  // programmatic dependent launch of the decode-chain kernels (SB_PDL=0 turns it off)

#ifdef __CUDACC__
// Programmatic dependent launch: a kernel started with the attribute below may begin (block scheduling, prologue)
// while its predecessor in the stream is still draining; ``pdl_wait`` blocks until the predecessor grid has completed
// and its writes are visible, so every access to memory that a predecessor may have produced -- or may still be
// reading -- comes after it.  Without the launch attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace sb
