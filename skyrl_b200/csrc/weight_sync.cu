// Trainer -> rollout weight sync as one kernel per source rank: gather / re-layout / push.
//
// The trainer's parameter shards (tensor-parallel slices of fused QKV, gate/up, o-proj and down-proj matrices, or a
// whole replicated model) have to arrive in the generation engines' own layout, which may use a different
// tensor-parallel degree.  Instead of all-gathering every parameter, re-slicing it and copying it into the engine
// (what the reference does: DTensor.full_tensor() per parameter, pack, IPC handle, load_weights), every source rank
// runs this kernel once: it walks a table of 2-D block copies -- "rows x row_bytes from my shard at this stride to
// that engine's buffer at that stride" -- and stores the data straight into the destination GPUs' engine buffers
// with plain 16-byte peer stores over NVLink.  Each byte of the model crosses NVLink exactly once per destination
// and nothing is staged.  An optional fp32 -> bf16 cast covers sources that are fp32 master shards.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

struct CopyDesc {
  const char* src;          // this GPU's memory
  char* dst;                // destination GPU's memory (or this GPU's)
  long long src_stride;     // bytes between rows at the source
  long long dst_stride;     // bytes between rows at the destination
  long long first_item;     // prefix sum of work items before this descriptor
  int rows;
  int vecs_per_row;         // 16-byte vectors of *destination* per row
  int cast_f32;             // 1: source rows are fp32 (32 source bytes per destination vector)
  int pad;
};

constexpr int kVecsPerItem = 2048;  // 32 KB of destination per work item

__global__ void relayout_push_kernel(const CopyDesc* __restrict__ descs, int n_desc, long long n_items) {
  for (long long item = blockIdx.x; item < n_items; item += gridDim.x) {
    // binary search for the descriptor that owns this item
    int lo = 0, hi = n_desc - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (descs[mid].first_item <= item) lo = mid; else hi = mid - 1;
    }
    const CopyDesc d = descs[lo];
    const long long v0 = (item - d.first_item) * kVecsPerItem;
    const long long total = static_cast<long long>(d.rows) * d.vecs_per_row;
    const long long v1 = v0 + kVecsPerItem < total ? v0 + kVecsPerItem : total;
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      const long long r = v / d.vecs_per_row;
      const long long c = v - r * d.vecs_per_row;
      uint4 o;
      if (d.cast_f32) {
        const float4* s = reinterpret_cast<const float4*>(d.src + r * d.src_stride + c * 32);
        const float4 a = s[0], b = s[1];
        o.x = pack_bf16x2(a.x, a.y);
        o.y = pack_bf16x2(a.z, a.w);
        o.z = pack_bf16x2(b.x, b.y);
        o.w = pack_bf16x2(b.z, b.w);
      } else {
        o = *reinterpret_cast<const uint4*>(d.src + r * d.src_stride + c * 16);
      }
      *reinterpret_cast<uint4*>(d.dst + r * d.dst_stride + c * 16) = o;
    }
  }
}

}  // namespace sb

extern "C" {

int sb_relayout_desc_bytes() { return static_cast<int>(sizeof(sb::CopyDesc)); }
int sb_relayout_vecs_per_item() { return sb::kVecsPerItem; }

// descs: device array of n_desc CopyDesc whose first_item fields are the running sum of
// ceil(rows * vecs_per_row / sb_relayout_vecs_per_item()); n_items is the total.
int sb_relayout_push(const void* descs, int n_desc, long long n_items, void* stream) {
  if (n_desc <= 0 || n_items <= 0) return SB_OK;
  if (!descs) return SB_ERR_ARG;
  long long grid = n_items;
  const long long cap = static_cast<long long>(sb::sm_count()) * 8;
  if (grid > cap) grid = cap;
  sb::relayout_push_kernel<<<static_cast<int>(grid), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const sb::CopyDesc*>(descs), n_desc, n_items);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
