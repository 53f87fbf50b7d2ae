// Parameters of the dense split-KV decode kernel.
#pragma once
#include "common.cuh"

namespace ra {

constexpr int kFdTile = 128;                        // tokens per pipeline stage
constexpr int kFdHalfBytes = kFdTile * 128;         // one [128 tokens][64 dims] swizzled half
constexpr int kFdStageBytes = 4 * kFdHalfBytes;     // K lo, K hi, V lo, V hi = 64 KiB
constexpr int kFdConsumerWarps = 8;                 // 16 tokens of a tile each
constexpr int kFdThreads = 32 * (kFdConsumerWarps + 1);
constexpr int kFdMaxStages = 3;
constexpr int kFdMaxGroup = 8;                      // query heads per kv head

struct FlashParams {
  CUtensorMap kmap, vmap;   // 4-D maps (64-dim boxes, 128-byte swizzle) over K and V
  const __half* q;          // [B,Hq,128]
  float* partials;          // [splits][B*Hq][130]: un-normalised sums, weight, maximum
  unsigned* status;
  int batch, hq, hkv, n_tokens;
  int group;                // hq / hkv
  int kv_per_batch;
  int num_splits, split_len;
  int nstages;
  int num_items;            // batch * hkv * num_splits
  float scale_log2e;
};

size_t flash_decode_smem_bytes(int nstages);
cudaError_t launch_flash_decode(const FlashParams& P, int grid, size_t smem, cudaStream_t stream);

}  // namespace ra
