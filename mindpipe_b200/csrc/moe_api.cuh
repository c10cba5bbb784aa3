// Launchers shared between the MoE chain (moe.cu) and the grouped tensor-core GEMMs (w8a8_gemm.cu).
#pragma once

#include <cuda_runtime.h>

namespace mp {

// Layout of expert-sorted rows: the plan counts tiles in units of 128 rows, and every expert's
// segment starts at a multiple of 256 rows (an even number of units), so that both the 128-row
// single-CTA tiles and the 256-row CTA-pair tiles of the grouped GEMMs stay inside one expert.
constexpr int kMoeTileRows = 128;
constexpr int kMoeSegmentAlign = 256;
__host__ __device__ constexpr int moe_segment_tiles(int rows) {
  return (rows + kMoeSegmentAlign - 1) / kMoeSegmentAlign * (kMoeSegmentAlign / kMoeTileRows);
}

// h[r, n] = f16(silu(f16(gate)) * f16(up)) for the expert-sorted int8 rows, plus per-row max |h|.
int launch_moe_gemm1_swiglu(const void* routed_q, const float* routed_scale, const void* w13_q, const float* w13_scale,
                            int padded_rows, int H, int I, int E, const int* num_tiles_dev, const int* tile_expert,
                            void* h_out, unsigned int* row_absmax, int* error_word, cudaStream_t st);

// d[r, :] = f16(acc * scale2[r] * w2_scale[e, :]) for the re-quantised rows.
int launch_moe_gemm2(const void* q2, const float* scale2, const void* w2_q, const float* w2_scale, int padded_rows,
                     int I, int H, int E, const int* num_tiles_dev, const int* tile_expert, void* d_out,
                     int* error_word, cudaStream_t st);

}  // namespace mp
