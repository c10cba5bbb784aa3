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

// Expert-parallel return path fused into the second GEMM: where does expert-sorted row i go home to?
// xplan is the receiving rank's extended plan (see ep_plan_kernel in moe_ep.cu), back[s] rank s's result
// buffer ([rows of rank s's routed buffer][H] fp16, peer-mapped).
constexpr int kMoeMaxRanks = 16;
struct RowScatter {
  const int* xplan;          // null: no scatter (rows are stored at their sorted position)
  int world, e_loc, ext;
  void* back[kMoeMaxRanks];
};

// Which (source rank, row of that rank's routed buffer) does sorted row i hold?  false = padding.
__device__ __forceinline__ bool ep_locate(const int* xplan, int world, int e_loc, int ext, int i, int& s_out,
                                          int& src_row) {
  const int* seg = xplan + 2 * e_loc;
  const int* cum = xplan + ext;
  const int* src_seg = xplan + ext + e_loc * (world + 1);
  if (i >= seg[e_loc]) return false;
  int e = 0;
  while (e + 1 < e_loc && i >= seg[e + 1]) ++e;
  const int j = i - seg[e];
  if (j >= cum[e * (world + 1) + world]) return false;
  int s = 0;
  while (s + 1 < world && j >= cum[e * (world + 1) + s + 1]) ++s;
  s_out = s;
  src_row = src_seg[e * world + s] + (j - cum[e * (world + 1) + s]);
  return true;
}

#ifdef __CUDACC__
// Wait (at most 2 s) until a peer's arrival word has reached `epoch`; the words only grow, and the comparison is
// wrap-safe.  On giving up the error word is set to 4 ("a peer did not arrive") and the caller carries on.
__device__ __forceinline__ void peer_flag_wait(const unsigned int* flag, unsigned int epoch, int* error_word) {
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (unsigned int it = 0;; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - epoch) >= 0) break;
    if ((it & 0xFF) == 0xFF) {
      uint64_t t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        if (error_word) atomicExch(error_word, 4);
        break;
      }
    }
  }
}
#endif

// h[r, n] = f16(silu(f16(gate)) * f16(up)) for the expert-sorted int8 rows, plus max |h| of every row within
// every 128-column tile: row_absmax[r * moe_absmax_slots(I) + tile] (plain stores, so nothing is zeroed first;
// rows of tiles that are not in use are left untouched).
__host__ __device__ constexpr int moe_absmax_slots(int I) { return (I + 127) / 128; }
int launch_moe_gemm1_swiglu(const void* routed_q, const float* routed_scale, const void* w13_q, const float* w13_scale,
                            int padded_rows, int H, int I, int E, const int* num_tiles_dev, const int* tile_expert,
                            void* h_out, float* row_absmax, int* error_word, cudaStream_t st, int tile_part = -1);

// d[r, :] = f16(acc * scale2[r] * w2_scale[e, :]) for the re-quantised rows.
int launch_moe_gemm2(const void* q2, const float* scale2, const void* w2_q, const float* w2_scale, int padded_rows,
                     int I, int H, int E, const int* num_tiles_dev, const int* tile_expert, void* d_out,
                     int* error_word, cudaStream_t st, const RowScatter* scatter = nullptr, int tile_part = -1);

// tile_part: -1 = every row tile; 0 / 1 = the first / second half of the 256-row tiles in use (the halves are
// split at (tiles + 1) / 2, the same split mp_moe_ep_pull_part / mp_moe_ep_push_part use for rows).
__host__ __device__ constexpr int moe_half_split_rows(int tiles_128) {     // first row of the second half
  return (((tiles_128 + 1) / 2 + 1) / 2) * kMoeSegmentAlign;
}

}  // namespace mp
