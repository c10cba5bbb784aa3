// W8A8 GEMM on the 5th-generation tensor cores: int8 x int8 -> int32 in TMEM,
// then a scale epilogue.  One persistent CTA per SM, warp specialised:
//
//   warp 0     TMA producer: 128-byte-swizzled [128 x 128 B] activation tile and
//              [BN x 128 B] weight tile per stage, multi-stage mbarrier ring
//   warp 1     MMA issuer: tcgen05.mma kind::i8 (M=128, N=BN, K=32), four per
//              stage; tcgen05.commit releases the stage / publishes the tile
//   warps 2-5  epilogue: tcgen05.ld the int32 accumulators (TMEM is double
//              buffered, so this overlaps the next tile's main loop), apply
//              acc * s_token[m] * s_channel[n] (+bias) and store
//
// Both operands are K-major: activations q[M,K] and weights w[N,K] (the
// reference's [out, in] layout).  The same kernel serves three uses, chosen
// by the epilogue: fp16 output (the npu_quant_matmul role,
// acceleration/runtime_patches/vllm_ascend.patch:4007-4015), raw int32
// accumulators (its output_dtype=int32 passthrough,
// acceleration/runtime_patches/vllm.patch:756-760), and the MoE gate/up GEMM
// with the SwiGLU epilogue.  In grouped (MoE) mode every 128-row tile of the
// expert-sorted activations belongs to one expert, whose weight rows start at
// expert * rows_per_expert (segments are 256-row aligned, so a CTA pair's 256-row
// tile belongs to one expert as well).
//
// Every mbarrier wait is bounded; on a timeout the block records an error
// word, lets its copies land, frees its TMEM and returns.
#include "common.cuh"
#include "tc.cuh"
#include "moe_api.cuh"

namespace mp {

using namespace tc;

constexpr int kBM = 128;
constexpr int kBK = 128;      // int8 elements (= bytes) of K per stage
constexpr int kUmmaK = 32;    // K of one kind::i8 instruction

enum : int { EPI_F16 = 0, EPI_I32 = 1, EPI_SWIGLU = 2, EPI_AFFINE = 3 };   // AFFINE: unsigned codes with zero points

struct GemmParams {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int k_split;                 // > 1: a tile's K range is cut into this many work items of kb_per_split k-blocks,
  int kb_per_split;            //      whose raw int32 partial tiles go to `partial` ([k_split][M][N])
  int* partial;
  RowScatter scatter;          // expert-parallel GEMM2: rows are stored at home (peer memory), see moe_api.cuh
  int group_m;                 // tile order: groups of this many M tiles are swept across all of N before the next group
  int tile_part;               // grouped: -1 = all row tiles, 0 / 1 = the first / second half of them (two launches whose
                               //          neighbours -- the pull of the other half, the push of this one -- overlap them)
  const int* m_tiles_dev;      // grouped: number of 128-row tiles in use (device side)
  const int* tile_expert;      // grouped: expert of each 128-row tile
  int b_rows_per_expert;       // grouped: weight rows per expert (2I for gate/up, H for down)
  int up_row_offset;           // SwiGLU: rows between a gate row and its up row (I)
  const float* a_scale;        // [M] per-token scales
  const float* b_scale;        // per-channel scales, indexed like the weight rows
  const __half* bias;          // [N] or null
  void* out;                   // f16 [M,N] or int32 [M,N]
  float* row_absmax;           // SwiGLU: max |h| of every (row, 128-column tile), [rows][n_tiles]
  const float* a_zero;         // AFFINE: per-token zero points (integer valued) and code row sums
  const int* a_rowsum;
  const float* b_zero;         // AFFINE: per-channel zero points and code row sums
  const int* b_rowsum;
  int* error_word;
};

// PAIR: two CTAs (a cluster of 2) share each MMA -- a 256 x BN tile, 128 rows of A and of the
// accumulator per CTA, and each CTA stages only its half of the BN weight rows.  Per CTA and k-block
// the shared memory then carries 16 KB (A) + BN/2 x 128 B (B) in and the same out, instead of
// 16 KB + BN x 128 B: at BN = 256 that is 64 KB rather than 96 KB per 512 tensor cycles, which takes
// the kernel off the 128 B/clk shared-memory limit that held the single-CTA form at ~70 % tensor use.
template <int BN, bool PAIR = false>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * kBK;
  static constexpr int kStages = PAIR ? (BN == 256 ? 6 : 8) : (BN == 256 ? 4 : 6);
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kBarBytes = 256;
  static constexpr int kScaleBytes = 3 * 4 * 256 * 4;   // per epilogue warp: 256 channel scales (+ zero points, row sums)
  static constexpr size_t kSmem = 1024 + (size_t)kStages * (kABytes + kBBytes) + kBarBytes + kScaleBytes;
};

// acc * s_token * s_channel (+ bias) with every fp32 operation rounded on its own (no contraction into
// an fma), so that the GEMM epilogue and the split-K reduce kernel produce the same bits.
__device__ __forceinline__ float scaled_output(int acc, float s_token, float s_channel) {
  return __fmul_rn(__fmul_rn(static_cast<float>(acc), s_token), s_channel);
}

// Tile order.  Concurrent CTAs work on consecutive tile numbers; a group of `group_m` M tiles is swept
// over all N tiles before the next group starts (M fastest inside the group).  The activation rows of
// one group (a few MB) and the weight tiles of a handful of N tiles are then the whole working set
// of a wave, so both operands come from HBM about once even when neither matrix fits in L2 -- in the
// MoE GEMMs a plain M-fastest order re-read the activations once per weight tile column (6 GB of DRAM
// reads for 1 GB of operands).
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int& m_tile, int& n_tile) {
  const int per_group = group_m * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int gsize = min(group_m, m_tiles - first_m);
  const int in_group = tile - group * per_group;
  m_tile = first_m + in_group % gsize;
  n_tile = in_group / gsize;
}

// Grouped mode: the tile groups follow the experts.  A group is the run of row tiles of one expert (cut evenly when
// it is longer than two default groups), swept over all column tiles before the next group starts, so an expert's
// weights stream from HBM once.  With fixed groups of eight row tiles a group straddled two experts whenever a
// segment was not a multiple of eight tiles, and the second expert's weights were streamed again for the
// straggler tiles (MoE GEMM1: 2.5 GB of DRAM reads for 1.0 GB of operands).
constexpr int kMaxTileGroups = 256;

__device__ __forceinline__ void tile_coords_grouped(int tile, int n_tiles, const int* g_first, int groups, int& m_tile,
                                                    int& n_tile) {
  int g = 0;
  while (g + 1 < groups && tile >= g_first[g + 1] * n_tiles) ++g;
  const int first = g_first[g], gsize = g_first[g + 1] - first;
  const int in_group = tile - first * n_tiles;
  m_tile = first + in_group % gsize;
  n_tile = in_group / gsize;
}

template <int BN, int EPI, bool PAIR>
__global__ void __launch_bounds__(192, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN, PAIR>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = smem;
  unsigned char* sB = smem + STAGES * Cfg::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * Cfg::kBBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_scales = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + Cfg::kBarBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // PAIR: rank 0 of the cluster leads (issues the MMAs, owns the "full" and "accumulator free"
  // barriers); both CTAs own a "stage empty" and an "accumulator full" barrier that the leader's
  // commits arrive on.  Every WAIT in the kernel is on a barrier of the waiting CTA.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, PAIR ? 8 : 4);     // one arrival per epilogue warp (of both CTAs)
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) {            // the peer's barriers exist before anything signals them
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // everything above touched only this block's shared and tensor memory: under programmatic dependent launch it
  // ran beside the previous kernel's tail; from here on that kernel's results are read
  chain_wait();
  chain_release();

  // tiles are 128 (PAIR: 256) rows of the activations; the grouped plan counts 128-row units
  const int m_units = p.m_tiles_dev ? min(*p.m_tiles_dev, p.m_tiles) : p.m_tiles;
  const int m_tiles_all = PAIR ? (m_units + 1) / 2 : m_units;
  // a launch may take one half of the row tiles (grouped mode): [m_lo, m_lo + m_tiles)
  const int m_mid = (m_tiles_all + 1) / 2;
  const int m_lo = p.tile_part == 1 ? m_mid : 0;
  const int m_tiles = p.tile_part < 0 ? m_tiles_all : (p.tile_part == 0 ? m_mid : m_tiles_all - m_mid);
  const int total = m_tiles * p.n_tiles * p.k_split;           // work items: (tile, K slice)
  const int first_tile = PAIR ? blockIdx.x >> 1 : blockIdx.x;
  const int tile_step = PAIR ? gridDim.x >> 1 : gridDim.x;
  constexpr int kRowsPerTile = PAIR ? 2 * kBM : kBM;
  __shared__ int s_gfirst[kMaxTileGroups + 1];
  __shared__ int s_groups;
  const bool grouped = p.tile_expert != nullptr;
  if (grouped) {
    if (threadIdx.x == 0) {
      int g = 0, i = 0;
      while (i < m_tiles && g < kMaxTileGroups) {      // indices relative to m_lo
        const int e = p.tile_expert[PAIR ? 2 * (m_lo + i) : m_lo + i];
        int j = i + 1;
        while (j < m_tiles && p.tile_expert[PAIR ? 2 * (m_lo + j) : m_lo + j] == e) ++j;
        const int len = j - i, parts = (len + 2 * p.group_m - 1) / (2 * p.group_m);
        for (int q = 0; q < parts && g < kMaxTileGroups; ++q) s_gfirst[g++] = i + (len * q) / parts;
        i = j;
      }
      s_gfirst[g] = m_tiles;               // (a table that filled up leaves the rest to its last group)
      s_groups = g;
    }
    __syncthreads();
  }
  auto coords = [&](int tile, int& m_tile, int& n_tile) {
    if (grouped) {
      tile_coords_grouped(tile, p.n_tiles, s_gfirst, s_groups, m_tile, n_tile);
      m_tile += m_lo;
    } else {
      tile_coords(tile, m_tiles, p.n_tiles, p.group_m, m_tile, n_tile);
    }
  };

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = first_tile; ok && work < total; work += tile_step) {
        const int tile = work / p.k_split;
        const int kb0 = (work - tile * p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        int m_tile, n_tile;
        coords(tile, m_tile, n_tile);
        const int m0 = m_tile * kRowsPerTile + static_cast<int>(rank) * kBM;
        const int e_row0 = p.tile_expert ? p.tile_expert[PAIR ? 2 * m_tile : m_tile] * p.b_rows_per_expert : 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag)) { ok = false; break; }
          if (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier
            const uint32_t full = map_to_cta(full0 + 8 * stage, 0);
            if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * (Cfg::kABytes + Cfg::kBBytes));
            tma_load_2d_pair(smem_u32(sA + stage * Cfg::kABytes), &tmap_a, full, kb * kBK, m0);
            // this CTA's half of the tile's weight rows; with SwiGLU the halves are the gate rows
            // (accumulator columns [0,128)) and the matching up rows (columns [128,256))
            const int b_row = EPI == EPI_SWIGLU
                                  ? e_row0 + (rank ? p.up_row_offset : 0) + n_tile * 128
                                  : e_row0 + n_tile * BN + static_cast<int>(rank) * (BN / 2);
            tma_load_2d_pair(smem_u32(sB + stage * Cfg::kBBytes), &tmap_b, full, kb * kBK, b_row);
          } else {
            const uint32_t full = full0 + 8 * stage;
            mbar_arrive_expect_tx(full, Cfg::kABytes + Cfg::kBBytes);
            tma_load_2d(smem_u32(sA + stage * Cfg::kABytes), &tmap_a, full, kb * kBK, m0);
            if (EPI == EPI_SWIGLU) {
              // gate rows then the matching up rows: the tile's columns [0,128) and [128,256)
              const uint32_t dst = smem_u32(sB + stage * Cfg::kBBytes);
              tma_load_2d(dst, &tmap_b, full, kb * kBK, e_row0 + n_tile * 128);
              tma_load_2d(dst + 128 * kBK, &tmap_b, full, kb * kBK, e_row0 + p.up_row_offset + n_tile * 128);
            } else {
              tma_load_2d(smem_u32(sB + stage * Cfg::kBBytes), &tmap_b, full, kb * kBK, e_row0 + n_tile * BN);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one()) {
      constexpr uint32_t idesc =
          umma_idesc(kIdescDFormatS32 | (EPI == EPI_AFFINE ? kIdescABFormatU8 : kIdescABFormatS8), kRowsPerTile, BN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int work = first_tile; ok && work < total; work += tile_step) {
        const int kb0 = (work % p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        if (!mbar_wait(tempty0 + 8 * buf, buf_phase ^ 1, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t a_desc = umma_desc_k_sw128(smem_u32(sA + stage * Cfg::kABytes));
          const uint64_t b_desc = umma_desc_k_sw128(smem_u32(sB + stage * Cfg::kBBytes));
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            // advancing K by 32 bytes inside the 128-byte swizzle row: +2 in 16-byte address units
            if (PAIR) {
              umma_i8_pair(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb != kb0 || kk != 0));
            } else {
              umma_i8(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb != kb0 || kk != 0));
            }
          }
          if (PAIR) {                      // release the stage in both CTAs
            umma_commit_pair(empty0 + 8 * stage);
            umma_commit_pair(map_to_cta(empty0 + 8 * stage, 1));
          } else {
            umma_commit(empty0 + 8 * stage);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) {                        // publish the accumulator halves to both CTAs' epilogues
          umma_commit_pair(tfull0 + 8 * buf);
          umma_commit_pair(map_to_cta(tfull0 + 8 * buf, 1));
        } else {
          umma_commit(tfull0 + 8 * buf);
        }
        if (++buf == 2) { buf = 0; buf_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;               // TMEM lanes [32*quarter, +32) belong to this warp
    float* my_scales = s_scales + quarter * 768; // this warp's copy of the tile's channel scales
    float* my_zero = my_scales + 256;             // AFFINE: channel zero points ...
    int* my_wsum = reinterpret_cast<int*>(my_scales + 512);   // ... and channel code sums
    int buf = 0;
    uint32_t buf_phase = 0;
    const uint32_t tempty_leader0 = PAIR ? map_to_cta(tempty0, 0) : tempty0;
    for (int work = first_tile; work < total; work += tile_step) {
      const int tile = work / p.k_split, split = work - tile * p.k_split;
      int m_tile, n_tile;
      coords(tile, m_tile, n_tile);
      const int e_row0 = p.tile_expert ? p.tile_expert[PAIR ? 2 * m_tile : m_tile] * p.b_rows_per_expert : 0;
      // channel scales of this tile -> shared memory (each warp keeps its own copy: no cross-warp barrier)
      if (EPI != EPI_I32) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = lane + 32 * i;             // column of the accumulator tile
          int n, src;
          if (EPI == EPI_SWIGLU) {
            n = n_tile * 128 + (c & 127);
            src = e_row0 + (c >= 128 ? p.up_row_offset : 0) + n;
          } else {
            n = n_tile * BN + c;
            src = e_row0 + n;
          }
          my_scales[c] = (c < BN && n < p.N) ? __ldg(p.b_scale + src) : 0.0f;
          if (EPI == EPI_AFFINE) {
            my_zero[c] = (c < BN && n < p.N) ? __ldg(p.b_zero + src) : 0.0f;
            my_wsum[c] = (c < BN && n < p.N) ? __ldg(p.b_rowsum + src) : 0;
          }
        }
        __syncwarp();
      }
      // the whole warp takes the same way out: the TMEM loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, buf_phase, abort_flag))) break;
      tcgen05_fence_after();
      const int row = m_tile * kRowsPerTile + static_cast<int>(rank) * kBM + quarter * 32 + lane;
      bool row_ok = row < p.M;
      // where this row's fp16 output goes: its sorted position, or (expert-parallel GEMM2) straight home
      // into the source rank's result buffer over NVLink; padding rows are not stored at all
      __half* out_row = static_cast<__half*>(p.out) + (size_t)row * p.N;
      if (EPI == EPI_F16 && p.scatter.xplan) {
        int home_rank = 0, home_row = 0;
        row_ok = row_ok && ep_locate(p.scatter.xplan, p.scatter.world, p.scatter.e_loc, p.scatter.ext, row, home_rank,
                                     home_row);
        out_row = static_cast<__half*>(p.scatter.back[home_rank]) + (size_t)home_row * p.N;
      }
      const float sa = (EPI != EPI_I32 && row_ok) ? p.a_scale[row] : 0.0f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      if (EPI == EPI_SWIGLU) {
        const int n0 = n_tile * 128;
        float hmax = 0.0f;
        __half* out = static_cast<__half*>(p.out);
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c0, rg);
          tmem_ld_32x32(taddr + 128 + c0, ru);
          tmem_ld_wait();
          uint32_t hp[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            __half h2v[2];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
              const float sg = my_scales[c0 + j + jj], su = my_scales[128 + c0 + j + jj];
              // the reference rounds gate/up (F.linear output), silu(gate) and the product to fp16
              const __half g16 = f2h(static_cast<float>(static_cast<int>(rg[j + jj])) * sa * sg);
              const __half u16 = f2h(static_cast<float>(static_cast<int>(ru[j + jj])) * sa * su);
              const float gf = h2f(g16);
              // silu in fp32 with the hardware exp2 / reciprocal: the result is rounded to fp16 right
              // away (as the reference does), which hides their ~2 ulp fp32 error
              const __half s16 = f2h(__fdividef(gf, 1.0f + __expf(-gf)));
              const __half h16 = hmul_t(s16, u16);
              h2v[jj] = h16;
              hmax = fmaxf(hmax, fabsf(h2f(h16)));
            }
            hp[j >> 1] = h2_as_u32(__halves2half2(h2v[0], h2v[1]));
          }
          if (row_ok) {
            __half* dst = out + (size_t)row * p.N + n0 + c0;
            if (n0 + c0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
              for (int v = 0; v < 4; ++v)
                reinterpret_cast<uint4*>(dst)[v] = make_uint4(hp[4 * v], hp[4 * v + 1], hp[4 * v + 2], hp[4 * v + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {                   // static indices keep hp in registers
                const uint32_t w = hp[j >> 1];
                if (n0 + c0 + j < p.N)
                  dst[j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
              }
            }
          }
        }
        if (row_ok) p.row_absmax[(size_t)row * p.n_tiles + n_tile] = hmax;   // one slot per (row, column tile): no atomics, nothing to zero
      } else {
        const int n0 = n_tile * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          if (EPI == EPI_I32 || p.k_split > 1) {
            // raw accumulators: the int32 output, or this K slice's partial tile (a second kernel adds the
            // slices -- integer sums, so the split changes no bit -- and applies the scales)
            if (row_ok) {
              int* dst = (p.k_split > 1 ? p.partial + (size_t)split * p.M * p.N : static_cast<int*>(p.out)) +
                         (size_t)row * p.N + n0 + c0;
              if (n0 + c0 + 32 <= p.N && (p.N % 4) == 0) {
#pragma unroll
                for (int v = 0; v < 8; ++v)
                  reinterpret_cast<uint4*>(dst)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n0 + c0 + j < p.N) dst[j] = static_cast<int>(r[j]);
              }
            }
          } else {
            uint32_t hp[16];
            long long zx = 0, xs = 0;
            if (EPI == EPI_AFFINE && row_ok) {
              zx = static_cast<long long>(p.a_zero[row]);
              xs = p.a_rowsum[row];
            }
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float v0, v1;
              if (EPI == EPI_AFFINE) {
                // sum (qx - zx)(qw - zw) = acc - zw * sum(qx) - zx * sum(qw) + K * zx * zw, exactly, in int64
                const long long zw0 = static_cast<long long>(my_zero[c0 + j]), zw1 = static_cast<long long>(my_zero[c0 + j + 1]);
                const long long t0 = static_cast<long long>(r[j]) - zw0 * xs - zx * my_wsum[c0 + j] + (long long)p.K * zx * zw0;
                const long long t1 = static_cast<long long>(r[j + 1]) - zw1 * xs - zx * my_wsum[c0 + j + 1] + (long long)p.K * zx * zw1;
                v0 = static_cast<float>(t0) * sa * my_scales[c0 + j];
                v1 = static_cast<float>(t1) * sa * my_scales[c0 + j + 1];
              } else {
                v0 = scaled_output(static_cast<int>(r[j]), sa, my_scales[c0 + j]);
                v1 = scaled_output(static_cast<int>(r[j + 1]), sa, my_scales[c0 + j + 1]);
              }
              if (p.bias) {
                if (n0 + c0 + j < p.N) v0 = __fadd_rn(v0, h2f(p.bias[n0 + c0 + j]));
                if (n0 + c0 + j + 1 < p.N) v1 = __fadd_rn(v1, h2f(p.bias[n0 + c0 + j + 1]));
              }
              hp[j >> 1] = h2_as_u32(__floats2half2_rn(v0, v1));
            }
            if (row_ok) {
              __half* dst = out_row + n0 + c0;
              if (n0 + c0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                  reinterpret_cast<uint4*>(dst)[v] = make_uint4(hp[4 * v], hp[4 * v + 1], hp[4 * v + 2], hp[4 * v + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {                 // static indices keep hp in registers
                  const uint32_t w = hp[j >> 1];
                  if (n0 + c0 + j < p.N)
                    dst[j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
                }
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) {
          mbar_arrive_cluster(tempty_leader0 + 8 * buf);
        } else {
          mbar_arrive(tempty0 + 8 * buf);
        }
      }
      if (++buf == 2) { buf = 0; buf_phase ^= 1; }
    }
  }

  __syncthreads();
  if (PAIR) {
    // a CTA that gave up tells its peer (whose waits poll the flag) before both meet at the cluster
    // barrier; the peer cannot have left yet, so its shared memory is still there
    if (*abort_flag && threadIdx.x == 0) st_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u), 1u);
    cluster_arrive();       // the leader's MMAs read the peer's shared memory: nobody leaves early
    cluster_wait();
  }
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.error_word) atomicExch(p.error_word, 1);
    // give copies still in flight time to land before the shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    if (PAIR) {
      tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    } else {
      tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
    g_last_cuda_error = static_cast<int>(e != cudaSuccess ? e : cudaErrorUnknown);
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                         uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                         bool swizzle_128b) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return MP_ERR_CUDA;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = 100000 + static_cast<int>(r);
    return MP_ERR_CUDA;
  }
  return MP_OK;
}

// Sum of the K slices' int32 partial tiles, then the epilogue of the unsplit kernel with the same
// operations in the same order (so a split changes no output bit): f16(float(acc) * s_token * s_channel (+ bias)),
// or the raw int32 sum.
template <bool F16OUT>
__global__ void __launch_bounds__(256)
w8a8_splitk_reduce_kernel(const int* __restrict__ partial, int k_split, int M, int N, const float* __restrict__ a_scale,
                          const float* __restrict__ b_scale, const __half* __restrict__ bias, void* __restrict__ out) {
  chain_wait();
  chain_release();
  const int quads = N >> 2;
  const size_t slice = (size_t)M * N;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += gridDim.x * blockDim.x) {
    const int m = i / quads, n = (i - m * quads) << 2;
    int4 acc = make_int4(0, 0, 0, 0);
    for (int s = 0; s < k_split; ++s) {
      const int4 v = *reinterpret_cast<const int4*>(partial + s * slice + (size_t)m * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (F16OUT) {
      const float sa = a_scale[m];
      float v0 = scaled_output(acc.x, sa, b_scale[n]), v1 = scaled_output(acc.y, sa, b_scale[n + 1]);
      float v2 = scaled_output(acc.z, sa, b_scale[n + 2]), v3 = scaled_output(acc.w, sa, b_scale[n + 3]);
      if (bias) {
        v0 = __fadd_rn(v0, h2f(bias[n])); v1 = __fadd_rn(v1, h2f(bias[n + 1]));
        v2 = __fadd_rn(v2, h2f(bias[n + 2])); v3 = __fadd_rn(v3, h2f(bias[n + 3]));
      }
      const __half2 lo = __floats2half2_rn(v0, v1), hi = __floats2half2_rn(v2, v3);
      *reinterpret_cast<uint2*>(static_cast<__half*>(out) + (size_t)m * N + n) = make_uint2(h2_as_u32(lo), h2_as_u32(hi));
    } else {
      *reinterpret_cast<int4*>(static_cast<int*>(out) + (size_t)m * N + n) = acc;
    }
  }
}

struct GemmCall {
  int k_split = 1; int* partial = nullptr;
  const RowScatter* scatter = nullptr;
  const float* a_zero = nullptr; const int* a_rowsum = nullptr; const float* b_zero = nullptr; const int* b_rowsum = nullptr;
  const void* a; const void* b;
  int M, N, K;
  int a_rows;                 // rows of the activation buffer (>= M; padded in grouped mode)
  int b_rows_total;           // rows of the weight buffer
  const float* a_scale; const float* b_scale; const __half* bias;
  void* out;
  const int* m_tiles_dev; const int* tile_expert; int b_rows_per_expert; int up_row_offset;
  float* row_absmax;
  int* error_word;
  int tile_part = -1;
};

template <int BN, int EPI, bool PAIR = false>
static int launch_gemm(const GemmCall& c, cudaStream_t st) {
  using Cfg = GemmCfg<BN, PAIR>;
  CUtensorMap ta, tb;
  int rc = encode_tensor_map_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.a, (uint64_t)c.K, (uint64_t)c.a_rows,
                                (uint64_t)c.K, kBK, kBM);
  if (rc != MP_OK) return rc;
  rc = encode_tensor_map_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.b, (uint64_t)c.K, (uint64_t)c.b_rows_total,
                            (uint64_t)c.K, kBK, PAIR ? BN / 2 : (EPI == EPI_SWIGLU ? 128 : BN));
  if (rc != MP_OK) return rc;
  GemmParams p{};
  p.M = c.M; p.N = c.N; p.K = c.K;
  p.m_tiles = (c.a_rows + kBM - 1) / kBM;
  p.n_tiles = (c.N + (EPI == EPI_SWIGLU ? 128 : BN) - 1) / (EPI == EPI_SWIGLU ? 128 : BN);
  p.k_blocks = (c.K + kBK - 1) / kBK;
  p.m_tiles_dev = c.m_tiles_dev; p.tile_expert = c.tile_expert;
  p.b_rows_per_expert = c.b_rows_per_expert; p.up_row_offset = c.up_row_offset;
  p.a_scale = c.a_scale; p.b_scale = c.b_scale; p.bias = c.bias; p.out = c.out;
  p.row_absmax = c.row_absmax; p.error_word = c.error_word;
  p.group_m = PAIR ? 8 : 16;            // 2048 activation rows per group
  p.tile_part = c.m_tiles_dev ? c.tile_part : -1;
  p.k_split = c.k_split > 1 ? c.k_split : 1;
  p.kb_per_split = (p.k_blocks + p.k_split - 1) / p.k_split;
  p.partial = c.partial;
  if (c.scatter) p.scatter = *c.scatter;
  p.a_zero = c.a_zero; p.a_rowsum = c.a_rowsum; p.b_zero = c.b_zero; p.b_rowsum = c.b_rowsum;
  auto kern = w8a8_gemm_kernel<BN, EPI, PAIR>;
  static thread_local int configured_device = -1;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmem));
    configured_device = device;
  }
  if (PAIR) {
    // one cluster of two CTAs per 256-row tile in flight: 74 pairs fill the 148 SMs
    const long long total = (long long)((p.m_tiles + 1) / 2) * p.n_tiles;
    const int pairs = (int)(total < kSmCount / 2 ? total : kSmCount / 2);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = decode_programmatic_launch() ? 2 : 1;
    MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
    return MP_OK;
  }
  const long long total = (long long)p.m_tiles * p.n_tiles * p.k_split;
  const int grid = (int)(total < kSmCount ? total : kSmCount);
  return launch_chained(kern, dim3(grid), dim3(192), Cfg::kSmem, st, ta, tb, p);
}

// Few output tiles (decode and small batches: the GEMM is a weight stream, and a CTA sustains only
// ~130 GB/s on its own): cut K until about one work item per SM exists.  Needs N % 4 == 0.
static int w8a8_k_split(int M, int N, int K) {
  if (N % 4 != 0 || N <= 128) return 1;
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  if (tiles256 >= kSmCount) return 1;                       // the 128 x 256 form fills the machine
  const int tiles = ((M + 127) / 128) * ((N + 127) / 128);  // 128 x 128 tiles are used below that
  const int k_blocks = (K + kBK - 1) / kBK;
  int ks = kSmCount / tiles;
  if (ks > k_blocks / 4) ks = k_blocks / 4;
  if (ks > 16) ks = 16;
  if (ks < 2) return 1;
  const int per = (k_blocks + ks - 1) / ks;
  return (k_blocks + per - 1) / per;                        // no empty slice
}

template <bool F16OUT>
static int launch_splitk_reduce(const GemmCall& c, cudaStream_t st) {
  int blocks = (c.M * (c.N / 4) + 255) / 256;
  if (blocks > 2 * kSmCount) blocks = 2 * kSmCount;
  return launch_chained(w8a8_splitk_reduce_kernel<F16OUT>, dim3(blocks), dim3(256), 0, st, c.partial, c.k_split, c.M, c.N,
                        c.a_scale, c.b_scale, c.bias, c.out);
}

// The CTA-pair form pays once there are enough 256-row tiles to occupy the 74 pairs.
static bool use_pair(int M, int N) {
  return (long long)((M + 255) / 256) * ((N + 255) / 256) >= kSmCount / 2 && N > 128;
}

static int check_gemm_args(const void* a, const void* b, void* out, int M, int N, int K) {
  if (!a || !b || !out || M <= 0 || N <= 0 || K <= 0) return MP_ERR_INVALID_ARG;
  if (K % 16 != 0) return MP_ERR_UNSUPPORTED;       // TMA needs 16-byte row pitches
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(out, 16)) return MP_ERR_ALIGNMENT;
  return MP_OK;
}

// Grouped GEMMs of the MoE expert chain (declared in moe_api.cuh).
int launch_moe_gemm1_swiglu(const void* routed_q, const float* routed_scale, const void* w13_q, const float* w13_scale,
                            int padded_rows, int H, int I, int E, const int* num_tiles_dev, const int* tile_expert,
                            void* h_out, float* row_absmax, int* error_word, cudaStream_t st, int tile_part) {
  GemmCall c{};
  c.a = routed_q; c.b = w13_q; c.M = padded_rows; c.N = I; c.K = H; c.a_rows = padded_rows;
  c.b_rows_total = E * 2 * I;
  c.a_scale = routed_scale; c.b_scale = w13_scale; c.out = h_out;
  c.m_tiles_dev = num_tiles_dev; c.tile_expert = tile_expert; c.b_rows_per_expert = 2 * I; c.up_row_offset = I;
  c.row_absmax = row_absmax; c.error_word = error_word;
  c.tile_part = tile_part;
  return launch_gemm<256, EPI_SWIGLU, true>(c, st);   // expert segments are 256-row aligned: pair tiles fit
}

int launch_moe_gemm2(const void* q2, const float* scale2, const void* w2_q, const float* w2_scale, int padded_rows,
                     int I, int H, int E, const int* num_tiles_dev, const int* tile_expert, void* d_out,
                     int* error_word, cudaStream_t st, const RowScatter* scatter, int tile_part) {
  GemmCall c{};
  c.a = q2; c.b = w2_q; c.M = padded_rows; c.N = H; c.K = I; c.a_rows = padded_rows; c.b_rows_total = E * H;
  c.a_scale = scale2; c.b_scale = w2_scale; c.out = d_out;
  c.m_tiles_dev = num_tiles_dev; c.tile_expert = tile_expert; c.b_rows_per_expert = H;
  c.error_word = error_word;
  c.scatter = scatter;
  c.tile_part = tile_part;
  return launch_gemm<256, EPI_F16, true>(c, st);
}

}  // namespace mp

using namespace mp;

extern "C" size_t mp_w8a8_gemm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || use_pair(M, N)) return 0;
  const int ks = w8a8_k_split(M, N, K);
  return ks > 1 ? (size_t)ks * M * N * sizeof(int) : 0;
}

extern "C" int mp_w8a8_gemm(const void* qx_i8, const void* x_scale_f32, const void* w_i8, const void* w_scale_f32,
                            const void* bias_f16, void* y_f16, int M, int N, int K, int* error_word,
                            mp_stream_t stream) {
  return mp_w8a8_gemm_ex(qx_i8, x_scale_f32, w_i8, w_scale_f32, bias_f16, y_f16, M, N, K, nullptr, 0, error_word,
                         stream);
}

extern "C" int mp_w8a8_gemm_ex(const void* qx_i8, const void* x_scale_f32, const void* w_i8, const void* w_scale_f32,
                               const void* bias_f16, void* y_f16, int M, int N, int K, void* workspace,
                               size_t workspace_bytes, int* error_word, mp_stream_t stream) {
  int rc = check_gemm_args(qx_i8, w_i8, y_f16, M, N, K);
  if (rc != MP_OK) return rc;
  if (!x_scale_f32 || !w_scale_f32) return MP_ERR_INVALID_ARG;
  GemmCall c{};
  c.a = qx_i8; c.b = w_i8; c.M = M; c.N = N; c.K = K; c.a_rows = M; c.b_rows_total = N;
  c.a_scale = static_cast<const float*>(x_scale_f32); c.b_scale = static_cast<const float*>(w_scale_f32);
  c.bias = static_cast<const __half*>(bias_f16); c.out = y_f16; c.error_word = error_word;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pair(M, N)) return launch_gemm<256, EPI_F16, true>(c, st);
  const int ks = workspace ? w8a8_k_split(M, N, K) : 1;        // without scratch: one K slice per tile
  if (ks > 1) {
    if (workspace_bytes < (size_t)ks * M * N * sizeof(int)) return MP_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return MP_ERR_ALIGNMENT;
    c.k_split = ks;
    c.partial = static_cast<int*>(workspace);
    rc = launch_gemm<128, EPI_F16>(c, st);
    if (rc != MP_OK) return rc;
    return launch_splitk_reduce<true>(c, st);
  }
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  if (N <= 128 || tiles256 < kSmCount) return launch_gemm<128, EPI_F16>(c, st);
  return launch_gemm<256, EPI_F16>(c, st);
}

extern "C" int mp_w8a8_gemm_i32(const void* qx_i8, const void* w_i8, void* acc_i32, int M, int N, int K,
                                int* error_word, mp_stream_t stream) {
  int rc = check_gemm_args(qx_i8, w_i8, acc_i32, M, N, K);
  if (rc != MP_OK) return rc;
  GemmCall c{};
  c.a = qx_i8; c.b = w_i8; c.M = M; c.N = N; c.K = K; c.a_rows = M; c.b_rows_total = N;
  c.out = acc_i32; c.error_word = error_word;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pair(M, N)) return launch_gemm<256, EPI_I32, true>(c, st);
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  if (N <= 128 || tiles256 < kSmCount) return launch_gemm<128, EPI_I32>(c, st);
  return launch_gemm<256, EPI_I32>(c, st);
}

extern "C" int mp_w8a8_affine_gemm(const void* qx_u8, const void* x_scale_f32, const void* x_zero_f32,
                                   const void* x_rowsum_i32, const void* w_u8, const void* w_scale_f32,
                                   const void* w_zero_f32, const void* w_rowsum_i32, const void* bias_f16,
                                   void* y_f16, int M, int N, int K, int* error_word, mp_stream_t stream) {
  int rc = check_gemm_args(qx_u8, w_u8, y_f16, M, N, K);
  if (rc != MP_OK) return rc;
  if (!x_scale_f32 || !x_zero_f32 || !x_rowsum_i32 || !w_scale_f32 || !w_zero_f32 || !w_rowsum_i32) return MP_ERR_INVALID_ARG;
  if ((long long)K * 255 * 255 > 2147483647LL) return MP_ERR_UNSUPPORTED;   // the unsigned sums must fit int32
  GemmCall c{};
  c.a = qx_u8; c.b = w_u8; c.M = M; c.N = N; c.K = K; c.a_rows = M; c.b_rows_total = N;
  c.a_scale = static_cast<const float*>(x_scale_f32); c.b_scale = static_cast<const float*>(w_scale_f32);
  c.a_zero = static_cast<const float*>(x_zero_f32); c.a_rowsum = static_cast<const int*>(x_rowsum_i32);
  c.b_zero = static_cast<const float*>(w_zero_f32); c.b_rowsum = static_cast<const int*>(w_rowsum_i32);
  c.bias = static_cast<const __half*>(bias_f16); c.out = y_f16; c.error_word = error_word;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pair(M, N)) return launch_gemm<256, EPI_AFFINE, true>(c, st);
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  if (N <= 128 || tiles256 < kSmCount) return launch_gemm<128, EPI_AFFINE>(c, st);
  return launch_gemm<256, EPI_AFFINE>(c, st);
}
