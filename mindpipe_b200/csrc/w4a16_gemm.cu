// W4A16 prefill GEMM: y[M,N] = x[M,K] @ dequant(W)[N,K]^T on the fp16 tensor
// cores, with the int4 unpack + group dequant fused in as a producer stage.
//
// One persistent CTA per SM, 14 warps (128-row tile, MT = 1) or 18 warps (256-row tile, MT = 2):
//   warp 0      TMA producer for the activation tile x[128 MT x 64] (128-byte swizzle)
//   warp 1      MMA issuer: tcgen05.mma kind::f16, M=128, N=256, K=16, fp32 in TMEM
//   next 4 MT   epilogue warps: tcgen05.ld -> (+bias) -> fp16 -> global
//               (for M > 256 two CTAs of a cluster share each MMA, see Cfg)
//   last 8      dequant producers: stream the packed int4 words of the weight tile
//               [256 rows x 64 columns] from global memory with 128-bit loads, expand
//               them with dequant8 (exactly f16((u - z) * s), the reference's Wdq) and
//               store them into shared memory in the canonical K-major 128-byte-swizzle
//               layout the MMA reads -- the dequantised weights never exist in HBM.
//
// A stage is full when the TMA bytes have landed and all dequant warps have
// arrived (after a fence that makes their generic-proxy stores visible to the
// tensor core).  Every wait is bounded (see tc.cuh).
#include "common.cuh"
#include "tc.cuh"

namespace mp {

using namespace tc;

namespace w4 {
constexpr int kBN = 256;
constexpr int kBK = 64;            // fp16 elements of K per stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kSubBytes = 128 * kBK * 2;   // one 128-row activation sub-tile: 16 KB
constexpr int kTmemCols = 2 * kBN;         // all 512 columns
constexpr int kDequantWarps = 8;
// MT = 128-row activation sub-tiles per block tile.  MT = 1: 128 x 256 tile, two accumulator
// buffers (the epilogue of a tile overlaps the next main loop).  MT = 2: 256 x 256 tile whose two
// accumulators share one dequantised weight tile -- half the dequant work per flop, one buffer.
// PAIR (with MT = 2): two CTAs of a cluster share every MMA (cta_group::2, M = 256 per instruction:
// 128 rows from each CTA), so a pair computes a 512 x 256 tile and each CTA dequantises and stages
// only 128 of the 256 weight rows -- half the dequant work and a third less shared-memory traffic
// per flop than the single-CTA 256 x 256 tile.
template <int MT, bool PAIR = false>
struct Cfg {
  static constexpr int kBM = 128 * MT;                       // activation rows per CTA
  static constexpr int kStages = PAIR ? 4 : (MT == 1 ? 4 : 3);
  static constexpr int kABytes = MT * kSubBytes;
  static constexpr int kBRows = PAIR ? kBN / 2 : kBN;        // weight rows this CTA dequantises
  static constexpr int kBStage = kBRows * kBK * 2;
  static constexpr int kBufs = MT == 1 ? 2 : 1;
  static constexpr int kEpiWarps = 4 * MT;
  static constexpr int kFirstDequantWarp = 2 + kEpiWarps;
  static constexpr int kThreads = 32 * (2 + kEpiWarps + kDequantWarps);
  static constexpr size_t kSmem = 1024 + (size_t)kStages * (kABytes + kBStage) + 256;
};
}  // namespace w4

struct W4GemmParams {
  const uint32_t* packed;   // [N, K/8]
  const uint32_t* sz;       // [K/group, N] (scale, zero) f16 pairs
  const __half* bias;
  __half* y;
  int M, N, K, group;
  int m_tiles, n_tiles, k_blocks;
  int k_split;              // > 1: each tile's K range is cut into this many work items ...
  int kb_per_split;         // ... of this many k-blocks, whose fp32 partial tiles go to `partial`
  float* partial;           // [k_split][M][N] fp32 (split-K only)
  int* error_word;
};

template <int MT, bool PAIR>
__global__ void __launch_bounds__(w4::Cfg<MT, PAIR>::kThreads, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const W4GemmParams p) {
  using namespace w4;
  using C = Cfg<MT, PAIR>;
  constexpr int kBStage = C::kBStage;
  constexpr int kStages = C::kStages;
  constexpr int kABytes = C::kABytes;
  constexpr int kBM = C::kBM;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = smem;
  unsigned char* sB = smem + kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + kStages * kBStage);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // PAIR: rank 0 of the cluster leads: it issues the MMAs and owns the "stage full" and "accumulator
  // free" barriers, on which the peer's TMA bytes, dequant warps and epilogue warps arrive remotely;
  // both CTAs own "stage empty" and "accumulator full" barriers that the leader's commits arrive on.
  // Every wait is on a barrier of the waiting CTA.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  constexpr int kCtas = PAIR ? 2 : 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      // leader: the TMA producer's expect_tx arrival + its dequant warps (+ one relayed arrival for the
      // peer's dequant warps); peer: its dequant warps only (its relay thread waits on this one)
      mbar_init(full0 + 8 * s, leader ? 1 + kDequantWarps + (PAIR ? 1 : 0) : kDequantWarps);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, kCtas * C::kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), kTmemCols);
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
  // work item = (tile, K slice); m_tiles counts tiles of kCtas * kBM rows
  const int total = p.m_tiles * p.n_tiles * p.k_split;
  const int first_tile = PAIR ? blockIdx.x >> 1 : blockIdx.x;
  const int tile_step = PAIR ? gridDim.x >> 1 : gridDim.x;
  const uint32_t full_leader0 = PAIR ? map_to_cta(full0, 0) : full0;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tensormap(&tmap_x);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = first_tile; ok && work < total; work += tile_step) {
        const int tile = work / p.k_split;
        const int kb0 = (work - tile * p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        const int m0 = (tile % p.m_tiles) * (kCtas * kBM) + static_cast<int>(rank) * kBM;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag)) { ok = false; break; }
          if (PAIR) {
            const uint32_t full = full_leader0 + 8 * stage;      // both CTAs' bytes are counted by the leader
            if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * kABytes);
#pragma unroll
            for (int sub = 0; sub < MT; ++sub)
              tma_load_2d_pair(smem_u32(sA + stage * kABytes + sub * kSubBytes), &tmap_x, full, kb * kBK,
                               m0 + sub * 128);
          } else {
            const uint32_t full = full0 + 8 * stage;
            mbar_arrive_expect_tx(full, kABytes);
#pragma unroll
            for (int sub = 0; sub < MT; ++sub)
              tma_load_2d(smem_u32(sA + stage * kABytes + sub * kSubBytes), &tmap_x, full, kb * kBK, m0 + sub * 128);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 && !leader) {
    // peer CTA: relay "my half of the weight tile is in place" to the leader with ONE cluster-scope
    // arrival per stage (the eight dequant warps arrive on the local barrier, which is cheap)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = first_tile; ok && work < total; work += tile_step) {
        const int kb0 = (work % p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          mbar_arrive_cluster(full_leader0 + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kIdescDFormatF32 | kIdescABFormatF16, kCtas * 128, kBN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int work = first_tile; ok && work < total; work += tile_step) {
        const int kb0 = (work % p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        if (!mbar_wait(tempty0 + 8 * buf, buf_phase ^ 1, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBN;        // MT == 2: the accumulators sit at columns 0 and 256
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t b_desc = umma_desc_k_sw128(smem_u32(sB + stage * kBStage));
#pragma unroll
          for (int sub = 0; sub < MT; ++sub) {
            const uint64_t a_desc = umma_desc_k_sw128(smem_u32(sA + stage * kABytes + sub * kSubBytes));
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {  // +32 bytes of K per step
              if (PAIR) {
                umma_f16_pair(d_tmem + sub * kBN, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb != kb0 || kk != 0));
              } else {
                umma_f16(d_tmem + sub * kBN, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb != kb0 || kk != 0));
              }
            }
          }
          if (PAIR) {                      // release the stage in both CTAs
            umma_commit_pair(empty0 + 8 * stage);
            umma_commit_pair(map_to_cta(empty0 + 8 * stage, 1));
          } else {
            umma_commit(empty0 + 8 * stage);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) {                        // publish the accumulators to both CTAs' epilogues
          umma_commit_pair(tfull0 + 8 * buf);
          umma_commit_pair(map_to_cta(tfull0 + 8 * buf, 1));
        } else {
          umma_commit(tfull0 + 8 * buf);
        }
        if (++buf == C::kBufs) { buf = 0; buf_phase ^= 1; }
      }
    }
  } else if (warp < C::kFirstDequantWarp) {
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, +32) belong to this warp
    const int sub = (warp - 2) >> 2;              // which 128-row accumulator (MT == 2)
    int buf = 0;
    uint32_t buf_phase = 0;
    const uint32_t tempty_leader0 = PAIR ? map_to_cta(tempty0, 0) : tempty0;
    for (int work = first_tile; work < total; work += tile_step) {
      const int tile = work / p.k_split, split = work - tile * p.k_split;
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, buf_phase, abort_flag))) break;
      tcgen05_fence_after();
      const int row = m_tile * (kCtas * kBM) + static_cast<int>(rank) * kBM + sub * 128 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int n0 = n_tile * kBN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (buf + sub) * kBN;
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (p.k_split > 1) {
          // split-K: this K slice's fp32 partial tile; a second kernel adds the slices in order
          if (row_ok) {
            float* dst = p.partial + ((size_t)split * p.M + row) * p.N + n0 + c0;
            if (n0 + c0 + 32 <= p.N && (p.N % 4) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                reinterpret_cast<uint4*>(dst)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + c0 + j < p.N) dst[j] = __uint_as_float(r[j]);
            }
          }
          continue;
        }
        uint32_t packed_out[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = n0 + c0 + 2 * j;
          float v0 = __uint_as_float(r[2 * j]), v1 = __uint_as_float(r[2 * j + 1]);
          if (p.bias) {
            if (n < p.N) v0 += h2f(p.bias[n]);
            if (n + 1 < p.N) v1 += h2f(p.bias[n + 1]);
          }
          packed_out[j] = h2_as_u32(__floats2half2_rn(v0, v1));
        }
        if (row_ok) {
          __half* dst = p.y + (size_t)row * p.N + n0 + c0;
          if (n0 + c0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v)
              reinterpret_cast<uint4*>(dst)[v] =
                  make_uint4(packed_out[4 * v], packed_out[4 * v + 1], packed_out[4 * v + 2], packed_out[4 * v + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {                     // static indices keep the values in registers
              const uint32_t w = packed_out[j >> 1];
              if (n0 + c0 + j < p.N)
                dst[j] = __ushort_as_half(static_cast<unsigned short>((j & 1) ? (w >> 16) : (w & 0xFFFFu)));
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
      if (++buf == C::kBufs) { buf = 0; buf_phase ^= 1; }
    }
  } else {
    // ---- dequant producers: 256 threads expand this CTA's rows of the weight tile; a thread owns one
    // row (all 64 columns of the k-block) or, with 128 rows per CTA (PAIR), one 32-column half of a row ----
    constexpr int kTPR = 256 / C::kBRows;                              // threads per row: 1 or 2
    constexpr int kVec = 2 / kTPR;                                     // 128-bit loads per thread and k-block
    const int dt = threadIdx.x - C::kFirstDequantWarp * 32;            // 0..255
    const int r = dt / kTPR;                                           // row of this CTA's weight tile
    const int part = dt % kTPR;                                        // which half of the row's k-block
    const int words_per_row = p.K >> 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const int row_off = (r >> 3) * 1024 + (r & 7) * 128;     // row r of a K-major tile with 128-byte rows
    const int sw = r & 7;
    for (int work = first_tile; ok && work < total; work += tile_step) {
      const int tile = work / p.k_split;
      const int kb0 = (work - tile * p.k_split) * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      const int n = (tile / p.m_tiles) * kBN + static_cast<int>(rank) * C::kBRows + r;
      const bool n_ok = n < p.N;
      const uint32_t* row = p.packed + (size_t)(n_ok ? n : 0) * words_per_row + part * 4;
      const uint32_t* szp = p.sz + (n_ok ? n : 0);
      // software pipeline: the words of the next kPrefetch k-blocks are in flight while one is
      // expanded (a k-block lasts about 1000 tensor cycles, a global load under load about as long)
      constexpr int kPrefetch = 3;
      uint4 q[kPrefetch][kVec];
      uint32_t szq[kPrefetch];
      auto fetch = [&](int kb, uint4 (&dst)[kVec], uint32_t& z) {
        const bool live = n_ok && kb < kb1;
        const uint32_t* src = row + kb * (kBK / 8);
#pragma unroll
        for (int v = 0; v < kVec; ++v) dst[v] = live ? ldg_stream_v4(src + 4 * v) : make_uint4(0, 0, 0, 0);
        z = live ? __ldg(szp + (size_t)((kb * kBK) / p.group) * p.N) : 0u;
      };
#pragma unroll
      for (int d = 0; d < kPrefetch; ++d) fetch(kb0 + d, q[d], szq[d]);
      for (int kb = kb0; kb < kb1; ++kb) {
        uint4 cur[kVec];
#pragma unroll
        for (int v = 0; v < kVec; ++v) cur[v] = q[0][v];
        const uint32_t szc = szq[0];
#pragma unroll
        for (int d = 0; d + 1 < kPrefetch; ++d) {
#pragma unroll
          for (int v = 0; v < kVec; ++v) q[d][v] = q[d + 1][v];
          szq[d] = szq[d + 1];
        }
        fetch(kb + kPrefetch, q[kPrefetch - 1], szq[kPrefetch - 1]);
        const __half2 hz = *reinterpret_cast<const __half2*>(&szc);
        const ScaleZero sp = make_scale_zero(__low2half(hz), __high2half(hz));
        if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag))) { ok = false; break; }
        const uint32_t row_base = smem_u32(sB + stage * kBStage + row_off);   // st.shared below, not generic stores
#pragma unroll
        for (int jj = 0; jj < 4 * kVec; ++jj) {                   // 16-byte chunk j = columns 8j..8j+7
          const int j = part * 4 + jj;
          const uint4& src = cur[jj >> 2];
          const uint32_t word = (jj & 3) == 0 ? src.x : (jj & 3) == 1 ? src.y : (jj & 3) == 2 ? src.z : src.w;
          __half2 v[4];
          dequant8(word, sp, v);
          const uint32_t a = h2_as_u32(v[0]), b = h2_as_u32(v[1]), c = h2_as_u32(v[2]), d = h2_as_u32(v[3]);
          uint4 o;                                                // natural column order for the MMA
          o.x = prmt(a, b, 0x5410);
          o.y = prmt(c, d, 0x5410);
          o.z = prmt(a, b, 0x7632);
          o.w = prmt(c, d, 0x7632);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_base + ((j ^ sw) << 4)), "r"(o.x), "r"(o.y),
                       "r"(o.z), "r"(o.w) : "memory");                // 128-byte swizzle
        }
        fence_proxy_async_smem();      // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * stage);      // this CTA's barrier (the peer's is relayed)
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
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
    if (threadIdx.x == 0 && p.error_word) atomicExch(p.error_word, 2);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    if (PAIR) {
      tmem_dealloc_pair(tmem_base, w4::kTmemCols);
    } else {
      tmem_dealloc(tmem_base, w4::kTmemCols);
    }
  }
}

// y = f16(sum of the K slices' partial tiles, in slice order (+ bias))
__global__ void __launch_bounds__(256)
w4a16_splitk_reduce_kernel(const float* __restrict__ partial, int k_split, int M, int N,
                           const __half* __restrict__ bias, __half* __restrict__ y) {
  const int quads = N >> 2;
  const size_t slice = (size_t)M * N;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += gridDim.x * blockDim.x) {
    const int m = i / quads, n = (i - m * quads) << 2;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < k_split; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + s * slice + (size_t)m * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
      acc.x += h2f(bias[n]); acc.y += h2f(bias[n + 1]); acc.z += h2f(bias[n + 2]); acc.w += h2f(bias[n + 3]);
    }
    const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
    *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = make_uint2(h2_as_u32(lo), h2_as_u32(hi));
  }
}

// With few output tiles (batch sizes just above the decode kernels' range, or a narrow N) most SMs
// would idle while a handful stream all the weights: cut K so that about one work item per SM (per
// CTA pair for M > 256) exists.  Returns 1 when the tiles alone fill the machine or N % 4 != 0.
static int prefill_k_split(int M, int N, int K) {
  if (N % 4 != 0) return 1;
  const int n_tiles = (N + w4::kBN - 1) / w4::kBN;
  int tiles, units;
  if (M > 256) {
    tiles = ((M + 511) / 512) * n_tiles;
    units = kSmCount / 2;
  } else {
    tiles = (M > 128 ? (M + 255) / 256 : (M + 127) / 128) * n_tiles;
    units = kSmCount;
  }
  const int k_blocks = K / w4::kBK;
  int ks = units / tiles;
  if (ks > k_blocks / 4) ks = k_blocks / 4;          // at least four k-blocks per slice
  if (ks > 16) ks = 16;
  if (ks < 2) return 1;
  const int per = (k_blocks + ks - 1) / ks;
  return (k_blocks + per - 1) / per;                  // no empty slice
}

template <int MT, bool PAIR = false>
static int launch_w4_gemm(const CUtensorMap& tx, W4GemmParams p, cudaStream_t st) {
  using C = w4::Cfg<MT, PAIR>;
  constexpr int kTileRows = (PAIR ? 2 : 1) * C::kBM;
  p.m_tiles = (p.M + kTileRows - 1) / kTileRows;
  auto kern = w4a16_gemm_kernel<MT, PAIR>;
  static thread_local int configured_device = -1;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmem));
    configured_device = device;
  }
  const long long total = (long long)p.m_tiles * p.n_tiles * p.k_split;
  if (PAIR) {
    const int pairs = (int)(total < kSmCount / 2 ? total : kSmCount / 2);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tx, p));
    return MP_OK;
  }
  const int grid = (int)(total < kSmCount ? total : kSmCount);
  kern<<<grid, C::kThreads, C::kSmem, st>>>(tx, p);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

}  // namespace mp

using namespace mp;

extern "C" size_t mp_w4a16_prefill_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || K % w4::kBK != 0) return 0;
  const int ks = prefill_k_split(M, N, K);
  return ks > 1 ? (size_t)ks * M * N * sizeof(float) : 0;
}

extern "C" int mp_w4a16_linear_prefill(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                       const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                       int* error_word, mp_stream_t stream) {
  return mp_w4a16_linear_prefill_ex(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, nullptr, 0,
                                    error_word, stream);
}

extern "C" int mp_w4a16_linear_prefill_ex(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                          const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                          void* workspace, size_t workspace_bytes, int* error_word,
                                          mp_stream_t stream) {
  if (!x_f16 || !packed_i32 || !sz_f16x2 || !y_f16 || M <= 0 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (K % w4::kBK != 0 || group % w4::kBK != 0 || K % group != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || !aligned(packed_i32, 16) || !aligned(sz_f16x2, 4) || !aligned(y_f16, 16)) return MP_ERR_ALIGNMENT;
  CUtensorMap tx;
  int rc = encode_tensor_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x_f16, (uint64_t)K, (uint64_t)M,
                                (uint64_t)K * 2, w4::kBK, 128);
  if (rc != MP_OK) return rc;
  W4GemmParams p{};
  p.packed = static_cast<const uint32_t*>(packed_i32);
  p.sz = static_cast<const uint32_t*>(sz_f16x2);
  p.bias = static_cast<const __half*>(bias_f16);
  p.y = static_cast<__half*>(y_f16);
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.n_tiles = (N + w4::kBN - 1) / w4::kBN;
  p.k_blocks = K / w4::kBK;
  p.error_word = error_word;
  p.k_split = 1;
  p.kb_per_split = p.k_blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ks = workspace ? prefill_k_split(M, N, K) : 1;    // without scratch: one K slice per tile
  if (ks > 1) {
    if (workspace_bytes < (size_t)ks * M * N * sizeof(float)) return MP_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return MP_ERR_ALIGNMENT;
    p.k_split = ks;
    p.kb_per_split = (p.k_blocks + ks - 1) / ks;
    p.partial = static_cast<float*>(workspace);
  }
  rc = M > 256 ? launch_w4_gemm<2, true>(tx, p, st)          // 512 x 256 tiles on CTA pairs
       : M > 128 ? launch_w4_gemm<2>(tx, p, st) : launch_w4_gemm<1>(tx, p, st);
  if (rc != MP_OK || ks == 1) return rc;
  int blocks = (M * (N / 4) + 255) / 256;
  if (blocks > 2 * kSmCount) blocks = 2 * kSmCount;
  w4a16_splitk_reduce_kernel<<<blocks, 256, 0, st>>>(p.partial, ks, M, N, p.bias, p.y);
  MP_LAUNCH_CHECK();
  return MP_OK;
}
