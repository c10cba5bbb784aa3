// W4A16 decode linear (M <= 16; 17..64 rows with a wider activation tile) on the tcgen05
// tensor core with the weights as the TENSOR-MEMORY operand: y = x @ dequant(W)^T.
//
// A thread owns ONE weight row: it reads 16 bytes (32 codes) of its row from
// the shared-memory ring, expands them with dequant8 -- exactly
// f16((u - z) * s) -- and stores the 16 packed registers straight into tensor
// memory (tcgen05.st, lane = row, column = pair of K).  One elected thread then
// issues tcgen05.mma kind::f16 with A = those TMEM columns (128 rows x 16 K per
// instruction), B = the activation tile in shared memory (16 token rows,
// K-major, 128-byte swizzle) and the fp32 accumulator [128 rows x 16 tokens] in
// TMEM.  No dequantised weight touches shared or global memory and no dequant
// warp issues an MMA, shuffles a fragment or touches an activation.
//
// Work is cut stream-K style: the (row block, 256-column stage) pairs, row
// block major, form one sequence that is divided evenly over a PERSISTENT grid
// of about two blocks per SM, so every SM streams the same number of bytes
// whatever the shape, the ring never drains between row blocks, and block
// start-up is paid once per launch.  A block's range crosses at most a few row
// blocks; for each it owns a "segment".  A segment that covers the whole K of
// its row block is written to y directly; otherwise its fp32 tile goes to the
// caller's workspace and the last segment of the row block to arrive (device
// counter) adds the tiles in block order -- a fixed order, so results are
// identical from run to run -- adds the bias and writes fp16.
//
//   warps 0-7   dequant: warp w serves TMEM lanes [32 (w & 3), +32) and the
//               (w >> 2)-th 128-column half of every 256-column stage; warps
//               0-3 also run the segment epilogues
//   warp 8      TMA producer (packed weights, (scale, zero) pairs, activations)
//   warp 9      TMEM allocation and the MMA issuer
//   warp 10     activation permuter: dequant8 emits the columns of a packed
//               word in the order (k0,k4,k1,k5,k2,k6,k3,k7); the same
//               permutation is applied in place to every 16-byte chunk of the
//               activation tile (a chunk is one token's eight columns of one
//               packed word, so the swizzle does not matter), off the dequant
//               warps' critical path
// TMEM (256 columns per block, two blocks per SM): accumulator at columns
// [0,TOK); three 64-column A slots (128 K each) after it, used round robin by the
// "units" (stage, half) in issue order.  TOK = 16, 32 or 64 token rows (the UMMA N):
// the wider tiles serve 17..64 rows with the weights still streamed once; their
// activation tile is 16 / 32 KB per stage, so the ring is 3 / 2 stages deep, and an
// MMA costs about 110 / 135 / 190 clocks at N = 16 / 32 / 64 (measured end to end on
// 28672x8192), which is why 32 rows cost 1.2x and 64 rows 1.9x the time of 16.  One accumulator is enough: the first MMA of a
// segment needs weights from warps 0-3, which they store only after they have
// read the previous segment's accumulator.
// Every mbarrier wait is bounded.
#include "common.cuh"
#include "tc.cuh"

namespace mp {

using namespace tc;

namespace du {
constexpr int kRows = 128;
constexpr int kStageK = 256;
constexpr int kDequantWarps = 8;
constexpr int kProducerWarp = 8, kMmaWarp = 9, kPermuteWarp = 10;
constexpr int kThreads = 11 * 32;
constexpr int kWBytes = kRows * (kStageK / 2);       // 16384
// TOK = token rows of the activation tile = UMMA N: 16, 32 or 64
__host__ __device__ constexpr int x_sub(int tok) { return tok * 128; }        // [TOK tokens x 64 columns] fp16
__host__ __device__ constexpr int x_bytes(int tok) { return 4 * x_sub(tok); }
constexpr int kMaxStages = 4;
constexpr int kBars = 3 * kMaxStages + 7;
constexpr size_t kSmemBlockMax = 113 * 1024;         // two blocks per SM
__host__ __device__ constexpr int stage_bytes(int tok, int groups_per_stage) {   // ring stride, a multiple of 1024
  return kWBytes + x_bytes(tok) + ((groups_per_stage * kRows * 4 + 1023) & ~1023);
}
__host__ __device__ constexpr size_t smem_bytes(int tok, int stages, int groups_per_stage) {
  return 1024 + (size_t)stages * stage_bytes(tok, groups_per_stage) + kBars * 8 + 64;
}
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kASlotCols = 64;                  // three A slots (128 K each) after the accumulator columns
__host__ __device__ constexpr uint32_t a_slot0(int tok) { return tok <= 32 ? 32u : 64u; }
constexpr int kASlots = 3;
constexpr int kMaxBlocks = 2 * kSmCount;
constexpr size_t kCounterBytes = 16384;              // one arrival counter per row block (<= 4096 of them)
__host__ __device__ constexpr size_t tile_floats(int tok) { return (size_t)tok * kRows; }
__host__ __device__ constexpr size_t workspace_bytes(int tok) {
  return kCounterBytes + (size_t)kMaxBlocks * 2 * tile_floats(tok) * sizeof(float);
}
__host__ __device__ constexpr int tokens_for(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }
}  // namespace du

struct DecodeUmmaParams {
  const __half* bias;
  __half* y;
  int M, N, K, group;
  int stages_per_row;      // ST = ceil(K / 256)
  int total;               // row blocks x ST
  int groups_per_stage;    // rows of the (scale, zero) box
  int gshift;              // log2(group) for groups shorter than 128 columns
  int* counters;           // workspace: [row blocks], zero between calls
  float* tiles;            // workspace: [grid][2][TOK][128] fp32 partial tiles
  int* error_word;
};

// the stage range of block b in a grid of g blocks: [range_start(b), range_start(b + 1))
__device__ __forceinline__ int range_start(int b, int g, int total) {
  return static_cast<int>((static_cast<long long>(b) * total) / g);
}
// the block whose range holds stage t
__device__ __forceinline__ int block_of(int t, int g, int total) {
  return static_cast<int>(((static_cast<long long>(t) + 1) * g - 1) / total);
}

__device__ __forceinline__ void tmem_st_32x32_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (lane = row, one 32-bit
// column = two consecutive K elements), 16 K per instruction.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Ring accesses by 32-bit shared-window address (the 1 KB-aligned ring pointer hides the address space from the
// compiler; plain dereferences of it are generic loads and stores).
__device__ __forceinline__ uint4 du_lds_v4(uint32_t addr) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// volatile instead of a memory clobber: keeps its place among the other volatile statements (barrier waits,
// stores) without being a compiler barrier between neighbouring loads
__device__ __forceinline__ uint4 du_lds_v4_ordered(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t du_lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void du_sts_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
}

// eight fp16 values (k0..k7) -> (k0,k4,k1,k5,k2,k6,k3,k7), the column order dequant8 emits
__device__ __forceinline__ uint4 pair_permute_u4(const uint4 in) {
  uint4 v;
  v.x = prmt(in.x, in.z, 0x5410);
  v.y = prmt(in.x, in.z, 0x7632);
  v.z = prmt(in.y, in.w, 0x5410);
  v.w = prmt(in.y, in.w, 0x7632);
  return v;
}

template <int STAGES, int TOK>
__global__ void __launch_bounds__(du::kThreads, 2)
w4a16_decode_umma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                         const __grid_constant__ CUtensorMap tmap_sz, const DecodeUmmaParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kXSub = du::x_sub(TOK), kXBytes = du::x_bytes(TOK);
  constexpr uint32_t kASlot0 = du::a_slot0(TOK);
  const int stage_bytes = du::stage_bytes(TOK, p.groups_per_stage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + STAGES * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + du::kBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_word = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [last?, first block, last block]
  const uint32_t full0 = smem_u32(bars);                      // stage landed (TMA bytes)
  const uint32_t empty0 = full0 + 8 * du::kMaxStages;         // stage may be overwritten
  const uint32_t xp0 = empty0 + 8 * du::kMaxStages;           // stage's activations are permuted
  const uint32_t afull0 = xp0 + 8 * du::kMaxStages;           // A slot holds a unit's dequantised weights
  const uint32_t aempty0 = afull0 + 8 * du::kASlots;          // A slot has been read by its MMAs
  const uint32_t dfull = aempty0 + 8 * du::kASlots;           // a segment's accumulator is final

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, du::kDequantWarps + 1);       // eight dequant warps + the MMAs' commit
      mbar_init(xp0 + 8 * s, 1);
    }
    for (int q = 0; q < du::kASlots; ++q) {
      mbar_init(afull0 + 8 * q, 4);                           // the four warps of one half
      mbar_init(aempty0 + 8 * q, 1);
    }
    mbar_init(dfull, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == du::kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), du::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int grid = static_cast<int>(gridDim.x), blk = static_cast<int>(blockIdx.x);
  const int ST = p.stages_per_row;
  const int t0 = range_start(blk, grid, p.total);
  const int n_stages = range_start(blk + 1, grid, p.total) - t0;

  if (warp == du::kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      prefetch_tensormap(&tmap_w);
      prefetch_tensormap(&tmap_x);
      prefetch_tensormap(&tmap_sz);
      const uint32_t tx_bytes = du::kWBytes + kXBytes + p.groups_per_stage * du::kRows * 4;
      auto issue_weights = [&](int i) {
        const int s = i % STAGES;
        const int t = t0 + i, rb = t / ST, st = t - rb * ST;
        const uint32_t full = full0 + 8 * s;
        unsigned char* base = ring + s * stage_bytes;
        mbar_arrive_expect_tx(full, tx_bytes);
        tma_load_2d(smem_u32(base), &tmap_w, full, st * (du::kStageK / 2), rb * du::kRows);
        tma_load_2d(smem_u32(base + du::kWBytes + kXBytes), &tmap_sz, full, rb * du::kRows,
                    (st * du::kStageK) / p.group);
      };
      auto issue_x = [&](int i) {
        const int s = i % STAGES;
        const int t = t0 + i, st = t % ST;
        const uint32_t full = full0 + 8 * s;
        unsigned char* xb = ring + s * stage_bytes + du::kWBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_load_2d(smem_u32(xb + j * kXSub), &tmap_x, full, st * du::kStageK + j * 64, 0);
      };
      const int prologue = min(n_stages, STAGES);
      for (int i = 0; i < prologue; ++i) issue_weights(i);     // weights never depend on the previous kernel
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < prologue; ++i) issue_x(i);
      for (int i = prologue; i < n_stages; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = ((i / STAGES) & 1) ^ 1;
        if (!mbar_wait_sleep(empty0 + 8 * s, phase, abort_flag, 400)) break;
        issue_weights(i);
        issue_x(i);
      }
    }
  } else if (warp == du::kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kIdescDFormatF32 | kIdescABFormatF16, du::kRows, TOK);
      bool ok = true;
      int st = t0 % ST;
      bool seg_first = true;
      for (int i = 0; ok && i < n_stages; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        const uint32_t xb = smem_u32(ring + s * stage_bytes + du::kWBytes);
        const bool seg_last = st == ST - 1 || i == n_stages - 1;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int u = 2 * i + h, q = u % du::kASlots;
          const uint32_t aphase = (u / du::kASlots) & 1;
          if (!mbar_wait_sleep(afull0 + 8 * q, aphase, abort_flag, 100)) { ok = false; break; }
          if (h == 0 && !mbar_wait_sleep(xp0 + 8 * s, phase, abort_flag, 100)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_tmem = tmem_base + kASlot0 + q * du::kASlotCols;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {     // 16 K per instruction: 8 TMEM columns of A, 32 bytes of B's rows
            const uint64_t b_desc = umma_desc_k_sw128(xb + (h * 2 + (kk >> 2)) * kXSub) + 2 * (kk & 3);
            umma_f16_ts(tmem_base, a_tmem + kk * 8, b_desc, idesc, !(seg_first && h == 0 && kk == 0));
          }
          umma_commit(aempty0 + 8 * q);
          if (h == 1) {
            umma_commit(empty0 + 8 * s);                        // the stage's activations have been read
            if (seg_last) umma_commit(dfull);
          }
        }
        seg_first = seg_last;
        if (++st == ST) st = 0;
      }
    }
  } else if (warp == du::kPermuteWarp) {
    // ------------------------------------------------------------ activation permuter
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < n_stages; ++i) {
      const int s = i % STAGES;
      const uint32_t phase = (i / STAGES) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_sleep(full0 + 8 * s, phase, abort_flag, 400))) break;
      const uint32_t xt = smem_u32(ring + s * stage_bytes + du::kWBytes);
      // four chunks per lane in flight: the loads are issued together, then permuted and stored
      for (int c = lane; c < kXBytes / 16; c += 128) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = du_lds_v4_ordered(xt + (c + 32 * j) * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) du_sts_v4(xt + (c + 32 * j) * 16, pair_permute_u4(v[j]));
      }
      fence_proxy_async_smem();                                // generic-proxy stores -> visible to the MMA's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(xp0 + 8 * s);
    }
  } else {
    // ------------------------------------------------------------ dequant warps (+ epilogues on warps 0-3)
    const int quarter = warp & 3, kh = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const int sw = row & 7;
    const bool short_groups = p.group < 128;
    const int grp0 = p.groups_per_stage > 1 ? (kh * 128) / p.group : 0;
    int w_off[4];                                  // this row's four 16-byte chunks of its half (128-byte swizzle)
#pragma unroll
    for (int j = 0; j < 4; ++j) w_off[j] = row * 128 + (((kh * 4 + j) ^ sw) << 4);
    const int sz_off = du::kWBytes + kXBytes + row * 4;
    const uint32_t ring_addr = smem_u32(ring);
    int rb = t0 / ST, st = t0 - rb * ST;
    int seg_begin_i = 0, seg_begin_st = st, seg_idx = 0;
    for (int i = 0; i < n_stages; ++i) {
      const int s = i % STAGES;
      const uint32_t phase = (i / STAGES) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, phase, abort_flag))) break;
      const uint32_t base = ring_addr + s * stage_bytes;
      uint4 q4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) q4[j] = du_lds_v4(base + w_off[j]);
      ScaleZero sp;
      {
        const uint32_t szw = du_lds_u32(base + sz_off + grp0 * (du::kRows * 4));
        const __half2 h = *reinterpret_cast<const __half2*>(&szw);
        sp = make_scale_zero(__low2half(h), __high2half(h));
      }
      const int u = 2 * i + kh, q = u % du::kASlots;
      const uint32_t aphase = ((u / du::kASlots) & 1) ^ 1;
      const uint32_t a_tmem = tmem_base + lane_field + kASlot0 + q * du::kASlotCols;
      // (waiting for the slot here, before the expansion, measured 8 % faster at 16 tokens than waiting
      // just before the first store)
      if (!__all_sync(0xffffffffu, mbar_wait(aempty0 + 8 * q, aphase, abort_flag))) break;
      tcgen05_fence_after();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j > 0 && short_groups && ((j * 32) & (p.group - 1)) == 0) {   // groups of 32 or 64 columns: next (scale, zero)
          const int grp = (kh * 128 + j * 32) >> p.gshift;
          const uint32_t szw = du_lds_u32(base + sz_off + grp * (du::kRows * 4));
          const __half2 h = *reinterpret_cast<const __half2*>(&szw);
          sp = make_scale_zero(__low2half(h), __high2half(h));
        }
        uint32_t r[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t word = c == 0 ? q4[j].x : c == 1 ? q4[j].y : c == 2 ? q4[j].z : q4[j].w;
          __half2 v[4];
          dequant8(word, sp, v);
#pragma unroll
          for (int e = 0; e < 4; ++e) r[4 * c + e] = h2_as_u32(v[e]);
        }
        tmem_st_32x32_x16(a_tmem + j * 16, r);
      }
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(afull0 + 8 * q);
        mbar_arrive(empty0 + 8 * s);
      }
      const bool seg_last = st == ST - 1 || i == n_stages - 1;
      if (seg_last) {
        if (kh == 0) {
          // ---- segment epilogue: lane = weight row, column = token
          if (!__all_sync(0xffffffffu, mbar_wait(dfull, seg_idx & 1, abort_flag))) break;
          tcgen05_fence_after();
          // 16 token columns at a time (more would not fit beside the dequant registers)
          asm volatile("griddepcontrol.wait;" ::: "memory");   // before anything of the previous kernel is overwritten
          const int n = rb * du::kRows + row;
          const float bias = (p.bias && n < p.N) ? h2f(p.bias[n]) : 0.0f;
          const bool whole = seg_begin_st == 0 && st == ST - 1;   // the whole K of this row block: final
          const int which = seg_begin_i == 0 ? 0 : 1;              // a block has at most two partial segments
          float* tile = p.tiles + ((size_t)blk * 2 + which) * du::tile_floats(TOK);
#pragma unroll 1
          for (int t0c = 0; t0c < TOK; t0c += 16) {
            uint32_t acc[16];
            tmem_ld_32x32_x16(tmem_base + lane_field + t0c, acc);
            tmem_ld_wait();
            if (whole) {
              if (n < p.N) {
#pragma unroll
                for (int m = 0; m < 16; ++m)
                  if (t0c + m < p.M) p.y[(size_t)(t0c + m) * p.N + n] = f2h(__uint_as_float(acc[m]) + bias);
              }
            } else {
#pragma unroll
              for (int m = 0; m < 16; ++m)
                if (t0c + m < p.M) tile[(t0c + m) * du::kRows + row] = __uint_as_float(acc[m]);
            }
          }
          if (!whole) {
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 0 && lane == 0) {
              const int fb = block_of(rb * ST, grid, p.total), lb = block_of(rb * ST + ST - 1, grid, p.total);
              const int old = atomicAdd(p.counters + rb, 1);
              const int last = old == lb - fb ? 1 : 0;
              if (last) p.counters[rb] = 0;                    // re-armed for the next call
              __threadfence();
              epi_word[0] = last; epi_word[1] = fb; epi_word[2] = lb;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (epi_word[0]) {
              const int fb = epi_word[1], lb = epi_word[2];
#pragma unroll 1
              for (int t0c = 0; t0c < TOK && t0c < p.M; t0c += 16) {
                float sum[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) sum[m] = 0.0f;
                for (int b2 = fb; b2 <= lb; ++b2) {            // block order: deterministic
                  const int w2 = range_start(b2, grid, p.total) >= rb * ST ? 0 : 1;
                  const float* t2 = p.tiles + ((size_t)b2 * 2 + w2) * du::tile_floats(TOK) + row;
#pragma unroll
                  for (int m = 0; m < 16; ++m)
                    if (t0c + m < p.M) sum[m] += __ldcg(t2 + (t0c + m) * du::kRows);
                }
                if (n < p.N) {
#pragma unroll
                  for (int m = 0; m < 16; ++m)
                    if (t0c + m < p.M) p.y[(size_t)(t0c + m) * p.N + n] = f2h(sum[m] + bias);
                }
              }
            }
          }
          tcgen05_fence_before();
        }
        ++seg_idx;
        seg_begin_i = i + 1;
        seg_begin_st = 0;
      }
      if (++st == ST) { st = 0; ++rb; }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0 && p.error_word) atomicExch(p.error_word, 4);
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 200000ull) __nanosleep(1000);  // let copies and MMAs in flight land
    __syncthreads();
  }
  if (warp == du::kMmaWarp) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, du::kTmemCols);
  }
}

int* decode_error_word_ptr(int* out_rc);   // w4a16_decode_tma.cu: device address of the decode error word

size_t decode_umma_workspace_bytes(int M) { return du::workspace_bytes(du::tokens_for(M)); }

static bool umma_shape_ok(int M, int N, int K, int group) {
  if (M > 64 || K % 64 != 0 || N % 4 != 0) return false;
  return group == 32 || group == 64 || group == 128 || group == du::kStageK || group % du::kStageK == 0;
}

template <int STAGES, int TOK>
static int launch_umma(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tsz, const DecodeUmmaParams& p,
                       int grid, size_t smem, cudaStream_t st, bool pdl) {
  auto kern = w4a16_decode_umma_kernel<STAGES, TOK>;
  static thread_local int configured_device = -1;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)du::kSmemBlockMax));
    configured_device = device;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(du::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  int n_attrs = 0;
  if (pdl) {
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    n_attrs = 1;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tw, tx, tsz, p));
  return MP_OK;
}

// Returns MP_ERR_UNSUPPORTED for shapes this kernel does not take (M > 16, K % 64 != 0, N % 4 != 0, groups
// other than 32, 64, 128, 256 or a multiple of 256) and when the workspace is missing or too small; the
// caller then uses a scratch-free kernel.  The workspace starts zeroed and is left ready for the next call;
// calls that share it must not overlap on the GPU.
int launch_decode_umma(const void* x, const void* packed, const void* sz, const void* bias, void* y, int M, int N, int K,
                       int group, void* workspace, size_t workspace_bytes, cudaStream_t st, bool pdl) {
  if (!umma_shape_ok(M, N, K, group)) return MP_ERR_UNSUPPORTED;
  const int tok = du::tokens_for(M);
  if (!workspace || workspace_bytes < du::workspace_bytes(tok) || !aligned(workspace, 16)) return MP_ERR_UNSUPPORTED;
  if (!aligned(x, 16) || !aligned(packed, 16) || !aligned(sz, 16)) return MP_ERR_UNSUPPORTED;
  const int row_blocks = (N + du::kRows - 1) / du::kRows;
  if ((size_t)row_blocks * sizeof(int) > du::kCounterBytes) return MP_ERR_UNSUPPORTED;
  CUtensorMap tw, tx, tsz;
  int rc = encode_tensor_map_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, packed, (uint64_t)K / 2, (uint64_t)N,
                                (uint64_t)K / 2, 128, du::kRows, true);
  if (rc != MP_OK) return rc;
  rc = encode_tensor_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64,
                            tok, true);
  if (rc != MP_OK) return rc;
  const int gps = group < du::kStageK ? du::kStageK / group : 1;
  rc = encode_tensor_map_2d(&tsz, CU_TENSOR_MAP_DATA_TYPE_UINT32, sz, (uint64_t)N, (uint64_t)(K / group),
                            (uint64_t)N * 4, du::kRows, gps, false);
  if (rc != MP_OK) return rc;
  DecodeUmmaParams p{};
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<__half*>(y);
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.stages_per_row = (K + du::kStageK - 1) / du::kStageK;
  p.total = row_blocks * p.stages_per_row;
  p.groups_per_stage = gps;
  p.gshift = group == 32 ? 5 : group == 64 ? 6 : 7;
  p.counters = static_cast<int*>(workspace);
  p.tiles = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + du::kCounterBytes);
  int rc_err = MP_OK;
  p.error_word = decode_error_word_ptr(&rc_err);
  if (rc_err != MP_OK) return rc_err;
  // two blocks per SM, each with at least two stages of work
  const int grid = max(1, min(du::kMaxBlocks, p.total / 2));
  // the deepest ring that still lets two blocks share an SM (groups of 32 columns carry 4 KB of (scale, zero)
  // pairs per stage; a 32-token activation tile is 16 KB per stage, a 64-token one 32 KB)
  auto fits = [&](int stages) { return du::smem_bytes(tok, stages, gps) <= du::kSmemBlockMax; };
  if (tok == 16) {
    if (fits(4)) return launch_umma<4, 16>(tw, tx, tsz, p, grid, du::smem_bytes(16, 4, gps), st, pdl);
    return launch_umma<3, 16>(tw, tx, tsz, p, grid, du::smem_bytes(16, 3, gps), st, pdl);
  }
  if (tok == 32) {
    if (fits(3)) return launch_umma<3, 32>(tw, tx, tsz, p, grid, du::smem_bytes(32, 3, gps), st, pdl);
    if (fits(2)) return launch_umma<2, 32>(tw, tx, tsz, p, grid, du::smem_bytes(32, 2, gps), st, pdl);
    return MP_ERR_UNSUPPORTED;
  }
  if (fits(2)) return launch_umma<2, 64>(tw, tx, tsz, p, grid, du::smem_bytes(64, 2, gps), st, pdl);
  return MP_ERR_UNSUPPORTED;
}

}  // namespace mp
