// W4A16 decode linear (M <= 16), TMA-fed: y = x @ dequant(W)^T streaming the
// packed weights through a shared-memory ring.
//
// A block owns 128 output rows and 1/CK of K (CK = cluster size along K).
//   warp 8      producer: per stage (256 columns of K) one TMA box of packed
//               weights [128 rows x 128 B, 128-byte swizzle], four boxes of
//               activations [M rows x 64 columns] and one box of (scale, zero)
//               pairs, all landing on one mbarrier; a 3-deep ring keeps up to
//               ~50 KB per block in flight without holding registers
//   warps 0-7   consumers (4 row-warps x 2 K-halves): read their 32-row x
//               128-column chunk from the ring (conflict-light swizzled
//               128-bit loads), expand it in registers with dequant8 (exactly
//               f16((u - z) * s)) and feed mma.sync m16n8k16 directly -- the
//               dequantised weights never touch shared or global memory.  (For
//               M <= 8 and groups of a multiple of 128 columns the folded form
//               described at nibble_pairs() applies scale and zero point per
//               group instead of per weight.)  The
//               packed nibble order yields column pairs (k, k+4); the
//               activation fragments are permuted to match when they are read.
//               For M <= 8 the operands swap roles (weights are the 16-row A
//               operand, the 8 tokens the B operand), which halves the number
//               of MMAs per weight.
// Reduction: the two K-halves are added in shared memory, then every block
// stores its [M x 128] partial tile into the shared memory of the blocks that
// own the columns (block r of the cluster owns columns [r*128/CK, ...)), one
// cluster barrier, and each owner adds the CK tiles in rank order
// (deterministic), adds the bias and writes fp16.  No scratch memory.
//
// Under programmatic dependent launch the weight and scale boxes of the first
// stages are requested before griddepcontrol.wait; activations, bias and the
// output are only touched after it.  Every mbarrier wait is bounded.
#include <cooperative_groups.h>

#include "common.cuh"
#include "tc.cuh"

namespace mp {

using namespace tc;

namespace dt {
constexpr int kRows = 128;
constexpr int kStageK = 256;
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStages = 3;
constexpr int kWBytes = kRows * (kStageK / 2);     // 16384
constexpr int kSzBytes = 4096;                      // up to 8 groups x 128 rows x 4 B
template <bool HALF>
struct Cfg {
  static constexpr int kMRows = HALF ? 8 : 16;
  static constexpr int kXSub = kMRows * 128;        // one [M x 64 columns] sub-tile
  static constexpr int kXBytes = 4 * kXSub;
  static constexpr int kStageBytes = kWBytes + kXBytes + kSzBytes;
  static constexpr int kSlotBytes = kMRows * kRows * 4;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kStageBytes + kSlotBytes + 128;
};
}  // namespace dt

struct DecodeTmaParams {
  const __half* bias;
  __half* y;
  int M, N, K, group;
  int stages_total;        // ceil(K / 256)
  int stages_per_block;    // per cluster rank
  int groups_per_stage;    // rows of the (scale, zero) box
  int* error_word;
  DecodePush push;         // row-parallel mode (PUSH kernels only)
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Ring reads by 32-bit shared-window address.  The ring pointer is derived by integer arithmetic (1 KB alignment),
// which hides the address space from the compiler: written as plain dereferences these were generic loads.
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  // not volatile: free to move among the MMAs; the memory clobber keeps it behind the stage's barrier wait
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// (k0..k7 in natural order) -> (k0,k4) (k1,k5) (k2,k6) (k3,k7), the order dequant8 emits
__device__ __forceinline__ uint4 pair_permute(const uint4 in) {
  uint4 v;
  v.x = prmt(in.x, in.z, 0x5410);
  v.y = prmt(in.x, in.z, 0x7632);
  v.z = prmt(in.y, in.w, 0x5410);
  v.w = prmt(in.y, in.w, 0x7632);
  return v;
}

// Folded form (groups that are a multiple of 128 columns): a 4-bit code u is fed to the tensor core as
// the fp16 SUBNORMAL with bit pattern u (value u * 2^-24) -- mma.sync honours fp16 subnormals -- so
// "dequantisation" is four ANDs and a shift per eight weights.  Odd nibbles are left in place (bit
// pattern 16u, value 16u * 2^-24) and the activations that meet them are scaled by 1/16 instead.  One
// extra MMA per step multiplies a row of ones (same two bit patterns) with the same activations, which
// yields sum_k x[k] for the group.  Per group and accumulator element the fp32 epilogue is
//     acc += (s * 2^24) * (raw - z * ones)       =  s * sum_k (u_k - z) * x_k
// i.e. the scale and zero point are applied to the group's dot product rather than to each weight; the
// result differs from the product with the fp16-rounded f16((u - z) * s) by that rounding only.
__device__ __forceinline__ void nibble_pairs(uint32_t w, uint32_t (&v)[4]) {
  v[0] = w & 0x000f000fu;            // (k0, k4)        value u * 2^-24
  v[1] = w & 0x00f000f0u;            // (k1, k5)        value 16u * 2^-24
  const uint32_t w8 = w >> 8;
  v[2] = w8 & 0x000f000fu;           // (k2, k6)
  v[3] = w8 & 0x00f000f0u;           // (k3, k7)
}
constexpr uint32_t kOnesLo = 0x00010001u, kOnesHi = 0x00100010u;

// D = A * B with a zero accumulator input (no register has to be cleared first)
__device__ __forceinline__ void mma_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// the (k1,k5) and (k3,k7) activation pairs meet nibbles left in place: scale them by 1/16
__device__ __forceinline__ uint4 scale_odd_pairs(uint4 v) {
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  __half2 y = __hmul2_rn(*reinterpret_cast<__half2*>(&v.y), sixteenth);
  __half2 w = __hmul2_rn(*reinterpret_cast<__half2*>(&v.w), sixteenth);
  v.y = *reinterpret_cast<uint32_t*>(&y);
  v.w = *reinterpret_cast<uint32_t*>(&w);
  return v;
}

// PUSH (row-parallel linear, K sharded over GPUs): instead of rounding to fp16 the owner blocks store
// their fp32 sums into this GPU's partial-sum buffer, and the last block of the grid publishes this
// rank's arrival on every peer with a system-scope release store; the peers' finish kernels then read
// the buffer over NVLink.  (Storing into the peers' buffers from every block was tried first: the
// system-scope fence each block then needs before it may count itself done waits for its NVLink writes
// and cost 18 us on a 31 us kernel.)
template <bool HALF, bool FOLD, bool PUSH>
__global__ void __launch_bounds__(dt::kThreads, 2)
w4a16_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_sz, const DecodeTmaParams p) {
  namespace cg = cooperative_groups;
  using C = dt::Cfg<HALF>;
  constexpr int MROWS = C::kMRows;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;
  float* slots = reinterpret_cast<float*>(smem + dt::kStages * C::kStageBytes);   // [src block][m][owned column]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(slots) + C::kSlotBytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * dt::kStages);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + dt::kStages);

  cg::cluster_group cluster = cg::this_cluster();
  const int ck = static_cast<int>(cluster.num_blocks());
  const int crank = static_cast<int>(cluster.block_rank());
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < dt::kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, dt::kConsumerWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "I am running"; waited on before the pushes
  __syncthreads();

  const int s_begin = min(p.stages_total, crank * p.stages_per_block);
  const int s_end = min(p.stages_total, s_begin + p.stages_per_block);
  const int n_stages = s_end - s_begin;
  const int row_block0 = blockIdx.x * dt::kRows;

  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[r][i] = 0.0f;

  if (warp == dt::kConsumerWarps) {
    // ------------------------------------------------------------ producer
    if (elect_one()) {
      prefetch_tensormap(&tmap_w);
      prefetch_tensormap(&tmap_x);
      prefetch_tensormap(&tmap_sz);
      const uint32_t stage_bytes = dt::kWBytes + C::kXBytes + p.groups_per_stage * dt::kRows * 4;
      auto issue_weights = [&](int i) {
        const int s = i % dt::kStages;
        const int st = s_begin + i;
        const uint32_t full = full0 + 8 * s;
        unsigned char* base = ring + s * C::kStageBytes;
        mbar_arrive_expect_tx(full, stage_bytes);
        tma_load_2d(smem_u32(base), &tmap_w, full, st * (dt::kStageK / 2), row_block0);
        tma_load_2d(smem_u32(base + dt::kWBytes + C::kXBytes), &tmap_sz, full, row_block0,
                    (st * dt::kStageK) / p.group);
      };
      auto issue_x = [&](int i) {
        const int s = i % dt::kStages;
        const int st = s_begin + i;
        const uint32_t full = full0 + 8 * s;
        unsigned char* xb = ring + s * C::kStageBytes + dt::kWBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_load_2d(smem_u32(xb + j * C::kXSub), &tmap_x, full, st * dt::kStageK + j * 64, 0);
      };
      const int prologue = min(n_stages, dt::kStages);
      for (int i = 0; i < prologue; ++i) issue_weights(i);     // weights never depend on the previous kernel
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < prologue; ++i) issue_x(i);
      for (int i = prologue; i < n_stages; ++i) {
        const int s = i % dt::kStages;
        const uint32_t phase = ((i / dt::kStages) & 1) ^ 1;
        if (!mbar_wait(empty0 + 8 * s, phase, abort_flag)) break;
        issue_weights(i);
        issue_x(i);
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int g = lane >> 2, t = lane & 3;
    const int wn = warp >> 1, kh = warp & 1;
    const int grp_local = p.groups_per_stage > 1 ? (kh * 128 + t * 32) / p.group : 0;
    // byte offsets inside a stage that do not change from stage to stage
    const int w_off = (wn * 32 + g) * 128 + (((kh * 4 + t) ^ g) << 4);                 // + r * 8 * 128
    const int x_off = dt::kWBytes + (kh * 2 + (t >> 1)) * C::kXSub + g * 128;          // + ((cc ^ g) << 4) (+ 8 rows)
    const int sz_off = dt::kWBytes + C::kXBytes + (grp_local * dt::kRows + wn * 32 + g) * 4;   // + r * 32
    const uint32_t ring_addr = smem_u32(ring);
    bool ok = true;
    for (int i = 0; i < n_stages; ++i) {
      const int s = i % dt::kStages;
      const uint32_t phase = (i / dt::kStages) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, phase, abort_flag));
      if (!ok) break;
      const uint32_t base = ring_addr + s * C::kStageBytes;
      if constexpr (FOLD) {
        static_assert(HALF || !FOLD, "the folded form is written for the swapped-operand (M <= 8) layout");
        uint4 q[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) q[r] = lds_v4(base + w_off + r * 1024);
        float raw[2][4];
        float ones[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int xo = x_off + ((((t & 1) * 4 + c) ^ g) << 4);
          const uint4 alo = scale_odd_pairs(pair_permute(lds_v4(base + xo)));
          if (c == 0) {
            mma_16816_first(ones, kOnesLo, kOnesLo, kOnesHi, kOnesHi, alo.x, alo.y);
          } else {
            mma_16816(ones, kOnesLo, kOnesLo, kOnesHi, kOnesHi, alo.x, alo.y);
          }
          mma_16816(ones, kOnesLo, kOnesLo, kOnesHi, kOnesHi, alo.z, alo.w);
#pragma unroll
          for (int rp = 0; rp < 2; ++rp) {
            const uint4& qa = q[2 * rp];
            const uint4& qb = q[2 * rp + 1];
            const uint32_t wa = c == 0 ? qa.x : c == 1 ? qa.y : c == 2 ? qa.z : qa.w;
            const uint32_t wb = c == 0 ? qb.x : c == 1 ? qb.y : c == 2 ? qb.z : qb.w;
            uint32_t va[4], vb[4];
            nibble_pairs(wa, va);
            nibble_pairs(wb, vb);
            if (c == 0) {
              mma_16816_first(raw[rp], va[0], vb[0], va[1], vb[1], alo.x, alo.y);
            } else {
              mma_16816(raw[rp], va[0], vb[0], va[1], vb[1], alo.x, alo.y);
            }
            mma_16816(raw[rp], va[2], vb[2], va[3], vb[3], alo.z, alo.w);
          }
        }
        // group epilogue: acc += (s * 2^24) * (raw - z * ones).
        // raw[rp]: [0],[1] = row g of row group 2rp, tokens 2t, 2t+1; [2],[3] = row g of row group 2rp+1
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t szw = lds_u32(base + sz_off + r * 32);
          const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&szw));
          const float s24 = szf.x * 16777216.0f;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int i = (r & 1) * 2 + j;
            acc[2 * (r >> 1)][i] = fmaf(s24, fmaf(-szf.y, ones[j], raw[r >> 1][i]), acc[2 * (r >> 1)][i]);
          }
        }
      } else {
        uint4 q[4];
        ScaleZero sp[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          q[r] = lds_v4(base + w_off + r * 1024);
          const uint32_t szw = lds_u32(base + sz_off + r * 32);
          const __half2 h = *reinterpret_cast<const __half2*>(&szw);
          sp[r] = make_scale_zero(__low2half(h), __high2half(h));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int xo = x_off + ((((t & 1) * 4 + c) ^ g) << 4);
          const uint4 alo = pair_permute(lds_v4(base + xo));
          if (HALF) {
            // weights are the A operand: the row groups 2rp and 2rp+1 fill one 16-row tile, the 8 token
            // rows are the B operand.  acc[2*rp] is the tile D[16 weight rows][8 tokens]:
            // [0],[1] = (row g of group 2rp; tokens 2t, 2t+1), [2],[3] = (row g of group 2rp+1; same tokens).
#pragma unroll
            for (int rp = 0; rp < 2; ++rp) {
              const uint4& qa = q[2 * rp];
              const uint4& qb = q[2 * rp + 1];
              const uint32_t wa = c == 0 ? qa.x : c == 1 ? qa.y : c == 2 ? qa.z : qa.w;
              const uint32_t wb = c == 0 ? qb.x : c == 1 ? qb.y : c == 2 ? qb.z : qb.w;
              __half2 va[4], vb[4];
              dequant8(wa, sp[2 * rp], va);
              dequant8(wb, sp[2 * rp + 1], vb);
              mma_16816(acc[2 * rp], h2_as_u32(va[0]), h2_as_u32(vb[0]), h2_as_u32(va[1]), h2_as_u32(vb[1]), alo.x, alo.y);
              mma_16816(acc[2 * rp], h2_as_u32(va[2]), h2_as_u32(vb[2]), h2_as_u32(va[3]), h2_as_u32(vb[3]), alo.z, alo.w);
            }
          } else {
            const uint4 ahi = pair_permute(lds_v4(base + xo + 1024));
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const uint32_t word = c == 0 ? q[r].x : c == 1 ? q[r].y : c == 2 ? q[r].z : q[r].w;
              __half2 v[4];
              dequant8(word, sp[r], v);
              mma_16816(acc[r], alo.x, ahi.x, alo.y, ahi.y, h2_as_u32(v[0]), h2_as_u32(v[1]));
              mma_16816(acc[r], alo.z, ahi.z, alo.w, ahi.w, h2_as_u32(v[2]), h2_as_u32(v[3]));
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    // add the two K-halves: the ring is idle now (every stage that was requested has been consumed)
    float* ksum = reinterpret_cast<float*>(ring);                       // [m][128 rows of the block]
    asm volatile("bar.sync 1, 256;" ::: "memory");                     // all eight consumer warps are done reading it
    if (kh == 1) {
      if (HALF) {
#pragma unroll
        for (int rp = 0; rp < 2; ++rp)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            ksum[(2 * t + (i & 1)) * dt::kRows + wn * 32 + (2 * rp + (i >> 1)) * 8 + g] = acc[2 * rp][i];
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float* d = ksum + g * dt::kRows + wn * 32 + r * 8 + 2 * t;
          *reinterpret_cast<float2*>(d) = make_float2(acc[r][0], acc[r][1]);
          *reinterpret_cast<float2*>(d + 8 * dt::kRows) = make_float2(acc[r][2], acc[r][3]);
        }
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");                     // the eight consumer warps
    if (kh == 0) {
      if (HALF) {
#pragma unroll
        for (int rp = 0; rp < 2; ++rp)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            acc[2 * rp][i] += ksum[(2 * t + (i & 1)) * dt::kRows + wn * 32 + (2 * rp + (i >> 1)) * 8 + g];
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float* d = ksum + g * dt::kRows + wn * 32 + r * 8 + 2 * t;
          const float2 lo = *reinterpret_cast<const float2*>(d);
          const float2 hi = *reinterpret_cast<const float2*>(d + 8 * dt::kRows);
          acc[r][0] += lo.x; acc[r][1] += lo.y;
          acc[r][2] += hi.x; acc[r][3] += hi.y;
        }
      }
    }
  }

  // ---- push the block's tile to the owners of its columns, one barrier, owners finish ----
  const int cols = dt::kRows / ck;
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // every block of the cluster is running
  if (warp < dt::kConsumerWarps && (warp & 1) == 0) {
    const int g = lane >> 2, t = lane & 3, wn = warp >> 1;
    if (HALF) {
#pragma unroll
      for (int rp = 0; rp < 2; ++rp)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n_local = wn * 32 + (2 * rp + (i >> 1)) * 8 + g, m = 2 * t + (i & 1);
          const int owner = n_local / cols, c_in = n_local - owner * cols;
          cluster.map_shared_rank(slots, owner)[(size_t)(crank * MROWS + m) * cols + c_in] = acc[2 * rp][i];
        }
    } else {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n_local = wn * 32 + r * 8 + 2 * t;
        const int owner = n_local / cols, c_in = n_local - owner * cols;
        float* dst = cluster.map_shared_rank(slots, owner) + ((size_t)(crank * MROWS + g) * cols + c_in);
        *reinterpret_cast<float2*>(dst) = make_float2(acc[r][0], acc[r][1]);
        *reinterpret_cast<float2*>(dst + 8 * cols) = make_float2(acc[r][2], acc[r][3]);
      }
    }
  }
  cluster.sync();                                    // remote stores are visible; nobody is written to after this
  // PUSH: this call's number; the counter is advanced by the grid's last block, after every block has
  // read it here, and its parity picks the partial buffer
  [[maybe_unused]] const unsigned int push_epoch = PUSH ? *p.push.epoch + 1u : 0u;
  [[maybe_unused]] float* push_dst = PUSH ? p.push.partial[push_epoch & 1u] : nullptr;
  if (!*abort_flag) {
    for (int e = tid; e < p.M * cols; e += dt::kThreads) {
      const int m = e / cols, c = e - m * cols;
      const int n = row_block0 + crank * cols + c;
      float s = 0.0f;
      for (int src = 0; src < ck; ++src) s += slots[(src * MROWS + m) * cols + c];   // rank order: deterministic
      if (n < p.N) {
        if constexpr (PUSH) {
          push_dst[(size_t)m * p.N + n] = s;
        } else {
          if (p.bias) s += h2f(p.bias[n]);
          p.y[(size_t)m * p.N + n] = f2h(s);
        }
      }
    }
    if constexpr (PUSH) {
      __syncthreads();                                  // the block's stores ...
      if (tid == 0) {
        __threadfence();                                // ... are ordered before its count (fences are cumulative)
        const int blocks = static_cast<int>(gridDim.x * gridDim.y);
        if (atomicAdd(p.push.block_counter, 1) == blocks - 1) {       // every block of this GPU has stored
          atomicExch(p.push.block_counter, 0);                        // re-armed for the next call
          *p.push.epoch = push_epoch;
          __threadfence_system();
          for (int q = 0; q < p.push.world; ++q) {
            unsigned int* flag = p.push.flags[q] + p.push.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(push_epoch) : "memory");
          }
        }
      }
    }
  } else {
    if (tid == 0 && p.error_word) atomicExch(p.error_word, 3);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);       // let copies in flight land
  }
}

static bool g_decode_pdl = false;
void set_decode_programmatic_launch(bool on) { g_decode_pdl = on; }
bool decode_programmatic_launch() { return g_decode_pdl; }

// Set to a non-zero value by a decode kernel whose bounded wait gave up.
static __device__ int g_decode_error = 0;

int read_and_clear_decode_error(int* value) {
  int v = 0;
  MP_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_decode_error, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    MP_CUDA_TRY(cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(int)));
  }
  *value = v;
  return MP_OK;
}

// Device address of g_decode_error on the current device (looked up once per thread and device).
int* decode_error_word_ptr(int* out_rc) {
  static thread_local int* err_ptr = nullptr;
  static thread_local int err_device = -1;
  *out_rc = MP_OK;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess && err_device != device) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_error);
    if (e == cudaSuccess) {
      err_ptr = static_cast<int*>(ptr);
      err_device = device;
    }
  }
  if (e != cudaSuccess) {
    *out_rc = cuda_fail(e);
    return nullptr;
  }
  return err_ptr;
}

template <bool HALF, bool FOLD, bool PUSH>
static int launch_tma(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tsz, const DecodeTmaParams& p,
                      int row_blocks, int ck, cudaStream_t st, bool pdl) {
  using C = dt::Cfg<HALF>;
  auto kern = w4a16_decode_tma_kernel<HALF, FOLD, PUSH>;
  static thread_local int configured_device = -1;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmem));
    configured_device = device;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(row_blocks, ck, 1);
  cfg.blockDim = dim3(dt::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 1;
  attrs[0].val.clusterDim.y = ck;
  attrs[0].val.clusterDim.z = 1;
  int n_attrs = 1;
  // (push launches too: their block counter and call number are touched only after griddepcontrol.wait, i.e. after
  // the previous push kernel and the finish kernel between them have completed; the early start lets the next
  // shard's weight fetch run under the exchange)
  if (pdl) {
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    n_attrs = 2;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tw, tx, tsz, p));
  return MP_OK;
}

// Returns MP_ERR_UNSUPPORTED for shapes this kernel does not take (the caller then uses the
// register-streaming kernel): M > 16, K % 64 != 0, N % 4 != 0, group sizes that neither divide nor
// are a multiple of 256.
int launch_decode_tma(const void* x, const void* packed, const void* sz, const void* bias, void* y, int M, int N, int K,
                      int group, cudaStream_t st, const DecodePush* push, int pdl_choice) {
  const bool pdl = pdl_choice < 0 ? g_decode_pdl : pdl_choice != 0;
  if (M > 16 || K % 64 != 0 || N % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!((group <= dt::kStageK && dt::kStageK % group == 0) || group % dt::kStageK == 0)) return MP_ERR_UNSUPPORTED;
  if (!aligned(x, 16) || !aligned(packed, 16) || !aligned(sz, 16)) return MP_ERR_UNSUPPORTED;
  const bool half = M <= 8;
  const int mrows = half ? 8 : 16;
  const int gps = group < dt::kStageK ? dt::kStageK / group : 1;
  // The three tensor maps depend on addresses and shapes only; a serving loop calls with the same handful of
  // (x, W, scales) triples over and over, so the encoded maps are kept in a small per-thread cache.
  struct MapEntry {
    const void *x, *packed, *sz;
    int M, N, K, group, device;
    CUtensorMap tw, tx, tsz;
  };
  constexpr int kMapCache = 32;
  static thread_local MapEntry cache[kMapCache];
  static thread_local int cache_used = 0, cache_next = 0;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  const MapEntry* hit = nullptr;
  for (int i = 0; i < cache_used; ++i) {
    const MapEntry& e = cache[i];
    if (e.x == x && e.packed == packed && e.sz == sz && e.M == M && e.N == N && e.K == K && e.group == group &&
        e.device == device) {
      hit = &e;
      break;
    }
  }
  if (!hit) {
    MapEntry e{};
    e.x = x; e.packed = packed; e.sz = sz; e.M = M; e.N = N; e.K = K; e.group = group; e.device = device;
    int rc = encode_tensor_map_2d(&e.tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, packed, (uint64_t)K / 2, (uint64_t)N,
                                  (uint64_t)K / 2, 128, dt::kRows, true);
    if (rc != MP_OK) return rc;
    rc = encode_tensor_map_2d(&e.tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64,
                              mrows, true);
    if (rc != MP_OK) return rc;
    rc = encode_tensor_map_2d(&e.tsz, CU_TENSOR_MAP_DATA_TYPE_UINT32, sz, (uint64_t)N, (uint64_t)(K / group),
                              (uint64_t)N * 4, dt::kRows, gps, false);
    if (rc != MP_OK) return rc;
    const int slot = cache_used < kMapCache ? cache_used++ : (cache_next++ % kMapCache);
    cache[slot] = e;
    hit = &cache[slot];
  }
  const CUtensorMap& tw = hit->tw;
  const CUtensorMap& tx = hit->tx;
  const CUtensorMap& tsz = hit->tsz;
  DecodeTmaParams p{};
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<__half*>(y);
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.stages_total = (K + dt::kStageK - 1) / dt::kStageK;
  p.groups_per_stage = gps;
  {
    int rc_err = MP_OK;
    p.error_word = decode_error_word_ptr(&rc_err);
    if (rc_err != MP_OK) return rc_err;
  }
  const int row_blocks = (N + dt::kRows - 1) / dt::kRows;
  // K is cut over a cluster of ck blocks: the smallest power of two (<= 8, the portable limit) that puts
  // about two blocks on every SM ...
  constexpr int kSlots = 2 * kSmCount;
  int ck = 1;
  while (ck < 8 && row_blocks * ck < kSlots && p.stages_total >= 2 * ck) ck <<= 1;
  // ... unless that grid needs more than one and a half waves: the second wave pays the launch ramp (first
  // TMA round trip) and the cluster reduction again, which costs more than the idle slots of one wave
  // filled to three quarters (8192x28672, M = 1: 512 blocks 35.9 us, 256 blocks 31.4 us; 8192x8192:
  // 15.7 -> 12.1 us; 28672x8192: 37.4 -> 35.0 us).  Grids of up to 1.5 waves keep the finer split: in a
  // back-to-back sequence of 7B-sized linears it measured better (12288x4096 as 384 rather than 192
  // blocks: 69.0 vs 72.2 us per layer set).
  if (ck > 1 && row_blocks * ck * 2 > kSlots * 3) ck >>= 1;
  p.stages_per_block = (p.stages_total + ck - 1) / ck;
  // Folded scales need each warp's 128-column half of a stage to lie inside one group.  They pay for
  // M <= 8 (measured 10-15 % faster on the 70B shapes, neutral on the 7B ones); with 9..16 tokens the
  // extra MMAs of the ones row cost what the shorter dequantisation saves, so that case keeps the
  // exact per-weight form.
  if (push) {
    p.push = *push;
    if (half && group % 128 == 0) return launch_tma<true, true, true>(tw, tx, tsz, p, row_blocks, ck, st, pdl);
    return half ? launch_tma<true, false, true>(tw, tx, tsz, p, row_blocks, ck, st, pdl)
                : launch_tma<false, false, true>(tw, tx, tsz, p, row_blocks, ck, st, pdl);
  }
  if (half && group % 128 == 0) return launch_tma<true, true, false>(tw, tx, tsz, p, row_blocks, ck, st, pdl);
  return half ? launch_tma<true, false, false>(tw, tx, tsz, p, row_blocks, ck, st, pdl)
              : launch_tma<false, false, false>(tw, tx, tsz, p, row_blocks, ck, st, pdl);
}

}  // namespace mp
