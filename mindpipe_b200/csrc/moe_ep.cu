// Expert-parallel MoE exchange over NVLink peer memory, driven from the device.
//
// Every rank keeps its routed int8 rows, their scales, its routing plan and a
// result buffer in symmetric memory (mapped by every peer).  The dispatch is a
// PULL: after a cross-rank barrier, each rank reads its peers' per-expert row
// counts, lays out its expert-sorted buffer, and copies the rows it owns
// straight out of the peers' routed buffers with plain peer loads.  The return
// is a PUSH: after the expert stage each result row is stored straight into
// the source rank's result buffer at the row's original position, so the
// weighted combine at home needs no re-ordering.  Row counts never visit the
// host, so a layer is a fixed sequence of launches with no synchronisation.
//
// Role in the reference: the all-to-all token dispatcher / combiner of the
// runtime (TokenDispatcherWithAll2AllV, acceleration/runtime_patches/
// vllm_ascend.patch:3228-3236; int8 payload as at :1668-1682).
//
// The barrier is a bounded wait: each rank stores the call's epoch into a flag
// slot on every peer and polls its own slots; if a peer does not show up within
// the limit the kernel records an error word and returns (no trap, no endless
// spin).  One process per GPU: the waiting kernels of different ranks run on
// different devices.  Only plain peer loads / stores are used.
#include "common.cuh"
#include "moe_api.cuh"

namespace mp {

constexpr int kMaxRanks = 16;
constexpr int kEpTile = kMoeTileRows;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ uint64_t ep_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// flags[r] on rank p is written by rank r.  Thread r < world: publish, then wait for peer r.
__device__ __forceinline__ void peer_barrier_body(const PeerPtrs& peer_flags, int world, int rank, unsigned int epoch,
                                                  int* error_word) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();                                           // everything this GPU wrote so far is visible
  unsigned int* remote = static_cast<unsigned int*>(peer_flags.p[r]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  peer_flag_wait(static_cast<const unsigned int*>(peer_flags.p[rank]) + r, epoch, error_word);   // peer r reached this epoch
  __threadfence_system();
}

__global__ void peer_barrier_kernel(PeerPtrs peer_flags, int world, int rank, unsigned int epoch, int* error_word) {
  peer_barrier_body(peer_flags, world, rank, epoch, error_word);
}

// Same, with the epoch kept in device memory and advanced by the kernel itself: the launch carries no
// per-call value, so a captured CUDA graph containing it can be replayed (every rank replays the same
// sequence of barriers, so the counters advance in step).
__global__ void peer_barrier_counted_kernel(PeerPtrs peer_flags, int world, int rank, unsigned int* epoch_counter,
                                            int* error_word) {
  chain_wait();
  chain_release();
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    *epoch_counter = s_epoch;
  }
  __syncthreads();
  peer_barrier_body(peer_flags, world, rank, s_epoch, error_word);
}

// Extended plan of the receiving rank (ints):
//   [0, plan_std)                       the standard plan the expert stage reads
//                                       (counts[El] | cursors[El] | seg[El+1] | num_tiles | tile_expert[...])
//   ext + e*(W+1) + s                   cum[e][s]: rows of local expert e that come from ranks < s
//   ext + El*(W+1) + e*W + s            src_seg[e][s]: first row of that segment in rank s's routed buffer
__device__ __forceinline__ void ep_plan_body(const PeerPtrs& peer_plans, int world, int rank, int e_total, int e_loc,
                                             int max_tiles, int ext, int* __restrict__ xplan) {
  // one thread per (local expert, source rank) fetches that peer's count and segment offset over NVLink
  __shared__ int s_cnt[256], s_seg[256];
  const int pairs = e_loc * world;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = i / world, s = i - e * world;
    const int ge = rank * e_loc + e;
    const int* pp = static_cast<const int*>(peer_plans.p[s]);       // rank s's plan over all e_total experts
    s_cnt[i] = pp[ge];                                               // counts[ge]
    s_seg[i] = pp[2 * e_total + ge];                                 // seg_offsets[ge]
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  int* counts = xplan;
  int* cursors = xplan + e_loc;
  int* seg = xplan + 2 * e_loc;
  int* num_tiles = xplan + 3 * e_loc + 1;
  int* tile_expert = xplan + 3 * e_loc + 2;
  int* cum = xplan + ext;
  int* src_seg = xplan + ext + e_loc * (world + 1);
  int off = 0, tiles = 0;
  for (int e = 0; e < e_loc; ++e) {
    int total = 0;
    for (int s = 0; s < world; ++s) {
      cum[e * (world + 1) + s] = total;
      total += s_cnt[e * world + s];
      src_seg[e * world + s] = s_seg[e * world + s];
    }
    cum[e * (world + 1) + world] = total;
    counts[e] = total;
    cursors[e] = 0;
    seg[e] = off;
    const int nt = moe_segment_tiles(total);
    for (int i = 0; i < nt && tiles < max_tiles; ++i) tile_expert[tiles++] = e;
    off += nt * kEpTile;
  }
  seg[e_loc] = off;
  *num_tiles = tiles;
}

__global__ void ep_plan_kernel(PeerPtrs peer_plans, int world, int rank, int e_total, int e_loc, int max_tiles,
                               int ext, int* __restrict__ xplan) {
  ep_plan_body(peer_plans, world, rank, e_total, e_loc, max_tiles, ext, xplan);
}

// The barrier in front of the plan and the plan itself in one launch: the block first meets its peers (bounded),
// then reads their counts.  One graph node less on the path of every layer.
__global__ void ep_barrier_plan_kernel(PeerPtrs peer_flags, PeerPtrs peer_plans, int world, int rank,
                                       unsigned int* epoch_counter, int e_total, int e_loc, int max_tiles, int ext,
                                       int* __restrict__ xplan, int* error_word) {
  chain_wait();
  chain_release();
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    *epoch_counter = s_epoch;
  }
  __syncthreads();
  peer_barrier_body(peer_flags, world, rank, s_epoch, error_word);
  __syncthreads();
  ep_plan_body(peer_plans, world, rank, e_total, e_loc, max_tiles, ext, xplan);
}

// The part of the extended plan that ep_locate reads (segment offsets, per-source cumulative counts, source
// segment starts), copied to shared memory once per block: a row's home is then found without a chain of
// dependent global loads in front of every row copy.
constexpr int kEpLocateInts = 2 * 64 + 1 + 64 * (kMaxRanks + 1) + 64 * kMaxRanks;   // up to 64 local experts

struct EpLocator {
  const int* seg;       // [e_loc + 1]
  const int* cum;       // [e_loc][world + 1]
  const int* src_seg;   // [e_loc][world]
  int world, e_loc;
  __device__ __forceinline__ bool locate(int i, int& s_out, int& src_row) const {
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
};

__device__ __forceinline__ EpLocator ep_cache_plan(const int* __restrict__ xplan, int world, int e_loc, int ext, int* s_buf) {
  int* s_seg = s_buf;
  int* s_cum = s_seg + e_loc + 1;
  int* s_src = s_cum + e_loc * (world + 1);
  for (int i = threadIdx.x; i <= e_loc; i += blockDim.x) s_seg[i] = xplan[2 * e_loc + i];
  for (int i = threadIdx.x; i < e_loc * (world + 1); i += blockDim.x) s_cum[i] = xplan[ext + i];
  for (int i = threadIdx.x; i < e_loc * world; i += blockDim.x) s_src[i] = xplan[ext + e_loc * (world + 1) + i];
  __syncthreads();
  return EpLocator{s_seg, s_cum, s_src, world, e_loc};
}

// Rows [row_lo, row_hi) a launch handles: all padded rows in use (part < 0), or the first / second half of the
// 256-row tiles (part 0 / 1), split where the grouped GEMMs split their row tiles.
__device__ __forceinline__ void ep_row_range(int rows_in_use, int part, int& row_lo, int& row_hi) {
  const int split = min(rows_in_use, moe_half_split_rows(rows_in_use / kEpTile));
  row_lo = part == 1 ? split : 0;
  row_hi = part == 0 ? split : rows_in_use;
}

// Sorted row i <- peer row (int8 codes and fp32 scale).  One warp per row: a lane requests all its 16-byte
// pieces of the row before it stores the first, so a row costs one NVLink round trip; warps stride over the
// rows in use.  VPL = 16-byte pieces per lane.
template <int VPL>
__global__ void __launch_bounds__(256)
ep_pull_kernel(PeerPtrs peer_q, PeerPtrs peer_scale, const int* __restrict__ xplan, int world, int e_loc, int ext,
               int vec_per_row, uint4* __restrict__ q_sorted, float* __restrict__ s_sorted, int part) {
  chain_wait();
  chain_release();
  __shared__ int s_plan[kEpLocateInts];
  const EpLocator loc = ep_cache_plan(xplan, world, e_loc, ext, s_plan);
  int row_lo, rows;                                                 // padded rows in use, or one half of them
  ep_row_range(loc.seg[e_loc], part, row_lo, rows);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = row_lo + blockIdx.x * 8 + warp; i < rows; i += gridDim.x * 8) {
    int s, src;
    if (!loc.locate(i, s, src)) {
      if (lane == 0) s_sorted[i] = 0.0f;                            // padding row: neutralised by a zero scale
      continue;
    }
    const uint4* from = static_cast<const uint4*>(peer_q.p[s]) + (size_t)src * vec_per_row;
    uint4* to = q_sorted + (size_t)i * vec_per_row;
    if (VPL > 0) {
      uint4 v[VPL > 0 ? VPL : 1];
#pragma unroll
      for (int j = 0; j < VPL; ++j) v[j] = from[lane + 32 * j];
      if (lane == 0) s_sorted[i] = static_cast<const float*>(peer_scale.p[s])[src];
#pragma unroll
      for (int j = 0; j < VPL; ++j) to[lane + 32 * j] = v[j];
    } else {
      for (int v = lane; v < vec_per_row; v += 32) to[v] = from[v];
      if (lane == 0) s_sorted[i] = static_cast<const float*>(peer_scale.p[s])[src];
    }
  }
}

// Optional tail of the push kernel: once every block's stores are out, raise this rank's arrival word on every
// peer with the next epoch (the second half of a barrier; the consumer of the rows does the waiting half).
struct EpSignal {
  PeerPtrs peer_flags;
  unsigned int* epoch_counter;   // null: no signal
  int* block_counter;            // zero between calls
  int world, rank;
};

// Result row i -> the source rank's result buffer, at the row's original position; one warp per row.
template <int VPL>
__global__ void __launch_bounds__(256)
ep_push_kernel(const uint4* __restrict__ d_sorted, const int* __restrict__ xplan, int world, int e_loc, int ext,
               int vec_per_row, PeerPtrs peer_back, int part, EpSignal sig) {
  chain_wait();
  chain_release();
  __shared__ int s_plan[kEpLocateInts];
  const EpLocator loc = ep_cache_plan(xplan, world, e_loc, ext, s_plan);
  int row_lo, rows;
  ep_row_range(loc.seg[e_loc], part, row_lo, rows);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = row_lo + blockIdx.x * 8 + warp; i < rows; i += gridDim.x * 8) {
    int s, src;
    if (!loc.locate(i, s, src)) continue;
    const uint4* from = d_sorted + (size_t)i * vec_per_row;
    uint4* to = static_cast<uint4*>(peer_back.p[s]) + (size_t)src * vec_per_row;
    if (VPL > 0) {
      uint4 v[VPL > 0 ? VPL : 1];
#pragma unroll
      for (int j = 0; j < VPL; ++j) v[j] = from[lane + 32 * j];
#pragma unroll
      for (int j = 0; j < VPL; ++j) to[lane + 32 * j] = v[j];
    } else {
      for (int v = lane; v < vec_per_row; v += 32) to[v] = from[v];
    }
  }
  if (sig.epoch_counter == nullptr) return;
  // the block that finishes last tells every peer that this rank's result rows have landed
  __shared__ bool s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(sig.block_counter, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x == 0) {
    *sig.block_counter = 0;                                          // ready for the next call
    *sig.epoch_counter += 1;
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < sig.world) {
    unsigned int* remote = static_cast<unsigned int*>(sig.peer_flags.p[threadIdx.x]) + sig.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(*sig.epoch_counter) : "memory");
  }
}

static int fill_peers(PeerPtrs& dst, const void* const* src, int world) {
  if (!src || world <= 0 || world > kMaxRanks) return MP_ERR_INVALID_ARG;
  for (int i = 0; i < kMaxRanks; ++i) dst.p[i] = i < world ? const_cast<void*>(src[i]) : nullptr;
  for (int i = 0; i < world; ++i)
    if (!dst.p[i]) return MP_ERR_INVALID_ARG;
  return MP_OK;
}

}  // namespace mp

using namespace mp;

extern "C" int mp_peer_barrier(const void* const* peer_flag_ptrs, int world, int rank, unsigned int epoch,
                               int* error_word, mp_stream_t stream) {
  PeerPtrs pf;
  int rc = fill_peers(pf, peer_flag_ptrs, world);
  if (rc != MP_OK) return rc;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, world, rank, epoch, error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_peer_barrier_counted(const void* const* peer_flag_ptrs, int world, int rank,
                                       void* epoch_counter_u32, int* error_word, mp_stream_t stream) {
  PeerPtrs pf;
  int rc = fill_peers(pf, peer_flag_ptrs, world);
  if (rc != MP_OK) return rc;
  if (rank < 0 || rank >= world || !epoch_counter_u32) return MP_ERR_INVALID_ARG;
  return launch_chained(peer_barrier_counted_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), pf, world,
                        rank, static_cast<unsigned int*>(epoch_counter_u32), error_word);
}

// ---- row-parallel W8A8 linear: K sharded over GPUs ------------------------------------------------------
// Every rank quantises its activation slice per token, multiplies it with its weight slice into raw
// int32 accumulators kept in peer-mapped memory, and announces them; every rank then reads all the
// accumulators and per-token scales over NVLink and sums the dequantised partial products in rank order.

// After this rank's GEMM (stream order): advance the call counter and raise it on every peer.
__global__ void peer_signal_kernel(PeerPtrs peer_flags, int world, int rank, unsigned int* epoch_counter) {
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    *epoch_counter = s_epoch;
  }
  __syncthreads();
  if (threadIdx.x >= world) return;
  __threadfence_system();                                           // the accumulators and scales are visible first
  unsigned int* remote = static_cast<unsigned int*>(peer_flags.p[threadIdx.x]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(s_epoch) : "memory");
}

struct PeerPair {
  const void* acc[kMaxRanks];
  const void* xscale[kMaxRanks];
};

// y[m, n] = f16(sum_r float(acc_r[m, n]) * xscale_r[m] * wscale[n] (+ bias)): each product rounded on its own,
// fp32 adds in rank order, one rounding to fp16 -- the same bits on every rank.
__global__ void __launch_bounds__(256)
w8a8_rowparallel_finish_kernel(PeerPair peers, const unsigned int* __restrict__ flags, int world,
                               const unsigned int* __restrict__ epoch_counter, int M, int N,
                               const float* __restrict__ w_scale, const __half* __restrict__ bias,
                               __half* __restrict__ y, int* error_word) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const unsigned int epoch = *epoch_counter;           // advanced by this rank's signal kernel before this launch
  if (threadIdx.x < world) {
    const unsigned int* f = flags + threadIdx.x;
    const uint64_t t0 = ep_timer_ns();
    for (unsigned int it = 0;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if ((it & 0xFF) == 0xFF && ep_timer_ns() - t0 > 2000000000ull) {  // 2 s: give up, report, write nothing
        s_ok = 0;
        if (error_word) atomicExch(error_word, 5);
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int quads = N >> 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += gridDim.x * blockDim.x) {
    const int m = i / quads, n = (i - m * quads) << 2;
    const float4 sw = *reinterpret_cast<const float4*>(w_scale + n);
    // all ranks' loads are issued before the first add: one NVLink round trip, not one per rank
    int4 a[kMaxRanks];
    float sx[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) {
        a[r] = *reinterpret_cast<const int4*>(static_cast<const int*>(peers.acc[r]) + (size_t)m * N + n);
        sx[r] = static_cast<const float*>(peers.xscale[r])[m];
      }
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) {
        sum.x = __fadd_rn(sum.x, __fmul_rn(__fmul_rn(static_cast<float>(a[r].x), sx[r]), sw.x));
        sum.y = __fadd_rn(sum.y, __fmul_rn(__fmul_rn(static_cast<float>(a[r].y), sx[r]), sw.y));
        sum.z = __fadd_rn(sum.z, __fmul_rn(__fmul_rn(static_cast<float>(a[r].z), sx[r]), sw.z));
        sum.w = __fadd_rn(sum.w, __fmul_rn(__fmul_rn(static_cast<float>(a[r].w), sx[r]), sw.w));
      }
    if (bias) {
      sum.x = __fadd_rn(sum.x, __half2float(bias[n])); sum.y = __fadd_rn(sum.y, __half2float(bias[n + 1]));
      sum.z = __fadd_rn(sum.z, __half2float(bias[n + 2])); sum.w = __fadd_rn(sum.w, __half2float(bias[n + 3]));
    }
    const __half2 lo = __floats2half2_rn(sum.x, sum.y), hi = __floats2half2_rn(sum.z, sum.w);
    uint2 out;
    out.x = *reinterpret_cast<const uint32_t*>(&lo);
    out.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = out;
  }
}

extern "C" int mp_peer_signal(const void* const* peer_flag_ptrs, int world, int rank, void* epoch_counter_u32,
                              mp_stream_t stream) {
  PeerPtrs pf;
  int rc = fill_peers(pf, peer_flag_ptrs, world);
  if (rc != MP_OK) return rc;
  if (rank < 0 || rank >= world || !epoch_counter_u32) return MP_ERR_INVALID_ARG;
  peer_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, world, rank,
                                                                     static_cast<unsigned int*>(epoch_counter_u32));
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w8a8_rowparallel_finish(const void* const* peer_acc_i32, const void* const* peer_xscale_f32,
                                          const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                                          int N, const void* w_scale_f32, const void* bias_f16, void* y_f16,
                                          int* error_word, mp_stream_t stream) {
  if (!peer_acc_i32 || !peer_xscale_f32 || !flags_u32 || !epoch_counter_u32 || !w_scale_f32 || !y_f16 || world < 1 ||
      world > kMaxRanks || M <= 0 || N <= 0)
    return MP_ERR_INVALID_ARG;
  if (N % 4 != 0) return MP_ERR_UNSUPPORTED;
  PeerPair pp{};
  for (int r = 0; r < world; ++r) {
    if (!peer_acc_i32[r] || !peer_xscale_f32[r]) return MP_ERR_INVALID_ARG;
    if (!aligned(peer_acc_i32[r], 16)) return MP_ERR_ALIGNMENT;
    pp.acc[r] = peer_acc_i32[r];
    pp.xscale[r] = peer_xscale_f32[r];
  }
  if (!aligned(w_scale_f32, 16) || !aligned(y_f16, 8)) return MP_ERR_ALIGNMENT;
  long long blocks = ((long long)M * (N / 4) + 255) / 256;
  if (blocks > 4 * kSmCount) blocks = 4 * kSmCount;
  w8a8_rowparallel_finish_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const unsigned int*>(flags_u32), world, static_cast<const unsigned int*>(epoch_counter_u32), M, N,
      static_cast<const float*>(w_scale_f32), static_cast<const __half*>(bias_f16), static_cast<__half*>(y_f16),
      error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" size_t mp_moe_ep_plan_ints(int world, int num_local_experts, int capacity_rows) {
  const int max_tiles = capacity_rows / kEpTile;
  const size_t std_ints = (size_t)3 * num_local_experts + 2 + max_tiles;
  return std_ints + (size_t)num_local_experts * (world + 1) + (size_t)num_local_experts * world;
}

extern "C" int mp_moe_ep_plan(const void* const* peer_plan_ptrs, int world, int rank, int num_experts,
                              int capacity_rows, void* xplan_i32, mp_stream_t stream) {
  PeerPtrs pp;
  int rc = fill_peers(pp, peer_plan_ptrs, world);
  if (rc != MP_OK) return rc;
  if (!xplan_i32 || num_experts <= 0 || num_experts % world != 0 || capacity_rows <= 0 || capacity_rows % kMoeSegmentAlign != 0)
    return MP_ERR_INVALID_ARG;
  if (num_experts > 256) return MP_ERR_UNSUPPORTED;   // (local expert, source) pairs are staged in shared memory
  const int e_loc = num_experts / world;
  const int max_tiles = capacity_rows / kEpTile;
  const int ext = 3 * e_loc + 2 + max_tiles;
  ep_plan_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, rank, num_experts, e_loc, max_tiles, ext,
                                                                  static_cast<int*>(xplan_i32));
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_moe_ep_barrier_plan(const void* const* peer_flag_ptrs, const void* const* peer_plan_ptrs, int world,
                                      int rank, void* epoch_counter_u32, int num_experts, int capacity_rows,
                                      void* xplan_i32, int* error_word, mp_stream_t stream) {
  PeerPtrs pf, pp;
  int rc = fill_peers(pf, peer_flag_ptrs, world);
  if (rc != MP_OK) return rc;
  rc = fill_peers(pp, peer_plan_ptrs, world);
  if (rc != MP_OK) return rc;
  if (rank < 0 || rank >= world || !epoch_counter_u32 || !xplan_i32 || num_experts <= 0 || num_experts % world != 0 ||
      capacity_rows <= 0 || capacity_rows % kMoeSegmentAlign != 0)
    return MP_ERR_INVALID_ARG;
  if (num_experts > 256) return MP_ERR_UNSUPPORTED;
  const int e_loc = num_experts / world;
  const int max_tiles = capacity_rows / kEpTile;
  const int ext = 3 * e_loc + 2 + max_tiles;
  return launch_chained(ep_barrier_plan_kernel, dim3(1), dim3(64), 0, static_cast<cudaStream_t>(stream), pf, pp, world,
                        rank, static_cast<unsigned int*>(epoch_counter_u32), num_experts, e_loc, max_tiles, ext,
                        static_cast<int*>(xplan_i32), error_word);
}

extern "C" int mp_moe_ep_pull_part(const void* const* peer_q_ptrs, const void* const* peer_scale_ptrs,
                                   const void* xplan_i32, int world, int num_local_experts, int capacity_rows, int H,
                                   void* q_sorted_i8, void* scale_sorted_f32, int part, mp_stream_t stream) {
  if (part < -1 || part > 1) return MP_ERR_INVALID_ARG;
  PeerPtrs pq, ps;
  int rc = fill_peers(pq, peer_q_ptrs, world);
  if (rc != MP_OK) return rc;
  rc = fill_peers(ps, peer_scale_ptrs, world);
  if (rc != MP_OK) return rc;
  if (!xplan_i32 || !q_sorted_i8 || !scale_sorted_f32 || H <= 0 || H % 16 != 0) return MP_ERR_INVALID_ARG;
  if (num_local_experts > 64) return MP_ERR_UNSUPPORTED;           // the locate tables are staged in shared memory
  const int ext = 3 * num_local_experts + 2 + capacity_rows / kEpTile;
  const int vec = H / 16;
  int grid = (capacity_rows + 7) / 8;                               // one warp per row, at most four blocks per SM
  if (grid > 4 * kSmCount) grid = 4 * kSmCount;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int* xp = static_cast<const int*>(xplan_i32);
  uint4* qd = static_cast<uint4*>(q_sorted_i8);
  float* sd = static_cast<float*>(scale_sorted_f32);
  auto kern = vec == 256 ? ep_pull_kernel<8> : (vec == 128 ? ep_pull_kernel<4> : ep_pull_kernel<0>);
  return launch_chained(kern, dim3(grid), dim3(256), 0, st, pq, ps, xp, world, num_local_experts, ext, vec, qd, sd, part);
}

extern "C" int mp_moe_ep_push_part(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                                   int capacity_rows, int H, const void* const* peer_back_ptrs, int part,
                                   mp_stream_t stream) {
  if (part < -1 || part > 1) return MP_ERR_INVALID_ARG;
  PeerPtrs pb;
  int rc = fill_peers(pb, peer_back_ptrs, world);
  if (rc != MP_OK) return rc;
  if (!d_sorted_f16 || !xplan_i32 || H <= 0 || H % 8 != 0) return MP_ERR_INVALID_ARG;
  if (num_local_experts > 64) return MP_ERR_UNSUPPORTED;
  const int ext = 3 * num_local_experts + 2 + capacity_rows / kEpTile;
  const int vec = H / 8;
  int grid = (capacity_rows + 7) / 8;
  if (grid > 4 * kSmCount) grid = 4 * kSmCount;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint4* dd = static_cast<const uint4*>(d_sorted_f16);
  const int* xp = static_cast<const int*>(xplan_i32);
  auto kern = vec == 512 ? ep_push_kernel<16> : (vec == 256 ? ep_push_kernel<8> : ep_push_kernel<0>);
  return launch_chained(kern, dim3(grid), dim3(256), 0, st, dd, xp, world, num_local_experts, ext, vec, pb, part,
                        EpSignal{});
}

extern "C" int mp_moe_ep_push_signal(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                                     int capacity_rows, int H, const void* const* peer_back_ptrs,
                                     const void* const* peer_flag_ptrs, int rank, void* epoch_counter_u32,
                                     void* block_counter_i32, mp_stream_t stream) {
  PeerPtrs pb;
  EpSignal sig{};
  int rc = fill_peers(pb, peer_back_ptrs, world);
  if (rc != MP_OK) return rc;
  rc = fill_peers(sig.peer_flags, peer_flag_ptrs, world);
  if (rc != MP_OK) return rc;
  if (!d_sorted_f16 || !xplan_i32 || H <= 0 || H % 8 != 0 || rank < 0 || rank >= world || !epoch_counter_u32 ||
      !block_counter_i32)
    return MP_ERR_INVALID_ARG;
  if (num_local_experts > 64) return MP_ERR_UNSUPPORTED;
  sig.epoch_counter = static_cast<unsigned int*>(epoch_counter_u32);
  sig.block_counter = static_cast<int*>(block_counter_i32);
  sig.world = world;
  sig.rank = rank;
  const int ext = 3 * num_local_experts + 2 + capacity_rows / kEpTile;
  const int vec = H / 8;
  int grid = (capacity_rows + 7) / 8;
  if (grid > 4 * kSmCount) grid = 4 * kSmCount;
  auto kern = vec == 512 ? ep_push_kernel<16> : (vec == 256 ? ep_push_kernel<8> : ep_push_kernel<0>);
  return launch_chained(kern, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                        static_cast<const uint4*>(d_sorted_f16), static_cast<const int*>(xplan_i32), world,
                        num_local_experts, ext, vec, pb, -1, sig);
}

extern "C" int mp_moe_ep_pull(const void* const* peer_q_ptrs, const void* const* peer_scale_ptrs, const void* xplan_i32,
                              int world, int num_local_experts, int capacity_rows, int H, void* q_sorted_i8,
                              void* scale_sorted_f32, mp_stream_t stream) {
  return mp_moe_ep_pull_part(peer_q_ptrs, peer_scale_ptrs, xplan_i32, world, num_local_experts, capacity_rows, H,
                             q_sorted_i8, scale_sorted_f32, -1, stream);
}

extern "C" int mp_moe_ep_push(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                              int capacity_rows, int H, const void* const* peer_back_ptrs, mp_stream_t stream) {
  return mp_moe_ep_push_part(d_sorted_f16, xplan_i32, world, num_local_experts, capacity_rows, H, peer_back_ptrs, -1,
                             stream);
}
