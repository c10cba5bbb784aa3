// Small device-driven collectives over NVLink peer memory for the tensor-parallel linears: an all-gather
// of output slices (column-parallel W4A16) and a two-phase all-reduce of fp32 partial sums (row-parallel
// W4A16).  They stand in for the runtime's tensor-parallel all-gather / all-reduce around its linear
// methods (acceleration/runtime_patches/vllm_ascend.patch:3260-3305) at decode sizes, where a library
// collective is all launch latency.
//
// One process per GPU; every buffer named "peer" is symmetric memory mapped by all ranks.  Data moves by
// plain peer stores / loads; a rank announces "my part of call number e is in place" by a system-scope
// release store of e into its slot of every peer's flag array, and waits (bounded: 2 s, then an error word)
// until all its own slots have reached e.  The call number lives in device memory and is advanced by the
// kernels, so no launch argument changes between calls and the launches can be replayed from a CUDA graph.
// Receive buffers are used alternately by call parity: a peer can push call n+1 while this rank still
// reads call n, and cannot push call n+2 before this rank has announced call n+1, i.e. finished call n.
#include "common.cuh"

namespace mp {

namespace {

constexpr int kPcMaxRanks = 16;
constexpr uint64_t kPcWaitNs = 2000000000ull;

struct PcPeers {
  void* p[kPcMaxRanks];
};

__device__ __forceinline__ uint64_t pc_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Threads r < world wait for slot r of this rank's flag array to reach `epoch`; returns false (all threads)
// when a peer did not show up in time.
__device__ __forceinline__ bool pc_wait_all(const unsigned int* my_flags, int world, unsigned int epoch, int* error_word,
                                            int error_code, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const unsigned int* f = my_flags + threadIdx.x;
    const uint64_t t0 = pc_timer_ns();
    for (unsigned int it = 0;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;                         // wrap-safe
      if ((it & 0xFF) == 0xFF && pc_timer_ns() - t0 > kPcWaitNs) {
        *s_ok = 0;
        if (error_word) atomicExch(error_word, error_code);
        break;
      }
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// The grid's last block (by the arrival counter, which it re-arms) publishes `epoch` on every peer.
__device__ __forceinline__ void pc_publish_when_grid_done(int* block_counter, const PcPeers& peer_flags, int world, int rank,
                                                          unsigned int epoch, unsigned int* epoch_counter) {
  __threadfence_system();                                  // this thread's peer stores are visible system-wide ...
  __syncthreads();                                         // ... and so are the whole block's
  if (threadIdx.x == 0) {
    const int blocks = static_cast<int>(gridDim.x);
    if (atomicAdd(block_counter, 1) == blocks - 1) {
      atomicExch(block_counter, 0);                        // re-armed for the next call
      if (epoch_counter) *epoch_counter = epoch;
      __threadfence_system();
      for (int q = 0; q < world; ++q) {
        unsigned int* flag = static_cast<unsigned int*>(peer_flags.p[q]) + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
      }
    }
  }
}

__device__ __forceinline__ uint4 pc_ld_l2(const void* p) {        // peers wrote it: read from L2, not a stale L1 line
  uint4 r;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// ---- all-gather of row slices -----------------------------------------------------------------------------
// src [rows][slice_bytes] (this rank's columns) -> every peer's gather[parity][rows][world * slice_bytes] at column
// offset rank * slice_bytes; then wait for all ranks and copy this rank's gathered buffer to `out`.
__global__ void __launch_bounds__(256)
peer_allgather_push_kernel(const unsigned char* __restrict__ src, int rows, int slice_bytes, PcPeers gather0,
                           PcPeers gather1, PcPeers peer_flags, unsigned int* epoch_counter, int* block_counter,
                           int world, int rank, unsigned char* __restrict__ out, int* error_word) {
  __shared__ int s_ok;
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(epoch_counter) + 1u;
  const PcPeers& gather = (epoch & 1u) ? gather1 : gather0;
  const int cpr = slice_bytes >> 4;                          // 16-byte chunks per slice row
  const size_t pitch = (size_t)world * slice_bytes;
  const int stride = gridDim.x * blockDim.x;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < rows * cpr; c += stride) {
    const int m = c / cpr, j = c - m * cpr;
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)c * 16);
    const size_t off = (size_t)m * pitch + (size_t)rank * slice_bytes + (size_t)j * 16;
    for (int q = 0; q < world; ++q) *reinterpret_cast<uint4*>(static_cast<unsigned char*>(gather.p[q]) + off) = v;
  }
  pc_publish_when_grid_done(block_counter, peer_flags, world, rank, epoch, epoch_counter);
  if (!pc_wait_all(static_cast<const unsigned int*>(peer_flags.p[rank]), world, epoch, error_word, 7, &s_ok)) return;
  const unsigned char* mine = static_cast<const unsigned char*>(gather.p[rank]);
  const int total = static_cast<int>((size_t)rows * pitch >> 4);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride)
    *reinterpret_cast<uint4*>(out + (size_t)c * 16) = pc_ld_l2(mine + (size_t)c * 16);
}

// ---- two-phase all-reduce of the row-parallel decode linear ---------------------------------------------
// partial[parity][r]: rank r's fp32 partial sums [M][N] (announced by the decode kernel through `arrival`).
// Phase 1: this rank adds the P partials of ITS N/P columns in rank order (+ bias), rounds to fp16 and stores
// the slice into every rank's gather[parity][M][N].  Phase 2: wait for all slices, copy to y.  Every output
// element is computed once, by its owner, so all ranks hold the same bits; a rank reads 4 M N (P-1)/P bytes
// over NVLink instead of 4 M N (P-1).
struct PcPartials {
  const float* p[2][kPcMaxRanks];
};

__global__ void __launch_bounds__(256)
rowparallel_finish2_kernel(PcPartials partial, const unsigned int* __restrict__ arrival, PcPeers gather0, PcPeers gather1,
                           PcPeers peer_flags2, const unsigned int* __restrict__ epoch_counter, int* block_counter,
                           int world, int rank, int M, int N, const __half* __restrict__ bias, __half* __restrict__ y,
                           int* error_word) {
  __shared__ int s_ok;
  const unsigned int epoch = *epoch_counter;                 // advanced by the decode kernel that ran before this one
  const float* const* src = partial.p[epoch & 1u];
  const PcPeers& gather = (epoch & 1u) ? gather1 : gather0;
  if (!pc_wait_all(arrival, world, epoch, error_word, 5, &s_ok)) return;
  const int n_loc = N / world, quads = n_loc >> 2, n0 = rank * n_loc;
  const int stride = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += stride) {
    const int m = i / quads, n = n0 + ((i - m * quads) << 2);
    float4 v[kPcMaxRanks];
#pragma unroll
    for (int r = 0; r < kPcMaxRanks; ++r)                    // all loads in flight before the first add
      if (r < world) v[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)m * N + n);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kPcMaxRanks; ++r)
      if (r < world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
    if (bias) {
      acc.x += h2f(bias[n]); acc.y += h2f(bias[n + 1]); acc.z += h2f(bias[n + 2]); acc.w += h2f(bias[n + 3]);
    }
    const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
    const uint2 o = make_uint2(h2_as_u32(lo), h2_as_u32(hi));
    for (int q = 0; q < world; ++q)
      *reinterpret_cast<uint2*>(static_cast<__half*>(gather.p[q]) + (size_t)m * N + n) = o;
  }
  pc_publish_when_grid_done(block_counter, peer_flags2, world, rank, epoch, nullptr);
  if (!pc_wait_all(static_cast<const unsigned int*>(peer_flags2.p[rank]), world, epoch, error_word, 5, &s_ok)) return;
  const unsigned char* mine = static_cast<const unsigned char*>(gather.p[rank]);
  const int total = static_cast<int>((size_t)M * N * 2 >> 4);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride)
    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(y) + (size_t)c * 16) = pc_ld_l2(mine + (size_t)c * 16);
}

// ---- publish: copy up to two local ranges into this rank's receive slot of the call's parity, then announce ---
// The producer kernels (a GEMM, an activation quantiser) write to ordinary local buffers; the slot peers read
// is chosen here, on the device, from the call number -- so a captured graph that contains an odd number of
// calls still alternates slots from replay to replay.
__global__ void __launch_bounds__(256)
peer_publish_kernel(const unsigned char* __restrict__ src_a, int bytes_a, int off_a, const unsigned char* __restrict__ src_b,
                    int bytes_b, int off_b, unsigned char* slot0, unsigned char* slot1, PcPeers peer_flags,
                    unsigned int* epoch_counter, int* block_counter, int world, int rank) {
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(epoch_counter) + 1u;
  unsigned char* slot = (epoch & 1u) ? slot1 : slot0;
  const int stride = gridDim.x * blockDim.x, t = blockIdx.x * blockDim.x + threadIdx.x;
  for (int c = t; c < (bytes_a >> 4); c += stride)
    *reinterpret_cast<uint4*>(slot + off_a + (size_t)c * 16) = *reinterpret_cast<const uint4*>(src_a + (size_t)c * 16);
  for (int c = t; c < (bytes_b >> 2); c += stride)
    *reinterpret_cast<uint32_t*>(slot + off_b + (size_t)c * 4) = *reinterpret_cast<const uint32_t*>(src_b + (size_t)c * 4);
  pc_publish_when_grid_done(block_counter, peer_flags, world, rank, epoch, epoch_counter);
}

struct PcPair {
  const void* acc[2][kPcMaxRanks];
  const void* xscale[2][kPcMaxRanks];
};

// y[m, n] = f16(sum_r float(acc_r[m, n]) * xscale_r[m] * wscale[n] (+ bias)): each product rounded on its own,
// fp32 adds in rank order, one rounding to fp16 -- the same bits on every rank.  The slot parity is the call
// number's (already advanced by this rank's publish kernel).
__global__ void __launch_bounds__(256)
w8a8_rowparallel_finish_parity_kernel(PcPair peers, const unsigned int* __restrict__ flags, int world,
                                      const unsigned int* __restrict__ epoch_counter, int M, int N,
                                      const float* __restrict__ w_scale, const __half* __restrict__ bias,
                                      __half* __restrict__ y, int* error_word) {
  __shared__ int s_ok;
  const unsigned int epoch = *epoch_counter;
  if (!pc_wait_all(flags, world, epoch, error_word, 5, &s_ok)) return;
  const void* const* accs = peers.acc[epoch & 1u];
  const void* const* scales = peers.xscale[epoch & 1u];
  const int quads = N >> 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += gridDim.x * blockDim.x) {
    const int m = i / quads, n = (i - m * quads) << 2;
    const float4 sw = *reinterpret_cast<const float4*>(w_scale + n);
    int4 a[kPcMaxRanks];
    float sx[kPcMaxRanks];
#pragma unroll
    for (int r = 0; r < kPcMaxRanks; ++r)                    // all loads in flight before the first add
      if (r < world) {
        a[r] = *reinterpret_cast<const int4*>(static_cast<const int*>(accs[r]) + (size_t)m * N + n);
        sx[r] = static_cast<const float*>(scales[r])[m];
      }
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kPcMaxRanks; ++r)
      if (r < world) {
        sum.x = __fadd_rn(sum.x, __fmul_rn(__fmul_rn(static_cast<float>(a[r].x), sx[r]), sw.x));
        sum.y = __fadd_rn(sum.y, __fmul_rn(__fmul_rn(static_cast<float>(a[r].y), sx[r]), sw.y));
        sum.z = __fadd_rn(sum.z, __fmul_rn(__fmul_rn(static_cast<float>(a[r].z), sx[r]), sw.z));
        sum.w = __fadd_rn(sum.w, __fmul_rn(__fmul_rn(static_cast<float>(a[r].w), sx[r]), sw.w));
      }
    if (bias) {
      sum.x = __fadd_rn(sum.x, h2f(bias[n])); sum.y = __fadd_rn(sum.y, h2f(bias[n + 1]));
      sum.z = __fadd_rn(sum.z, h2f(bias[n + 2])); sum.w = __fadd_rn(sum.w, h2f(bias[n + 3]));
    }
    const __half2 lo = __floats2half2_rn(sum.x, sum.y), hi = __floats2half2_rn(sum.z, sum.w);
    *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = make_uint2(h2_as_u32(lo), h2_as_u32(hi));
  }
}

int pc_fill(PcPeers& dst, const void* const* src, int world) {
  if (!src || world <= 0 || world > kPcMaxRanks) return MP_ERR_INVALID_ARG;
  for (int i = 0; i < kPcMaxRanks; ++i) dst.p[i] = i < world ? const_cast<void*>(src[i]) : nullptr;
  for (int i = 0; i < world; ++i) {
    if (!dst.p[i]) return MP_ERR_INVALID_ARG;
    if (!aligned(dst.p[i], 16)) return MP_ERR_ALIGNMENT;
  }
  return MP_OK;
}

// few blocks: the waits inside the kernels assume the whole grid is resident
int pc_grid(int work_items) {
  int blocks = (work_items + 255) / 256;
  return blocks < 1 ? 1 : (blocks > 32 ? 32 : blocks);
}

}  // namespace
}  // namespace mp

using namespace mp;

extern "C" int mp_peer_allgather_push(const void* src, int rows, int slice_bytes, void* const* peer_gather0,
                                      void* const* peer_gather1, void* const* peer_flags_u32, void* epoch_counter_u32,
                                      int* block_counter, int world, int rank, void* out, int* error_word,
                                      mp_stream_t stream) {
  if (!src || !out || !epoch_counter_u32 || !block_counter || rows <= 0 || slice_bytes <= 0) return MP_ERR_INVALID_ARG;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (slice_bytes % 16 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(src, 16) || !aligned(out, 16)) return MP_ERR_ALIGNMENT;
  PcPeers g0, g1, pf;
  int rc = pc_fill(g0, peer_gather0, world);
  if (rc != MP_OK) return rc;
  if ((rc = pc_fill(g1, peer_gather1, world)) != MP_OK) return rc;
  if ((rc = pc_fill(pf, peer_flags_u32, world)) != MP_OK) return rc;
  const int grid = pc_grid(rows * (slice_bytes / 16) * world);
  peer_allgather_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(src), rows, slice_bytes, g0, g1, pf, static_cast<unsigned int*>(epoch_counter_u32),
      block_counter, world, rank, static_cast<unsigned char*>(out), error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w4a16_rowparallel_finish2(void* const* peer_partial0_f32, void* const* peer_partial1_f32,
                                            const void* arrival_flags_u32, void* const* peer_gather0_f16,
                                            void* const* peer_gather1_f16, void* const* peer_flags2_u32,
                                            int* block_counter, int world, int rank, const void* epoch_counter_u32, int M,
                                            int N, const void* bias_f16, void* y_f16, int* error_word,
                                            mp_stream_t stream) {
  if (!arrival_flags_u32 || !epoch_counter_u32 || !block_counter || !y_f16 || M <= 0 || N <= 0) return MP_ERR_INVALID_ARG;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (world > kPcMaxRanks || N % world != 0 || (N / world) % 4 != 0 || ((size_t)M * N * 2) % 16 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(y_f16, 16)) return MP_ERR_ALIGNMENT;
  PcPeers p0, p1, g0, g1, pf2;
  int rc = pc_fill(p0, peer_partial0_f32, world);
  if (rc != MP_OK) return rc;
  if ((rc = pc_fill(p1, peer_partial1_f32, world)) != MP_OK) return rc;
  if ((rc = pc_fill(g0, peer_gather0_f16, world)) != MP_OK) return rc;
  if ((rc = pc_fill(g1, peer_gather1_f16, world)) != MP_OK) return rc;
  if ((rc = pc_fill(pf2, peer_flags2_u32, world)) != MP_OK) return rc;
  PcPartials pp{};
  for (int r = 0; r < world; ++r) {
    pp.p[0][r] = static_cast<const float*>(p0.p[r]);
    pp.p[1][r] = static_cast<const float*>(p1.p[r]);
  }
  const int grid = pc_grid(M * N / 8);
  rowparallel_finish2_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const unsigned int*>(arrival_flags_u32), g0, g1, pf2,
      static_cast<const unsigned int*>(epoch_counter_u32), block_counter, world, rank, M, N,
      static_cast<const __half*>(bias_f16), static_cast<__half*>(y_f16), error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_peer_publish(const void* src_a, int bytes_a, int offset_a, const void* src_b, int bytes_b, int offset_b,
                               void* slot0, void* slot1, void* const* peer_flags_u32, void* epoch_counter_u32,
                               int* block_counter, int world, int rank, mp_stream_t stream) {
  if (!src_a || !slot0 || !slot1 || !epoch_counter_u32 || !block_counter || bytes_a <= 0 || bytes_b < 0 || offset_a < 0 ||
      offset_b < 0 || (bytes_b > 0 && !src_b))
    return MP_ERR_INVALID_ARG;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (bytes_a % 16 != 0 || offset_a % 16 != 0 || bytes_b % 4 != 0 || offset_b % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(src_a, 16) || !aligned(slot0, 16) || !aligned(slot1, 16) || (src_b && !aligned(src_b, 4))) return MP_ERR_ALIGNMENT;
  PcPeers pf;
  const int rc = pc_fill(pf, peer_flags_u32, world);
  if (rc != MP_OK) return rc;
  const int grid = pc_grid(bytes_a / 16);
  peer_publish_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(src_a), bytes_a, offset_a, static_cast<const unsigned char*>(src_b), bytes_b,
      offset_b, static_cast<unsigned char*>(slot0), static_cast<unsigned char*>(slot1), pf,
      static_cast<unsigned int*>(epoch_counter_u32), block_counter, world, rank);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w8a8_rowparallel_finish_parity(const void* const* peer_acc0_i32, const void* const* peer_acc1_i32,
                                                 const void* const* peer_xscale0_f32, const void* const* peer_xscale1_f32,
                                                 const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                                                 int N, const void* w_scale_f32, const void* bias_f16, void* y_f16,
                                                 int* error_word, mp_stream_t stream) {
  if (!peer_acc0_i32 || !peer_acc1_i32 || !peer_xscale0_f32 || !peer_xscale1_f32 || !flags_u32 || !epoch_counter_u32 ||
      !w_scale_f32 || !y_f16 || world < 1 || world > kPcMaxRanks || M <= 0 || N <= 0)
    return MP_ERR_INVALID_ARG;
  if (N % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(y_f16, 8) || !aligned(w_scale_f32, 16)) return MP_ERR_ALIGNMENT;
  PcPair pp{};
  for (int r = 0; r < world; ++r) {
    const void* ptrs[4] = {peer_acc0_i32[r], peer_acc1_i32[r], peer_xscale0_f32[r], peer_xscale1_f32[r]};
    for (const void* q : ptrs)
      if (!q) return MP_ERR_INVALID_ARG;
    if (!aligned(ptrs[0], 16) || !aligned(ptrs[1], 16)) return MP_ERR_ALIGNMENT;
    pp.acc[0][r] = ptrs[0]; pp.acc[1][r] = ptrs[1];
    pp.xscale[0][r] = ptrs[2]; pp.xscale[1][r] = ptrs[3];
  }
  int blocks = (M * (N / 4) + 255) / 256;
  if (blocks > kSmCount) blocks = kSmCount;
  w8a8_rowparallel_finish_parity_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const unsigned int*>(flags_u32), world, static_cast<const unsigned int*>(epoch_counter_u32), M, N,
      static_cast<const float*>(w_scale_f32), static_cast<const __half*>(bias_f16), static_cast<__half*>(y_f16), error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}
