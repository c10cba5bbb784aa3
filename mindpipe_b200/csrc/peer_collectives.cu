// Small device-driven collectives over NVLink peer memory for the tensor-parallel linears: an all-gather
// of output slices (column-parallel W4A16), a reduce-scatter + all-gather of fp32 partial sums (row-parallel
// W4A16), and the slot publication of the row-parallel W8A8 linear.  They stand in for the runtime's tensor-parallel all-gather / all-reduce around its linear
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

bool decode_programmatic_launch();   // w4a16_decode_tma.cu: the process-wide programmatic-dependent-launch switch

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

// ---- flag-in-data transfers ------------------------------------------------------------------------------
// A message that is announced by a separate arrival word costs a full NVLink round trip before the word may
// be stored (the system-scope fence waits for the data stores to be acknowledged) plus the word's own flight.
// At decode sizes that is most of the collective.  Here every 8 bytes on the wire carry 4 bytes of payload and
// the call number (the low-latency form of a library collective's wire protocol): a 16-byte store holds
// {w0, epoch, w1, epoch}; the receiver polls the very words it needs until both numbers match and no fence,
// arrival word or grid-wide step is needed.  8-byte halves of a store are never torn, and a slot is reused
// only two calls later with a different number, so a stale word cannot be mistaken for a fresh one.
__device__ __forceinline__ void ll_store(void* p, uint32_t w0, uint32_t w1, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w0), "r"(epoch), "r"(w1), "r"(epoch)
               : "memory");
}

struct LlWait {
  uint64_t t0;
  bool ok;
};

// Polls one 16-byte unit until both call numbers equal `epoch` (bounded); false after a timeout.
__device__ __forceinline__ bool ll_load(const void* p, uint32_t epoch, uint32_t& w0, uint32_t& w1, LlWait& w) {
  if (!w.ok) { w0 = w1 = 0; return false; }
  for (unsigned int it = 0;; ++it) {
    uint32_t e0, e1;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w0), "=r"(e0), "=r"(w1), "=r"(e1) : "l"(p) : "memory");
    if (e0 == epoch && e1 == epoch) return true;
    if ((it & 0x3FF) == 0x3FF && pc_timer_ns() - w.t0 > kPcWaitNs) {
      w.ok = false;
      w0 = w1 = 0;
      return false;
    }
  }
}

// The grid's last block (by the arrival counter, which it re-arms) stores the new call number.
__device__ __forceinline__ void pc_count_call(int* block_counter, unsigned int* epoch_counter, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(block_counter, 1) == static_cast<int>(gridDim.x) - 1) {
    atomicExch(block_counter, 0);
    *epoch_counter = epoch;
  }
}

// ---- all-gather of row slices -----------------------------------------------------------------------------
// src [rows][slice_bytes] (this rank's columns) -> every peer's receive buffer of the call's parity,
// [rows][world][slice_bytes * 2] in the flag-in-data form; this rank's own slice goes straight to `out`
// [rows][world * slice_bytes], the others are polled out of the local receive buffer.
__global__ void __launch_bounds__(256)
peer_allgather_push_kernel(const unsigned char* __restrict__ src, int rows, int slice_bytes, PcPeers recv0,
                           PcPeers recv1, unsigned int* epoch_counter, int* block_counter, int world, int rank,
                           unsigned char* __restrict__ out, int* error_word) {
  // under programmatic dependent launch: wait for the producer of `src`, then let the next kernel of the stream
  // begin its own prologue (e.g. a decode linear's weight fetch) while this one is on the wire
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(epoch_counter) + 1u;
  const PcPeers& recv = (epoch & 1u) ? recv1 : recv0;
  const int cpr = slice_bytes >> 4;                          // 16-byte payload chunks per slice row
  const size_t out_pitch = (size_t)world * slice_bytes;
  const int stride = gridDim.x * blockDim.x, tid = blockIdx.x * blockDim.x + threadIdx.x;
  for (int c = tid; c < rows * cpr; c += stride) {
    const int m = c / cpr, j = c - m * cpr;
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)c * 16);
    const size_t off = (((size_t)m * world + rank) * cpr + j) * 32;      // 32 wire bytes per payload chunk
    for (int q = 0; q < world; ++q) {
      if (q == rank) continue;
      unsigned char* dst = static_cast<unsigned char*>(recv.p[q]) + off;
      ll_store(dst, v.x, v.y, epoch);
      ll_store(dst + 16, v.z, v.w, epoch);
    }
    *reinterpret_cast<uint4*>(out + (size_t)m * out_pitch + (size_t)rank * slice_bytes + (size_t)j * 16) = v;
  }
  LlWait w{pc_timer_ns(), true};
  const unsigned char* mine = static_cast<const unsigned char*>(recv.p[rank]);
  const int others = world - 1;
  for (int c = tid; c < rows * others * cpr; c += stride) {
    const int m = c / (others * cpr), rem = c - m * (others * cpr);
    int r = rem / cpr;
    const int j = rem - r * cpr;
    r += (r >= rank);                                        // skip this rank's own slice
    const unsigned char* p = mine + (((size_t)m * world + r) * cpr + j) * 32;
    uint4 v;
    ll_load(p, epoch, v.x, v.y, w);
    ll_load(p + 16, epoch, v.z, v.w, w);
    if (w.ok) *reinterpret_cast<uint4*>(out + (size_t)m * out_pitch + (size_t)r * slice_bytes + (size_t)j * 16) = v;
  }
  if (!w.ok && error_word) atomicExch(error_word, 7);
  pc_count_call(block_counter, epoch_counter, epoch);
}

// ---- all-reduce of the row-parallel decode linear: reduce-scatter, then all-gather, both flag-in-data -------
// partial: this rank's fp32 partial sums [M][N] (written by the decode kernel that ran before on the stream).
// Step 1: the columns that rank q owns (N / P of them) are sent to q's receive buffer
//         recv1[parity][this rank][M][N / P] (8 wire bytes per sum).
// Step 2: for its own columns this rank polls the P - 1 peers' sums, adds all P in rank order (+ bias), rounds
//         to fp16, writes y and sends the fp16 pairs to every peer's recv2[parity][M][N] (8 wire bytes per pair).
// Step 3: the other ranks' columns are polled out of recv2 into y.
// Every output element is computed once, by its owner, in a fixed order: the same bits on all ranks.  A rank
// sends 4 M N (P-1)/P * 2 bytes in step 1 and 2 M N (P-1)/P * 2 bytes in step 2, and waits twice for one
// one-way flight -- no acknowledged fence, no arrival words.
__global__ void __launch_bounds__(256)
rowparallel_finish_ll_kernel(const float* __restrict__ partial0, const float* __restrict__ partial1, PcPeers recv1_0,
                             PcPeers recv1_1, PcPeers recv2_0, PcPeers recv2_1,
                             const unsigned int* __restrict__ epoch_counter, int world, int rank, int M, int N,
                             const __half* __restrict__ bias, __half* __restrict__ y, int* error_word) {
  asm volatile("griddepcontrol.wait;" ::: "memory");         // the decode kernel's partial sums and call number
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned int epoch = *epoch_counter;                 // advanced by the decode kernel that ran before this one
  const float* partial = (epoch & 1u) ? partial1 : partial0;
  const PcPeers& recv1 = (epoch & 1u) ? recv1_1 : recv1_0;
  const PcPeers& recv2 = (epoch & 1u) ? recv2_1 : recv2_0;
  const int n_loc = N / world, quads_loc = n_loc >> 2, quads = N >> 2;
  const int stride = gridDim.x * blockDim.x, tid = blockIdx.x * blockDim.x + threadIdx.x;
  // step 1: scatter the peers' columns
  for (int i = tid; i < M * quads; i += stride) {
    const int m = i / quads, n = (i - m * quads) << 2;
    const int q = n / n_loc;
    if (q == rank) continue;
    const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)m * N + n);
    unsigned char* dst = static_cast<unsigned char*>(recv1.p[q]) +
                         (((size_t)rank * M + m) * n_loc + (n - q * n_loc)) * 8;
    ll_store(dst, __float_as_uint(v.x), __float_as_uint(v.y), epoch);
    ll_store(dst + 16, __float_as_uint(v.z), __float_as_uint(v.w), epoch);
  }
  LlWait w{pc_timer_ns(), true};
  // step 2: reduce this rank's columns
  const unsigned char* in1 = static_cast<const unsigned char*>(recv1.p[rank]);
  for (int i = tid; i < M * quads_loc; i += stride) {
    const int m = i / quads_loc, nl = (i - m * quads_loc) << 2, n = rank * n_loc + nl;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      float4 v;
      if (r == rank) {
        v = *reinterpret_cast<const float4*>(partial + (size_t)m * N + n);
      } else {
        const unsigned char* p = in1 + (((size_t)r * M + m) * n_loc + nl) * 8;
        uint32_t a, b, c, d;
        ll_load(p, epoch, a, b, w);
        ll_load(p + 16, epoch, c, d, w);
        v = make_float4(__uint_as_float(a), __uint_as_float(b), __uint_as_float(c), __uint_as_float(d));
      }
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
      acc.x += h2f(bias[n]); acc.y += h2f(bias[n + 1]); acc.z += h2f(bias[n + 2]); acc.w += h2f(bias[n + 3]);
    }
    const uint32_t lo = h2_as_u32(__floats2half2_rn(acc.x, acc.y)), hi = h2_as_u32(__floats2half2_rn(acc.z, acc.w));
    if (!w.ok) continue;                                     // a peer never showed up: send nothing half-made
    *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = make_uint2(lo, hi);
    const size_t off = ((size_t)m * N + n) * 4;             // 8 wire bytes per fp16 pair
    for (int q = 0; q < world; ++q)
      if (q != rank) ll_store(static_cast<unsigned char*>(recv2.p[q]) + off, lo, hi, epoch);
  }
  // step 3: collect the other ranks' columns
  const unsigned char* in2 = static_cast<const unsigned char*>(recv2.p[rank]);
  for (int i = tid; i < M * quads; i += stride) {
    const int m = i / quads, n = (i - m * quads) << 2;
    if (n / n_loc == rank) continue;
    uint32_t lo, hi;
    if (ll_load(in2 + ((size_t)m * N + n) * 4, epoch, lo, hi, w))
      *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = make_uint2(lo, hi);
  }
  if (!w.ok && error_word) atomicExch(error_word, 5);
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



// Launch with the programmatic-stream-serialization attribute when the switch is on: the kernel may then be
// scheduled while the previous kernel of the stream drains (it waits for it with griddepcontrol.wait).
template <typename... KArgs, typename... Args>
int pc_launch(void (*kernel)(KArgs...), int grid, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = decode_programmatic_launch() ? 1 : 0;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
  return MP_OK;
}

// at most one block per SM: peers wait on what every block of the grid stores, so the whole grid is resident
int pc_grid(int work_items) {
  int blocks = (work_items + 255) / 256;
  return blocks < 1 ? 1 : (blocks > kSmCount ? kSmCount : blocks);
}

}  // namespace
}  // namespace mp

using namespace mp;

extern "C" size_t mp_peer_allgather_recv_bytes(int rows, int slice_bytes, int world) {
  if (rows <= 0 || slice_bytes <= 0 || world <= 0) return 0;
  return (size_t)rows * world * slice_bytes * 2;
}

extern "C" int mp_peer_allgather_push(const void* src, int rows, int slice_bytes, void* const* peer_recv0,
                                      void* const* peer_recv1, void* epoch_counter_u32, int* block_counter, int world,
                                      int rank, void* out, int* error_word, mp_stream_t stream) {
  if (!src || !out || !epoch_counter_u32 || !block_counter || rows <= 0 || slice_bytes <= 0) return MP_ERR_INVALID_ARG;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (slice_bytes % 16 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(src, 16) || !aligned(out, 16)) return MP_ERR_ALIGNMENT;
  PcPeers r0, r1;
  int rc = pc_fill(r0, peer_recv0, world);
  if (rc != MP_OK) return rc;
  if ((rc = pc_fill(r1, peer_recv1, world)) != MP_OK) return rc;
  const int grid = pc_grid(rows * (slice_bytes / 16) * (world > 1 ? world - 1 : 1));
  return pc_launch(peer_allgather_push_kernel, grid, static_cast<cudaStream_t>(stream),
                   static_cast<const unsigned char*>(src), rows, slice_bytes, r0, r1,
                   static_cast<unsigned int*>(epoch_counter_u32), block_counter, world, rank,
                   static_cast<unsigned char*>(out), error_word);
}

extern "C" size_t mp_w4a16_rowparallel_recv_bytes(int M, int N, int which) {
  if (M <= 0 || N <= 0) return 0;
  return which == 1 ? (size_t)M * N * 8 : (size_t)M * N * 4;
}

extern "C" int mp_w4a16_rowparallel_finish_ll(const void* partial0_f32, const void* partial1_f32,
                                              void* const* peer_recv1_0, void* const* peer_recv1_1,
                                              void* const* peer_recv2_0, void* const* peer_recv2_1, int world, int rank,
                                              const void* epoch_counter_u32, int M, int N, const void* bias_f16,
                                              void* y_f16, int* error_word, mp_stream_t stream) {
  if (!partial0_f32 || !partial1_f32 || !epoch_counter_u32 || !y_f16 || M <= 0 || N <= 0) return MP_ERR_INVALID_ARG;
  if (rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (world > kPcMaxRanks || N % world != 0 || (N / world) % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(y_f16, 8) || !aligned(partial0_f32, 16) || !aligned(partial1_f32, 16)) return MP_ERR_ALIGNMENT;
  PcPeers a0, a1, b0, b1;
  int rc = pc_fill(a0, peer_recv1_0, world);
  if (rc != MP_OK) return rc;
  if ((rc = pc_fill(a1, peer_recv1_1, world)) != MP_OK) return rc;
  if ((rc = pc_fill(b0, peer_recv2_0, world)) != MP_OK) return rc;
  if ((rc = pc_fill(b1, peer_recv2_1, world)) != MP_OK) return rc;
  int grid = (M * (N / 4) + 255) / 256;
  if (grid > kSmCount) grid = kSmCount;                      // one resident wave: peers wait on every block's stores
  return pc_launch(rowparallel_finish_ll_kernel, grid, static_cast<cudaStream_t>(stream),
                   static_cast<const float*>(partial0_f32), static_cast<const float*>(partial1_f32), a0, a1, b0, b1,
                   static_cast<const unsigned int*>(epoch_counter_u32), world, rank, M, N,
                   static_cast<const __half*>(bias_f16), static_cast<__half*>(y_f16), error_word);
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
