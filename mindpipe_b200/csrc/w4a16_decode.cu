// W4A16 decode-shaped linear (M <= 64): y = x @ dequant(W)^T, streaming the
// packed weights once at HBM rate.
//
// Work split: a block owns ROWS_PER_BLOCK output rows and one slice of K; its
// warps are arranged WN (rows) x 4 (K).  A warp step covers 32 rows x 128
// columns: every lane fetches, per 8-row group, one 128-bit word vector (32
// codes of one row) with a no-allocate streaming load plus one (scale, zero)
// pair, dequantises in registers (dequant8) and feeds the result straight
// into mma.sync m16n8k16 as the B fragment -- the weights never touch shared
// memory.  The packed nibble order makes dequant8 emit column pairs
// (k, k+4); instead of shuffling them, the activations are staged in shared
// memory with the same permutation, in fragment order, so each A fragment is
// one conflict-free 128-bit load that is reused across the four row groups.
// Partial sums are reduced across the K-warps in shared memory, then across
// the K slices through a workspace: every block stores its partial tile,
// bumps a per-row-block counter, and the block that arrives last adds the
// slices in a fixed order (deterministic), adds the bias, writes fp16 and
// re-arms the counter for the next call.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

#ifndef MP_TRACE_POINT
#define MP_TRACE_POINT(i)   // debugging builds may record a timestamp here
#endif

namespace mp {

// TMA-fed kernel for M <= 16 (w4a16_decode_tma.cu)
// pdl_choice: -1 = the process-wide setting, 0 / 1 = programmatic dependent launch off / on for this call
int launch_decode_tma(const void* x, const void* packed, const void* sz, const void* bias, void* y, int M, int N, int K,
                      int group, cudaStream_t st, const DecodePush* push = nullptr, int pdl_choice = -1);
void set_decode_programmatic_launch(bool on);
bool decode_programmatic_launch();
int read_and_clear_decode_error(int* value);
// tcgen05 kernel for M <= 16 with the weights as the tensor-memory operand (w4a16_decode_umma.cu)
int launch_decode_umma(const void* x, const void* packed, const void* sz, const void* bias, void* y, int M, int N, int K,
                       int group, void* workspace, size_t workspace_bytes, cudaStream_t st, bool pdl);
size_t decode_umma_workspace_bytes(int M);   // M <= 64: the activation tile is 16, 32 or 64 token rows
// Which kernel serves M <= 16 when a call does not say: one of the MP_DECODE_KERNEL_* values.  Shapes the
// chosen one does not take fall through to the next.
static int g_decode_kernel = MP_DECODE_KERNEL_AUTO;

// AUTO: the tcgen05 kernel for 9 to 16 tokens (below that the mma.sync kernel's folded scales are cheaper
// still) on weights of at least 40 MiB packed with at least 128 row blocks -- the shapes where the mma.sync
// kernel cannot cut K without a second wave and stream-K's even split pays (28672x8192, M = 16: 43.9 vs
// 52.2 us; 22016x4096: 23.4 vs 26.3 us, and 66.1 vs 69.4 us per 7B layer set when the fused gate/up
// projection alone takes it).  With fewer row blocks the mma.sync kernel's one-wave cluster split is as
// fast or faster (8192x28672: 45.1 vs 46.3 us; 8192x8192: 16.2 vs 21.9 us; 12288x4096 inside the layer
// set: 71.1 us per set when it also goes to the tcgen05 kernel).
static int decode_kernel_for(int kind, int M, int N, int K, bool have_workspace) {
  if (kind != MP_DECODE_KERNEL_AUTO) return kind;
  if (have_workspace && M > 8 && N >= 16384 && (size_t)N * (size_t)K / 2 >= (size_t)40 << 20) return MP_DECODE_KERNEL_UMMA;
  return MP_DECODE_KERNEL_MMA_SYNC;
}

// 17..64 rows: the tcgen05 kernel with a 32- or 64-token activation tile streams the weights once, where the
// register-streaming kernel re-reads its activations per chunk; taken when the call names it.
// AUTO (measured against the split-K tensor-core GEMM, chains under programmatic dependent launch): up to 32
// rows on at least 24 MiB of packed weights with at least 8192 output rows (28672x8192: 54 vs 98 us, 22016x4096:
// 31 vs 53, 8192x28672: 58 vs 90, 12288x4096: 24 vs 26; 4096x11008 loses 35 vs 24), and 33..64 rows on the
// 70B-sized weights of the M <= 16 rule (28672x8192: 83 vs 98, 22016x4096: 47 vs 53; 8192x8192 loses 53 vs 33).
static bool umma_above_16_rows(int kind, int M, int N, int K) {
  if (kind == MP_DECODE_KERNEL_UMMA) return true;
  if (kind != MP_DECODE_KERNEL_AUTO) return false;
  const size_t packed = (size_t)N * (size_t)K / 2;
  if (M <= 32) return N >= 8192 && packed >= ((size_t)24 << 20);
  return N >= 16384 && packed >= ((size_t)40 << 20);
}

constexpr int kWarpsK = 4;        // warps along K inside a block
constexpr int kRowGroups = 4;     // 8-row groups per warp -> 32 rows per warp
constexpr int kChunk = 128;       // columns one warp step covers

struct DecodeParams {
  const __half* x;
  const uint32_t* packed;
  const uint32_t* sz;     // [K/group, N] (scale, zero) f16 pairs
  const __half* bias;
  __half* y;
  float* partials;        // [k_split, M, N]
  int* counters;          // one per row block
  int M, N, K, group;
  int chunks;             // K / 128
  int chunks_per_split;
  int k_split;
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MB: 16-row token blocks held per warp; HALF: only token rows 0..7 exist
// (M <= 8, MB == 1); WN: warps along the row dimension; STAGE: chunks of
// activations staged in shared memory at a time (multiple of 4).
template <int MB, bool HALF, int WN, int STAGE>
__global__ void __launch_bounds__(WN * kWarpsK * 32)
w4a16_decode_kernel(const DecodeParams p) {
  constexpr int THREADS = WN * kWarpsK * 32;
  constexpr int ROWS = WN * 32;                    // output rows per block
  constexpr int HR = HALF ? 1 : 2;                 // 8-row halves per token block
  constexpr int TOK = MB * HR * 8;                 // token rows staged
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);                      // STAGE*4*MB*HR*32 units
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)STAGE * 4 * MB * HR * 32 * 16);
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wk = warp % kWarpsK, wn = warp / kWarpsK;
  const int row0 = blockIdx.x * ROWS + wn * 32;    // first output row of this warp
  const int split = blockIdx.y;
  const int cs = split * p.chunks_per_split;
  const int ce = min(p.chunks, cs + p.chunks_per_split);
  const int words_per_row = p.K >> 3;

  float acc[MB][kRowGroups][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int r = 0; r < kRowGroups; ++r)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mb][r][i] = 0.0f;

  uint4 qn[kRowGroups];
  uint32_t szn[kRowGroups];
  auto prefetch = [&](int chunk) {
    const int kabs = chunk * kChunk + t * 32;
    const int grp = kabs / p.group;
#pragma unroll
    for (int r = 0; r < kRowGroups; ++r) {
      const int n = row0 + r * 8 + g;
      if (n < p.N) {
        qn[r] = ldg_stream_v4(p.packed + (size_t)n * words_per_row + (kabs >> 3));
        szn[r] = __ldg(p.sz + (size_t)grp * p.N + n);
      } else {
        qn[r] = make_uint4(0, 0, 0, 0);
        szn[r] = 0;
      }
    }
  };

  int my = cs + wk;
  if (my < ce) prefetch(my);

  for (int stage0 = cs; stage0 < ce; stage0 += STAGE) {
    const int nch = min(STAGE, ce - stage0);
    __syncthreads();  // the previous stage's fragments have been consumed
    // Stage activations: 16-byte units of 8 columns, permuted to (k0,k4,k1,k5,k2,k6,k3,k7)
    // and stored at [chunk][c][mb][half][g][t] so that a warp's fragment load is contiguous.
    const int units = nch * 16;
    for (int idx = tid; idx < TOK * units; idx += THREADS) {
      const int m = idx / units, u = idx - m * units;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < p.M) {
        const uint4 in = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + (size_t)(stage0 * kChunk + u * 8));
        v.x = prmt(in.x, in.z, 0x5410);  // (k0, k4)
        v.y = prmt(in.x, in.z, 0x7632);  // (k1, k5)
        v.z = prmt(in.y, in.w, 0x5410);  // (k2, k6)
        v.w = prmt(in.y, in.w, 0x7632);  // (k3, k7)
      }
      const int kc = u >> 4, tt = (u >> 2) & 3, c = u & 3;
      const int mb = m / (HR * 8), hr = (m / 8) % HR, gg = m & 7;
      xs[((((kc * 4 + c) * MB + mb) * HR + hr) * 8 + gg) * 4 + tt] = v;
    }
    __syncthreads();

#pragma unroll 1
    for (int j = 0; j < STAGE / kWarpsK; ++j) {
      if (my >= stage0 + nch) break;
      uint4 q[kRowGroups];
      ScaleZero sp[kRowGroups];
#pragma unroll
      for (int r = 0; r < kRowGroups; ++r) {
        q[r] = qn[r];
        const __half2 h = *reinterpret_cast<const __half2*>(&szn[r]);
        sp[r] = make_scale_zero(__low2half(h), __high2half(h));
      }
      if (my + kWarpsK < ce) prefetch(my + kWarpsK);
      const int kc = my - stage0;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 alo[MB], ahi[MB];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int base = (((kc * 4 + c) * MB + mb) * HR) * 32 + lane;
          alo[mb] = xs[base];
          ahi[mb] = HALF ? make_uint4(0, 0, 0, 0) : xs[base + 32];
        }
#pragma unroll
        for (int r = 0; r < kRowGroups; ++r) {
          const uint32_t word = c == 0 ? q[r].x : c == 1 ? q[r].y : c == 2 ? q[r].z : q[r].w;
          __half2 v[4];
          dequant8(word, sp[r], v);
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            mma_m16n8k16(acc[mb][r], alo[mb].x, ahi[mb].x, alo[mb].y, ahi[mb].y, h2_as_u32(v[0]), h2_as_u32(v[1]));
            mma_m16n8k16(acc[mb][r], alo[mb].z, ahi[mb].z, alo[mb].w, ahi[mb].w, h2_as_u32(v[2]), h2_as_u32(v[3]));
          }
        }
      }
      my += kWarpsK;
    }
  }

  // ---- reduce the K-warps of this block: red[wk][wn][m][32 rows] ----
  constexpr int MROWS = MB * 16;
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int r = 0; r < kRowGroups; ++r) {
      float* base = red + (((size_t)(wk * WN + wn) * MROWS + mb * 16 + g) * 32 + r * 8 + 2 * t);
      *reinterpret_cast<float2*>(base) = make_float2(acc[mb][r][0], acc[mb][r][1]);
      if (!HALF) *reinterpret_cast<float2*>(base + 8 * 32) = make_float2(acc[mb][r][2], acc[mb][r][3]);
    }
  __syncthreads();

  const int nl = tid & 31;                 // row inside a 32-row warp tile
  const int grp_m = tid >> 5;              // THREADS/32 (m, wn) pairs per pass
  const bool direct = p.k_split == 1;
  for (int e = grp_m; e < WN * p.M; e += THREADS / 32) {
    const int wn2 = e / p.M, m = e - wn2 * p.M;
    const int n = blockIdx.x * ROWS + wn2 * 32 + nl;
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kWarpsK; ++k) s += red[((size_t)(k * WN + wn2) * MROWS + m) * 32 + nl];
    if (n < p.N) {
      if (direct) {
        if (p.bias) s += h2f(p.bias[n]);
        p.y[(size_t)m * p.N + n] = f2h(s);
      } else {
        p.partials[((size_t)split * p.M + m) * p.N + n] = s;
      }
    }
  }
  if (direct) return;

  // ---- cross-slice reduction by the block that arrives last ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(p.counters + blockIdx.x, 1);
    s_last = (prev == p.k_split - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = grp_m; e < WN * p.M; e += THREADS / 32) {
    const int wn2 = e / p.M, m = e - wn2 * p.M;
    const int n = blockIdx.x * ROWS + wn2 * 32 + nl;
    if (n >= p.N) continue;
    float s = 0.0f;
    for (int k = 0; k < p.k_split; ++k) s += __ldcg(p.partials + ((size_t)k * p.M + m) * p.N + n);
    if (p.bias) s += h2f(p.bias[n]);
    p.y[(size_t)m * p.N + n] = f2h(s);
  }
  if (tid == 0) p.counters[blockIdx.x] = 0;  // ready for the next call
}


// ---------------------------------------------------------------------------
// M <= 16: split K across a thread-block cluster and reduce through
// distributed shared memory -- no scratch, no atomics, no second pass.
//
// A block of 16 warps (4 row-warps x 4 K-warps) owns 128 output rows and 1/CK
// of K; the CK blocks of a cluster cover all of K for the same rows.  Work is
// cut fine so that thousands of warps are in flight on a problem of a few
// megabytes: one warp step is one 128-column chunk of 32 rows (four independent
// 128-bit loads per lane).  Per round the block stages the four chunks of
// activations its K-warps need once, for all four row-warps; every per-warp
// index is computed once, outside the round loop.  The reduction is a push:
// block r of the cluster owns output columns [r*128/CK, (r+1)*128/CK); after
// its last round every warp stores its accumulator fragments straight into
// the owner's shared memory (one slot per (block, K-warp), so nothing is
// overwritten), one cluster barrier makes the stores visible, and each owner
// adds its 4*CK slots in a fixed order (deterministic), adds the bias and
// writes fp16.  A barrier arrive at kernel entry, waited on just before the
// first remote store, guarantees every block of the cluster is running.
//
// The first round's weight loads are issued before griddepcontrol.wait, so
// that under programmatic dependent launch they overlap the tail of the
// preceding kernel; everything that touches x, bias or y comes after it.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

constexpr int kClusterRows = 128;   // output rows per block of the cluster kernel
constexpr int kClusterThreads = 512;

template <bool HALF>
__global__ void __launch_bounds__(kClusterThreads, 2)
w4a16_decode_cluster_kernel(const DecodeParams p) {
  namespace cg = cooperative_groups;
  constexpr int HR = HALF ? 1 : 2;
  constexpr int MROWS = HALF ? 8 : 16;
  __shared__ __align__(16) uint4 xs[kWarpsK * 4 * HR * 32];            // one round: 4 chunks
  // slots[(src block * 4 + K-warp)][m][column of this owner]: 4*CK slots of MROWS x (128/CK) floats
  __shared__ __align__(16) float slots[kWarpsK * MROWS * kClusterRows];

  cg::cluster_group cluster = cg::this_cluster();
  const int ck = static_cast<int>(cluster.num_blocks());
  const int crank = static_cast<int>(cluster.block_rank());
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "I am running"; waited on before the pushes
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wk = warp & 3, wn = warp >> 2;
  const int row0 = blockIdx.x * kClusterRows + wn * 32;
  const int cs = min(p.chunks, crank * p.chunks_per_split);
  const int ce = min(p.chunks, cs + p.chunks_per_split);
  const int words_per_row = p.K >> 3;
  const bool group_is_chunk = p.group == kChunk;

  float acc[kRowGroups][4];
#pragma unroll
  for (int r = 0; r < kRowGroups; ++r)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[r][i] = 0.0f;

  // per-lane weight pointer: row (row0 + g), 16-byte column slot t, this warp's first chunk; the
  // other row groups are 8 rows further each.  N % 8 == 0, so a row group is valid as a whole.
  const int rows_left = p.N - row0;                                      // valid rows of this warp
  const int vec_per_row = words_per_row >> 2;                            // uint4 per weight row
  const uint4* wptr = reinterpret_cast<const uint4*>(p.packed) +
                      (size_t)(rows_left > 0 ? row0 + g : 0) * vec_per_row + t + (cs + wk) * (kChunk / 32);
  const uint32_t* szptr = p.sz + (rows_left > 0 ? row0 + g : 0);

  // staging slot of this thread: unit u (8 columns) of token row m_lo (and m_lo + 8)
  const int st_u = tid & 63, st_m = tid >> 6;                           // 64 units x 8 rows per pass
  const int st_dst = (((st_u >> 4) * 4 + (st_u & 3)) * HR * 8 + st_m) * 4 + ((st_u >> 2) & 3);
  const __half* st_src = p.x + (size_t)st_m * p.K + st_u * 8;

  uint4 q[kRowGroups];
  uint32_t szv[kRowGroups];
  auto load_chunk = [&](int chunk) {
    const int grp = group_is_chunk ? chunk : (chunk * kChunk + t * 32) / p.group;
    const uint32_t* sp = szptr + (size_t)grp * p.N;
#pragma unroll
    for (int r = 0; r < kRowGroups; ++r) {
      if (chunk < ce && r * 8 < rows_left) {
        q[r] = ldg_stream_v4(wptr + (size_t)r * 8 * vec_per_row);
        szv[r] = __ldg(sp + r * 8);
      } else {
        q[r] = make_uint4(0, 0, 0, 0);
        szv[r] = 0;
      }
    }
    wptr += kWarpsK * (kChunk / 32);                                    // next round: four chunks on
  };

  MP_TRACE_POINT(0);
  load_chunk(cs + wk);
  grid_launch_dependents();
  grid_dependency_wait();
  MP_TRACE_POINT(1);

  for (int c_begin = cs; c_begin < ce; c_begin += kWarpsK) {
    if (c_begin != cs) {
      __syncthreads();                       // the previous round's fragments have been consumed
      load_chunk(c_begin + wk);
    }
    // stage x[:, 4 chunks]: unit (m, u) -> fragment order [chunk][c][half][g][t], nibble-permuted
#pragma unroll
    for (int hr = 0; hr < HR; ++hr) {
      const int m = st_m + hr * 8;
      const int col = c_begin * kChunk + st_u * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < p.M && col < p.K) {
        const uint4 in = *reinterpret_cast<const uint4*>(st_src + (size_t)hr * 8 * p.K + c_begin * kChunk);
        v.x = prmt(in.x, in.z, 0x5410);
        v.y = prmt(in.x, in.z, 0x7632);
        v.z = prmt(in.y, in.w, 0x5410);
        v.w = prmt(in.y, in.w, 0x7632);
      }
      xs[st_dst + hr * 32] = v;
    }
    __syncthreads();
    MP_TRACE_POINT(2);
    if (c_begin + wk < ce) {
      ScaleZero sp[kRowGroups];
#pragma unroll
      for (int r = 0; r < kRowGroups; ++r) {
        const __half2 h = *reinterpret_cast<const __half2*>(&szv[r]);
        sp[r] = make_scale_zero(__low2half(h), __high2half(h));
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int base = ((wk * 4 + c) * HR) * 32 + lane;
        const uint4 alo = xs[base];
        const uint4 ahi = HALF ? make_uint4(0, 0, 0, 0) : xs[base + 32];
#pragma unroll
        for (int r = 0; r < kRowGroups; ++r) {
          const uint32_t word = c == 0 ? q[r].x : c == 1 ? q[r].y : c == 2 ? q[r].z : q[r].w;
          __half2 v[4];
          dequant8(word, sp[r], v);
          mma_m16n8k16(acc[r], alo.x, ahi.x, alo.y, ahi.y, h2_as_u32(v[0]), h2_as_u32(v[1]));
          mma_m16n8k16(acc[r], alo.z, ahi.z, alo.w, ahi.w, h2_as_u32(v[2]), h2_as_u32(v[3]));
        }
      }
    }
  }

  MP_TRACE_POINT(3);
  // push the fragments to the owners of their columns
  const int cols = kClusterRows / ck;              // columns each block owns
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // every block of the cluster has started
  MP_TRACE_POINT(4);
#pragma unroll
  for (int r = 0; r < kRowGroups; ++r) {
    const int n_local = wn * 32 + r * 8 + 2 * t;
    const int owner = n_local / cols, c_in = n_local - owner * cols;
    float* dst = cluster.map_shared_rank(slots, owner) + ((size_t)((crank * kWarpsK + wk) * MROWS + g) * cols + c_in);
    *reinterpret_cast<float2*>(dst) = make_float2(acc[r][0], acc[r][1]);
    if (!HALF) *reinterpret_cast<float2*>(dst + 8 * cols) = make_float2(acc[r][2], acc[r][3]);
  }
  MP_TRACE_POINT(5);
  cluster.sync();                                  // remote stores are visible; nobody is written to after this
  MP_TRACE_POINT(6);
  const int n_slots = ck * kWarpsK;
  for (int e = tid; e < p.M * cols; e += kClusterThreads) {
    const int m = e / cols, c = e - m * cols;
    const int n = blockIdx.x * kClusterRows + crank * cols + c;
    float s = 0.0f;
    for (int sl = 0; sl < n_slots; ++sl) s += slots[(sl * MROWS + m) * cols + c];   // fixed order: deterministic
    if (n < p.N) {
      if (p.bias) s += h2f(p.bias[n]);
      p.y[(size_t)m * p.N + n] = f2h(s);
    }
  }
  MP_TRACE_POINT(7);
}

static bool g_programmatic_launch = false;

template <bool HALF>
static int launch_decode_cluster(const DecodeParams& p, int row_blocks, int ck, cudaStream_t st) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(row_blocks, ck, 1);
  cfg.blockDim = dim3(kClusterThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 1;
  attrs[0].val.clusterDim.y = ck;
  attrs[0].val.clusterDim.z = 1;
  int n_attrs = 1;
  if (g_programmatic_launch) {
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    n_attrs = 2;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a16_decode_cluster_kernel<HALF>, p));
  return MP_OK;
}

struct DecodePlan {
  int mb;        // 16-row token blocks
  bool half;     // M <= 8
  int wn;        // warps along rows
  int stage;     // staged chunks
  int rows;      // rows per block
  int row_blocks;
  int k_split;
  int chunks_per_split;
  size_t smem;
};

static DecodePlan plan_decode(int M, int N, int K, int k_split_req) {
  DecodePlan pl{};
  pl.mb = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  pl.half = M <= 8;
  pl.wn = M <= 8 ? 1 : 2;
  pl.stage = pl.mb == 1 ? 8 : 4;
  pl.rows = pl.wn * 32;
  pl.row_blocks = (N + pl.rows - 1) / pl.rows;
  const int chunks = K / kChunk;
  int ks = k_split_req;
  if (ks <= 0) {
    // Aim at roughly 512 resident warps' worth of blocks over the 148 SMs while
    // keeping at least one chunk per K-warp in every slice.
    const int target_blocks = kSmCount * (pl.wn == 1 ? 6 : 3);
    ks = (target_blocks + pl.row_blocks / 2) / pl.row_blocks;
  }
  ks = ks < 1 ? 1 : ks;
  int cps = (chunks + ks - 1) / ks;
  if (cps < kWarpsK && chunks >= kWarpsK) cps = kWarpsK;
  pl.chunks_per_split = cps;
  pl.k_split = (chunks + cps - 1) / cps;
  const int hr = pl.half ? 1 : 2;
  pl.smem = (size_t)pl.stage * 4 * pl.mb * hr * 32 * 16 + (size_t)kWarpsK * pl.wn * pl.mb * 16 * 32 * sizeof(float);
  return pl;
}

constexpr size_t kCounterBytes = 16384;  // room for 4096 row blocks

template <int MB, bool HALF, int WN, int STAGE>
static int launch_decode(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st) {
  auto kern = w4a16_decode_kernel<MB, HALF, WN, STAGE>;
  // Static + dynamic shared memory can pass the 48 KB default together; opt in once per device.
  static thread_local int configured_device = -1;
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    MP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    configured_device = device;
  }
  dim3 grid(pl.row_blocks, pl.k_split);
  kern<<<grid, WN * kWarpsK * 32, pl.smem, st>>>(p);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

}  // namespace mp

using namespace mp;

extern "C" size_t mp_w4a16_decode_workspace_bytes_ex(int M, int N, int K, int k_split) {
  if (M <= 0 || M > 64 || N <= 0 || K <= 0 || K % kChunk != 0) return 0;
  if (M <= 16 && k_split <= 0) {             // partial tiles of the persistent tcgen05 kernels; the mma.sync kernels need none
    return g_decode_kernel == MP_DECODE_KERNEL_MMA_SYNC ? 0 : decode_umma_workspace_bytes(M);
  }
  const DecodePlan pl = plan_decode(M, N, K, k_split);
  const size_t split_k = kCounterBytes + (size_t)pl.k_split * (size_t)M * (size_t)N * sizeof(float);
  if (k_split <= 0 && g_decode_kernel != MP_DECODE_KERNEL_MMA_SYNC && decode_umma_workspace_bytes(M) > split_k)
    return decode_umma_workspace_bytes(M);   // 17..64 rows may take the tcgen05 kernel with a wider activation tile
  return split_k;
}

extern "C" size_t mp_w4a16_decode_workspace_bytes(int M, int N, int K) {
  return mp_w4a16_decode_workspace_bytes_ex(M, N, K, 0);
}

static int decode_linear(const void* x_f16, const void* packed_i32, const void* sz_f16x2, const void* bias_f16,
                         void* y_f16, int M, int N, int K, int group, void* workspace, size_t workspace_bytes,
                         int k_split, int kind, int pdl_choice, mp_stream_t stream);

extern "C" int mp_w4a16_linear_decode_ex(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                         const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                         void* workspace, size_t workspace_bytes, int k_split,
                                         mp_stream_t stream) {
  return decode_linear(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, workspace, workspace_bytes,
                       k_split, g_decode_kernel, -1, stream);
}

extern "C" int mp_w4a16_linear_decode_opts(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                           const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                           void* workspace, size_t workspace_bytes, unsigned int options,
                                           mp_stream_t stream) {
  const unsigned int k = options & MP_DECODE_OPT_KERNEL_MASK;
  int kind = g_decode_kernel;
  if (k == MP_DECODE_OPT_KERNEL_MMA_SYNC) kind = MP_DECODE_KERNEL_MMA_SYNC;
  else if (k == MP_DECODE_OPT_KERNEL_UMMA) kind = MP_DECODE_KERNEL_UMMA;
  else if (k == MP_DECODE_OPT_KERNEL_AUTO) kind = MP_DECODE_KERNEL_AUTO;
  else if (k != 0) return MP_ERR_INVALID_ARG;
  const unsigned int pd = options & MP_DECODE_OPT_PDL_MASK;
  if (pd == MP_DECODE_OPT_PDL_MASK) return MP_ERR_INVALID_ARG;
  const int pdl_choice = pd == MP_DECODE_OPT_PDL_ON ? 1 : pd == MP_DECODE_OPT_PDL_OFF ? 0 : -1;
  if (M > 64) return MP_ERR_UNSUPPORTED;
  return decode_linear(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, workspace, workspace_bytes, 0,
                       kind, pdl_choice, stream);
}

static int decode_linear(const void* x_f16, const void* packed_i32, const void* sz_f16x2, const void* bias_f16,
                         void* y_f16, int M, int N, int K, int group, void* workspace, size_t workspace_bytes,
                         int k_split, int kind, int pdl_choice, mp_stream_t stream) {
  if (!x_f16 || !packed_i32 || !sz_f16x2 || !y_f16 || M <= 0 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (M > 64 || K % kChunk != 0 || group % 32 != 0 || K % group != 0 || N % 8 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || !aligned(packed_i32, 16) || !aligned(sz_f16x2, 4) || !aligned(y_f16, 2)) return MP_ERR_ALIGNMENT;
  DecodeParams p{};
  p.x = static_cast<const __half*>(x_f16);
  p.packed = static_cast<const uint32_t*>(packed_i32);
  p.sz = static_cast<const uint32_t*>(sz_f16x2);
  p.bias = static_cast<const __half*>(bias_f16);
  p.y = static_cast<__half*>(y_f16);
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.chunks = K / kChunk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M <= 16 && k_split <= 0) {
    const bool pdl = pdl_choice < 0 ? decode_programmatic_launch() : pdl_choice != 0;
    const int chosen = decode_kernel_for(kind, M, N, K, workspace != nullptr && workspace_bytes > 0);
    if (chosen == MP_DECODE_KERNEL_UMMA) {
      const int rc_umma = launch_decode_umma(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, workspace,
                                             workspace_bytes, st, pdl);
      if (rc_umma != MP_ERR_UNSUPPORTED) return rc_umma;
    }
    // the TMA-fed mma.sync ring kernel; shapes it does not take fall through to the register-streaming one
    const int rc_tma = launch_decode_tma(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, st, nullptr,
                                         pdl ? 1 : 0);
    if (rc_tma != MP_ERR_UNSUPPORTED) return rc_tma;
    // cluster split-K: the smallest power of two (<= 8, the portable limit) that puts about two
    // 16-warp blocks on every SM, as long as every block keeps at least one chunk per K-warp
    const int row_blocks_ = (N + kClusterRows - 1) / kClusterRows;
    int ck = 1;
    while (ck < 8 && row_blocks_ * ck < 2 * kSmCount && p.chunks >= 2 * ck * kWarpsK) ck <<= 1;
    p.chunks_per_split = (p.chunks + ck - 1) / ck;
    p.k_split = ck;
    const int row_blocks = (N + kClusterRows - 1) / kClusterRows;
    return M <= 8 ? launch_decode_cluster<true>(p, row_blocks, ck, st)
                  : launch_decode_cluster<false>(p, row_blocks, ck, st);
  }
  if (M > 16 && k_split <= 0 && umma_above_16_rows(kind, M, N, K)) {
    const bool pdl = pdl_choice < 0 ? decode_programmatic_launch() : pdl_choice != 0;
    const int rc_umma = launch_decode_umma(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, workspace,
                                           workspace_bytes, st, pdl);
    if (rc_umma != MP_ERR_UNSUPPORTED) return rc_umma;
  }
  const DecodePlan pl = plan_decode(M, N, K, k_split);
  if ((size_t)pl.row_blocks * sizeof(int) > kCounterBytes) return MP_ERR_UNSUPPORTED;
  p.chunks_per_split = pl.chunks_per_split;
  p.k_split = pl.k_split;
  if (pl.k_split > 1) {
    const size_t need = kCounterBytes + (size_t)pl.k_split * M * N * sizeof(float);
    if (!workspace || workspace_bytes < need) return MP_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return MP_ERR_ALIGNMENT;
    p.counters = static_cast<int*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kCounterBytes);
  }
  if (pl.mb == 1 && pl.half) return launch_decode<1, true, 1, 8>(p, pl, st);
  if (pl.mb == 1) return launch_decode<1, false, 2, 8>(p, pl, st);
  if (pl.mb == 2) return launch_decode<2, false, 2, 4>(p, pl, st);
  return launch_decode<4, false, 2, 4>(p, pl, st);
}

// ---- row-parallel decode: K sharded over GPUs; every rank leaves its partial sums in its own buffer,
// raises its arrival word on the peers, and each rank adds all buffers ------------------------------------
struct PeerPartials {
  const float* p[2][kMaxPeerRanks];     // [buffer parity][rank]
};

// out[m, n] = f16(sum_r partial_r[m][n] (+ bias)), ranks in ascending order (every GPU computes the same
// bits); partial_r is read from rank r's memory over NVLink.  Each block first waits (bounded) until every
// rank's arrival word has reached `epoch`.
__global__ void __launch_bounds__(256)
rowparallel_finish_kernel(PeerPartials partial, const unsigned int* __restrict__ flags, int world,
                          const unsigned int* __restrict__ epoch_counter, int M, int N,
                          const __half* __restrict__ bias, __half* __restrict__ y, int* error_word) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const unsigned int epoch = *epoch_counter;           // advanced by the push kernel that ran before this one
  const float* const* src = partial.p[epoch & 1u];
  if (threadIdx.x < world) {
    const unsigned int* f = flags + threadIdx.x;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned int it = 0;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;                  // rank threadIdx.x has stored (wrap-safe)
      if ((it & 0xFF) == 0xFF) {
        uint64_t now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > 2000000000ull) {                              // 2 s: give up, report, write nothing
          s_ok = 0;
          if (error_word) atomicExch(error_word, 5);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int quads = N >> 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * quads; i += gridDim.x * blockDim.x) {
    const int m = i / quads, n = (i - m * quads) << 2;
    // all ranks' loads are issued before the first add: one NVLink round trip, not one per rank
    float4 v[kMaxPeerRanks];
#pragma unroll
    for (int r = 0; r < kMaxPeerRanks; ++r)
      if (r < world) v[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)m * N + n);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxPeerRanks; ++r)
      if (r < world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
    if (bias) {
      acc.x += h2f(bias[n]); acc.y += h2f(bias[n + 1]); acc.z += h2f(bias[n + 2]); acc.w += h2f(bias[n + 3]);
    }
    const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
    *reinterpret_cast<uint2*>(y + (size_t)m * N + n) = make_uint2(h2_as_u32(lo), h2_as_u32(hi));
  }
}

extern "C" int mp_w4a16_rowparallel_push(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                         void* partial0_f32, void* partial1_f32, void* const* peer_flags_u32,
                                         int* block_counter, void* epoch_counter_u32, int world, int rank, int M, int N,
                                         int K_local, int group, mp_stream_t stream) {
  if (!x_f16 || !packed_i32 || !sz_f16x2 || !partial0_f32 || !partial1_f32 || !peer_flags_u32 || !block_counter ||
      !epoch_counter_u32 || M <= 0 || N <= 0 || K_local <= 0 || group <= 0)
    return MP_ERR_INVALID_ARG;
  if (world < 1 || world > kMaxPeerRanks || rank < 0 || rank >= world) return MP_ERR_INVALID_ARG;
  if (M > 16 || K_local % group != 0 || N % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(partial0_f32, 16) || !aligned(partial1_f32, 16)) return MP_ERR_ALIGNMENT;
  DecodePush push{};
  for (int q = 0; q < world; ++q) {
    if (!peer_flags_u32[q]) return MP_ERR_INVALID_ARG;
    push.flags[q] = static_cast<unsigned int*>(peer_flags_u32[q]);
  }
  push.partial[0] = static_cast<float*>(partial0_f32);
  push.partial[1] = static_cast<float*>(partial1_f32);
  push.block_counter = block_counter;
  push.epoch = static_cast<unsigned int*>(epoch_counter_u32);
  push.world = world; push.rank = rank;
  // only the TMA-fed kernel has this epilogue; shapes it does not take are reported as unsupported
  return launch_decode_tma(x_f16, packed_i32, sz_f16x2, nullptr, nullptr, M, N, K_local, group,
                           static_cast<cudaStream_t>(stream), &push);
}

extern "C" int mp_w4a16_rowparallel_finish(void* const* peer_partial0_f32, void* const* peer_partial1_f32,
                                           const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                                           int N, const void* bias_f16, void* y_f16, int* error_word,
                                           mp_stream_t stream) {
  if (!peer_partial0_f32 || !peer_partial1_f32 || !flags_u32 || !epoch_counter_u32 || !y_f16 || world < 1 ||
      world > kMaxPeerRanks || M <= 0 || N <= 0)
    return MP_ERR_INVALID_ARG;
  if (N % 4 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(y_f16, 8)) return MP_ERR_ALIGNMENT;
  PeerPartials pp{};
  for (int r = 0; r < world; ++r) {
    if (!peer_partial0_f32[r] || !peer_partial1_f32[r]) return MP_ERR_INVALID_ARG;
    if (!aligned(peer_partial0_f32[r], 16) || !aligned(peer_partial1_f32[r], 16)) return MP_ERR_ALIGNMENT;
    pp.p[0][r] = static_cast<const float*>(peer_partial0_f32[r]);
    pp.p[1][r] = static_cast<const float*>(peer_partial1_f32[r]);
  }
  int blocks = (M * (N / 4) + 255) / 256;
  if (blocks > kSmCount) blocks = kSmCount;
  rowparallel_finish_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const unsigned int*>(flags_u32), world, static_cast<const unsigned int*>(epoch_counter_u32), M, N,
      static_cast<const __half*>(bias_f16), static_cast<__half*>(y_f16), error_word);
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w4a16_linear_decode_host_ws(const void* x_host_f16, void* x_stage_f16, const void* packed_i32,
                                              const void* sz_f16x2, const void* bias_f16, void* y_stage_f16,
                                              void* y_host_f16, int M, int N, int K, int group, void* workspace,
                                              size_t workspace_bytes, mp_stream_t stream) {
  if (!x_host_f16 || !x_stage_f16 || !y_stage_f16) return MP_ERR_INVALID_ARG;
  if (M > 16) return MP_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MP_CUDA_TRY(cudaMemcpyAsync(x_stage_f16, x_host_f16, (size_t)M * K * sizeof(__half), cudaMemcpyHostToDevice, st));
  // without a workspace: the scratch-free kernels only
  const int rc = mp_w4a16_linear_decode_ex(x_stage_f16, packed_i32, sz_f16x2, bias_f16, y_stage_f16, M, N, K, group,
                                           workspace, workspace ? workspace_bytes : 0, 0, stream);
  if (rc != MP_OK) return rc;
  // no y_host: the result stays where the kernel stored it (y_stage may be the device alias of a pinned host
  // buffer, see mp_host_buffer_device_alias: the kernel's stores then are the device-to-host transfer)
  if (y_host_f16)
    MP_CUDA_TRY(cudaMemcpyAsync(y_host_f16, y_stage_f16, (size_t)M * N * sizeof(__half), cudaMemcpyDeviceToHost, st));
  return MP_OK;
}

extern "C" int mp_w4a16_linear_decode_host(const void* x_host_f16, void* x_stage_f16, const void* packed_i32,
                                           const void* sz_f16x2, const void* bias_f16, void* y_stage_f16,
                                           void* y_host_f16, int M, int N, int K, int group, mp_stream_t stream) {
  return mp_w4a16_linear_decode_host_ws(x_host_f16, x_stage_f16, packed_i32, sz_f16x2, bias_f16, y_stage_f16, y_host_f16,
                                        M, N, K, group, nullptr, 0, stream);
}

extern "C" int mp_w4a16_linear_decode_host_many(const mp_host_linear* linears, int count, mp_stream_t stream) {
  if (!linears || count <= 0) return MP_ERR_INVALID_ARG;
  for (int i = 0; i < count; ++i) {
    const mp_host_linear& c = linears[i];
    if (!c.x_host_f16 || !c.x_stage_f16 || !c.y_stage_f16 || c.M <= 0 || c.K <= 0 || c.N <= 0) return MP_ERR_INVALID_ARG;
    if (c.M > 16) return MP_ERR_UNSUPPORTED;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < count; ++i) {
    const mp_host_linear& c = linears[i];
    MP_CUDA_TRY(cudaMemcpyAsync(c.x_stage_f16, c.x_host_f16, (size_t)c.M * c.K * sizeof(__half), cudaMemcpyHostToDevice, st));
  }
  for (int i = 0; i < count; ++i) {
    const mp_host_linear& c = linears[i];
    const int rc = mp_w4a16_linear_decode_ex(c.x_stage_f16, c.packed_i32, c.sz_f16x2, c.bias_f16, c.y_stage_f16, c.M, c.N,
                                             c.K, c.group, c.workspace, c.workspace ? c.workspace_bytes : 0, 0, stream);
    if (rc != MP_OK) return rc;
  }
  for (int i = 0; i < count; ++i) {
    const mp_host_linear& c = linears[i];
    if (c.y_host_f16)
      MP_CUDA_TRY(cudaMemcpyAsync(c.y_host_f16, c.y_stage_f16, (size_t)c.M * c.N * sizeof(__half), cudaMemcpyDeviceToHost, st));
  }
  return MP_OK;
}

extern "C" int mp_host_buffer_device_alias(const void* host_ptr, size_t bytes, void** device_ptr) {
  if (!host_ptr || !device_ptr || bytes == 0) return MP_ERR_INVALID_ARG;
  *device_ptr = nullptr;
  cudaPointerAttributes first{}, last{};
  MP_CUDA_TRY(cudaPointerGetAttributes(&first, host_ptr));
  MP_CUDA_TRY(cudaPointerGetAttributes(&last, static_cast<const char*>(host_ptr) + bytes - 1));
  if (first.type != cudaMemoryTypeHost || last.type != cudaMemoryTypeHost || !first.devicePointer ||
      !last.devicePointer)
    return MP_ERR_UNSUPPORTED;                      // pageable memory, or not mapped for this device
  if (static_cast<const char*>(last.devicePointer) - static_cast<const char*>(first.devicePointer) !=
      static_cast<ptrdiff_t>(bytes - 1))
    return MP_ERR_UNSUPPORTED;                      // the range spans two registrations
  if (!aligned(first.devicePointer, 16)) return MP_ERR_ALIGNMENT;
  *device_ptr = first.devicePointer;
  return MP_OK;
}

extern "C" int mp_w4a16_linear_decode(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                      const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                      void* workspace, size_t workspace_bytes, mp_stream_t stream) {
  return mp_w4a16_linear_decode_ex(x_f16, packed_i32, sz_f16x2, bias_f16, y_f16, M, N, K, group, workspace,
                                   workspace_bytes, 0, stream);
}

extern "C" int mp_w4a16_decode_kernel_choice(int M, int N, int K, int have_workspace) {
  if (M <= 0 || M > 64 || N <= 0 || K <= 0) return MP_ERR_INVALID_ARG;
  if (M > 16) return have_workspace && umma_above_16_rows(g_decode_kernel, M, N, K) ? MP_DECODE_KERNEL_UMMA
                                                                                    : MP_DECODE_KERNEL_MMA_SYNC;
  return decode_kernel_for(g_decode_kernel, M, N, K, have_workspace != 0);
}

extern "C" int mp_set_decode_kernel(int kind) {
  if (kind != MP_DECODE_KERNEL_MMA_SYNC && kind != MP_DECODE_KERNEL_UMMA && kind != MP_DECODE_KERNEL_AUTO)
    return MP_ERR_INVALID_ARG;
  const int prev = g_decode_kernel;
  g_decode_kernel = kind;
  return prev;
}

extern "C" int mp_set_programmatic_launch(int enabled) {
  const int prev = g_programmatic_launch ? 1 : 0;
  g_programmatic_launch = enabled != 0;
  set_decode_programmatic_launch(g_programmatic_launch);
  return prev;
}

// ---------------------------------------------------------------------------
// Split-K decode linear for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain scratch for the split-K
// partial sums: a plugin running inside another runtime's forward pass whose
// memory pool is closed to it, code executing in a context where cudaMalloc is
// off limits (inside a capture region set up by someone else, in a callback, in
// a process with a frozen memory budget).  For them the workspace of the
// split-K kernel lives in the fixed array below, which every GPU that loads the
// library holds until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB: counters + partial sums
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_ptr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

// The array's name is only a host-side handle; the address kernels can use comes
// from the runtime, once per device, with that device current.
static int static_scratch_for_current_device(void** out) {
  int device = 0;
  MP_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return MP_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    MP_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_decode_scratch));
    if (ptr == nullptr) return MP_ERR_CUDA;
    g_static_scratch_ptr[device] = ptr;
  }
  *out = g_static_scratch_ptr[device];
  return MP_OK;
}

extern "C" size_t mp_w4a16_linear_decode_static_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int mp_w4a16_linear_decode_static(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                             const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                             mp_stream_t stream) {
  if (!x_f16 || !packed_i32 || !sz_f16x2 || !y_f16 || M <= 0 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (M > 64 || K % kChunk != 0 || group % 32 != 0 || K % group != 0 || N % 8 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || !aligned(packed_i32, 16) || !aligned(sz_f16x2, 4) || !aligned(y_f16, 2)) return MP_ERR_ALIGNMENT;
  const DecodePlan pl = plan_decode(M, N, K, 0);
  if ((size_t)pl.row_blocks * sizeof(int) > kCounterBytes) return MP_ERR_UNSUPPORTED;
  const size_t need = kCounterBytes + (pl.k_split > 1 ? (size_t)pl.k_split * M * N * sizeof(float) : 0);
  if (need > kStaticScratchBytes) return MP_ERR_WORKSPACE;     // beyond the fixed scratch: use the workspace entry point
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != MP_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left; the arrival counters must start at zero.
  MP_CUDA_TRY(cudaMemsetAsync(scratch, 0, kCounterBytes, st));
  DecodeParams p{};
  p.x = static_cast<const __half*>(x_f16);
  p.packed = static_cast<const uint32_t*>(packed_i32);
  p.sz = static_cast<const uint32_t*>(sz_f16x2);
  p.bias = static_cast<const __half*>(bias_f16);
  p.y = static_cast<__half*>(y_f16);
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.chunks = K / kChunk;
  p.chunks_per_split = pl.chunks_per_split;
  p.k_split = pl.k_split;
  p.counters = static_cast<int*>(scratch);
  p.partials = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kCounterBytes);
  if (pl.mb == 1 && pl.half) return launch_decode<1, true, 1, 8>(p, pl, st);
  if (pl.mb == 1) return launch_decode<1, false, 2, 8>(p, pl, st);
  if (pl.mb == 2) return launch_decode<2, false, 2, 4>(p, pl, st);
  return launch_decode<4, false, 2, 4>(p, pl, st);
}

extern "C" int mp_read_decode_error(int* value) {
  if (!value) return MP_ERR_INVALID_ARG;
  return read_and_clear_decode_error(value);
}
